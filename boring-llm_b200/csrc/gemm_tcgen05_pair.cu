// Matrix product for many rows on PAIRS of SMs: out[M, N] = epilogue(x[M, K] . W[N, K]^T), bfloat16 operands,
// 32-bit accumulation in tensor memory, tcgen05.mma with cta_group::2, persistent blocks.
//
// Two blocks of a cluster compute 256 x BN tiles of the output (BN 256, or 128 where 256 would leave SMs idle).
// Each block loads its own 128 rows of x and HALF of the tile's rows of W per 64-wide k block, but the pair
// multiplies 256 x BN x 64 with them: twice the arithmetic per byte that crosses from L2 into shared memory.
// The leader block (cluster rank 0) issues the MMAs for both; the hardware reads x tiles and W halves from both
// blocks' shared memory and writes each block's 128 rows of the accumulator into that block's tensor memory.
//
// One pair per two SMs stays resident and walks over tiles (tile t, t + pairs, ...). The round trip "stage free ->
// TMA -> data landed -> MMA done -> stage free" takes a couple of microseconds, so five to seven stages are kept in flight,
// and the accumulator is double buffered in tensor memory (2 x 256 columns): while the eight epilogue warps drain
// one tile, the issuer already fills the next, and the loaders never stop.
//
//   warp 0, one thread in EACH block (loader): waits for its own stage to be free, TMA-loads its x tile and its half
//     of W. Both blocks' copies report their bytes to the LEADER's "full" barrier (the .cta_group::2 form of
//     cp.async.bulk.tensor, barrier address with the peer bit cleared); the leader expects the bytes of both.
//     No multicast: every block fetches its own tiles.
//   warp 1, one thread in the leader (issuer): waits until both blocks have drained the accumulator buffer, then per
//     stage waits for "full", issues four K = 16 MMAs (M 256, N BN) per k block of the stage and commits with multicast to the "empty"
//     barrier of that stage in BOTH blocks; after a tile, to both blocks' "accumulator full" barriers.
//   warps 2..9 of each block (epilogue, two per quarter of the rows, taking chunks in turn): tcgen05.ld of the block's own 128 x BN accumulator, 32 x 32 chunks passed
//     through shared memory, 16-byte stores, then an arrival on the leader's "accumulator empty" barrier. For
//     SwiGLU the leader's half of W holds gate rows and the peer's half the matching up rows, so the first BN/2
//     columns are gates and the rest their ups.
// Every mbarrier wait is bounded (a status word records the first that ran out); the cluster barriers are hardware
// barriers that both blocks always reach.
#include "tcgen05.cuh"

namespace {

constexpr const char* WHO = "bl_gemm_tc_pair";

constexpr int BM = 128;                 // rows per block (256 per pair)
constexpr int BK = 64;
constexpr int A_BYTES = BM * BK * 2;
// A stage holds the block's 128 rows of x and its half of the tile's rows of W. The ring is as deep as shared memory
// allows: five stages of 32 KB for 256-wide tiles, three of 48 KB (two k blocks each) for 128-wide ones.
// (KS k blocks of 64 per stage: two for the 128-wide tiles, whose main loop is bound by the hand-over of stages
// between loader, issuer and tensor cores and not by the tensor cores themselves: fewer, larger steps)
constexpr int ksub(int bn) { return bn == 256 ? 1 : 2; }
constexpr int b_bytes(int bn) { return (bn / 2) * BK * 2; }
constexpr int stage_bytes(int bn) { return ksub(bn) * (A_BYTES + b_bytes(bn)); }
constexpr int stages_for(int bn) { return bn == 256 ? 5 : 3; }
constexpr int RING_BYTES = stages_for(128) * stage_bytes(128) > stages_for(256) * stage_bytes(256)
                               ? stages_for(128) * stage_bytes(128) : stages_for(256) * stage_bytes(256);
constexpr int MAX_STAGES = 7;
constexpr int EPI_WARPS = 8, THREADS = 32 * (2 + EPI_WARPS);    // two warps per quarter of the accumulator's rows
constexpr int PITCH = 36;                                            // floats per staged row of the epilogue
constexpr int STAGING_BYTES = EPI_WARPS * 32 * PITCH * 4;
constexpr int SMEM_BYTES = RING_BYTES + STAGING_BYTES + 1024 + 256;
constexpr int TMEM_COLS = 512;                                       // two accumulators of up to 256 columns
constexpr uint32_t WAIT_LIMIT = 1u << 22;
constexpr uint32_t PEER_BIT_MASK = 0xFEFFFFFFu;      // clears the bit that selects the odd block of a pair

__device__ int g_status2 = 0;

// An epilogue of this file only: the joined q/k/v product of an attention layer, finished in place. A tile of 128
// columns is whole heads (head size 64 or 128); the accumulator gets its bias, q and k heads are rotated by the
// token's position (pairs j, j + head size / 2; cos and sin from the step's table), and the bfloat16 results go
// where the attention kernels read them: q rows, and the key and value pages of the token's request.
constexpr int EPI_QKV_ROPE = 100;
struct QkvOut {
    const int* tok_req; const int* positions; const int* block_table; int max_pages;
    const float* cs; const float* sn;            // [M, dh / 2]
    __nv_bfloat16* q; __nv_bfloat16* k_cache; __nv_bfloat16* v_cache;   // caches may be null (nothing is cached)
    int H, KV, dh;
};

// An RMS norm between two products, without a pass of its own. The product that adds into the residual stream
// (producer) also writes the new stream times the norm's weight as bfloat16 rows (hw) and, per row, the sums of
// squares of its tiles' columns (ss_out: [M, 2 * tiles], one value per tile and epilogue warp, always added in the
// same order); the product that reads the normed rows (consumer: SwiGLU, or q/k/v with rotation) takes hw as its x
// and multiplies each accumulator row by 1 / sqrt(sum of the row's ss_in / dim + eps): the row's scale commutes with
// the product. Statistics and scale are 32-bit.
struct NormLink {
    const void* norm_w; int norm_w_dtype; __nv_bfloat16* hw; float* ss_out;      // producer (null hw: none)
    const float* ss_in; int parts_in; float inv_dim, eps;                        // consumer (null ss_in: none)
};

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* give_up, int code) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if (*give_up) return false;
    }
    *give_up = 1;
    atomicCAS(&g_status2, 0, code);
    return false;
}
// Both blocks of the pair issue this; the bytes are reported to the barrier of the EVEN block (the leader).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t leader_bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(dst), "l"(map), "r"(leader_bar & PEER_BIT_MASK), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
                 :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {      // arrives on `bar` in both blocks
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 :: "r"(bar), "h"((unsigned short)3) : "memory");
}
// Arrives on the barrier at this address in the LEADER block (own block when it is the leader).
__device__ __forceinline__ void mbar_arrive_leader(uint32_t bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" :: "r"(bar & PEER_BIT_MASK) : "memory");
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// D 32-bit, A and B bfloat16 and K-major, N >> 3 at bit 17, M = 256 over the pair (>> 4 at bit 24)
__host__ __device__ constexpr uint32_t idesc_for(int bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

template <int EPI, typename TO, int BN>
__global__ void __launch_bounds__(THREADS)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const void* __restrict__ bias, int bias_dtype, TO* __restrict__ out, int M, int N, int K,
                    int m_pairs, int n_tiles, const QkvOut qo, const NormLink nl) {
    constexpr bool GLU = EPI == BL_EPI_SWIGLU;
    constexpr int STAGE_BYTES = stage_bytes(BN), STAGES = stages_for(BN), KS = ksub(BN), B_BYTES = b_bytes(BN);
    static_assert(STAGES <= MAX_STAGES && STAGES * STAGE_BYTES <= RING_BYTES && STAGE_BYTES % 1024 == 0, "ring does not fit");
    constexpr int COLS = GLU ? BN / 2 : BN;                          // output columns per tile
    extern __shared__ unsigned char smem_raw[];
    if (threadIdx.x == 0) { tma_prefetch_map(&map_a); tma_prefetch_map(&map_b); }
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* aligned = smem_raw + (base - smem_u32(smem_raw));
    float* staging = reinterpret_cast<float*>(aligned + RING_BYTES);
    const uint32_t bars = base + RING_BYTES + STAGING_BYTES;
    volatile int* give_up = reinterpret_cast<volatile int*>(aligned + RING_BYTES + STAGING_BYTES + 192);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(aligned + RING_BYTES + STAGING_BYTES + 200);
    const uint32_t full0 = bars, empty0 = bars + 8 * MAX_STAGES, acc_full0 = bars + 16 * MAX_STAGES, acc_empty0 = acc_full0 + 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const bool leader = rank == 0;
    const int pair = blockIdx.x / 2, n_pairs = gridDim.x / 2;
    const int total_tiles = m_pairs * n_tiles;
    const int kblocks = ((K + BK - 1) / BK + KS - 1) / KS;           // steps of KS k blocks (a block past K arrives as zeros)

    if (threadIdx.x == 0) {
        *give_up = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full0 + 8 * b, 1); mbar_init(acc_empty0 + 8 * b, 2 * EPI_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    cluster_sync();                                                  // both blocks' barriers exist before anyone signals them
    // W does not depend on the kernel before this one: the loader starts this block's half of W for the first ring of
    // k blocks before the dependent-launch wait, so that those copies (the first touch of this layer's weights) run
    // while the predecessor finishes. The stage's barrier expects the bytes of x and W together; x follows after the wait.
    int early = 0;                                                   // loader: k blocks whose W is already on its way
    if (warp == 0 && lane == 0 && pair < total_tiles) {
        const int n0 = (pair / m_pairs) * COLS;
        const int w_row0 = GLU ? (int)rank * N + n0 : n0 + (int)rank * (BN / 2);
        for (; early < STAGES && early < kblocks; ++early) {
            if (leader) mbar_expect_tx(full0 + 8 * early, 2 * STAGE_BYTES);   // the bytes of both blocks
#pragma unroll
            for (int u = 0; u < KS; ++u)
                tma_load_2d_pair(base + early * STAGE_BYTES + KS * A_BYTES + u * B_BYTES, &map_b, full0 + 8 * early, (early * KS + u) * BK, w_row0);
        }
    }
    __syncwarp();
    bl_pdl_wait();                                                   // x, the residual stream and tensor memory belong to the predecessor until here
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(smem_u32((const void*)tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    fence_before_sync();
    __syncthreads();
    cluster_sync();                                                  // both blocks hold their tensor memory before the leader writes into it
    fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    bl_pdl_trigger();                                                // the next kernel may start its own preamble (it waits before it touches data)

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;                                              // k blocks loaded so far, over all tiles
            for (int t = pair; t < total_tiles && !*give_up; t += n_pairs) {
                const int m0 = ((t % m_pairs) * 2 + (int)rank) * BM;
                const int n0 = (t / m_pairs) * COLS;
                // this block's half of W. Plain: rows n0 + rank * BN/2. SwiGLU: gate rows (leader) or the up rows that match.
                const int w_row0 = GLU ? (int)rank * N + n0 : n0 + (int)rank * (BN / 2);
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1, give_up, 1)) break;
                    const uint32_t a_dst = base + s * STAGE_BYTES, b_dst = a_dst + KS * A_BYTES;   // stage: KS tiles of x, then KS of W
                    if (it >= early) {                                // (the first ring's W was started before the wait)
                        if (leader) mbar_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);   // the bytes of both blocks
#pragma unroll
                        for (int u = 0; u < KS; ++u) tma_load_2d_pair(b_dst + u * B_BYTES, &map_b, full0 + 8 * s, (kb * KS + u) * BK, w_row0);
                    }
#pragma unroll
                    for (int u = 0; u < KS; ++u) tma_load_2d_pair(a_dst + u * A_BYTES, &map_a, full0 + 8 * s, (kb * KS + u) * BK, m0);
                }
            }
        }
    } else if (warp == 1) {
        if (leader && lane == 0) {
            int it = 0, local = 0;
            for (int t = pair; t < total_tiles && !*give_up; t += n_pairs, ++local) {
                const int buf = local & 1;
                // both blocks must have drained this accumulator buffer (its first two uses find it free)
                if (local >= 2 && !mbar_wait(acc_empty0 + 8 * buf, ((local / 2) & 1) ^ 1, give_up, 4)) break;
                fence_after_sync();
                const uint32_t d_tmem = tmem + buf * 256;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(full0 + 8 * s, (it / STAGES) & 1, give_up, 2)) break;
                    fence_after_sync();
#pragma unroll
                    for (int u = 0; u < KS; ++u) {
                        const uint64_t a_desc = smem_desc(base + s * STAGE_BYTES + u * A_BYTES);
                        const uint64_t b_desc = smem_desc(base + s * STAGE_BYTES + KS * A_BYTES + u * B_BYTES);
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k)
                            umma_bf16_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc_for(BN), (kb | u | k) != 0);
                    }
                    umma_commit_pair(empty0 + 8 * s);
                }
                umma_commit_pair(acc_full0 + 8 * buf);
            }
        }
    } else {
        const int ew = warp - 2;                                     // epilogue warp 0..7
        const int quarter = warp & 3;                                // the 32 accumulator rows this warp may read
        const int half = ew >> 2;                                    // of the two warps of a quarter: even or odd chunks
        float* tile = staging + ew * 32 * PITCH;
        const int r_sub = lane >> 3, c4 = (lane & 7) * 4;
        const bool vec_ok = (N % 4) == 0;
        constexpr int CHUNKS = COLS / 32;
        int local = 0;
        for (int t = pair; t < total_tiles; t += n_pairs, ++local) {
            const int buf = local & 1;
            const int m0 = ((t % m_pairs) * 2 + (int)rank) * BM;
            const int n0 = (t / m_pairs) * COLS;
            // The residual epilogue reads what it adds to. Those reads do not depend on the product: the eight 16-byte
            // words a lane needs for a chunk are requested before the chunk's accumulator is fetched (for the first
            // chunk: before the accumulator is even waited for), so that their trip to L2 is not paid row by row.
            constexpr bool PRELOAD = EPI == BL_EPI_RESIDUAL && sizeof(TO) == 4;
            // consumer of a pending norm: the scale of this lane's row (a lane owns a row where the accumulator is read)
            float row_scale = 1.0f;
            if ((GLU || EPI == EPI_QKV_ROPE) && nl.ss_in != nullptr) {
                const int m = m0 + quarter * 32 + lane;
                if (m < M) {
                    float sum = 0.f;
                    for (int q = 0; q < nl.parts_in; ++q) sum += nl.ss_in[(size_t)m * nl.parts_in + q];
                    row_scale = rsqrtf(sum * nl.inv_dim + nl.eps);
                }
            }
            float ssum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};     // producer of a pending norm: sums of squares of this lane's columns, per row
            float4 res[8];
            auto preload = [&](int c) {
#pragma unroll
                for (int it2 = 0; it2 < 8; ++it2) {
                    const int m = m0 + quarter * 32 + it2 * 4 + r_sub, n = n0 + c * 32 + c4;
                    res[it2] = (vec_ok && m < M && n + 3 < N) ? *reinterpret_cast<const float4*>(out + (size_t)m * N + n)
                                                               : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            };
            if (EPI == EPI_QKV_ROPE) {
                // This lane's row of the accumulator is one token. The tile's 128 columns are 128 / dh heads; an item is
                // 32 columns of a head's first half with the 32 that turn with them (dh / 2 further on); the two warps
                // of a quarter take an item each. Everything that does not depend on the product (where the row goes,
                // its cosines and sines, the bias) is asked for before the accumulator is waited for.
                const int dh = qo.dh, half_cols = dh >> 1;
                const int m = m0 + quarter * 32 + lane;
                const int c_lo = dh == 64 ? 2 * half : half, c_hi = c_lo + (dh >> 6);     // 32-column chunks of the tile
                const int n_lo = n0 + c_lo * 32;                                          // first column of the item's low half
                const int head = n_lo / dh;                                               // q heads, then k heads, then v heads
                const int j0 = n_lo % dh;                                                 // first pair of the item (0, or 32 for dh 128)
                const bool turn = head < qo.H + qo.KV;
                // where this token's row of the head goes (elements from the start of q, or of a cache)
                __nv_bfloat16* dst_base = nullptr;
                size_t dst_row = 0;
                bool row_ok = m < M && n_lo < N;                                          // (the last tile of an odd number of 64-wide heads is half empty)
                if (head < qo.H) {
                    dst_base = qo.q;
                    dst_row = ((size_t)(row_ok ? m : 0) * qo.H + head) * dh;
                } else {
                    const bool keys = head < qo.H + qo.KV;
                    dst_base = keys ? qo.k_cache : qo.v_cache;
                    const int kvh = keys ? head - qo.H : head - qo.H - qo.KV;
                    if (dst_base == nullptr) row_ok = false;
                    if (row_ok) {
                        const int pos = qo.positions[m];
                        const int page = qo.block_table[(size_t)qo.tok_req[m] * qo.max_pages + pos / 16];
                        if (page < 0) row_ok = false;                                     // the host never schedules this; keep memory safe anyway
                        dst_row = (((size_t)(page < 0 ? 0 : page) * qo.KV + kvh) * 16 + (size_t)(pos % 16)) * dh;
                    }
                }
                const float4* cs4 = reinterpret_cast<const float4*>(qo.cs + (size_t)(m < M ? m : 0) * half_cols + j0);
                const float4* sn4 = reinterpret_cast<const float4*>(qo.sn + (size_t)(m < M ? m : 0) * half_cols + j0);
                float4 cw[4], sw[4];                                                      // pairs 0..15 of the item
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    cw[i] = turn ? cs4[i] : make_float4(1.f, 1.f, 1.f, 1.f);
                    sw[i] = turn ? sn4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                // the bias of the item's 2 x 32 columns (the same for every row): bfloat16 as eight 16-byte words
                const bool b16 = bias != nullptr && bias_dtype == BL_BF16 && n_lo < N;
                uint4 bl4[4], bh4[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    bl4[i] = b16 ? reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(bias) + n_lo)[i] : make_uint4(0u, 0u, 0u, 0u);
                    bh4[i] = b16 ? reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(bias) + n_lo + half_cols)[i] : make_uint4(0u, 0u, 0u, 0u);
                }
                const bool b32 = bias != nullptr && bias_dtype == BL_F32 && n_lo < N;
                if (!mbar_wait(acc_full0 + 8 * buf, (local / 2) & 1, give_up, 3)) break;
                fence_after_sync();
                const uint32_t lane_addr = tmem + buf * 256 + ((uint32_t)(quarter * 32) << 16);
                uint32_t lo[32], hi[32];
                tmem_ld32(lane_addr + c_lo * 32, lo);
                tmem_ld32(lane_addr + c_hi * 32, hi);
                tmem_ld_wait();
                float4 cw2[4], sw2[4];                                                    // pairs 16..31: on their way while the first are used
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    cw2[i] = turn ? cs4[4 + i] : make_float4(1.f, 1.f, 1.f, 1.f);
                    sw2[i] = turn ? sn4[4 + i] : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                uint32_t* st = reinterpret_cast<uint32_t*>(tile);                          // [32 rows][lo 16 words | hi 16 words | 4 unused]
                const uint32_t* blw = reinterpret_cast<const uint32_t*>(bl4);
                const uint32_t* bhw = reinterpret_cast<const uint32_t*>(bh4);
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    const float4 c4v = j < 16 ? cw[j >> 2] : cw2[(j - 16) >> 2], s4v = j < 16 ? sw[j >> 2] : sw2[(j - 16) >> 2];
                    const float c[4] = {c4v.x, c4v.y, c4v.z, c4v.w}, sv[4] = {s4v.x, s4v.y, s4v.z, s4v.w};
                    float a[4], b[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        // two bfloat16 per word: the even one in the low half
                        const uint32_t wl = blw[(j + e) >> 1], wh = bhw[(j + e) >> 1];
                        float ba = __uint_as_float((e & 1) ? (wl & 0xffff0000u) : (wl << 16));
                        float bb = __uint_as_float((e & 1) ? (wh & 0xffff0000u) : (wh << 16));
                        if (b32) { ba = reinterpret_cast<const float*>(bias)[n_lo + j + e]; bb = reinterpret_cast<const float*>(bias)[n_lo + half_cols + j + e]; }
                        const float x0 = __uint_as_float(lo[j + e]) * row_scale + ba, x1 = __uint_as_float(hi[j + e]) * row_scale + bb;
                        a[e] = x0 * c[e] - x1 * sv[e];
                        b[e] = x0 * sv[e] + x1 * c[e];
                    }
                    __nv_bfloat162 p0 = __floats2bfloat162_rn(a[0], a[1]), p1 = __floats2bfloat162_rn(a[2], a[3]);
                    __nv_bfloat162 p2 = __floats2bfloat162_rn(b[0], b[1]), p3 = __floats2bfloat162_rn(b[2], b[3]);
                    // through shared memory, so that a row's 64 bytes of each half leave as whole 16-byte words side by side
                    *reinterpret_cast<uint2*>(st + lane * PITCH + (j >> 1)) = make_uint2(*reinterpret_cast<unsigned*>(&p0), *reinterpret_cast<unsigned*>(&p1));
                    *reinterpret_cast<uint2*>(st + lane * PITCH + 16 + (j >> 1)) = make_uint2(*reinterpret_cast<unsigned*>(&p2), *reinterpret_cast<unsigned*>(&p3));
                }
                __syncwarp();
#pragma unroll
                for (int it2 = 0; it2 < 8; ++it2) {
                    const int row = it2 * 4 + r_sub;
                    const bool ok = __shfl_sync(0xffffffffu, row_ok ? 1 : 0, row) != 0;
                    const unsigned long long at = __shfl_sync(0xffffffffu, (unsigned long long)dst_row, row);
                    if (!ok) continue;
                    const int w8 = lane & 7;                                              // 16-byte word of the row: 0-3 the low half, 4-7 the high half
                    const uint4 v = *reinterpret_cast<const uint4*>(st + row * PITCH + 4 * w8);
                    __nv_bfloat16* dst = dst_base + at + j0 + (w8 < 4 ? w8 * 8 : half_cols + (w8 - 4) * 8);   // (one destination tensor per item)
                    *reinterpret_cast<uint4*>(dst) = v;
                }
                __syncwarp();
                fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_leader(acc_empty0 + 8 * buf);
                continue;
            }
            if (PRELOAD && half < CHUNKS) preload(half);
            if (!mbar_wait(acc_full0 + 8 * buf, (local / 2) & 1, give_up, 3)) break;
            fence_after_sync();
            const uint32_t lane_addr = tmem + buf * 256 + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
            for (int c = half; c < CHUNKS; c += 2) {
                uint32_t r[32];
                tmem_ld32(lane_addr + c * 32, r);
                if (GLU) {
                    uint32_t u[32];
                    tmem_ld32(lane_addr + BN / 2 + c * 32, u);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(bl_silu_fast(__uint_as_float(r[j]) * row_scale) * (__uint_as_float(u[j]) * row_scale));
                } else {
                    tmem_ld_wait();
                }
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    *reinterpret_cast<uint4*>(tile + lane * PITCH + 4 * j) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                __syncwarp();
                float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);              // a lane writes the same four columns in all eight rows
                if (EPI == BL_EPI_BIAS && vec_ok && n0 + c * 32 + c4 + 3 < N) {
                    const int n = n0 + c * 32 + c4;
                    b4 = make_float4(bl_load_any(bias, bias_dtype, n), bl_load_any(bias, bias_dtype, n + 1),
                                     bl_load_any(bias, bias_dtype, n + 2), bl_load_any(bias, bias_dtype, n + 3));
                }
                const bool link = EPI == BL_EPI_RESIDUAL && nl.hw != nullptr;
                float4 nw4 = make_float4(0.f, 0.f, 0.f, 0.f);              // the norm's weight of this lane's four columns
                if (link && n0 + c * 32 + c4 + 3 < N) {
                    const int n = n0 + c * 32 + c4;
                    nw4 = make_float4(bl_load_any(nl.norm_w, nl.norm_w_dtype, n), bl_load_any(nl.norm_w, nl.norm_w_dtype, n + 1),
                                      bl_load_any(nl.norm_w, nl.norm_w_dtype, n + 2), bl_load_any(nl.norm_w, nl.norm_w_dtype, n + 3));
                }
#pragma unroll
                for (int it2 = 0; it2 < 8; ++it2) {
                    const int row = it2 * 4 + r_sub;
                    const int m = m0 + quarter * 32 + row;
                    const int n = n0 + c * 32 + c4;
                    if (m >= M || n >= N) continue;
                    float4 v = *reinterpret_cast<const float4*>(tile + row * PITCH + c4);
                    TO* dst = out + (size_t)m * N + n;
                    if (vec_ok && n + 3 < N) {
                        if (EPI == BL_EPI_BIAS) { v.x += b4.x; v.y += b4.y; v.z += b4.z; v.w += b4.w; }
                        if (sizeof(TO) == 4) {
                            if (EPI == BL_EPI_RESIDUAL) { v.x += res[it2].x; v.y += res[it2].y; v.z += res[it2].z; v.w += res[it2].w; }
                            if (link) {
                                __nv_bfloat162 h0 = __floats2bfloat162_rn(v.x * nw4.x, v.y * nw4.y), h1 = __floats2bfloat162_rn(v.z * nw4.z, v.w * nw4.w);
                                uint2 hk;
                                hk.x = *reinterpret_cast<unsigned*>(&h0); hk.y = *reinterpret_cast<unsigned*>(&h1);
                                *reinterpret_cast<uint2*>(nl.hw + (size_t)m * N + n) = hk;
                                ssum[it2] += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                            }
                            *reinterpret_cast<float4*>(dst) = v;
                        } else {
                            __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
                            uint2 pk;
                            pk.x = *reinterpret_cast<unsigned*>(&lo); pk.y = *reinterpret_cast<unsigned*>(&hi);
                            *reinterpret_cast<uint2*>(dst) = pk;
                        }
                    } else {
                        const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            if (n + j >= N) break;
                            float x1 = e[j];
                            if (EPI == BL_EPI_BIAS) x1 += bl_load_any(bias, bias_dtype, n + j);
                            if (EPI == BL_EPI_RESIDUAL) x1 += bl_load(dst + j);
                            bl_store(dst + j, x1);
                        }
                    }
                }
                __syncwarp();
                if (PRELOAD && c + 2 < CHUNKS) preload(c + 2);           // on its way while the next accumulator chunk is fetched
            }
            if (EPI == BL_EPI_RESIDUAL && nl.hw != nullptr) {
                // the eight lanes that share a row add up; one value per row, tile and epilogue warp of the quarter
                const int parts = 2 * n_tiles, part = (t / m_pairs) * 2 + half;
#pragma unroll
                for (int it2 = 0; it2 < 8; ++it2) {
                    float q = ssum[it2];
                    q += __shfl_xor_sync(0xffffffffu, q, 1);
                    q += __shfl_xor_sync(0xffffffffu, q, 2);
                    q += __shfl_xor_sync(0xffffffffu, q, 4);
                    const int m = m0 + quarter * 32 + it2 * 4 + r_sub;
                    if ((lane & 7) == 0 && m < M) nl.ss_out[(size_t)m * parts + part] = q;
                }
            }
            // this warp is done with the buffer: tell the issuer (in the leader block)
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(acc_empty0 + 8 * buf);
        }
    }
    __syncwarp();
    fence_before_sync();
    __syncthreads();
    cluster_sync();                                                  // neither block leaves while the other may still read its memory
    if (warp == 0) {
        fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

template <int EPI, typename TO, int BN>
int launch_bn(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int M, int N, int K, int sms,
              cudaStream_t s, const QkvOut& qo = QkvOut(), const NormLink& nl = NormLink()) {
    static bool configured = false;
    if (!configured) {
        BL_CUDA(cudaFuncSetAttribute(gemm_tc_pair_kernel<EPI, TO, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        BL_CUDA(bl_same_carveout(gemm_tc_pair_kernel<EPI, TO, BN>));
        configured = true;
    }
    const bool glu = EPI == BL_EPI_SWIGLU;
    CUtensorMap a, b;
    if (bl_make_map_bf16(WHO, &a, x, M, K, BM, BK)) return 1;
    if (bl_make_map_bf16(WHO, &b, w, glu ? 2 * N : N, K, BN / 2, BK)) return 1;
    const int cols = glu ? BN / 2 : BN;
    const int m_pairs = (M + 2 * BM - 1) / (2 * BM), n_tiles = (N + cols - 1) / cols;
    int pairs = m_pairs * n_tiles;
    if (pairs > sms / 2) pairs = sms / 2;                            // one resident pair per two SMs walks over the tiles
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    // The block waits (griddepcontrol.wait) before it allocates tensor memory or touches x and out, so it may be
    // launched while its predecessor still runs: its preamble and the first copies of W overlap the predecessor's tail.
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = bl_pdl_enabled() ? 1 : 0;
    cfg.attrs = attr; cfg.numAttrs = 2;
    BL_CUDA(cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<EPI, TO, BN>, a, b, bias, bias_dtype, (TO*)out, M, N, K, m_pairs, n_tiles, qo, nl));
    return 0;
}

int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 2;
    }
    return n;
}

// 256-column tiles unless they would leave SM pairs without a tile while 128-column tiles would not.
template <int EPI, typename TO>
int launch(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int M, int N, int K, cudaStream_t s,
           const NormLink& nl = NormLink()) {
    const int sms = sm_count();
    const int cols256 = EPI == BL_EPI_SWIGLU ? 128 : 256;
    const int m_pairs = (M + 2 * BM - 1) / (2 * BM);
    const int tiles256 = m_pairs * ((N + cols256 - 1) / cols256);
    if (tiles256 < sms / 2) return launch_bn<EPI, TO, 128>(x, w, bias, bias_dtype, out, M, N, K, sms, s, QkvOut(), nl);
    return launch_bn<EPI, TO, 256>(x, w, bias, bias_dtype, out, M, N, K, sms, s, QkvOut(), nl);
}

}  // namespace

// Same contract as bl_gemm_tc; meant for M of a few hundred rows and more (a pair covers 256 rows).
extern "C" int bl_gemm_tc_pair(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int out_dtype,
                               int M, int N, int K, int epilogue, void* stream) {
    if (M <= 0) return 0;
    if (N <= 0 || K <= 0) BL_FAIL("bl_gemm_tc_pair: bad sizes N=%d K=%d", N, K);
    if (K % 8 != 0) BL_FAIL("bl_gemm_tc_pair: K=%d is not a multiple of 8 (TMA rows must be 16-byte multiples)", K);
    if (((uintptr_t)x | (uintptr_t)w) & 15) BL_FAIL("bl_gemm_tc_pair: x and W must be 16-byte aligned");
    if (epilogue == BL_EPI_BIAS && (bias == nullptr || (bias_dtype != BL_F32 && bias_dtype != BL_BF16)))
        BL_FAIL("bl_gemm_tc_pair: bias epilogue needs a float32 or bfloat16 bias");
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == BL_F32) {
        switch (epilogue) {
            case BL_EPI_NONE: return launch<BL_EPI_NONE, float>(x, w, bias, bias_dtype, out, M, N, K, s);
            case BL_EPI_BIAS: return launch<BL_EPI_BIAS, float>(x, w, bias, bias_dtype, out, M, N, K, s);
            case BL_EPI_RESIDUAL: return launch<BL_EPI_RESIDUAL, float>(x, w, bias, bias_dtype, out, M, N, K, s);
            case BL_EPI_SWIGLU: return launch<BL_EPI_SWIGLU, float>(x, w, bias, bias_dtype, out, M, N, K, s);
        }
    } else if (out_dtype == BL_BF16) {
        switch (epilogue) {
            case BL_EPI_NONE: return launch<BL_EPI_NONE, __nv_bfloat16>(x, w, bias, bias_dtype, out, M, N, K, s);
            case BL_EPI_BIAS: return launch<BL_EPI_BIAS, __nv_bfloat16>(x, w, bias, bias_dtype, out, M, N, K, s);
            case BL_EPI_SWIGLU: return launch<BL_EPI_SWIGLU, __nv_bfloat16>(x, w, bias, bias_dtype, out, M, N, K, s);
            case BL_EPI_RESIDUAL: BL_FAIL("bl_gemm_tc_pair: the residual stream is 32-bit; output dtype must be float32");
        }
    } else {
        BL_FAIL("bl_gemm_tc_pair: unknown output dtype %d", out_dtype);
    }
    BL_FAIL("bl_gemm_tc_pair: unknown epilogue %d", epilogue);
}

// Values per row that bl_gemm_tc_pair_residual_norm writes into `ss` for these sizes (two per tile of columns).
extern "C" int bl_gemm_tc_pair_norm_parts(int M, int N) {
    const int sms = sm_count();
    const int m_pairs = (M + 2 * BM - 1) / (2 * BM);
    const int cols = m_pairs * ((N + 255) / 256) < sms / 2 ? 128 : 256;
    return 2 * ((N + cols - 1) / cols);
}

// out (float32, in place) += x . W^T, as bl_gemm_tc_pair with the residual epilogue, and for the RMS norm that reads
// `out` next: hw[M, N] = bfloat16(out * norm_w) and ss[M, parts] = sums of squares of out's columns by tile (parts =
// bl_gemm_tc_pair_norm_parts(M, N)). A product that takes hw as its x and scales its rows by
// 1 / sqrt(sum(ss[m, :]) / N + eps) computes what it would from the normed rows. N must be a multiple of 4.
extern "C" int bl_gemm_tc_pair_residual_norm(const void* x, const void* w, void* out, int M, int N, int K, const void* norm_w,
                                             int norm_w_dtype, void* hw, float* ss, void* stream) {
    if (M <= 0) return 0;
    if (N <= 0 || K <= 0 || N % 4 != 0) BL_FAIL("bl_gemm_tc_pair_residual_norm: bad sizes N=%d K=%d (N a multiple of 4)", N, K);
    if (K % 8 != 0) BL_FAIL("bl_gemm_tc_pair_residual_norm: K=%d is not a multiple of 8", K);
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out | (uintptr_t)hw) & 15) BL_FAIL("bl_gemm_tc_pair_residual_norm: x, W, out and hw must be 16-byte aligned");
    if (norm_w == nullptr || (norm_w_dtype != BL_F32 && norm_w_dtype != BL_BF16) || hw == nullptr || ss == nullptr)
        BL_FAIL("bl_gemm_tc_pair_residual_norm: needs the norm's weight (float32 or bfloat16), hw and ss");
    NormLink nl = NormLink();
    nl.norm_w = norm_w; nl.norm_w_dtype = norm_w_dtype; nl.hw = (__nv_bfloat16*)hw; nl.ss_out = ss;
    return launch<BL_EPI_RESIDUAL, float>(x, w, nullptr, 0, out, M, N, K, (cudaStream_t)stream, nl);
}

// out[M, N] (bfloat16) = silu(r g) * (r u) with g, u = hw . Wg^T, hw . Wu^T and r[m] = 1 / sqrt(sum(ss[m, :parts]) * inv_dim + eps):
// the SwiGLU product of the rows whose norm bl_gemm_tc_pair_residual_norm left pending.
extern "C" int bl_gemm_tc_pair_swiglu_scaled(const void* hw, const void* w, void* out, int M, int N, int K, const float* ss,
                                             int parts, float inv_dim, float eps, void* stream) {
    if (M <= 0) return 0;
    if (N <= 0 || K <= 0 || K % 8 != 0) BL_FAIL("bl_gemm_tc_pair_swiglu_scaled: bad sizes N=%d K=%d", N, K);
    if (((uintptr_t)hw | (uintptr_t)w) & 15) BL_FAIL("bl_gemm_tc_pair_swiglu_scaled: x and W must be 16-byte aligned");
    if (ss == nullptr || parts <= 0) BL_FAIL("bl_gemm_tc_pair_swiglu_scaled: needs the rows' sums of squares");
    NormLink nl = NormLink();
    nl.ss_in = ss; nl.parts_in = parts; nl.inv_dim = inv_dim; nl.eps = eps;
    return launch<BL_EPI_SWIGLU, __nv_bfloat16>(hw, w, nullptr, 0, out, M, N, K, (cudaStream_t)stream, nl);
}

// Whether bl_gemm_tc_pair_qkv_rope takes this layer: head size 64 or 128, pages of 16, K as for the other products.
extern "C" int bl_gemm_tc_pair_qkv_rope_supported(int H, int KV, int dh, int page_size, int K) {
    return (dh == 64 || dh == 128) && page_size == 16 && H > 0 && KV > 0 && K % 8 == 0;
}

// The joined q/k/v product of M tokens with its bias, the rotation of q and k (pairs j, j + dh / 2, every pair of a
// head; cs and sn: [M, dh / 2] from bl_rope_table) and the writes of q (bfloat16 [M, H * dh]) and of k and v into the
// pages of each token's request (null caches: nothing is cached). W: [(H + 2 KV) * dh, K] bfloat16, q rows first.
extern "C" int bl_gemm_tc_pair_qkv_rope(const void* x, const void* w, const void* bias, int bias_dtype, int M, int K,
                                        const int* tok_req, const int* positions, const int* block_table, int max_pages,
                                        const float* cs, const float* sn, void* q_out, void* k_cache, void* v_cache,
                                        int H, int KV, int dh, int page_size, const float* ss, int parts, float inv_dim,
                                        float eps, void* stream) {
    if (M <= 0) return 0;
    if (!bl_gemm_tc_pair_qkv_rope_supported(H, KV, dh, page_size, K))
        BL_FAIL("bl_gemm_tc_pair_qkv_rope: head size %d, pages of %d, %d + 2 x %d heads, K = %d is not built", dh, page_size, H, KV, K);
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)cs | (uintptr_t)sn) & 15)
        BL_FAIL("bl_gemm_tc_pair_qkv_rope: x, W, q, the caches and the rotation table must be 16-byte aligned");
    if (bias != nullptr && bias_dtype != BL_F32 && bias_dtype != BL_BF16) BL_FAIL("bl_gemm_tc_pair_qkv_rope: the bias must be float32 or bfloat16");
    if ((k_cache == nullptr) != (v_cache == nullptr)) BL_FAIL("bl_gemm_tc_pair_qkv_rope: key and value cache must both be given or both be null");
    if (max_pages <= 0) BL_FAIL("bl_gemm_tc_pair_qkv_rope: bad table width");
    QkvOut qo;
    qo.tok_req = tok_req; qo.positions = positions; qo.block_table = block_table; qo.max_pages = max_pages;
    qo.cs = cs; qo.sn = sn; qo.q = (__nv_bfloat16*)q_out; qo.k_cache = (__nv_bfloat16*)k_cache; qo.v_cache = (__nv_bfloat16*)v_cache;
    qo.H = H; qo.KV = KV; qo.dh = dh;
    NormLink nl = NormLink();                     // x may be rows whose norm is pending (ss != null): see bl_gemm_tc_pair_residual_norm
    if (ss != nullptr) { nl.ss_in = ss; nl.parts_in = parts; nl.inv_dim = inv_dim; nl.eps = eps; }
    return launch_bn<EPI_QKV_ROPE, __nv_bfloat16, 128>(x, w, bias, bias_dtype, nullptr, M, (H + 2 * KV) * dh, K, sm_count(), (cudaStream_t)stream, qo, nl);
}

extern "C" int bl_gemm_tc_pair_status(int* status) {
    int v = 0, zero = 0;
    BL_CUDA(cudaMemcpyFromSymbol(&v, g_status2, sizeof(int)));
    if (v != 0) BL_CUDA(cudaMemcpyToSymbol(g_status2, &zero, sizeof(int)));
    *status = v;
    return 0;
}
