// Paged causal grouped-query attention for prefill on the fifth-generation tensor cores (head size 64).
//
// A block is 256 consecutive new tokens of one request (two row tiles of 128) and one query head; a thread owns
// one row. It walks the request's keys in blocks of 128 (eight 16-token pages) up to the diagonal; per tile:
//   S = Q . K^T      tcgen05.mma, M 128 x N 128 x K 64, Q and the key block in shared memory (TMA, 128-byte
//                    swizzle, K-major), S in tensor memory;
//   softmax          every thread reads its row of S with tcgen05.ld (lane r of tensor memory is row r, so the
//                    row maximum and sum need no shuffles), keeps the running maximum and sum in 32-bit, and
//                    writes P = 2^(s - m) as bfloat16 into shared memory in the swizzled K-major layout;
//   O_b = P . V      tcgen05.mma, M 128 x N 64 x K 128, V as it lies in its pages (keys x head size: the
//                    MN-major form of the B operand), O_b in tensor memory;
//   out = out * 2^(m_old - m) + O_b   in registers.
// Eleven warps: four per row tile own the rows, one issues the MMAs of both tiles (lane 0), two issue the TMA
// copies of keys and of values (a box costs its issuing lane about 0.1 us, so the sixteen boxes of a block are
// kept off the MMAs' path). They meet only at mbarriers. Keys and values (shared by the two tiles), P and the
// shares of the output have two buffers each, the scores one per tile: while one tile's warps wait for their
// next scores the other tile's warps have the SM's arithmetic (the 2^x of the special-function unit above all,
// which bounds the kernel), and the products run beside both. One block per SM (224 KB of shared memory, all
// 512 tensor-memory columns).
// Pages come from the request's block table, one TMA box (16 keys x 64) per page and tensor.
//
// Every wait on an mbarrier is bounded; when a bound runs out the block records a code in a status word, its
// warps leave their loops (the others see the flag at their next wait), its own copies are waited for, and it
// frees its tensor memory and returns (bl_attention_prefill_tc_status).
// Softmax is the online form of the reference's flash kernels (FlashAttnRegKernel, src/math_gpu.br:3309-3504);
// scores are scaled after the dot product (src/math.br:319-322); a key j is visible to a query at position p
// when j <= p and, with a window, j + window > p (:327-328).
#include "common.cuh"
#include "api.h"
#include <cuda.h>

namespace {

constexpr int DH = 64;                 // head size
constexpr int ROWS = 128;              // query rows per block
constexpr int KBLK = 128;              // keys per block
constexpr int PAGE = 16;
constexpr int PAGES = KBLK / PAGE;     // TMA boxes per tensor and block
constexpr int PAGE_BYTES = PAGE * DH * 2;
constexpr int TILES = 2;               // row tiles of 128 per block: two groups of four warps take turns on the SM
constexpr int THREADS = TILES * ROWS + 96;   // the row warps, one warp that issues the MMAs, two that copy
constexpr int Q_BYTES = TILES * ROWS * DH * 2, KV_BYTES = KBLK * DH * 2, P_BYTES = ROWS * KBLK * 2;
constexpr int OFF_Q = 0, OFF_K = Q_BYTES, OFF_V = OFF_K + 2 * KV_BYTES, OFF_P = OFF_V + 2 * KV_BYTES;
constexpr int OFF_BARS = OFF_P + 2 * TILES * P_BYTES;                // P: [tile][stage]
constexpr int SMEM_BYTES = OFF_BARS + 256;
constexpr int TMEM_COLS = 512;         // scores: 128 columns per tile; shares of the output: [tile][stage] x 64 columns from column 256
constexpr uint32_t WAIT_LIMIT = 1u << 22;

__device__ int g_status = 0;           // 0 = fine; else the code of the first wait that ran out

struct Params {
    __nv_bfloat16* out;
    const int* cu_q; const int* ctx_len; const int* block_table; int max_pages;
    const int* tiles;                  // [n][2] (request, first token of the 128-row tile within the request)
    int H, KV, window; float scale_log2;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}
// Bounded wait. False when the bound ran out or another thread of the block has given up. SLEEP: the waiter is one
// of the copy or issue warps, which wait most of the time; it naps between tries so that its spinning does not
// take issue slots from the row warps of its scheduler.
template <bool SLEEP = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* give_up, int code) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if (*give_up) return false;
        if (SLEEP) __nanosleep(40);
    }
    *give_up = 1;
    atomicCAS(&g_status, 0, code);
    return false;
}
// Bounded wait that does not look at the give-up flag (a block that has given up waits for its own copies).
__device__ __forceinline__ void mbar_wait_plain(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return;
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// what the threads wrote into shared memory becomes visible to the tensor cores and to TMA
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 128-byte swizzle, rows of 128 bytes, groups of 8 rows 1024 bytes apart. The same descriptor serves a K-major
// operand (rows = M or N, 64 elements of K per row) and an MN-major one (rows = K, 64 elements of N per row).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    const uint32_t lo = ((addr >> 4) & 0x3FFFu) | (1u << 16);                 // start address, leading offset 1 (unused: one 64-wide atom)
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);               // stride offset, version 1, SWIZZLE_128B
    return ((uint64_t)hi << 32) | lo;
}
// kind::f16 instruction descriptors: D 32-bit, A and B bfloat16, N >> 3 at bit 17, M >> 4 at bit 24;
// bit 16 set: B is MN-major (V lies keys x head size).
constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(KBLK >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(DH >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);

// 2^x on the special-function unit (about 2 ulp; 2^-inf = 0, tiny results flush to 0)
__device__ __forceinline__ float bl_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

__global__ void __launch_bounds__(THREADS, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const Params p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    const uint32_t base = smem_u32(smem);
    const uint32_t bars = base + OFF_BARS;
    // barriers, 8 bytes each. [stage] is the stage of keys and values (block i uses stage i & 1), [t] the row tile.
    const uint32_t full_q = bars;
    const uint32_t full_k0 = bars + 8;          // [stage] keys copied
    const uint32_t full_v0 = bars + 24;         // [stage] values copied
    const uint32_t k_free0 = bars + 40;         // [stage] every tile's scores of the block are done: the keys may go
    const uint32_t v_free0 = bars + 56;         // [stage] every tile's product of the block is done: the values may go
    const uint32_t s_done0 = bars + 72;         // [t] the tile's scores are in tensor memory
    const uint32_t o_done0 = bars + 88;         // [t][stage] the tile's share of the output is in tensor memory
    const uint32_t p_ready0 = bars + 120;       // [t][stage] the tile's P is in shared memory (and its scores have been read)
    volatile int* give_up = reinterpret_cast<volatile int*>(smem + OFF_BARS + 160);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + OFF_BARS + 168);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int ROW_WARPS = TILES * ROWS / 32;
    const bool issuer = warp == ROW_WARPS;                               // after the row warps: the MMA issuer, then two copy warps

    // late tiles of a request see the most keys: they go first, so that the short ones fill the tail
    const int tile = gridDim.x - 1 - blockIdx.x;
    const int r = p.tiles[3 * tile], tok0 = p.tiles[3 * tile + 1], row_limit = p.tiles[3 * tile + 2];
    const int head = blockIdx.y, kvh = head / (p.H / p.KV);
    const int q_begin = p.cu_q[r], q_len = p.cu_q[r + 1] - q_begin, ctx = p.ctx_len[r];
    const int* table = p.block_table + (size_t)r * p.max_pages;
    const int rows_here = min(min(TILES * ROWS, row_limit), q_len - tok0);   // > 0 by construction of the tiles
    const int n_tiles = rows_here > ROWS ? 2 : 1;                        // a short last tile leaves the second half idle
    const int p_first = ctx - q_len + tok0, p_last = p_first + rows_here - 1;
    const int lo = p.window > 0 ? max(0, p_first - p.window + 1) : 0, hi = p_last;
    const int b_begin = lo / KBLK, nb = rows_here > 0 ? hi / KBLK + 1 - b_begin : 0;

    if (threadIdx.x == 0) {
        *give_up = (base & 1023u) ? 1 : 0;                               // the swizzled tiles need 1024-byte alignment
        if (base & 1023u) atomicCAS(&g_status, 0, 9);
        mbar_init(full_q, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(full_k0 + 8 * i, 1); mbar_init(full_v0 + 8 * i, 1);
            mbar_init(k_free0 + 8 * i, n_tiles); mbar_init(v_free0 + 8 * i, n_tiles);
            mbar_init(s_done0 + 8 * i, 1);
            for (int j = 0; j < 2; ++j) { mbar_init(o_done0 + 16 * i + 8 * j, 1); mbar_init(p_ready0 + 16 * i + 8 * j, ROWS); }
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // q, the newest keys and values, the output buffer and the tensor memory of the SM belong to the kernels before
    // this one until here; the block's preamble above may run while they finish
    bl_pdl_wait();
    if (issuer) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(smem_u32((const void*)tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    bl_pdl_trigger();                                                    // the next kernel may start its own preamble (it waits before it touches data)
    // tensor memory: scores of tile t in columns 128 t ..; the share of the output of tile t and block i in columns
    // 256 + 128 t + 64 (i & 1) ..
    bool ok = !*give_up;

    if (warp > ROW_WARPS) {
        // ================= two warps: the copies of the keys (and q) and of the values, a page per lane 0..7.
        // Issuing a box costs its lane about 0.1 us, one lane after the other: two warps keep the sixteen boxes of a
        // block off the path of the MMAs.
        const bool keys = warp == ROW_WARPS + 1;
        const CUtensorMap* map = keys ? &map_k : &map_v;
        const uint32_t full0 = keys ? full_k0 : full_v0, free0 = keys ? k_free0 : v_free0, off = keys ? OFF_K : OFF_V;
        auto page_of = [&](int b, int pg) -> int {                       // -1: no row may see a key of this page
            const int first = b * KBLK + pg * PAGE;
            if (first > hi || first + PAGE - 1 < lo) return -1;
            return table[first / PAGE];
        };
        int loads[2] = {0, 0};                                           // copies started per stage
        ok = __all_sync(0xffffffffu, ok);
        if (ok && keys && lane == 0) {
            mbar_expect_tx(full_q, Q_BYTES);
            tma_load_2d(base + OFF_Q, &map_q, full_q, head * DH, q_begin + tok0);
        }
        int page = lane < PAGES && nb > 0 ? page_of(b_begin, lane) : -1;
        for (int i = 0; ok && i < nb; ++i) {
            const int st = i & 1;
            const int page_next = lane < PAGES && i + 1 < nb ? page_of(b_begin + i + 1, lane) : -1;   // on its way during this block's copies
            if (i >= 2) {                                                // the stage is free once block i - 2 has been multiplied
                if (lane == 0) ok = mbar_wait<true>(free0 + 8 * st, (uint32_t)(((i - 2) >> 1) & 1), give_up, keys ? 3 : 7);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            const uint32_t bar = full0 + 8 * st, dst = base + off + st * KV_BYTES;
            const unsigned have = __ballot_sync(0xffffffffu, lane < PAGES && page >= 0);
            if (lane == 0) {
                if (have) mbar_expect_tx(bar, (uint32_t)__popc(have) * PAGE_BYTES); else mbar_arrive(bar);
            }
            __syncwarp();
            if (lane < PAGES && page >= 0) tma_load_2d(dst + lane * PAGE_BYTES, map, bar, 0, (page * p.KV + kvh) * PAGE);
            __syncwarp();
            ++loads[st];
            page = page_next;
        }
        // a block that gave up lets its own copies land before its shared memory goes to the next block
        if (lane == 0 && *give_up && !(base & 1023u)) {
            if (keys) mbar_wait_plain(full_q, 0);
            for (int s2 = 0; s2 < 2; ++s2)
                if (loads[s2] > 0) mbar_wait_plain(full0 + 8 * s2, (uint32_t)((loads[s2] - 1) & 1));
        }
    } else if (issuer) {
        // ================= one warp: lane 0 issues the MMAs of both tiles
        auto issue_s = [&](int t, int i) {                               // S_t = Q_t . K^T of the i-th block
            const uint64_t a = smem_desc(base + OFF_Q + t * (ROWS * DH * 2)), b = smem_desc(base + OFF_K + (i & 1) * KV_BYTES);
#pragma unroll
            for (int k = 0; k < DH / 16; ++k) umma_bf16(tmem + t * KBLK, a + 2 * k, b + 2 * k, IDESC_S, k != 0);
            umma_commit(s_done0 + 8 * t);
            umma_commit(k_free0 + 8 * (i & 1));
        };
        if (lane == 0 && ok && nb > 0) {
            ok = mbar_wait<true>(full_q, 0, give_up, 1) && mbar_wait<true>(full_k0, 0, give_up, 2);
            if (ok) {
                fence_after_sync();
                for (int t = 0; t < n_tiles; ++t) issue_s(t, 0);
            }
            for (int i = 0; ok && i < nb; ++i) {
                const int st = i & 1;
                const uint32_t par = (uint32_t)((i >> 1) & 1);
                for (int t = 0; ok && t < n_tiles; ++t) {
                    // P_t of block i is in shared memory and the tile's scores have been read
                    ok = mbar_wait<true>(p_ready0 + 16 * t + 8 * st, par, give_up, 4);
                    if (!ok) break;
                    fence_after_sync();
                    if (i + 1 < nb) {                                    // the next scores first: the tile's row warps wait for them
                        ok = mbar_wait<true>(full_k0 + 8 * (st ^ 1), (uint32_t)(((i + 1) >> 1) & 1), give_up, 6);
                        if (!ok) break;
                        fence_after_sync();
                        issue_s(t, i + 1);
                    }
                    ok = mbar_wait<true>(full_v0 + 8 * st, par, give_up, 5);
                    if (!ok) break;
                    fence_after_sync();
                    const uint64_t a0 = smem_desc(base + OFF_P + (2 * t + st) * P_BYTES), bv = smem_desc(base + OFF_V + st * KV_BYTES);
#pragma unroll
                    for (int kk = 0; kk < KBLK / 16; ++kk)              // 16 keys a step: 32 bytes along P's rows, two 8-row groups of V
                        umma_bf16(tmem + TILES * KBLK + (2 * t + st) * DH, a0 + (uint64_t)((kk >> 2) * (ROWS * 128 >> 4) + 2 * (kk & 3)),
                                  bv + (uint64_t)(kk * (2048 >> 4)), IDESC_PV, kk != 0);
                    umma_commit(o_done0 + 16 * t + 8 * st);
                    umma_commit(v_free0 + 8 * st);
                }
            }
        }
        __syncwarp();
    } else if (warp / (ROWS / 32) < n_tiles) {
        // ================= four warps per tile: a thread owns one query row
        const int t = warp / (ROWS / 32);
        const int row = threadIdx.x - t * ROWS;                          // row of the tile = lane of tensor memory
        const bool valid = t * ROWS + row < rows_here;
        const int pos = valid ? p_first + t * ROWS + row : -1;           // an invalid row sees nothing
        const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;     // this warp's 32 lanes of tensor memory
        const uint32_t t_s = tmem + t * KBLK + lane_off;
        float o[DH];
#pragma unroll
        for (int j = 0; j < DH; ++j) o[j] = 0.f;
        float m = -INFINITY, l = 0.f, alpha_prev = 0.f;
        // out = out * alpha + O_i, read from tensor memory one block late (the product runs meanwhile)
        auto add_output = [&](int i, float alpha) {
            const uint32_t t_o = tmem + TILES * KBLK + (2 * t + (i & 1)) * DH + lane_off;
#pragma unroll
            for (int c = 0; c < DH / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(t_o + c * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) o[c * 32 + j] = o[c * 32 + j] * alpha + __uint_as_float(v[j]);
            }
        };
        for (int i = 0; i < nb; ++i) {
            const int b = b_begin + i, st = i & 1;
            ok = mbar_wait(s_done0 + 8 * t, (uint32_t)(i & 1), give_up, 8) && ok;
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            fence_after_sync();
            const int k0 = b * KBLK;
            // blocks that lie wholly inside what this row may see need no per-key test
            const bool all_seen = k0 + KBLK - 1 <= pos && (p.window <= 0 || k0 + p.window > pos);
            // Local key j of chunk c (keys k0 + 32 c + j) is visible when lo_c < j <= hi_c. Everything below is free of
            // branches per key: a masked key becomes -inf before the maximum and before 2^x (2^-inf = 0).
            const int hi_l = pos - k0, lo_l = p.window > 0 ? pos - p.window - k0 : -(1 << 30);
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 1
            for (int c = 0; c < KBLK / 32; ++c) {                        // first pass: the row's maximum (of the raw scores)
                uint32_t s[32];
                tmem_ld32(t_s + c * 32, s);
                tmem_ld_wait();
                if (all_seen) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) mx[j & 3] = fmaxf(mx[j & 3], __uint_as_float(s[j]));
                } else {
                    const int hi_c = hi_l - c * 32, lo_c = lo_l - c * 32;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        mx[j & 3] = fmaxf(mx[j & 3], (j <= hi_c && j > lo_c) ? __uint_as_float(s[j]) : -INFINITY);
                }
            }
            // the scale is positive: the maximum of the scaled scores is the scaled maximum
            const float m_new = fmaxf(m, fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;        // a row that has seen no key yet
            const float alpha = bl_ex2(m - m_use);                       // 2^-inf = 0 on the first block
            m = m_new;
            float sm4[4] = {0.f, 0.f, 0.f, 0.f};
            unsigned char* p_tile = smem + OFF_P + (2 * t + st) * P_BYTES;
#pragma unroll 1
            for (int c = 0; c < KBLK / 32; ++c) {                        // second pass: P into shared memory
                uint32_t s[32];
                tmem_ld32(t_s + c * 32, s);
                tmem_ld_wait();
                float e[32];
                if (all_seen) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        e[j] = bl_ex2(fmaf(__uint_as_float(s[j]), p.scale_log2, -m_use));
                        sm4[j & 3] += e[j];
                    }
                } else {
                    const int hi_c = hi_l - c * 32, lo_c = lo_l - c * 32;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float x = fmaf(__uint_as_float(s[j]), p.scale_log2, -m_use);
                        e[j] = bl_ex2((j <= hi_c && j > lo_c) ? x : -INFINITY);
                        sm4[j & 3] += e[j];
                    }
                }
                // 16-byte chunk cc of the row's 256 bytes: sub-tile cc / 8 (64 keys each), chunk cc % 8, swizzled by the row
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const int cc = c * 4 + q4;
                    unsigned char* dst = p_tile + (cc >> 3) * (ROWS * 128) + row * 128 + (((cc & 7) ^ (row & 7)) << 4);
                    *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16(e[8 * q4], e[8 * q4 + 1]), pack_bf16(e[8 * q4 + 2], e[8 * q4 + 3]),
                                                                pack_bf16(e[8 * q4 + 4], e[8 * q4 + 5]), pack_bf16(e[8 * q4 + 6], e[8 * q4 + 7]));
                }
            }
            l = l * alpha + ((sm4[0] + sm4[1]) + (sm4[2] + sm4[3]));
            // the values of this block: rows that were not copied, or that lie past the last key, become zeros
            // (their P is 0, and 0 times whatever an old request left in a page must stay 0). Both tiles write the
            // same zeros: neither has to wait for the other.
            if (k0 + KBLK - 1 > hi || k0 < lo) {
                ok = mbar_wait(full_v0 + 8 * st, (uint32_t)((i >> 1) & 1), give_up, 10) && ok;
                if (ok) {
                    for (int idx = row; idx < KBLK * 8; idx += ROWS) {   // (key row, 16-byte chunk); a row's chunks stay in the row
                        const int key = k0 + (idx >> 3);
                        const int first = key / PAGE * PAGE;
                        const bool copied = !(first > hi || first + PAGE - 1 < lo) && table[first / PAGE] >= 0;
                        if (!copied || key > hi)
                            *reinterpret_cast<uint4*>(smem + OFF_V + st * KV_BYTES + (idx << 4)) = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
            }
            fence_async_smem();
            fence_before_sync();
            mbar_arrive(p_ready0 + 16 * t + 8 * st);
            // the share of the block before: its product has had a whole softmax to finish
            if (i > 0) {
                ok = mbar_wait(o_done0 + 16 * t + 8 * (st ^ 1), (uint32_t)(((i - 1) >> 1) & 1), give_up, 11) && ok;
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                fence_after_sync();
                add_output(i - 1, alpha_prev);
            }
            alpha_prev = alpha;
        }
        if (nb > 0) {
            ok = mbar_wait(o_done0 + 16 * t + 8 * ((nb - 1) & 1), (uint32_t)(((nb - 1) >> 1) & 1), give_up, 12) && ok;
            ok = __all_sync(0xffffffffu, ok);
            if (ok) {
                fence_after_sync();
                add_output(nb - 1, alpha_prev);
                if (valid) {
                    const float inv = l > 0.f ? 1.0f / l : 0.f;
                    __nv_bfloat16* dst = p.out + ((size_t)(q_begin + tok0 + t * ROWS + row) * p.H + head) * DH;
#pragma unroll
                    for (int j = 0; j < DH; j += 8)
                        *reinterpret_cast<uint4*>(dst + j) = make_uint4(pack_bf16(o[j] * inv, o[j + 1] * inv), pack_bf16(o[j + 2] * inv, o[j + 3] * inv),
                                                                        pack_bf16(o[j + 4] * inv, o[j + 5] * inv), pack_bf16(o[j + 6] * inv, o[j + 7] * inv));
                }
            }
        }
    }
    fence_before_sync();
    __syncthreads();
    if (issuer) {
        fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
    static EncodeTiled fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiled)ptr;
    }
    return fn;
}

// A row-major [rows, cols] bfloat16 matrix as a 2-D tensor map with boxes of box_rows x 64 elements, 128-byte swizzle.
int make_map(CUtensorMap* map, const void* ptr, long long rows, int cols, int box_rows) {
    EncodeTiled enc = encode_fn();
    if (enc == nullptr) BL_FAIL("bl_attention_prefill_tc: cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult res = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (res != CUDA_SUCCESS)
        BL_FAIL("bl_attention_prefill_tc: cuTensorMapEncodeTiled failed with code %d (rows %lld, cols %d)", (int)res, rows, cols);
    return 0;
}

}  // namespace

extern "C" int bl_attention_prefill_tc_supported(int dh, int page_size) { return dh == DH && page_size == PAGE; }

// tiles[n_tiles][3] = (request, first token of the block's rows within the request's new tokens, rows of the block:
// 256, or 128 for a block that takes one row tile only). T: rows of q and out; n_pages: pages of the cache tensors
// (their first dimension).
extern "C" int bl_attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache, const int* cu_q,
                                       const int* ctx_len, const int* block_table, int max_pages, const int* tiles,
                                       int n_tiles, void* out, int T, int n_pages, int H, int KV, int dh, int page_size,
                                       int window, float scale, void* stream) {
    if (n_tiles <= 0) return 0;
    if (dh != DH || page_size != PAGE)
        BL_FAIL("bl_attention_prefill_tc: head size %d with pages of %d tokens is not built (64 with 16 only)", dh, page_size);
    if (H <= 0 || KV <= 0 || H % KV != 0) BL_FAIL("bl_attention_prefill_tc: %d heads cannot share %d key/value heads", H, KV);
    if (max_pages <= 0 || window < 0 || T <= 0 || n_pages <= 0) BL_FAIL("bl_attention_prefill_tc: bad sizes");
    if (!(scale > 0.f)) BL_FAIL("bl_attention_prefill_tc: the scale of the scores must be positive (got %g)", (double)scale);
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) & 15)
        BL_FAIL("bl_attention_prefill_tc: q, the caches and out must be 16-byte aligned");
    CUtensorMap mq, mk, mv;
    if (make_map(&mq, q, T, H * DH, TILES * ROWS)) return 1;
    if (make_map(&mk, k_cache, (long long)n_pages * KV * PAGE, DH, PAGE)) return 1;
    if (make_map(&mv, v_cache, (long long)n_pages * KV * PAGE, DH, PAGE)) return 1;
    Params p;
    p.out = (__nv_bfloat16*)out; p.cu_q = cu_q; p.ctx_len = ctx_len; p.block_table = block_table; p.max_pages = max_pages;
    p.tiles = tiles; p.H = H; p.KV = KV; p.window = window; p.scale_log2 = scale * 1.4426950408889634f;
    static bool configured = false;
    if (!configured) {
        BL_CUDA(cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        configured = true;
    }
    // A block waits (griddepcontrol.wait) before it allocates tensor memory or touches data, so it may be launched
    // while the kernel before it still runs.
    BL_CUDA(bl_launch_dependent(attention_tc_kernel, dim3(n_tiles, H, 1), dim3(THREADS), (size_t)SMEM_BYTES, (cudaStream_t)stream,
                                mq, mk, mv, p));
    BL_CHECK_LAUNCH("bl_attention_prefill_tc");
    return 0;
}

// Reads and clears the status word: 0 when no block has given up on a wait since the last call. Codes name the
// wait: 1 q, 2 first keys, 3 / 7 a stage of keys / values to become free, 4 P, 5 values, 6 keys of the block after
// next, 8 scores, 10 values (row warps), 11 / 12 a share of the output, 9 shared memory not 1024-byte aligned.
// Synchronises the device.
extern "C" int bl_attention_prefill_tc_status(int* status) {
    int v = 0, zero = 0;
    BL_CUDA(cudaMemcpyFromSymbol(&v, g_status, sizeof(int)));
    if (v != 0) BL_CUDA(cudaMemcpyToSymbol(g_status, &zero, sizeof(int)));
    *status = v;
    return 0;
}
