// Paged causal grouped-query attention for prefill on the fifth-generation tensor cores (head sizes 64 and 128).
//
// A block is a tile of 128 consecutive new tokens of one request and one query head. It walks the request's keys
// in blocks of 128 (eight 16-token pages) up to the diagonal:
//   S = Q . K^T      tcgen05.mma, M 128 x N 128 x K 64, Q and the key block in shared memory (TMA, 128-byte
//                    swizzle, K-major), S in tensor memory;
//   softmax          a thread reads its row of S with tcgen05.ld (lane r of tensor memory is row r, so the row
//                    maximum and sum need no shuffles), keeps a reference maximum m and the sum in 32-bit, and writes
//                    P = 2^(s - m) as bfloat16 pairs back into tensor memory (tcgen05.st), where the second
//                    product takes its A operand from: P never passes through shared memory, whose bandwidth
//                    the products' other operands and the TMA copies need;
//   O += P . V       tcgen05.mma, M 128 x N 64 x K 128, V as it lies in its pages (keys x head size: the
//                    MN-major form of the B operand), O accumulated in tensor memory over the key blocks;
//   m moves only when a block's maximum passes it by 2^8; O (load, scale, store) and the sum are then rescaled.
// Twelve warps: eight own the rows, in two groups of four that take the even and the odd key blocks (each with a
// running maximum, sum and output of its own, merged at the end as the slices of a split are); one issues the
// first product and one the second (lane 0 each), two issue the TMA copies of keys and of values (a box costs its
// issuing lane about 0.1 us, so the sixteen boxes of a block are kept off the MMAs' path). They meet only at
// mbarriers. The scores rotate through three buffers of tensor memory (P lies over the upper half of the scores
// it was made from), each group has its own share of the output and stage of keys and values: a group's next
// scores are computed while it is in its current block, and while one group waits for a product the other has the
// SM's arithmetic (the 2^x of the special-function unit above all). The loops over a row's scores stay rolled in pairs of
// 32-score loads, and the bounded waits are not unrolled: warps at different places of the code must all find it
// in the instruction cache. One block per SM.
// Pages come from the request's block table, one TMA box (16 keys x 64) per page and tensor.
//
// Every wait on an mbarrier is bounded; when a bound runs out the block records a code in a status word, its
// warps leave their loops (the others see the flag at their next wait), its own copies are waited for, and it
// frees its tensor memory and returns (bl_attention_prefill_tc_status).
// Softmax is the online form of the reference's flash kernels (FlashAttnRegKernel, src/math_gpu.br:3309-3504);
// scores are scaled after the dot product (src/math.br:319-322); a key j is visible to a query at position p
// when j <= p and, with a window, j + window > p (:327-328).
#include "tcgen05.cuh"

namespace {

constexpr const char* WHO = "bl_attention_prefill_tc";

constexpr int ROWS = 128;              // query rows per block
constexpr int KBLK = 128;              // keys per block
constexpr int PAGE = 16;
constexpr int PAGES = KBLK / PAGE;     // pages per key block
constexpr int ATOM_BYTES = ROWS * 128; // a 128-row operand tile lies in shared memory as atoms of 64 elements (128 bytes) a row
constexpr int TMEM_COLS = 512;         // three buffers of scores of 128 columns (P, as bfloat16 pairs, takes the upper 64 of its scores' buffer), shares of the output 128
constexpr int SBUFS = 3;
constexpr int COL_P = KBLK / 2;        // within a buffer of scores
constexpr int COL_O = SBUFS * KBLK;
constexpr uint32_t WAIT_LIMIT = 1u << 22;

// The two shapes that are built. Head size 64: two groups of row warps, each with its own share of the output (2 x 64
// columns of tensor memory). Head size 128: one group (a row's 128 outputs, its scores and the 2^x batch fill a
// thread's registers; twice the tensor-core work per score leaves the single group less to wait for), one share of
// the output of 128 columns, written by block i + 1 only after block i's has been taken (the row warps take it before
// they post P of block i + 1). Keys, values and q lie as DH / 64 atoms of 64 dimensions.
template <int DH_, int GROUPS_>
struct Shape {
    static constexpr int DH = DH_, GROUPS = GROUPS_;
    static constexpr int ATOMS = DH / 64;
    static constexpr int PAGE_BYTES = PAGE * DH * 2;
    static constexpr int THREADS = GROUPS * ROWS + 128;  // the row warps, a warp that issues S = Q K^T, two that copy, one that issues O = P V
    static constexpr int Q_BYTES = ROWS * DH * 2, KV_BYTES = KBLK * DH * 2;
    static constexpr int MERGE_ROW = DH / 2 + 1;                          // half of a group's output at the merge, rows padded by one float
    static constexpr int MERGE_BYTES = GROUPS == 2 ? ROWS * MERGE_ROW * 4 : 0;
    static constexpr int OFF_Q = 0, OFF_K = Q_BYTES, OFF_V = OFF_K + 2 * KV_BYTES, OFF_MERGE = OFF_V + 2 * KV_BYTES;
    static constexpr int OFF_XCH = OFF_MERGE + 2 * MERGE_BYTES;          // the groups' maxima and sums at the merge: 4 x 128 floats
    static constexpr int OFF_BARS = OFF_XCH + 4 * ROWS * 4;
    static constexpr int SMEM_BYTES = OFF_BARS + 256;
    static_assert(DH % 64 == 0 && COL_O + GROUPS * DH <= TMEM_COLS && SMEM_BYTES <= 227 * 1024, "shape does not fit an SM");
};

__device__ int g_status = 0;           // 0 = fine; else the code of the first wait that ran out

struct Params {
    __nv_bfloat16* out;
    const int* cu_q; const int* ctx_len; const int* block_table; int max_pages;
    const int* tiles;                  // [n][2] (request, first token of the 128-row tile within the request)
    int H, KV, window; float scale_log2;
};

// Bounded wait. False when the bound ran out or another thread of the block has given up. SLEEP: the waiter is one
// of the copy or issue warps, which wait most of the time; it naps between tries so that its spinning does not
// take issue slots from the row warps of its scheduler.
template <bool SLEEP = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* give_up, int code) {
    if (!SLEEP) {
        // most of these waits find their phase complete: the test that cannot block answers in half the time of
        // the one that may
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
#pragma unroll 1
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
#pragma unroll 1
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return;
    }
}
// Two 32-bit floats in one 64-bit register, for the instructions that work on both at once (half the issue slots of
// the scalar forms; each lane is rounded as the scalar instruction rounds it).
__device__ __forceinline__ uint64_t f2_pack(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
// D (+)= A . B with the A operand in tensor memory (lane = row, a 32-bit column = two bfloat16 along K)
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
                 :: "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// 16 columns of this warp's 32 lanes of tensor memory, written: thread t's register j to lane t, column j
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                 :: "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                    "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// tcgen05.wait::ld tied to the registers of the load it completes: nothing that reads them may be moved above it.
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                   "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                   "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :: "memory");
}
// what the threads wrote into shared memory becomes visible to the tensor cores and to TMA
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// kind::f16 instruction descriptors: D 32-bit, A and B bfloat16, N >> 3 at bit 17, M >> 4 at bit 24;
// bit 16 set: B is MN-major (V lies keys x head size).
constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(KBLK >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);   // 64 dimensions of the head at a time

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

template <class S>
__global__ void __launch_bounds__(S::THREADS, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const Params p) {
    constexpr int DH = S::DH, GROUPS = S::GROUPS, ATOMS = S::ATOMS, PAGE_BYTES = S::PAGE_BYTES;
    constexpr int Q_BYTES = S::Q_BYTES, KV_BYTES = S::KV_BYTES, MERGE_BYTES = S::MERGE_BYTES, MERGE_ROW = S::MERGE_ROW;
    constexpr int OFF_Q = S::OFF_Q, OFF_K = S::OFF_K, OFF_V = S::OFF_V, OFF_MERGE = S::OFF_MERGE, OFF_XCH = S::OFF_XCH;
    constexpr int OFF_BARS = S::OFF_BARS;
    extern __shared__ __align__(1024) unsigned char smem[];
    if (threadIdx.x == 0) { tma_prefetch_map(&map_q); tma_prefetch_map(&map_k); tma_prefetch_map(&map_v); }
    const uint32_t base = smem_u32(smem);
    const uint32_t bars = base + OFF_BARS;
    // barriers, 8 bytes each; [i & 1] of block i for the pairs, [i % 3] for the triples
    const uint32_t full_q = bars;
    const uint32_t full_k0 = bars + 8;          // keys copied
    const uint32_t full_v0 = bars + 24;         // values copied
    const uint32_t o_done0 = bars + 40;         // share of the output in tensor memory (and the values' stage free again)
    const uint32_t s_done0 = bars + 56;         // x 3: scores in tensor memory (and the keys' stage free again)
    const uint32_t p_ready0 = bars + 80;        // x 3: P in tensor memory, scores read: 128 arrivals
    const uint32_t l_ready = bars + 104;        // both groups have posted their maxima, sums and half of their output
    const uint32_t buf_free0 = bars + 128;      // x 3: the second product has read P: the buffer may take the scores of block i + 3
    const uint32_t o_final0 = bars + 152;       // x GROUPS: the group's last second product has been added (one phase)
    volatile int* give_up = reinterpret_cast<volatile int*>(smem + OFF_BARS + 112);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + OFF_BARS + 120);
    float* xch = reinterpret_cast<float*>(smem + OFF_XCH);               // [2 groups][maximum, sum][128 rows]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int ROW_WARPS = GROUPS * ROWS / 32;                        // one thread per row in each group
    // after the row warps: the issuer of the first product (it also owns the tensor memory), two copy warps, the
    // issuer of the second product. One thread issuing both was the kernel's bottleneck: twelve MMAs, two commits and
    // three waits a key block took it 1,800 cycles, as long as a group of row warps needs for the block's softmax.
    const bool issuer = warp == ROW_WARPS, issuer_pv = warp == ROW_WARPS + 3;

    // Blocks start in the order of their index: all heads of the list's last tile, then all heads of the tile before.
    // The list is sorted by keys, so the launch runs longest tile first and the short ones fill the tail (with the
    // heads outermost, the long tiles of the last heads would start when the SMs are nearly through).
    const int tile = gridDim.x / p.H - 1 - blockIdx.x / p.H;
    const int r = p.tiles[2 * tile], tok0 = p.tiles[2 * tile + 1];
    const int head = blockIdx.x % p.H, kvh = head / (p.H / p.KV);
    const int q_begin = p.cu_q[r], q_len = p.cu_q[r + 1] - q_begin, ctx = p.ctx_len[r];
    const int* table = p.block_table + (size_t)r * p.max_pages;
    const int rows_here = min(ROWS, q_len - tok0);                       // <= 0 only for the padding entries of a replayed step's list
    const int p_first = ctx - q_len + tok0, p_last = p_first + rows_here - 1;
    const int lo = p.window > 0 ? max(0, p_first - p.window + 1) : 0, hi = p_last;
    const int b_begin = lo / KBLK, nb = rows_here > 0 ? hi / KBLK + 1 - b_begin : 0;

    if (threadIdx.x == 0) {
        *give_up = (base & 1023u) ? 1 : 0;                               // the swizzled tiles need 1024-byte alignment
        if (base & 1023u) atomicCAS(&g_status, 0, 9);
        mbar_init(full_q, 1);
        mbar_init(l_ready, GROUPS * ROWS);
        for (int i = 0; i < 2; ++i) {
            mbar_init(full_k0 + 8 * i, 1); mbar_init(full_v0 + 8 * i, 1); mbar_init(o_done0 + 8 * i, 1);
        }
        for (int i = 0; i < SBUFS; ++i) {
            mbar_init(s_done0 + 8 * i, 1); mbar_init(p_ready0 + 8 * i, ROWS); mbar_init(buf_free0 + 8 * i, 1);
        }
        for (int i = 0; i < GROUPS; ++i) mbar_init(o_final0 + 8 * i, 1);
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
    // tensor memory: scores of block i in columns 128 (i % 3) .., its P over the upper 64 of them, its share of the
    // output in columns 384 + 64 (i & 1) .. (head size 128: 384 ..)
    bool ok = !*give_up;

    if (warp == ROW_WARPS + 1 || warp == ROW_WARPS + 2) {
        // ================= two warps: the copies of the keys (and q) and of the values, a page per lane 0..7.
        // Issuing a box costs its lane about 0.1 us, one lane after the other: two warps keep the sixteen boxes of a
        // block off the path of the MMAs.
        const bool keys = warp == ROW_WARPS + 1;
        const CUtensorMap* map = keys ? &map_k : &map_v;
        const uint32_t full0 = keys ? full_k0 : full_v0, off = keys ? OFF_K : OFF_V;
        auto page_of = [&](int b, int pg) -> int {                       // -1: no row may see a key of this page
            const int first = b * KBLK + pg * PAGE;
            if (first > hi || first + PAGE - 1 < lo) return -1;
            return table[first / PAGE];
        };
        int loads[2] = {0, 0};                                           // copies started per stage
        ok = __all_sync(0xffffffffu, ok);
        if (ok && keys && lane == 0 && nb > 0) {                         // (a tile without rows copies nothing and waits for nothing)
            mbar_expect_tx(full_q, Q_BYTES);
#pragma unroll
            for (int a = 0; a < ATOMS; ++a)
                tma_load_2d(base + OFF_Q + a * ATOM_BYTES, &map_q, full_q, head * DH + a * 64, q_begin + tok0);
        }
        int page = lane < PAGES && nb > 0 ? page_of(b_begin, lane) : -1;
        for (int i = 0; ok && i < nb; ++i) {
            const int st = i & 1;
            const int page_next = lane < PAGES && i + 1 < nb ? page_of(b_begin + i + 1, lane) : -1;   // on its way during this block's copies
            if (i >= 2) {                                                // the stage is free once block i - 2 has been multiplied
                if (lane == 0)
                    ok = keys ? mbar_wait<true>(s_done0 + 8 * ((i - 2) % SBUFS), (uint32_t)(((i - 2) / SBUFS) & 1), give_up, 3)
                              : mbar_wait<true>(o_done0 + 8 * st, (uint32_t)(((i - 2) >> 1) & 1), give_up, 7);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            const uint32_t bar = full0 + 8 * st, dst = base + off + st * KV_BYTES;
            const unsigned have = __ballot_sync(0xffffffffu, lane < PAGES && page >= 0);
            if (lane == 0) {
                if (have) mbar_expect_tx(bar, (uint32_t)__popc(have) * PAGE_BYTES); else mbar_arrive(bar);
            }
            __syncwarp();
            if (lane < PAGES && page >= 0) {
#pragma unroll
                for (int a = 0; a < ATOMS; ++a)                         // 16 keys x 64 dimensions a box
                    tma_load_2d(dst + a * ATOM_BYTES + lane * (PAGE * 128), map, bar, a * 64, (page * p.KV + kvh) * PAGE);
            }
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
        // ================= one warp: lane 0 issues the MMAs
        auto issue_s = [&](int i) {                                      // S = Q . K^T of the i-th block of this tile
#pragma unroll
            for (int at = 0; at < ATOMS; ++at) {                         // 64 dimensions of the head an atom, 16 a step
                const uint64_t a = smem_desc(base + OFF_Q + at * ATOM_BYTES);
                const uint64_t b = smem_desc(base + OFF_K + (i & 1) * KV_BYTES + at * ATOM_BYTES);
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_bf16(tmem + (i % SBUFS) * KBLK, a + 2 * k, b + 2 * k, IDESC_S, (at | k) != 0);
            }
            umma_commit(s_done0 + 8 * (i % SBUFS));
        };
        if (lane == 0 && ok && nb > 0) {
            ok = mbar_wait<true>(full_q, 0, give_up, 1) && mbar_wait<true>(full_k0, 0, give_up, 2);
            if (ok) { fence_after_sync(); issue_s(0); }
            if (ok && nb > 1) {
                ok = mbar_wait<true>(full_k0 + 8, 0, give_up, 2);
                if (ok) { fence_after_sync(); issue_s(1); }
            }
            // The scores of block j go where block j - 3 had its scores and its P, once the second product of that
            // block has read P. With three buffers a group's next scores are computed while it works on its
            // current block (with two, each group had one buffer, and waited through copy-free 500 ns for the
            // product after every block).
            for (int j = 2; ok && j < nb; ++j) {
                // (the keys have long been copied when the buffer becomes free: that wait first, off the path)
                ok = mbar_wait(full_k0 + 8 * (j & 1), (uint32_t)((j >> 1) & 1), give_up, 6);
                if (ok && j >= SBUFS) ok = mbar_wait(buf_free0 + 8 * ((j - SBUFS) % SBUFS), (uint32_t)(((j - SBUFS) / SBUFS) & 1), give_up, 4);
                if (!ok) break;
                fence_after_sync();
                issue_s(j);
            }
        }
        __syncwarp();
    } else if (issuer_pv) {
        // ================= one warp: lane 0 issues O_i = P . V once the group has written P of block i (and has taken
        // the share of its block before out of the columns that this one goes to)
        if (lane == 0 && ok) {
            for (int i = 0; ok && i < nb; ++i) {
                const int st = i & 1, buf = i % SBUFS;
                ok = mbar_wait(full_v0 + 8 * st, (uint32_t)((i >> 1) & 1), give_up, 5) &&       // copied long before P is there
                     mbar_wait(p_ready0 + 8 * buf, (uint32_t)((i / SBUFS) & 1), give_up, 12);
                if (!ok) break;
                fence_after_sync();
#pragma unroll
                for (int at = 0; at < ATOMS; ++at) {                     // 64 dimensions of the head at a time
                    const uint64_t bv = smem_desc(base + OFF_V + st * KV_BYTES + at * ATOM_BYTES);
#pragma unroll
                    for (int kk = 0; kk < KBLK / 16; ++kk)              // 16 keys a step: 8 columns of P, two 8-row groups of V
                        umma_bf16_ts(tmem + COL_O + (GROUPS == 2 ? st * DH : 0) + at * 64, tmem + buf * KBLK + COL_P + kk * 8,
                                     bv + (uint64_t)(kk * (2048 >> 4)), IDESC_PV, (kk == 0 && i < GROUPS) ? 0u : 1u);   // the group's first block starts its sum
                }
                umma_commit(o_done0 + 8 * st);
                umma_commit(buf_free0 + 8 * buf);
                if (i + GROUPS >= nb) umma_commit(o_final0 + 8 * (GROUPS == 2 ? st : 0));   // the group's last block
            }
        }
        __syncwarp();
    } else {
        // ================= the row warps, in GROUPS groups of four: group g takes the key blocks i = g, g + GROUPS, ...
        // of the tile, a thread of it one query row, with a running maximum, sum and output of the group's own (merged
        // at the end). With two groups, one is in its exponentials while the other reads scores, rescales or waits for
        // its product. Block i has its scores, P, stage of keys and values and barriers at index i & 1.
        const int grp = GROUPS == 2 ? warp >> 2 : 0;
        const int row = (warp & 3) * 32 + lane;                          // row of the tile = lane of tensor memory
        const bool valid = row < rows_here;
        const int pos = valid ? p_first + row : -1;                      // an invalid row sees nothing
        const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;     // this warp's 32 lanes of tensor memory
        // The group's output accumulates in tensor memory over its key blocks (the second product adds to it). m is
        // the reference the row's weights are taken against: the running maximum as of the last time it was moved,
        // which is when a block's maximum exceeds it by more than RESCALE (weights then reach 2^RESCALE at most: far
        // inside bfloat16 and 32-bit range, with the same relative rounding). Moving it costs a pass over the
        // accumulated output (load, scale, store), which after a row's first blocks is rare.
        constexpr float RESCALE = 8.f;
        float m = -INFINITY, l = 0.f;
        const uint32_t t_o = tmem + COL_O + (GROUPS == 2 ? grp * DH : 0) + lane_off;
        // Waits until the second product of block `blk` has been added. A wait on a barrier's phase is valid only
        // while the barrier is at most one phase behind the one asked for (phases are told apart by parity alone).
        // The group does not look at every one of these phases; what keeps it in step is the rotation of the score
        // buffers: the scores of block i, which the group has seen, were issued after the second product of block
        // i - 3 had completed, and with it all before it. So inside block i the products up to i - 3 are done, and a
        // wait for the product of the group's block before (i - 2, or i - 1 with one group) is valid. After the
        // last block nothing bounds how far the barrier has come (a question about a phase two back, or one
        // ahead, gets the wrong answer): the end of the group's last product has a barrier of its own.
        auto output_done = [&](int blk) -> bool {
            bool fine = mbar_wait(o_done0 + 8 * (blk & 1), (uint32_t)((blk >> 1) & 1), give_up, 11);
            fine = __all_sync(0xffffffffu, fine);
            if (fine) fence_after_sync();
            return fine;
        };
        int last = -1;                                                   // the group's last block
        for (int i = grp; i < nb; i += GROUPS) {
            const int b = b_begin + i, st = i & 1, buf = i % SBUFS;
            const uint32_t par = (uint32_t)((i >> 1) & 1);
            // P goes over the upper half of the scores it is made from: by the time a chunk of P is written, the
            // scores under it are in registers (chunks are taken in the order 3, 2, 1, 0; P of chunk c lies under
            // the scores of chunk 2 + c / 2)
            const uint32_t t_s = tmem + buf * KBLK + lane_off, t_p = t_s + COL_P;
            const uint32_t s_done = s_done0 + 8 * buf, p_ready = p_ready0 + 8 * buf, full_v = full_v0 + 8 * st;
            ok = mbar_wait(s_done, (uint32_t)((i / SBUFS) & 1), give_up, 8) && ok;
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            fence_after_sync();
            const int k0 = b * KBLK;
            // blocks that lie wholly inside what this row may see need no per-key test
            const bool all_seen = k0 + KBLK - 1 <= pos && (p.window <= 0 || k0 + p.window > pos);
            // Local key j of chunk c (keys k0 + 32 c + j) is visible when lo_c < j <= hi_c. Everything below is free of
            // branches per key: a masked key becomes -inf before the maximum and before 2^x (2^-inf = 0).
            const int hi_l = pos - k0, lo_l = p.window > 0 ? pos - p.window - k0 : -(1 << 30);
            // a masked key becomes -inf before the maximum and before 2^x (2^-inf = 0): no branch per key
            auto mask = [&](uint32_t (&s)[32], int c) {
                const int hi_c = hi_l - c * 32, lo_c = lo_l - c * 32;
#pragma unroll
                for (int j = 0; j < 32; ++j) s[j] = (j <= hi_c && j > lo_c) ? s[j] : 0xff800000u;
            };
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            auto chunk_max = [&](uint32_t (&s)[32], int c) {
                if (!all_seen) mask(s, c);
#pragma unroll
                for (int j = 0; j < 32; j += 2) mx[(j >> 1) & 3] = max3(mx[(j >> 1) & 3], __uint_as_float(s[j]), __uint_as_float(s[j + 1]));
            };
            // First pass, the maximum of the raw scores; 32 scores a load, the next load on its way meanwhile. The
            // loops over pairs of chunks stay rolled: both groups, at different places of this code, must find it in
            // the instruction cache.
            uint32_t sa[32], sb[32];
            tmem_ld32(t_s, sa);
#pragma unroll 1
            for (int cp = 0; cp < 2; ++cp) {                             // chunks 2 cp (in sa) and 2 cp + 1 (in sb)
                tmem_ld_wait(sa); tmem_ld32(t_s + (2 * cp + 1) * 32, sb); chunk_max(sa, 2 * cp);
                tmem_ld_wait(sb); tmem_ld32(t_s + 64, sa); chunk_max(sb, 2 * cp + 1);   // chunk 2: next here, first of the second pass
            }
            // the scale is positive: the maximum of the scaled scores is the scaled maximum
            const float m_new = fmaxf(m, fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2);
            float alpha = 1.f;
            // (a row's first keys: -inf + RESCALE is -inf, below any score; a row without keys so far stays as it is)
            if (__any_sync(0xffffffffu, m_new > m + RESCALE)) {
                alpha = bl_ex2(m - (m_new == -INFINITY ? 0.f : m_new));   // 2^-inf = 0 on the first keys
                m = m_new;
                if (last >= 0) {                                          // what has been added so far moves to the new reference
                    if (!output_done(last)) { ok = false; break; }
#pragma unroll
                    for (int h = 0; h < DH / 32; ++h) {
                        uint32_t v[32];
                        tmem_ld32(t_o + h * 32, v);
                        tmem_ld_wait(v);
                        uint32_t lo16[16], hi16[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            lo16[j] = __float_as_uint(__uint_as_float(v[j]) * alpha);
                            hi16[j] = __float_as_uint(__uint_as_float(v[16 + j]) * alpha);
                        }
                        tmem_st16(t_o + h * 32, lo16);
                        tmem_st16(t_o + h * 32 + 16, hi16);
                    }
                }
            }
            const float m_use = m == -INFINITY ? 0.f : m;                // a row that has seen no key yet
            // sums of the row's weights in four parts: keys 0, 4, 8, .. and 1, 5, 9, .. (sum2[0]), 2, 6, .. and 3, 7, .. (sum2[1])
            uint64_t sum2[2] = {f2_pack(0.f, 0.f), f2_pack(0.f, 0.f)};
            const uint64_t scale2 = f2_pack(p.scale_log2, p.scale_log2), minus_m2 = f2_pack(-m_use, -m_use);
            // Second pass, chunks 3 (still in sb), 2, 1, 0: P = 2^(s * scale - m) as bfloat16 into tensor memory, the A
            // operand of the second product: lane = row, two keys to a 32-bit column, 16 columns a chunk.
            auto chunk_exp = [&](uint32_t (&s)[32], int c) {
                if (!all_seen) mask(s, c);
                // in batches, so that the special-function unit's queue stays full: 32 scaled differences, 32 x 2^x
                // back to back (volatile keeps them together), then the sums and the pairs
                float x[32];
#pragma unroll
                for (int j = 0; j < 32; j += 2)
                    f2_unpack(f2_fma(f2_pack(__uint_as_float(s[j]), __uint_as_float(s[j + 1])), scale2, minus_m2), x[j], x[j + 1]);
#pragma unroll
                for (int j = 0; j < 32; ++j) asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+f"(x[j]));
                uint32_t pk[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    sum2[j & 1] = f2_add(sum2[j & 1], f2_pack(x[2 * j], x[2 * j + 1]));
                    pk[j] = pack_bf16(x[2 * j], x[2 * j + 1]);
                }
                tmem_st16(t_p + 16 * c, pk);
            };
#pragma unroll 1
            for (int cp = 1; cp >= 0; --cp) {                            // chunks 2 cp + 1 (in sb) and 2 cp (on its way into sa)
                chunk_exp(sb, 2 * cp + 1);
                tmem_ld_wait(sa);
                if (cp) tmem_ld32(t_s + 32, sb);
                chunk_exp(sa, 2 * cp);
                if (cp) { tmem_ld_wait(sb); tmem_ld32(t_s, sa); }
            }
            float s_a, s_b, s_c, s_d;
            f2_unpack(sum2[0], s_a, s_c);
            f2_unpack(sum2[1], s_b, s_d);
            l = l * alpha + ((s_a + s_b) + (s_c + s_d));
            // the values of this block: rows that were not copied, or that lie past the last key, become zeros
            // (their P is 0, and 0 times whatever an old request left in a page must stay 0)
            if (k0 + KBLK - 1 > hi || k0 < lo) {
                // (once the product before has been added, the values of two blocks ago have been copied: the
                // barrier of this block's values is one phase behind at most)
                if (last >= 0 && !output_done(last)) { ok = false; break; }
                ok = mbar_wait(full_v, par, give_up, 10) && ok;
                if (ok) {
                    // (atom, key row, 16-byte chunk); the swizzle keeps a row's chunks in the row
                    for (int idx = threadIdx.x & (ROWS - 1); idx < ATOMS * KBLK * 8; idx += ROWS) {
                        const int in_atom = idx % (KBLK * 8);
                        const int key = k0 + (in_atom >> 3);
                        const int first = key / PAGE * PAGE;
                        const bool copied = !(first > hi || first + PAGE - 1 < lo) && table[first / PAGE] >= 0;
                        if (!copied || key > hi)
                            *reinterpret_cast<uint4*>(smem + OFF_V + st * KV_BYTES + (idx / (KBLK * 8)) * ATOM_BYTES + (in_atom << 4)) = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
            }
            fence_async_smem();
            tmem_st_wait();
            fence_before_sync();
            mbar_arrive(p_ready);
            last = i;
        }
        ok = __all_sync(0xffffffffu, ok);
        float o[DH];                                                     // the row's output against m, not yet divided by l
#pragma unroll
        for (int j = 0; j < DH; ++j) o[j] = 0.f;
        if (ok && last >= 0) {
            ok = mbar_wait(o_final0 + 8 * grp, 0, give_up, 13);
            ok = __all_sync(0xffffffffu, ok);
            if (ok) fence_after_sync();
            if (ok) {
#pragma unroll
                for (int h = 0; h < DH / 32; ++h) {
                    uint32_t v[32];
                    tmem_ld32(t_o + h * 32, v);
                    tmem_ld_wait(v);
#pragma unroll
                    for (int j = 0; j < 32; ++j) o[h * 32 + j] = __uint_as_float(v[j]);
                }
            }
        }
        if (GROUPS == 1) {
            // one group holds the whole row: out = o / l
            ok = __all_sync(0xffffffffu, ok);
            if (ok && valid) {
                const float inv = l > 0.f ? 1.0f / l : 0.f;
                __nv_bfloat16* dst = p.out + ((size_t)(q_begin + tok0 + row) * p.H + head) * DH;
#pragma unroll
                for (int j = 0; j < DH; j += 8)
                    *reinterpret_cast<uint4*>(dst + j) = make_uint4(pack_bf16(o[j] * inv, o[j + 1] * inv), pack_bf16(o[j + 2] * inv, o[j + 3] * inv),
                                                                    pack_bf16(o[j + 4] * inv, o[j + 5] * inv), pack_bf16(o[j + 6] * inv, o[j + 7] * inv));
            }
        } else {
            // The groups merge: each finishes half of the head's dimensions, and hands the other half of its output,
            // with its maximum and sum, to the other group through shared memory.
            float* mine = reinterpret_cast<float*>(smem + OFF_MERGE + grp * MERGE_BYTES);          // [row][MERGE_ROW]
            const float* theirs = reinterpret_cast<const float*>(smem + OFF_MERGE + (grp ^ 1) * MERGE_BYTES);
#pragma unroll
            for (int j = 0; j < DH / 2; ++j) mine[row * MERGE_ROW + j] = grp ? o[j] : o[DH / 2 + j];
            xch[(grp * 2) * ROWS + row] = m;
            xch[(grp * 2 + 1) * ROWS + row] = l;
            mbar_arrive(l_ready);
            ok = mbar_wait(l_ready, 0, give_up, 14) && ok;
            ok = __all_sync(0xffffffffu, ok);
            if (ok && valid) {
                const float m_o = xch[((grp ^ 1) * 2) * ROWS + row], l_o = xch[((grp ^ 1) * 2 + 1) * ROWS + row];
                const float mm = fmaxf(m, m_o), m_use = mm == -INFINITY ? 0.f : mm;
                const float a = bl_ex2(m - m_use), a_o = bl_ex2(m_o - m_use);
                const float total = l * a + l_o * a_o;
                const float inv = total > 0.f ? 1.0f / total : 0.f;
                const float wa = a * inv, wo = a_o * inv;
                float r[DH / 2];
#pragma unroll
                for (int j = 0; j < DH / 2; ++j) r[j] = (grp ? o[DH / 2 + j] : o[j]) * wa + theirs[row * MERGE_ROW + j] * wo;
                __nv_bfloat16* dst = p.out + ((size_t)(q_begin + tok0 + row) * p.H + head) * DH + grp * (DH / 2);
#pragma unroll
                for (int j = 0; j < DH / 2; j += 8)
                    *reinterpret_cast<uint4*>(dst + j) = make_uint4(pack_bf16(r[j], r[j + 1]), pack_bf16(r[j + 2], r[j + 3]),
                                                                    pack_bf16(r[j + 4], r[j + 5]), pack_bf16(r[j + 6], r[j + 7]));
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

}  // namespace

extern "C" int bl_attention_prefill_tc_supported(int dh, int page_size) { return (dh == 64 || dh == 128) && page_size == PAGE; }

namespace {

template <class S>
int launch(const void* q, const void* k_cache, const void* v_cache, const Params& p, int n_tiles, int T, int n_pages, cudaStream_t stream) {
    CUtensorMap mq, mk, mv;
    if (bl_make_map_bf16(WHO, &mq, q, T, p.H * S::DH, ROWS, 64)) return 1;
    if (bl_make_map_bf16(WHO, &mk, k_cache, (long long)n_pages * p.KV * PAGE, S::DH, PAGE, 64)) return 1;
    if (bl_make_map_bf16(WHO, &mv, v_cache, (long long)n_pages * p.KV * PAGE, S::DH, PAGE, 64)) return 1;
    static bool configured = false;                                      // per shape
    if (!configured) {
        BL_CUDA(cudaFuncSetAttribute(attention_tc_kernel<S>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM_BYTES));
        configured = true;
    }
    // A block waits (griddepcontrol.wait) before it allocates tensor memory or touches data, so it may be launched
    // while the kernel before it still runs.
    BL_CUDA(bl_launch_dependent(attention_tc_kernel<S>, dim3(n_tiles * p.H, 1, 1), dim3(S::THREADS), (size_t)S::SMEM_BYTES, stream,
                                mq, mk, mv, p));
    BL_CHECK_LAUNCH("bl_attention_prefill_tc");
    return 0;
}

}  // namespace

// tiles[n_tiles][2] = (request, first token of the tile's 128 rows within the request's new tokens); the last
// entries start first. T: rows of q and out; n_pages: pages of the cache tensors (their first dimension).
extern "C" int bl_attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache, const int* cu_q,
                                       const int* ctx_len, const int* block_table, int max_pages, const int* tiles,
                                       int n_tiles, void* out, int T, int n_pages, int H, int KV, int dh, int page_size,
                                       int window, float scale, void* stream) {
    if (n_tiles <= 0) return 0;
    if ((dh != 64 && dh != 128) || page_size != PAGE)
        BL_FAIL("bl_attention_prefill_tc: head size %d with pages of %d tokens is not built (64 or 128 with 16 only)", dh, page_size);
    if (H <= 0 || KV <= 0 || H % KV != 0) BL_FAIL("bl_attention_prefill_tc: %d heads cannot share %d key/value heads", H, KV);
    if (max_pages <= 0 || window < 0 || T <= 0 || n_pages <= 0) BL_FAIL("bl_attention_prefill_tc: bad sizes");
    if (!(scale > 0.f)) BL_FAIL("bl_attention_prefill_tc: the scale of the scores must be positive (got %g)", (double)scale);
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) & 15)
        BL_FAIL("bl_attention_prefill_tc: q, the caches and out must be 16-byte aligned");
    if ((long long)n_tiles * H > 2147483647LL) BL_FAIL("bl_attention_prefill_tc: %d tiles x %d heads are more blocks than a launch takes", n_tiles, H);
    Params p;
    p.out = (__nv_bfloat16*)out; p.cu_q = cu_q; p.ctx_len = ctx_len; p.block_table = block_table; p.max_pages = max_pages;
    p.tiles = tiles; p.H = H; p.KV = KV; p.window = window; p.scale_log2 = scale * 1.4426950408889634f;
    if (dh == 64) return launch<Shape<64, 2>>(q, k_cache, v_cache, p, n_tiles, T, n_pages, (cudaStream_t)stream);
    return launch<Shape<128, 1>>(q, k_cache, v_cache, p, n_tiles, T, n_pages, (cudaStream_t)stream);
}

// Reads and clears the status word: 0 when no block has given up on a wait since the last call. Codes name the
// wait: 1 q, 2 first keys, 3 / 7 a stage of keys / values to become free, 4 a buffer of scores to become free, 12 P,
// 5 values, 6 keys, 8 scores, 13 the group's last product, 10 values (row warps), 11 a share of the output, 14 the other group at the merge, 9 shared
// memory not 1024-byte aligned.
// Synchronises the device.
extern "C" int bl_attention_prefill_tc_status(int* status) {
    int v = 0, zero = 0;
    BL_CUDA(cudaMemcpyFromSymbol(&v, g_status, sizeof(int)));
    if (v != 0) BL_CUDA(cudaMemcpyToSymbol(g_status, &zero, sizeof(int)));
    *status = v;
    return 0;
}
