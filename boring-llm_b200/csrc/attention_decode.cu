// Paged grouped-query attention for requests with one new token (decode), head sizes 64 and 128.
//
// A block is one request, one key/value head (up to 16 of the query heads that share it) and one slice of the
// request's keys. The product is laid out the other way round than in the prefill kernels, so that the eight
// columns of an MMA are query heads and none of its rows is padding:
//   S^T = K . Q^T     m16n8k16: 16 keys x 8 heads per instruction, K from shared memory (ldmatrix), Q^T in registers;
//   P^T               2^(s - m) per (key, head); the accumulator layout (key rows) becomes the B operand's layout
//                     (key pairs along K) with one movmatrix per 8 keys;
//   O^T += V^T . P^T  m16n8k16: 16 dimensions of the head x 8 heads, V^T from the values as they lie in their pages
//                     (ldmatrix.trans).
// Each of the four warps walks units of 32 keys (two pages) of its own through a ring of its own: keys and values
// come page by page as TMA boxes (16 keys x 64 dimensions, 128-byte swizzle: ldmatrix reads them without bank
// conflicts and without padding), each stage with an mbarrier that counts the boxes' bytes; one lane per box issues
// them. The page numbers of 16 stages sit in the warp's registers (one table entry a lane, fetched a round ahead).
// There is no barrier of the block inside the loop. The running maximum of a head moves only when some lane meets a
// larger score (one vote per unit); the exchange across lanes happens then and only then, and gives exactly the
// running maximum of the online softmax (FlashAttnRegKernel, src/math_gpu.br:3309-3504).
// Cached keys and values of earlier tokens do not depend on the kernel before: their boxes are issued before the
// dependent-launch wait; only the unit with the newest token waits for it.
//
// The slices of a request are the blocks of one thread-block cluster (FlashDecodeKernel and
// FlashDecodeCombineKernel, src/math_gpu.br:3520-3679, split one query's keys the same way). After its own four
// warps have been merged, a block sends each row (head) of its partial result to the block that owns the row
// (row mod slices) with st.async into that block's shared memory; the stores count their bytes on the owner's
// mbarrier, so the owner waits for exactly the rows it is owed and for nothing else, merges them in slice order and
// writes the head's output. A cluster barrier before any store (mbarriers initialised) and one at the end (nobody
// leaves while stores to it may be in flight) frame this; neither lies between the last key and the output.
//
// A key j is visible when j <= p and, with a window, j + window > p, p being the new token's position
// (src/math.br:327-328); scores are scaled after the dot product (:319-322). Keys outside that range in a page that
// was copied whole get the score -inf, and their rows of V are zeroed in shared memory, whatever an earlier
// request left there.
//
// Every wait on an mbarrier is bounded. When a bound runs out the warp records a code in a status word, waits
// (bounded again) for the copies it has in flight, and goes on to the barriers that its cluster expects of it; the
// host reads the status word (bl_attention_decode_tma_status) and discards the launch.
#include "tcgen05.cuh"

namespace {

constexpr const char* WHO = "bl_attention_decode_tma";
constexpr int PAGE = 16;
constexpr int UNIT = 32;               // keys per stage: two pages
constexpr int WARPS = 4;
constexpr int THREADS = 32 * WARPS;
constexpr int MAX_SPLITS = 16;         // blocks of a cluster (above 8: the non-portable size)
constexpr int TAB = 16;                // stages whose page numbers a warp's registers hold at a time
constexpr uint32_t WAIT_LIMIT = 1u << 20;

template <int DH_>
struct Shape {
    static constexpr int DH = DH_;
    static constexpr int ATOMS = DH / 64;                         // a row of keys lies as atoms of 64 dimensions (128 bytes)
    static constexpr int KSTEPS = DH / 16;
    static constexpr int BOX_BYTES = PAGE * 128;                  // one page of one atom
    static constexpr int ATOM_BYTES = UNIT * 128;
    static constexpr int TENSOR_BYTES = ATOMS * ATOM_BYTES;       // the keys (or the values) of a stage
    static constexpr int STAGE_BYTES = 2 * TENSOR_BYTES;
    static constexpr int STAGES = DH == 64 ? 3 : 2;
    static constexpr int RING_BYTES = STAGES * STAGE_BYTES;      // per warp
    static constexpr int ROWF = DH + 4;                           // floats of a row in flight: outputs, maximum, sum, two unused
    static constexpr int RECV_SLOTS = 2 * MAX_SPLITS;             // (row / slices) * slices + sender < 16 + slices
    static constexpr int OFF_RECV = WARPS * RING_BYTES;
    static constexpr int OFF_STATS = OFF_RECV + RECV_SLOTS * ROWF * 4;   // the warps' maxima and sums: 2 x [4][16] floats
    static constexpr int OFF_BARS = OFF_STATS + 2 * WARPS * 16 * 4;
    static constexpr int SMEM_BYTES = OFF_BARS + (WARPS * STAGES + 1) * 8 + 16 + 1024;    // + flag, + room to align to 1,024 bytes
    static_assert(DH % 64 == 0 && 16 * ROWF * 4 <= RING_BYTES, "a warp's partial result must fit its ring");
};

__device__ int g_status = 0;           // 0 = fine; else the code of the first wait that ran out

struct Params {
    const __nv_bfloat16* q; __nv_bfloat16* out;
    const int* cu_q; const int* ctx_len; const int* block_table; int max_pages;
    const int* reqs; int n_splits;
    int H, KV, window; float scale_log2;
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
// An 8 x 8 matrix of 16-bit elements held one row per quad (the accumulator's layout), transposed across the warp.
__device__ __forceinline__ unsigned movmatrix_trans(unsigned a) {
    unsigned d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ float ex2(float x) {                  // 2^x on the special-function unit; 2^-inf = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t peer_shared(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
// 16 (8) bytes from registers into a block of the cluster's shared memory; their count is taken off that block's mbarrier
__device__ __forceinline__ void st_async_f4(uint32_t addr, float4 v, uint32_t bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];"
                 :: "r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w), "r"(bar) : "memory");
}
__device__ __forceinline__ void st_async_f2(uint32_t addr, float2 v, uint32_t bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.f32 [%0], {%1, %2}, [%3];"
                 :: "r"(addr), "f"(v.x), "f"(v.y), "r"(bar) : "memory");
}
// One try of a wait whose completion other blocks of the cluster bring about
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait. False when the bound ran out (the code of the first such wait is kept in the status word).
template <bool CLUSTER>
__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, int code) {
#pragma unroll 1
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i)
        if (CLUSTER ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity)) return true;
    atomicCAS(&g_status, 0, code);
    return false;
}

// One unit of 32 keys: scores, running maximum, 2^x, and the product with the values. NH: n-tiles of 8 heads.
// EDGE: some of the unit's keys lie outside [lo, hi] (their rows of V are zero already).
template <int DH, int NH, bool EDGE>
__device__ __forceinline__ void unit_step(uint32_t stage, const uint32_t (&koff)[4], const uint32_t (&voff)[4],
                                          const unsigned (&qb)[NH][DH / 16][2], float (&o)[NH][DH / 16][4],
                                          float (&m)[NH][2], float (&l)[NH][2], int k0, int lo, int hi, float scale_log2) {
    using S = Shape<DH>;
    const int g = (threadIdx.x & 31) >> 2;
    float s[2][NH][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
        for (int nh = 0; nh < NH; ++nh) { s[mt][nh][0] = s[mt][nh][1] = s[mt][nh][2] = s[mt][nh][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < S::KSTEPS; ++kk) {
            unsigned a[4];
            ldmatrix_x4(a, stage + (kk >> 2) * S::ATOM_BYTES + mt * (16 * 128) + koff[kk & 3]);
#pragma unroll
            for (int nh = 0; nh < NH; ++nh) mma_bf16(s[mt][nh], a, qb[nh][kk][0], qb[nh][kk][1]);
        }
    }
    if (EDGE) {
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int j = k0 + mt * 16 + g + 8 * (c >> 1);
                if (j < lo || j > hi) {
#pragma unroll
                    for (int nh = 0; nh < NH; ++nh) s[mt][nh][c] = -INFINITY;
                }
            }
        }
    }
    // this lane's largest raw score per head (columns 2t and 2t + 1 of each n-tile); the scale is positive
    float mx[NH][2];
    bool grows = false;
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[nh][h] = fmaxf(fmaxf(s[0][nh][h], s[0][nh][h + 2]), fmaxf(s[1][nh][h], s[1][nh][h + 2]));
            grows |= mx[nh][h] * scale_log2 > m[nh][h];
        }
    }
    if (__any_sync(0xffffffffu, grows)) {                         // (after the first units the maximum seldom moves)
#pragma unroll
        for (int nh = 0; nh < NH; ++nh) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float v = mx[nh][h];
                v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
                v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
                v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
                const float m_new = fmaxf(m[nh][h], v * scale_log2);
                if (m_new != m[nh][h]) {
                    const float alpha = ex2(m[nh][h] - m_new);    // 2^-inf = 0 for a head that had seen no key
                    m[nh][h] = m_new;
                    l[nh][h] *= alpha;
#pragma unroll
                    for (int mt = 0; mt < DH / 16; ++mt) { o[nh][mt][h] *= alpha; o[nh][mt][h + 2] *= alpha; }
                }
            }
        }
    }
    unsigned pb[2][NH][2];                                        // P^T as B operands: [16 keys][n-tile][k 0-7, k 8-15]
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) {
        const float m0 = m[nh][0] == -INFINITY ? 0.f : m[nh][0], m1 = m[nh][1] == -INFINITY ? 0.f : m[nh][1];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
            const float e0 = ex2(fmaf(s[mt][nh][0], scale_log2, -m0)), e1 = ex2(fmaf(s[mt][nh][1], scale_log2, -m1));
            const float e2 = ex2(fmaf(s[mt][nh][2], scale_log2, -m0)), e3 = ex2(fmaf(s[mt][nh][3], scale_log2, -m1));
            l[nh][0] += e0 + e2;
            l[nh][1] += e1 + e3;
            pb[mt][nh][0] = movmatrix_trans(pack_bf16(e0, e1));   // keys g of this 16: (head 2t, head 2t + 1) -> (key 2t, key 2t + 1) of head g
            pb[mt][nh][1] = movmatrix_trans(pack_bf16(e2, e3));   // keys g + 8
        }
    }
    const uint32_t vs = stage + S::TENSOR_BYTES;
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
        for (int mt = 0; mt < DH / 16; ++mt) {
            unsigned a[4];
            ldmatrix_x4_trans(a, vs + (mt >> 2) * S::ATOM_BYTES + ks * (16 * 128) + voff[mt & 3]);
#pragma unroll
            for (int nh = 0; nh < NH; ++nh) mma_bf16(o[nh][mt], a, pb[ks][nh][0], pb[ks][nh][1]);
        }
    }
}

template <int DH, int NH>
__global__ void __launch_bounds__(THREADS)
attention_decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const Params p) {
    using S = Shape<DH>;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                 // the swizzle of a TMA box follows the address: tiles start on 1,024 bytes
    unsigned char* gen = smem_raw + (base - raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    if (threadIdx.x == 0) { tma_prefetch_map(&map_k); tma_prefetch_map(&map_v); }
    bl_pdl_trigger();
    // the step's index arrays are written before its first kernel: they may be read before the wait
    const int r = p.reqs[blockIdx.z];
    const int G = p.H / p.KV, per_block = 8 * NH;
    const int groups = (G + per_block - 1) / per_block;
    const int kvh = blockIdx.y / groups;
    const int head0 = kvh * G + (blockIdx.y % groups) * per_block;
    const int rows_here = min(per_block, (kvh + 1) * G - head0);
    const int split = blockIdx.x, n_splits = p.n_splits;
    const int q_begin = p.cu_q[r], q_len = p.cu_q[r + 1] - q_begin, ctx = p.ctx_len[r];
    const int* table = p.block_table + (size_t)r * p.max_pages;
    const int hi = ctx - 1;                                       // the new token's position
    const int lo = p.window > 0 ? max(0, hi - p.window + 1) : 0;
    // this block's units of 32 keys, and this warp's among them
    const int u_lo = lo / UNIT, u_end = q_len > 0 ? hi / UNIT + 1 : u_lo;
    const int per = (u_end - u_lo + n_splits - 1) / n_splits;
    const int u0 = min(u_lo + split * per, u_end), u1 = min(u0 + per, u_end);
    const int n_mine = u1 - u0 > warp ? (u1 - u0 - warp + WARPS - 1) / WARPS : 0;
    const uint32_t ring = base + warp * S::RING_BYTES;
    const uint32_t bars = base + S::OFF_BARS, my_bars = bars + warp * S::STAGES * 8, recv_bar = bars + WARPS * S::STAGES * 8;
    const uint32_t recv = base + S::OFF_RECV;
    // rows (heads) whose merge this block owns: split, split + n_splits, ...
    const int rows_owned = n_splits > 1 && rows_here > split ? (rows_here - split + n_splits - 1) / n_splits : 0;
    if (threadIdx.x == 0) {
        for (int i = 0; i < WARPS * S::STAGES + 1; ++i) mbar_init(bars + i * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (rows_owned > 0 && q_len > 0) mbar_expect_tx(recv_bar, (uint32_t)(rows_owned * n_splits * (DH * 4 + 8)));
    }
    __syncthreads();
    if (n_splits > 1) cluster_sync_all();                         // every block's mbarriers exist before anything is sent to them

    // page numbers of stages [TAB * round, TAB * round + TAB): lane 2 j + h holds page h of stage j
    auto load_tab = [&](int round) -> int {
        const int i = TAB * round + (lane >> 1);
        const int pg = (u0 + warp + WARPS * i) * (UNIT / PAGE) + (lane & 1);
        return (i < n_mine && pg * PAGE <= hi && pg * PAGE + PAGE - 1 >= lo) ? table[pg] : -1;
    };
    // stage i of this warp: one lane per box (page, keys or values, atom); an absent page brings no bytes
    auto issue = [&](int i, int tab) {
        const int pg = __shfl_sync(0xffffffffu, tab, 2 * (i & (TAB - 1)) + (lane & 1));
        const int other = __shfl_xor_sync(0xffffffffu, pg, 1);
        const uint32_t bar = my_bars + (i % S::STAGES) * 8;
        const uint32_t dst = ring + (i % S::STAGES) * S::STAGE_BYTES;
        if (lane == 0) mbar_expect_tx(bar, (uint32_t)(((pg >= 0) + (other >= 0)) * 2 * S::ATOMS * S::BOX_BYTES));
        if (lane < 4 * S::ATOMS && pg >= 0) {
            const int values = (lane >> 1) & 1, atom = lane >> 2;
            tma_load_2d(dst + values * S::TENSOR_BYTES + atom * S::ATOM_BYTES + (lane & 1) * S::BOX_BYTES,
                        values ? &map_v : &map_k, bar, atom * 64, (pg * p.KV + kvh) * PAGE);
        }
    };
    int tab = load_tab(0), tab_next = load_tab(1);
    int issued = 0;
    // units that end before the new token: on their way before the kernel before this one has finished
    while (issued < S::STAGES && issued < n_mine && (u0 + warp + WARPS * issued) * UNIT + UNIT <= hi) {
        issue(issued, tab);
        ++issued;
    }
    // ldmatrix addresses inside a swizzled tile: row * 128 + ((16-byte chunk ^ (row & 7)) << 4)
    const int mi = lane >> 3, ri = lane & 7;
    uint32_t koff[4], voff[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        koff[j] = (uint32_t)((ri + 8 * (mi & 1)) * 128 + (((2 * j + (mi >> 1)) ^ ri) << 4));   // keys: rows 0-7 / 8-15, then the next 8 dimensions
        voff[j] = (uint32_t)((ri + 8 * (mi >> 1)) * 128 + (((2 * j + (mi & 1)) ^ ri) << 4));   // values: 8 dimensions on, then keys 8-15
    }
    bl_pdl_wait();                                                // q and the newest key and value come from the kernel before
    while (issued < S::STAGES && issued < n_mine) {
        issue(issued, tab);
        ++issued;
    }
    unsigned qb[NH][DH / 16][2];
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) {
        const bool valid = nh * 8 + g < rows_here && q_len > 0;
        const __nv_bfloat16* qp = p.q + ((size_t)q_begin * p.H + head0 + nh * 8 + g) * DH + 2 * t;
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
            qb[nh][kk][0] = valid ? *reinterpret_cast<const unsigned*>(qp + kk * 16) : 0u;
            qb[nh][kk][1] = valid ? *reinterpret_cast<const unsigned*>(qp + kk * 16 + 8) : 0u;
        }
    }
    float o[NH][DH / 16][4], m[NH][2], l[NH][2];
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) {
        m[nh][0] = m[nh][1] = -INFINITY; l[nh][0] = l[nh][1] = 0.f;
#pragma unroll
        for (int mt = 0; mt < DH / 16; ++mt) { o[nh][mt][0] = o[nh][mt][1] = o[nh][mt][2] = o[nh][mt][3] = 0.f; }
    }
    bool fine = true;
    for (int i = 0; i < n_mine; ++i) {
        const uint32_t stage = ring + (i % S::STAGES) * S::STAGE_BYTES;
        if (!wait_bounded<false>(my_bars + (i % S::STAGES) * 8, (uint32_t)((i / S::STAGES) & 1), 1)) {
            // gave up: the copies still on their way must land before this block's shared memory is given up
            for (int j = i + 1; j < issued; ++j) wait_bounded<false>(my_bars + (j % S::STAGES) * 8, (uint32_t)((j / S::STAGES) & 1), 2);
            fine = false;
            break;
        }
        const int k0 = (u0 + warp + WARPS * i) * UNIT;
        if (k0 < lo || k0 + UNIT - 1 > hi) {
            // rows of V whose keys are not to be seen become zeros (their scores become -inf)
            for (int row = 0; row < UNIT; ++row) {
                if (k0 + row >= lo && k0 + row <= hi) continue;
#pragma unroll
                for (int a = 0; a < S::ATOMS; ++a)
                    *reinterpret_cast<uint32_t*>(gen + (stage - base) + S::TENSOR_BYTES + a * S::ATOM_BYTES + row * 128 + lane * 4) = 0u;
            }
            __syncwarp();
            unit_step<DH, NH, true>(stage, koff, voff, qb, o, m, l, k0, lo, hi, p.scale_log2);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the zeros were plain stores; the stage's next filling is a TMA copy
        } else {
            unit_step<DH, NH, false>(stage, koff, voff, qb, o, m, l, k0, lo, hi, p.scale_log2);
        }
        __syncwarp();                                             // every lane has read the stage
        if (issued < n_mine) {                                    // the stage just used takes the unit STAGES on
            if ((issued & (TAB - 1)) == 0) { tab = tab_next; tab_next = load_tab(issued / TAB + 1); }
            issue(issued, tab);
            ++issued;
        }
    }
    (void)fine;
    // ---- the four warps' partial results become the block's -------------------------------------------------
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float v = l[nh][h];
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            v += __shfl_xor_sync(0xffffffffu, v, 8);
            v += __shfl_xor_sync(0xffffffffu, v, 16);
            l[nh][h] = v;
        }
    }
    constexpr int ROWF = S::ROWF;
    float* so = reinterpret_cast<float*>(gen + warp * S::RING_BYTES);              // [heads][ROWF]: rows 4 floats over a multiple of 16, so that
    float* sm = reinterpret_cast<float*>(gen + S::OFF_STATS);                      // a quad's four heads and the eight dimensions of its lanes
    float* sl = sm + WARPS * 16;                                                   // fall on distinct banks
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int head = nh * 8 + 2 * t + (c & 1);
#pragma unroll
            for (int mt = 0; mt < DH / 16; ++mt) so[head * ROWF + mt * 16 + g + 8 * (c >> 1)] = o[nh][mt][c];
        }
        if (g == 0) {
#pragma unroll
            for (int h = 0; h < 2; ++h) { sm[warp * 16 + nh * 8 + 2 * t + h] = m[nh][h]; sl[warp * 16 + nh * 8 + 2 * t + h] = l[nh][h]; }
        }
    }
    __syncthreads();
    constexpr int D4 = DH / 4;
    if (q_len > 0) {
        for (int i = threadIdx.x; i < rows_here * D4; i += THREADS) {
            const int row = i / D4, d = (i % D4) * 4;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) M = fmaxf(M, sm[w * 16 + row]);
            float L = 0.f;
            float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const float mw = sm[w * 16 + row];
                const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
                const float4 a = *reinterpret_cast<const float4*>(gen + w * S::RING_BYTES + (row * ROWF + d) * 4);
                L += sl[w * 16 + row] * f;
                O.x += a.x * f; O.y += a.y * f; O.z += a.z * f; O.w += a.w * f;
            }
            if (n_splits == 1) {
                const float inv = L > 0.f ? 1.0f / L : 0.f;
                *reinterpret_cast<uint2*>(p.out + ((size_t)q_begin * p.H + head0 + row) * DH + d) =
                    make_uint2(pack_bf16(O.x * inv, O.y * inv), pack_bf16(O.z * inv, O.w * inv));
            } else {
                const uint32_t owner = (uint32_t)(row % n_splits);
                const uint32_t slot = recv + (uint32_t)((row / n_splits) * n_splits + split) * (ROWF * 4);
                const uint32_t bar = peer_shared(recv_bar, owner);
                st_async_f4(peer_shared(slot + d * 4, owner), O, bar);
                if (d == 0) st_async_f2(peer_shared(slot + DH * 4, owner), make_float2(M, L), bar);
            }
        }
    }
    if (n_splits == 1) return;
    // ---- the slices' partial results of the rows this block owns --------------------------------------------
    if (rows_owned > 0 && q_len > 0 && wait_bounded<true>(recv_bar, 0u, 3)) {
        const float* rv = reinterpret_cast<const float*>(gen + S::OFF_RECV);
        for (int i = threadIdx.x; i < rows_owned * D4; i += THREADS) {
            const int k = i / D4, d = (i % D4) * 4, row = split + k * n_splits;
            const float* slot = rv + (size_t)(k * n_splits) * ROWF;
            float M = -INFINITY;
            for (int s2 = 0; s2 < n_splits; ++s2) M = fmaxf(M, slot[s2 * ROWF + DH]);
            float L = 0.f;
            float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s2 = 0; s2 < n_splits; ++s2) {               // out = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M), in slice order
                const float2 ml = *reinterpret_cast<const float2*>(slot + s2 * ROWF + DH);
                const float f = ml.x == -INFINITY ? 0.f : exp2f(ml.x - M);
                const float4 a = *reinterpret_cast<const float4*>(slot + s2 * ROWF + d);
                L += ml.y * f;
                O.x += a.x * f; O.y += a.y * f; O.z += a.z * f; O.w += a.w * f;
            }
            const float inv = L > 0.f ? 1.0f / L : 0.f;
            *reinterpret_cast<uint2*>(p.out + ((size_t)q_begin * p.H + head0 + row) * DH + d) =
                make_uint2(pack_bf16(O.x * inv, O.y * inv), pack_bf16(O.z * inv, O.w * inv));
        }
    }
    cluster_sync_all();                                           // nobody leaves while a store to its shared memory may be in flight
}

template <int DH, int NH>
int configure(int* smem_bytes) {
    static bool done = false;
    *smem_bytes = Shape<DH>::SMEM_BYTES;
    if (!done) {
        BL_CUDA(cudaFuncSetAttribute(attention_decode_kernel<DH, NH>, cudaFuncAttributeMaxDynamicSharedMemorySize, Shape<DH>::SMEM_BYTES));
        BL_CUDA(bl_same_carveout(attention_decode_kernel<DH, NH>));
        // clusters of more than 8 blocks need the kernel's consent; a device that refuses it keeps 8
        if (cudaFuncSetAttribute(attention_decode_kernel<DH, NH>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess)
            (void)cudaGetLastError();
        done = true;
    }
    return 0;
}

// early: the kernel may be launched while its predecessor still runs (programmatic dependent launch); it then starts
// its copies of the cached keys and values under the predecessor's tail. Large clusters of a launch with more blocks
// than SMs are better launched late: placed while the predecessor's blocks still hold SMs, they pile up two to an SM
// beside SMs that stay empty, and a long context then runs at the pace of the doubly loaded SMs.
template <int DH, int NH>
int launch(const CUtensorMap& mk, const CUtensorMap& mv, const Params& p, dim3 grid, bool early, cudaStream_t s) {
    int bytes = 0;
    if (configure<DH, NH>(&bytes)) return 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(THREADS); cfg.dynamicSmemBytes = (size_t)bytes; cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = bl_pdl_enabled() && early ? 1 : 0;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = p.n_splits; attr[1].val.clusterDim.y = 1; attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = p.n_splits > 1 ? 2 : 1;
    BL_CUDA(cudaLaunchKernelEx(&cfg, attention_decode_kernel<DH, NH>, mk, mv, p));
    BL_CHECK_LAUNCH(WHO);
    return 0;
}

template <int DH, int NH>
int resident() {
    int bytes = 0, dev = 0, sms = 0, per_sm = 0;
    if (configure<DH, NH>(&bytes)) return 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_decode_kernel<DH, NH>, THREADS, (size_t)bytes) != cudaSuccess) return 0;
    return sms * per_sm;
}

// Clusters of `cluster` blocks that the current device runs at once (0 when such a cluster cannot be launched).
template <int DH, int NH>
int max_clusters(int cluster) {
    int bytes = 0, n = 0;
    if (configure<DH, NH>(&bytes)) return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cluster, 1, 1); cfg.blockDim = dim3(THREADS); cfg.dynamicSmemBytes = (size_t)bytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = cluster; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr; cfg.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&n, attention_decode_kernel<DH, NH>, &cfg) != cudaSuccess) { (void)cudaGetLastError(); return 0; }
    return n;
}

bool built(int dh, int page_size) { return page_size == PAGE && (dh == 64 || dh == 128); }

}  // namespace

extern "C" int bl_attention_decode_tma_supported(int dh, int page_size) { return built(dh, page_size) ? 1 : 0; }

// Blocks that the current device holds at once (SMs x blocks per SM) for this head size and this many query heads per
// key/value head; 0 when the shape is not built.
extern "C" int bl_attention_decode_tma_resident_blocks(int dh, int heads_per_kv) {
    const bool two = heads_per_kv > 8;
    if (dh == 64) return two ? resident<64, 2>() : resident<64, 1>();
    if (dh == 128) return two ? resident<128, 2>() : resident<128, 1>();
    return 0;
}

// Clusters of `cluster` blocks (the slices of one request and key/value head) that the device runs at once: a launch
// of more of them runs in rounds. 0: the shape is not built or the cluster size cannot be launched.
extern "C" int bl_attention_decode_tma_max_clusters(int dh, int heads_per_kv, int cluster) {
    if (cluster < 1 || cluster > MAX_SPLITS) return 0;
    const bool two = heads_per_kv > 8;
    if (dh == 64) return two ? max_clusters<64, 2>(cluster) : max_clusters<64, 1>(cluster);
    if (dh == 128) return two ? max_clusters<128, 2>(cluster) : max_clusters<128, 1>(cluster);
    return 0;
}

extern "C" int bl_attention_decode_tma(const void* q, const void* k_cache, const void* v_cache, int n_pages, const int* cu_q,
                                       const int* ctx_len, const int* block_table, int max_pages, const int* reqs, int n,
                                       int n_splits, void* out, int H, int KV, int dh, int page_size, int window,
                                       float scale, int early, void* stream) {
    if (n <= 0) return 0;
    if (!(scale > 0.f)) BL_FAIL("%s: the scale of the scores must be positive (got %g)", WHO, (double)scale);
    if (H <= 0 || KV <= 0 || H % KV != 0) BL_FAIL("%s: %d heads cannot share %d key/value heads", WHO, H, KV);
    if (!built(dh, page_size)) BL_FAIL("%s: head size %d with pages of %d is not built (64 or 128, pages of 16)", WHO, dh, page_size);
    if (max_pages <= 0 || window < 0 || n_pages <= 0) BL_FAIL("%s: bad table width, window or page count", WHO);
    if (n_splits < 1 || n_splits > MAX_SPLITS) BL_FAIL("%s: %d slices (1..%d: the blocks of one cluster)", WHO, n_splits, MAX_SPLITS);
    if ((((uintptr_t)q | (uintptr_t)out) & 7) != 0) BL_FAIL("%s: q and out must be 8-byte aligned", WHO);
    Params p;
    p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out; p.cu_q = cu_q; p.ctx_len = ctx_len;
    p.block_table = block_table; p.max_pages = max_pages; p.reqs = reqs; p.n_splits = n_splits;
    p.H = H; p.KV = KV; p.window = window; p.scale_log2 = scale * 1.4426950408889634f;
    CUtensorMap mk, mv;
    if (bl_make_map_bf16(WHO, &mk, k_cache, (long long)n_pages * KV * PAGE, dh, PAGE, 64)) return 1;
    if (bl_make_map_bf16(WHO, &mv, v_cache, (long long)n_pages * KV * PAGE, dh, PAGE, 64)) return 1;
    const int G = H / KV;
    const bool two = G > 8;
    const dim3 grid(n_splits, KV * ((G + (two ? 16 : 8) - 1) / (two ? 16 : 8)), n);
    cudaStream_t s = (cudaStream_t)stream;
    if (dh == 64) return two ? launch<64, 2>(mk, mv, p, grid, early != 0, s) : launch<64, 1>(mk, mv, p, grid, early != 0, s);
    return two ? launch<128, 2>(mk, mv, p, grid, early != 0, s) : launch<128, 1>(mk, mv, p, grid, early != 0, s);
}

// Reads and clears the status word: 0 when no warp has given up on a wait since the last call. 1: a stage's keys
// and values did not arrive; 2: nor did the copies still in flight after that; 3: the other slices' partial results
// did not arrive. Synchronises the device.
extern "C" int bl_attention_decode_tma_status(int* status) {
    int v = 0;
    const int zero = 0;
    BL_CUDA(cudaMemcpyFromSymbol(&v, g_status, sizeof(int)));
    if (v != 0) BL_CUDA(cudaMemcpyToSymbol(g_status, &zero, sizeof(int)));
    *status = v;
    return 0;
}
