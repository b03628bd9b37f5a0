// Paged causal grouped-query attention on tensor cores (bfloat16 operands, 32-bit accumulation and
// softmax statistics), in two shapes that share their inner loops:
//   prefill: a block is 64 consecutive tokens of one request and one query head, 16 rows per warp, and
//            walks the request's keys in blocks of 64 (four 16-token pages) up to the diagonal;
//   decode:  a block is one single-token request, one key/value head and one slice of its keys; the 16 MMA
//            rows are the query heads that share that key/value head (every key and value is read once
//            for all of them); each of the four warps streams a page of every 64-key block through a
//            cp.async ring of its own, with no barrier of the block in the loop; the slices of long contexts
//            are merged from partial (max, sum, output) triples: up to 16 slices are the blocks of one
//            thread-block cluster and merge through distributed shared memory, each block finishing a share
//            of the outputs; more slices (or a caller that brings scratch memory) go through global scratch,
//            merged by whichever block of the (request, head group) finishes last.
// Keys and values come from the request's pages through its block table with 16-byte cp.async copies into
// padded shared-memory tiles. Softmax is the online form of the reference's flash kernels
// (FlashAttnRegKernel, src/math_gpu.br:3309-3504: running max m, sum l, rescale by exp(m - m_new)); the
// split of one query's keys and its merge follow FlashDecodeKernel / FlashDecodeCombineKernel
// (:3520-3679) and the sharing of key/value reads across a group follows FlashDecodeWarpTail128Kernel
// (:3793-3925). Scores are scaled after the dot product (src/math.br:319-322); a key j is visible to a query
// at position p when j <= p and, with a window, j + window > p (:327-328).
#include "common.cuh"
#include "api.h"

namespace {

constexpr int PAGE = 16;
constexpr int KB = 64;            // keys per block
constexpr int THREADS = 128;
constexpr int PAD = 8;            // bfloat16 elements of padding per shared-memory row (keeps ldmatrix conflict-free)

struct AttnParams {
    const __nv_bfloat16* q; const __nv_bfloat16* kc; const __nv_bfloat16* vc; __nv_bfloat16* out;
    const int* cu_q; const int* ctx_len; const int* block_table; int max_pages;
    const int* work;              // prefill: [n][2] (request, first token of the tile within the request); decode: [n] requests
    float* part_o; float* part_ml; int n_splits;
    int* counters;                // decode with slices: one per (request, head group), zero between launches
    int H, KV, window; float scale_log2;
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" :: "r"(addr), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" :: "n"(N)); }
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

constexpr int MAX_CLUSTER_SPLITS = 16;     // slices merged through distributed shared memory (a cluster of 16 needs the non-portable size)
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t peer_shared(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t a) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ float2 ld_cluster_f2(uint32_t a) {
    float2 v;
    asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a) : "memory");
    return v;
}

template <int DH>
struct Tiles {
    static constexpr int ROW = DH + PAD;
    static constexpr int STAGE = 2 * KB * ROW;                    // elements: K tile then V tile
    static constexpr int BYTES = 2 * STAGE * (int)sizeof(__nv_bfloat16);
    // decode: every warp has a ring of its own, one page of keys and values per stage
    static constexpr int WSTAGE = 2 * PAGE * ROW;
    static constexpr int WSTAGES = DH <= 128 ? 3 : 2;
    static constexpr int DECODE_BYTES = 4 * WSTAGES * WSTAGE * (int)sizeof(__nv_bfloat16);
};

// Decode: one warp copies the page of keys [key0, key0 + 16) of one key/value head, and its values, into a stage
// of its own. A page outside [lo, hi] or no longer in the table, and keys past hi, become zeros (see load_block).
template <int DH>
__device__ __forceinline__ void load_page(__nv_bfloat16* stage, const AttnParams& p, const int* table, int kvh,
                                          int key0, int lo, int hi) {
    constexpr int CH = DH / 8;
    constexpr int ROW = Tiles<DH>::ROW;
    const int lane = threadIdx.x & 31;
    const int page = (key0 + PAGE - 1 >= lo && key0 <= hi) ? table[key0 / PAGE] : -1;
    const size_t base = page >= 0 ? ((size_t)page * p.KV + kvh) * (PAGE * DH) : 0;
#pragma unroll
    for (int it = 0; it < (PAGE * CH + 31) / 32; ++it) {
        const int i = lane + 32 * it;
        if (i >= PAGE * CH) break;
        const int row = i / CH, c = i % CH;
        __nv_bfloat16* kd = stage + row * ROW + c * 8;
        __nv_bfloat16* vd = kd + PAGE * ROW;
        if (page >= 0 && key0 + row <= hi) {
            cp_async16(kd, p.kc + base + i * 8);
            cp_async16(vd, p.vc + base + i * 8);
        } else {
            *reinterpret_cast<uint4*>(kd) = make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(vd) = make_uint4(0u, 0u, 0u, 0u);
        }
    }
}

// Copies keys [key0, key0 + 64) of one key/value head into a stage. The 16 keys of a page lie together in global
// memory, so a page is copied as one contiguous run of 16-byte chunks (only the destination rows are padded).
// Pages outside [lo, hi] or no longer in the table, and keys past hi on the last page, become zeros: they are
// masked anyway, and zeros keep the value product finite whatever an old request left in a reused page.
template <int DH>
__device__ __forceinline__ void load_block(__nv_bfloat16* stage, const AttnParams& p, const int* table, int kvh,
                                           int key0, int lo, int hi) {
    constexpr int CH = DH / 8;                                    // 16-byte chunks per row
    constexpr int CPP = PAGE * CH;                                // chunks per page
    constexpr int ROW = Tiles<DH>::ROW;
    __nv_bfloat16* ks = stage;
    __nv_bfloat16* vs = stage + KB * ROW;
    int pages[KB / PAGE];
#pragma unroll
    for (int q = 0; q < KB / PAGE; ++q) {
        const int first = key0 + q * PAGE;
        pages[q] = (first + PAGE - 1 >= lo && first <= hi) ? table[first / PAGE] : -1;
    }
#pragma unroll
    for (int it = 0; it < (KB * CH + THREADS - 1) / THREADS; ++it) {
        const int i = threadIdx.x + it * THREADS;
        if (i >= KB * CH) break;
        const int pg = i / CPP, j = i % CPP;
        const int row = j / CH, c = j % CH;
        const int page = pages[pg];
        const int r = pg * PAGE + row;
        __nv_bfloat16* kd = ks + r * ROW + c * 8;
        __nv_bfloat16* vd = vs + r * ROW + c * 8;
        if (page >= 0 && key0 + r <= hi) {
            const size_t off = ((size_t)page * p.KV + kvh) * (PAGE * DH) + j * 8;
            cp_async16(kd, p.kc + off);
            cp_async16(vd, p.vc + off);
        } else {
            *reinterpret_cast<uint4*>(kd) = make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(vd) = make_uint4(0u, 0u, 0u, 0u);
        }
    }
}

// One warp, 16 rows, NT n-tiles of 8 keys starting at key `koff` of the staged block (KROWS keys, then their values).
template <int DH, int NT, int KROWS = KB>
__device__ __forceinline__ void block_step(const __nv_bfloat16* stage, int koff, int key_abs0,
                                           const unsigned (&qf)[DH / 16][4], float (&o)[DH / 8][4],
                                           float (&m)[2], float (&l)[2], const int (&pos)[2], int window,
                                           float scale_log2) {
    constexpr int ROW = Tiles<DH>::ROW;
    const __nv_bfloat16* ks = stage;
    const __nv_bfloat16* vs = stage + KROWS * ROW;
    const int lane = threadIdx.x & 31, t = lane & 3;
    const int mi = lane >> 3, ri = lane & 7;                      // ldmatrix: which 8x8 matrix, which row of it
    float s[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
            unsigned b[4];
            ldmatrix_x4(b, ks + (koff + np * 16 + (mi >> 1) * 8 + ri) * ROW + kk * 16 + (mi & 1) * 8);
            mma_bf16(s[2 * np], qf[kk], b[0], b[1]);
            mma_bf16(s[2 * np + 1], qf[kk], b[2], b[3]);
        }
    }
    // mask, running maximum. The maximum is taken over the raw scores (the scale is positive) and scaled once;
    // 2^(s * scale - m) is then one multiply-add and one special-function instruction per score.
    float mx[2] = {-INFINITY, -INFINITY};
    // most blocks lie wholly inside what both rows may see: no per-key test there
    const int k_first = key_abs0 + koff, k_last = k_first + NT * 8 - 1;
    const bool all_seen = k_last <= min(pos[0], pos[1]) && (window <= 0 || k_first + window > max(pos[0], pos[1]));
    if (all_seen) {
#pragma unroll
        for (int n = 0; n < NT; ++n) {
#pragma unroll
            for (int c = 0; c < 4; ++c) mx[c >> 1] = fmaxf(mx[c >> 1], s[n][c]);
        }
    } else {
#pragma unroll
        for (int n = 0; n < NT; ++n) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int j = k_first + n * 8 + 2 * t + (c & 1);
                const int p = pos[c >> 1];
                const bool seen = j <= p && (window <= 0 || j + window > p);
                const float v = seen ? s[n][c] : -INFINITY;
                s[n][c] = v;
                mx[c >> 1] = fmaxf(mx[c >> 1], v);
            }
        }
    }
    float m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m[h], mx[h] * scale_log2);
        m_use[h] = m_new == -INFINITY ? 0.f : m_new;              // a row that has seen no key yet
        if (m_new != m[h]) {                                       // (after the first blocks the maximum seldom moves)
            const float alpha = bl_ex2(m[h] - m_use[h]);           // 2^-inf = 0 on the first block
            m[h] = m_new;
            l[h] *= alpha;
#pragma unroll
            for (int n = 0; n < DH / 8; ++n) { o[n][2 * h] *= alpha; o[n][2 * h + 1] *= alpha; }
        }
    }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const float e = bl_ex2(fmaf(s[n][c], scale_log2, -m_use[c >> 1]));   // a masked score is -inf: 2^-inf = 0
            s[n][c] = e;
            l[c >> 1] += e;
        }
    }
    // out += P . V, P rounded to bfloat16 as the tensor cores' left operand
#pragma unroll
    for (int kk = 0; kk < NT / 2; ++kk) {
        unsigned a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int np = 0; np < DH / 16; ++np) {
            unsigned b[4];
            ldmatrix_x4_trans(b, vs + (koff + kk * 16 + (mi & 1) * 8 + ri) * ROW + np * 16 + (mi >> 1) * 8);
            mma_bf16(o[2 * np], a, b[0], b[1]);
            mma_bf16(o[2 * np + 1], a, b[2], b[3]);
        }
    }
}

template <int DH, bool DECODE>
__global__ void __launch_bounds__(THREADS, DH <= 64 ? 4 : 1)
attention_mma_kernel(const AttnParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int G = p.H / p.KV;
    bl_pdl_trigger();
    int r, kvh, head0, tok0, split = 0;
    if (DECODE) {
        r = p.work[blockIdx.z];
        const int groups16 = (G + 15) / 16;
        kvh = blockIdx.y / groups16;
        head0 = kvh * G + (blockIdx.y % groups16) * 16;           // first of up to 16 query heads of this block
        split = blockIdx.x;
        tok0 = 0;
    } else {
        // Blocks start in the order of their index: all heads of the last tile, then all heads of the tile before.
        // Late tiles of a request see the most keys: they go first, so that the short ones fill the tail (with the
        // heads outermost, the long tiles of the last heads would start when the SMs are nearly through).
        const int tile = gridDim.x / p.H - 1 - blockIdx.x / p.H;
        r = p.work[2 * tile];
        tok0 = p.work[2 * tile + 1];
        head0 = blockIdx.x % p.H;
        kvh = head0 / G;
    }
    // the step's index arrays are written before its first kernel: they may be read before the wait
    const int q_begin = p.cu_q[r], q_len = p.cu_q[r + 1] - q_begin, ctx = p.ctx_len[r];
    const int* table = p.block_table + (size_t)r * p.max_pages;
    // rows g and g + 8 of this warp
    int pos[2], tok[2], head[2];
    bool valid[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = g + 8 * h;
        if (DECODE) {
            tok[h] = 0; head[h] = head0 + row;
            valid[h] = head[h] < (kvh + 1) * G && q_len > 0;
        } else {
            tok[h] = tok0 + warp * 16 + row; head[h] = head0;
            valid[h] = tok[h] < q_len;
        }
        pos[h] = valid[h] ? ctx - q_len + tok[h] : -1;            // an invalid row sees nothing
    }
    // the block's range of keys
    const int first_tok = DECODE ? 0 : tok0;
    const int last_tok = DECODE ? 0 : min(q_len, tok0 + KB) - 1;
    const int p_first = ctx - q_len + first_tok, p_last = ctx - q_len + last_tok;
    const int lo = p.window > 0 ? max(0, p_first - p.window + 1) : 0;
    const int hi = p_last;
    int b_begin = lo / KB, b_end = hi / KB + 1;
    if (q_len <= 0) b_end = b_begin;
    if (DECODE) {
        const int nb = b_end - b_begin;
        const int per = (nb + p.n_splits - 1) / p.n_splits;
        const int s0 = b_begin + split * per;
        b_end = min(b_end, s0 + per);
        b_begin = min(s0, b_end);
    }
    constexpr int STAGE = Tiles<DH>::STAGE;
    constexpr int WSTAGE = Tiles<DH>::WSTAGE, WSTAGES = Tiles<DH>::WSTAGES;
    const int nb = b_end - b_begin;
    int issued = 0;                                   // blocks whose copies into shared memory have been started
    __nv_bfloat16* wring = smem + warp * WSTAGES * WSTAGE;        // decode: this warp's ring
    if (DECODE) {
        // The cached keys and values of earlier tokens do not depend on the kernel before: pages that do not hold
        // the newest token are copied into the warp's stages right away, and the rest of this slice is started on
        // its way into L2 (the newest token's row is written there by that kernel; L2 stays coherent with it).
        while (issued < WSTAGES && issued < nb && (b_begin + issued) * KB + warp * PAGE + PAGE <= hi) {
            load_page<DH>(wring + issued * WSTAGE, p, table, kvh, (b_begin + issued) * KB + warp * PAGE, lo, hi);
            cp_async_commit();
            ++issued;
        }
        constexpr int LINES = PAGE * DH * 2 / 128 > 0 ? PAGE * DH * 2 / 128 : 1;     // 128-byte lines per (page, head)
        const int first_page = (b_begin + min(nb, WSTAGES)) * (KB / PAGE), last_page = min(b_end * (KB / PAGE), hi / PAGE + 1);
        // (only the next two blocks: asking for a long slice at once, from hundreds of blocks, slowed the copies that are
        // actually waited for; measured 4% of a step at batch 64, nothing at batch 8)
        for (int i = threadIdx.x; i < min(last_page - first_page, 2 * KB / PAGE) * LINES; i += THREADS) {
            const int pg = first_page + i / LINES;
            const int page = pg * PAGE + PAGE - 1 >= lo ? table[pg] : -1;
            if (page >= 0) {
                const size_t off = (((size_t)page * p.KV + kvh) * PAGE) * DH * 2 + (size_t)(i % LINES) * 128;
                bl_prefetch_l2(reinterpret_cast<const char*>(p.kc) + off);
                bl_prefetch_l2(reinterpret_cast<const char*>(p.vc) + off);
            }
        }
    }
    bl_pdl_wait();                                    // q and the newest keys and values come from the kernel before
    unsigned qf[DH / 16][4];
#pragma unroll
    for (int kk = 0; kk < DH / 16; ++kk) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            unsigned lo32 = 0u, hi32 = 0u;
            if (valid[h]) {
                const __nv_bfloat16* qp = p.q + ((size_t)(q_begin + tok[h]) * p.H + head[h]) * DH + kk * 16 + 2 * t;
                lo32 = *reinterpret_cast<const unsigned*>(qp);
                hi32 = *reinterpret_cast<const unsigned*>(qp + 8);
            }
            qf[kk][h] = lo32; qf[kk][2 + h] = hi32;
        }
    }
    float o[DH / 8][4];
#pragma unroll
    for (int n = 0; n < DH / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    if (DECODE) {
        // Every warp walks its own pages (page `warp` of each 64-key block) through its own ring: no barrier of the
        // block inside the loop, and up to WSTAGES pages on their way per warp.
        while (issued < WSTAGES && issued < nb) {
            load_page<DH>(wring + issued * WSTAGE, p, table, kvh, (b_begin + issued) * KB + warp * PAGE, lo, hi);
            cp_async_commit();
            ++issued;
        }
        for (int i = 0; i < nb; ++i) {
            const int pending = issued - (i + 1);     // copies started after page i's
            if (pending >= 3) cp_async_wait<3>(); else if (pending == 2) cp_async_wait<2>();
            else if (pending == 1) cp_async_wait<1>(); else cp_async_wait<0>();
            __syncwarp();
            __nv_bfloat16* st = wring + (i % WSTAGES) * WSTAGE;
            block_step<DH, 2, PAGE>(st, 0, (b_begin + i) * KB + warp * PAGE, qf, o, m, l, pos, p.window, p.scale_log2);
            __syncwarp();
            if (issued < nb) {                        // the stage just used takes the page WSTAGES blocks on
                load_page<DH>(st, p, table, kvh, (b_begin + issued) * KB + warp * PAGE, lo, hi);
                cp_async_commit();
                ++issued;
            }
        }
    } else {
        while (issued < 2 && issued < nb) {           // two blocks in flight before the first is used
            load_block<DH>(smem + (issued & 1) * STAGE, p, table, kvh, (b_begin + issued) * KB, lo, hi);
            cp_async_commit();
            ++issued;
        }
        for (int i = 0; i < nb; ++i) {
            const int b = b_begin + i, st = i & 1;
            if (issued - (i + 1) >= 1) cp_async_wait<1>(); else cp_async_wait<0>();   // block i has landed
            __syncthreads();
            block_step<DH, 8>(smem + st * STAGE, 0, b * KB, qf, o, m, l, pos, p.window, p.scale_log2);
            __syncthreads();
            if (issued < nb) {                        // the stage just used takes the block after next
                load_block<DH>(smem + st * STAGE, p, table, kvh, (b_begin + issued) * KB, lo, hi);
                cp_async_commit();
                ++issued;
            }
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
    if (!DECODE) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            if (!valid[h]) continue;
            const float inv = l[h] > 0.f ? 1.0f / l[h] : 0.f;
            __nv_bfloat16* op = p.out + ((size_t)(q_begin + tok[h]) * p.H + head[h]) * DH + 2 * t;
#pragma unroll
            for (int n = 0; n < DH / 8; ++n)
                *reinterpret_cast<unsigned*>(op + n * 8) = pack_bf16(o[n][2 * h] * inv, o[n][2 * h + 1] * inv);
        }
        return;
    }
    // decode: merge the four warps (same 16 rows, different keys), then write the slice's result.
    // Every thread scales its own accumulators to the rows' common maximum; the sums over the warps
    // are then plain additions of 16-byte words. Rows are DH + 8 floats apart, which keeps the
    // 8-byte stores of a half-warp and the 16-byte loads of a quarter-warp on distinct banks.
    __syncthreads();
    constexpr int SO = DH + 8;
    float* so = reinterpret_cast<float*>(smem_raw);               // [4 warps][16 rows][SO]
    float* sm = so + 4 * 16 * SO;                                 // [4][16] maxima
    float* sl = sm + 4 * 16;                                      // [4][16] sums, then sums at the common maximum
    if (t == 0) {
#pragma unroll
        for (int h = 0; h < 2; ++h) { sm[warp * 16 + g + 8 * h] = m[h]; sl[warp * 16 + g + 8 * h] = l[h]; }
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = g + 8 * h;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, sm[w * 16 + row]);
        const float f = m[h] == -INFINITY ? 0.f : exp2f(m[h] - M);
        if (t == 0) sl[warp * 16 + row] = l[h] * f;
        float* dst = so + (warp * 16 + row) * SO + 2 * t;
#pragma unroll
        for (int n = 0; n < DH / 8; ++n)
            *reinterpret_cast<float2*>(dst + n * 8) = make_float2(o[n][2 * h] * f, o[n][2 * h + 1] * f);
    }
    __syncthreads();
    const int rows_here = min(16, (kvh + 1) * G - head0);
    const int q_tok = q_begin;
    float* cp_ml = sl + 4 * 16;                                   // [16 rows][max, sum] of this slice, for the cluster's merge
    float* cp_o = cp_ml + 32;                                     // [16 rows][DH]
    constexpr int D4 = DH / 4;
    if (q_len > 0) {
        for (int i = threadIdx.x; i < rows_here * D4; i += THREADS) {
            const int row = i / D4, d = (i % D4) * 4;
            float M = -INFINITY, L = 0.f;
            float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                M = fmaxf(M, sm[w * 16 + row]);
                L += sl[w * 16 + row];
                const float4 a = *reinterpret_cast<const float4*>(so + (w * 16 + row) * SO + d);
                O.x += a.x; O.y += a.y; O.z += a.z; O.w += a.w;
            }
            const int hd = head0 + row;
            if (p.n_splits == 1) {
                const float inv = L > 0.f ? 1.0f / L : 0.f;
                *reinterpret_cast<uint2*>(p.out + ((size_t)q_tok * p.H + hd) * DH + d) =
                    make_uint2(pack_bf16(O.x * inv, O.y * inv), pack_bf16(O.z * inv, O.w * inv));
            } else if (p.part_o == nullptr) {                             // the slices are the blocks of one cluster: the partial result stays here
                *reinterpret_cast<float4*>(cp_o + row * DH + d) = O;
                if (d == 0) *reinterpret_cast<float2*>(cp_ml + row * 2) = make_float2(M, L);
            } else {
                const size_t slot = ((size_t)blockIdx.z * p.H + hd) * p.n_splits + split;
                *reinterpret_cast<float4*>(p.part_o + slot * DH + d) = O;
                if (d == 0) *reinterpret_cast<float2*>(p.part_ml + slot * 2) = make_float2(M, L);
            }
        }
    }
    if (p.n_splits == 1 || q_len <= 0) return;
    if (p.part_o == nullptr) {
        // The slices of this (request, head group) are the blocks of one cluster, in slice order. Their partial results
        // meet in distributed shared memory: no scratch in global memory, no fence, no ticket. Every block finishes a
        // share of the (row, four dimensions) items: out = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M), slices
        // added in slice order (FlashDecodeCombineKernel, src/math_gpu.br:3597-3631).
        cluster_sync_all();                                           // every slice's partial result is written
        const uint32_t ml_base = (uint32_t)__cvta_generic_to_shared(cp_ml), o_base = (uint32_t)__cvta_generic_to_shared(cp_o);
        for (int i = split + (int)threadIdx.x * p.n_splits; i < rows_here * D4; i += THREADS * p.n_splits) {
            const int row = i / D4, d = (i % D4) * 4;
            float2 ml[MAX_CLUSTER_SPLITS];
            float4 po[MAX_CLUSTER_SPLITS];
#pragma unroll
            for (int s2 = 0; s2 < MAX_CLUSTER_SPLITS; ++s2) {             // all loads on their way before any is used
                if (s2 >= p.n_splits) break;
                ml[s2] = ld_cluster_f2(peer_shared(ml_base + (uint32_t)(row * 2) * 4u, (uint32_t)s2));
                po[s2] = ld_cluster_f4(peer_shared(o_base + (uint32_t)(row * DH + d) * 4u, (uint32_t)s2));
            }
            float M = -INFINITY;
#pragma unroll
            for (int s2 = 0; s2 < MAX_CLUSTER_SPLITS; ++s2) { if (s2 >= p.n_splits) break; M = fmaxf(M, ml[s2].x); }
            float L = 0.f;
            float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int s2 = 0; s2 < MAX_CLUSTER_SPLITS; ++s2) {
                if (s2 >= p.n_splits) break;
                const float f = ml[s2].x == -INFINITY ? 0.f : exp2f(ml[s2].x - M);
                L += ml[s2].y * f;
                O.x += po[s2].x * f; O.y += po[s2].y * f; O.z += po[s2].z * f; O.w += po[s2].w * f;
            }
            const float inv = L > 0.f ? 1.0f / L : 0.f;
            *reinterpret_cast<uint2*>(p.out + ((size_t)q_tok * p.H + head0 + row) * DH + d) =
                make_uint2(pack_bf16(O.x * inv, O.y * inv), pack_bf16(O.z * inv, O.w * inv));
        }
        cluster_sync_all();                                           // no block leaves while another may still read its partial result
        return;
    }
    // The block that finishes last among the slices of this (request, head group) merges them:
    // out = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M) (FlashDecodeCombineKernel, src/math_gpu.br:3597-3631).
    // Slices are added in slice order whoever merges, so the result does not depend on which block was last.
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int* counter = p.counters + (size_t)blockIdx.z * gridDim.y + blockIdx.y;
        const int ticket = atomicAdd(counter, 1);
        s_last = ticket == p.n_splits - 1;
        if (s_last) *counter = 0;                                  // ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    float* wts = reinterpret_cast<float*>(smem_raw);               // [rows_here][n_splits] weights 2^(m_s - M), then L per row
    float* sL = wts + 16 * p.n_splits;
    // One thread per (row, four dimensions). Its first PRE slices are requested before the weights are
    // worked out, so that the two round trips to L2 overlap.
    const int mine = threadIdx.x;                                  // rows_here * D4 <= 16 * 64: up to 8 items a thread
    const bool first_item = mine < rows_here * D4;
    constexpr int PRE = 8;
    float4 a0[PRE];
    {
        const int row = first_item ? mine / D4 : 0, d = first_item ? (mine % D4) * 4 : 0;
        const float4* po = reinterpret_cast<const float4*>(p.part_o + (((size_t)blockIdx.z * p.H + head0 + row) * p.n_splits) * DH + d);
#pragma unroll
        for (int j = 0; j < PRE; ++j)
            a0[j] = first_item && j < p.n_splits ? __ldcg(po + (size_t)j * D4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int row = warp; row < rows_here; row += 4) {
        const float2* ml = reinterpret_cast<const float2*>(p.part_ml) + ((size_t)blockIdx.z * p.H + head0 + row) * p.n_splits;
        // every lane's (max, sum) pairs are loaded at once (up to 8 per lane: 256 slices), then used twice
        float2 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int s2 = lane + 32 * i;
            v[i] = s2 < p.n_splits ? __ldcg(ml + s2) : make_float2(-INFINITY, 0.f);
        }
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < 8; ++i) mx = fmaxf(mx, v[i].x);
        mx = bl_warp_max(mx);
        float lsum = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {                              // lanes in slice order, 32 slices at a time
            if (32 * i >= p.n_splits) break;
            const int s2 = lane + 32 * i;
            const float f = v[i].x == -INFINITY ? 0.f : exp2f(v[i].x - mx);
            float lv = v[i].y * f;
            if (s2 < p.n_splits) wts[row * p.n_splits + s2] = f;
#pragma unroll
            for (int o2 = 1; o2 < 32; o2 <<= 1) {                  // a prefix sum keeps the order of the additions fixed
                const float up = __shfl_up_sync(0xffffffffu, lv, o2);
                if (lane >= o2) lv += up;
            }
            lsum += __shfl_sync(0xffffffffu, lv, 31);
        }
        if (lane == 0) sL[row] = lsum;
    }
    __syncthreads();
    // sixteen 16-byte loads in flight, slices added in slice order
    for (int i = threadIdx.x; i < rows_here * D4; i += THREADS) {
        const int row = i / D4, d = (i % D4) * 4;
        const float4* po = reinterpret_cast<const float4*>(p.part_o + (((size_t)blockIdx.z * p.H + head0 + row) * p.n_splits) * DH + d);
        float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s0 = 0; s0 < p.n_splits; s0 += 16) {
            float4 a[16];
            const bool have = i == mine && s0 == 0;               // the first PRE slices are already here
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                if (j < PRE && have) a[j] = a0[j];
                else a[j] = s0 + j < p.n_splits ? __ldcg(po + (size_t)(s0 + j) * D4) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float f = s0 + j < p.n_splits ? wts[row * p.n_splits + s0 + j] : 0.f;
                O.x += a[j].x * f; O.y += a[j].y * f; O.z += a[j].z * f; O.w += a[j].w * f;
            }
        }
        const float L = sL[row];
        const float inv = L > 0.f ? 1.0f / L : 0.f;
        __nv_bfloat16* dst = p.out + ((size_t)q_tok * p.H + head0 + row) * DH + d;
        *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(O.x * inv, O.y * inv), pack_bf16(O.z * inv, O.w * inv));
    }
}

template <int DH, bool DECODE>
int launch(const AttnParams& p, dim3 grid, cudaStream_t s) {
    static bool configured = false;                               // per template instance
    int bytes = DECODE ? Tiles<DH>::DECODE_BYTES : Tiles<DH>::BYTES;  // the stages; reused by the merges
    if (bytes < (int)((4 * 16 * (DH + 8) + 128) * sizeof(float))) bytes = (int)((4 * 16 * (DH + 8) + 128) * sizeof(float));
    if (bytes < (int)((16 * 256 + 16) * sizeof(float))) bytes = (int)((16 * 256 + 16) * sizeof(float));
    if (!configured) {
        BL_CUDA(cudaFuncSetAttribute(attention_mma_kernel<DH, DECODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
        configured = true;
    }
    if (DECODE && p.n_splits > 1 && p.part_o == nullptr) {
        // the slices of a request are the blocks of one cluster (grid.x = slices = cluster size)
        static int allowed = 0;                                   // largest cluster this kernel may be launched with (0: not asked yet)
        if (allowed == 0) {
            BL_CUDA(bl_same_carveout(attention_mma_kernel<DH, DECODE>));
            allowed = cudaFuncSetAttribute(attention_mma_kernel<DH, DECODE>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess
                          ? MAX_CLUSTER_SPLITS : 8;
            (void)cudaGetLastError();
        }
        if (p.n_splits > allowed)
            BL_FAIL("bl_attention_decode: %d slices without scratch memory (clusters of up to %d blocks merge in shared memory)", p.n_splits, allowed);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid; cfg.blockDim = dim3(THREADS); cfg.dynamicSmemBytes = (size_t)bytes; cfg.stream = s;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = p.n_splits; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = bl_pdl_enabled() ? 1 : 0;
        cfg.attrs = attr; cfg.numAttrs = 2;
        BL_CUDA(cudaLaunchKernelEx(&cfg, attention_mma_kernel<DH, DECODE>, p));
        BL_CHECK_LAUNCH("bl_attention_mma");
        return 0;
    }
    BL_CUDA(bl_launch_dependent(attention_mma_kernel<DH, DECODE>, grid, dim3(THREADS), (size_t)bytes, s, p));
    BL_CHECK_LAUNCH("bl_attention_mma");
    return 0;
}

template <int DH>
int decode_resident() {
    int bytes = Tiles<DH>::DECODE_BYTES;
    if (bytes < (int)((4 * 16 * (DH + 8) + 128) * sizeof(float))) bytes = (int)((4 * 16 * (DH + 8) + 128) * sizeof(float));
    if (bytes < (int)((16 * 256 + 16) * sizeof(float))) bytes = (int)((16 * 256 + 16) * sizeof(float));
    int dev = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    if (cudaFuncSetAttribute(attention_mma_kernel<DH, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_mma_kernel<DH, true>, THREADS, (size_t)bytes) != cudaSuccess) return 0;
    return sms * per_sm;
}

template <bool DECODE>
int dispatch(int dh, const AttnParams& p, dim3 grid, cudaStream_t s) {
    switch (dh) {
        case 16: return launch<16, DECODE>(p, grid, s);
        case 32: return launch<32, DECODE>(p, grid, s);
        case 48: return launch<48, DECODE>(p, grid, s);
        case 64: return launch<64, DECODE>(p, grid, s);
        case 96: return launch<96, DECODE>(p, grid, s);
        case 128: return launch<128, DECODE>(p, grid, s);
        default: BL_FAIL("bl_attention_mma: head size %d is not built (16, 32, 48, 64, 96, 128); use the plain kernel", dh);
    }
}

int check(int H, int KV, int dh, int page_size, int max_pages, int window, float scale) {
    if (!(scale > 0.f)) BL_FAIL("bl_attention_mma: the scale of the scores must be positive (got %g)", (double)scale);
    if (H <= 0 || KV <= 0 || H % KV != 0) BL_FAIL("bl_attention_mma: %d heads cannot share %d key/value heads", H, KV);
    if (page_size != PAGE) BL_FAIL("bl_attention_mma: pages of %d tokens are not built (16 only); use the plain kernel", page_size);
    if (max_pages <= 0 || window < 0) BL_FAIL("bl_attention_mma: bad table width or window");
    if (dh != 16 && dh != 32 && dh != 48 && dh != 64 && dh != 96 && dh != 128)
        BL_FAIL("bl_attention_mma: head size %d is not built (16, 32, 48, 64, 96, 128); use the plain kernel", dh);
    return 0;
}

}  // namespace

extern "C" int bl_attention_mma_supported(int dh, int page_size) {
    return page_size == PAGE && (dh == 16 || dh == 32 || dh == 48 || dh == 64 || dh == 96 || dh == 128);
}

// Blocks of the decode shape that the current device holds at once (SMs x blocks per SM for this head size), 0 when
// the head size is not built: launches of about this many blocks fill the device in one round.
extern "C" int bl_attention_decode_resident_blocks(int dh) {
    switch (dh) {
        case 16: return decode_resident<16>();
        case 32: return decode_resident<32>();
        case 48: return decode_resident<48>();
        case 64: return decode_resident<64>();
        case 96: return decode_resident<96>();
        case 128: return decode_resident<128>();
        default: return 0;
    }
}

// Prefill shape. tiles: [n_tiles][2] = (request, first token of a 64-token tile inside the request's new tokens).
extern "C" int bl_attention_prefill(const void* q, const void* k_cache, const void* v_cache, const int* cu_q,
                                    const int* ctx_len, const int* block_table, int max_pages, const int* tiles,
                                    int n_tiles, void* out, int H, int KV, int dh, int page_size, int window,
                                    float scale, void* stream) {
    if (n_tiles <= 0) return 0;
    if (check(H, KV, dh, page_size, max_pages, window, scale)) return 1;
    AttnParams p;
    p.q = (const __nv_bfloat16*)q; p.kc = (const __nv_bfloat16*)k_cache; p.vc = (const __nv_bfloat16*)v_cache;
    p.out = (__nv_bfloat16*)out; p.cu_q = cu_q; p.ctx_len = ctx_len; p.block_table = block_table; p.max_pages = max_pages;
    p.work = tiles; p.part_o = nullptr; p.part_ml = nullptr; p.counters = nullptr; p.n_splits = 1; p.H = H; p.KV = KV; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    if ((long long)n_tiles * H > 2147483647LL) BL_FAIL("bl_attention_prefill: %d tiles x %d heads are more blocks than a launch takes", n_tiles, H);
    return dispatch<false>(dh, p, dim3(n_tiles * H, 1, 1), (cudaStream_t)stream);
}

// Floats of scratch that bl_attention_decode needs for n requests and n_splits slices (0 when n_splits is 1).
extern "C" long long bl_attention_decode_scratch_floats(int n, int H, int dh, int n_splits) {
    return n_splits <= 1 ? 0 : (long long)n * H * n_splits * (dh + 2);
}

// Decode shape. reqs: [n] indices of single-token requests. scratch: bl_attention_decode_scratch_floats() floats.
extern "C" int bl_attention_decode(const void* q, const void* k_cache, const void* v_cache, const int* cu_q,
                                   const int* ctx_len, const int* block_table, int max_pages, const int* reqs, int n,
                                   int n_splits, float* scratch, int* counters, void* out, int H, int KV, int dh,
                                   int page_size, int window, float scale, void* stream) {
    if (n <= 0) return 0;
    if (check(H, KV, dh, page_size, max_pages, window, scale)) return 1;
    if (n_splits < 1 || n_splits > 256) BL_FAIL("bl_attention_decode: %d slices (1..256)", n_splits);
    if (n_splits > 1 && scratch != nullptr && counters == nullptr)
        BL_FAIL("bl_attention_decode: slices merged through scratch memory need zeroed counters");
    if (n_splits > MAX_CLUSTER_SPLITS && scratch == nullptr)
        BL_FAIL("bl_attention_decode: more than %d slices need scratch memory and zeroed counters", MAX_CLUSTER_SPLITS);
    AttnParams p;
    p.q = (const __nv_bfloat16*)q; p.kc = (const __nv_bfloat16*)k_cache; p.vc = (const __nv_bfloat16*)v_cache;
    p.out = (__nv_bfloat16*)out; p.cu_q = cu_q; p.ctx_len = ctx_len; p.block_table = block_table; p.max_pages = max_pages;
    p.work = reqs; p.n_splits = n_splits; p.H = H; p.KV = KV; p.window = window;
    p.part_o = scratch; p.part_ml = scratch ? scratch + (size_t)n * H * n_splits * dh : nullptr;
    p.counters = counters;
    p.scale_log2 = scale * 1.4426950408889634f;
    const int G = H / KV;
    return dispatch<true>(dh, p, dim3(n_splits, KV * ((G + 15) / 16), n), (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------------
// Decode attention for callers that must not allocate. See no_alloc.h.
// ---------------------------------------------------------------------------------------------------
#include "no_alloc.h"

namespace {

// Partial results of the slices live here instead of in memory the caller allocates. The array is part of the
// library's image on every GPU that loads it (8 MiB each, until the process exits).
static __device__ __align__(256) float g_static_scratch[BL_NO_ALLOC_SCRATCH_FLOATS];

// One counter per (request, head group) for the merge; zero when the library is loaded, and every launch leaves
// them at zero again.
static __device__ __align__(256) int g_static_counters[BL_NO_ALLOC_COUNTERS];

}  // namespace

extern "C" int bl_attention_decode_no_alloc(const void* q, const void* k_cache, const void* v_cache, const int* cu_q,
                                            const int* ctx_len, const int* block_table, int max_pages,
                                            const int* reqs, int n, int n_splits, void* out, int H, int KV, int dh,
                                            int page_size, int window, float scale, void* stream) {
    if (n <= 0) return 0;
    // every argument is checked before any arithmetic on it (a caller's KV = 0 must be an error, not a division)
    if (check(H, KV, dh, page_size, max_pages, window, scale)) return 1;
    if (n_splits < 1 || n_splits > 256) BL_FAIL("bl_attention_decode_no_alloc: %d slices (1..256)", n_splits);
    const long long need = bl_attention_decode_scratch_floats(n, H, dh, n_splits);
    if (need > (long long)BL_NO_ALLOC_SCRATCH_FLOATS)
        BL_FAIL("bl_attention_decode_no_alloc: %d requests x %d heads x %d slices x head size %d need %lld floats of "
                "scratch, the built-in array holds %d; use fewer slices or the allocating entry point",
                n, H, n_splits, dh, need, BL_NO_ALLOC_SCRATCH_FLOATS);
    const long long n_counters = (long long)n * KV * ((H / KV + 15) / 16);
    if (n_splits > 1 && n_counters > (long long)BL_NO_ALLOC_COUNTERS)
        BL_FAIL("bl_attention_decode_no_alloc: %d requests x %d head groups need more than the %d built-in counters",
                n, KV * ((H / KV + 15) / 16), BL_NO_ALLOC_COUNTERS);
    float* scratch = nullptr;
    int* counters = nullptr;
    if (n_splits > 1) {
        // In host code the array's name stands for a host-side shadow, not for device memory: a kernel handed
        // `g_static_scratch` itself would fault or touch the wrong memory. The device address has to be asked for,
        // with the device that will run the kernel current, and it differs from device to device. It is asked for
        // on every call (a table look-up inside the runtime, no allocation): nothing is cached here, so there is
        // nothing that two threads could fill at once or that a device reset could leave stale.
        BL_CUDA(cudaGetSymbolAddress((void**)&scratch, g_static_scratch));
        BL_CUDA(cudaGetSymbolAddress((void**)&counters, g_static_counters));
        if (scratch == nullptr || counters == nullptr)
            BL_FAIL("bl_attention_decode_no_alloc: the built-in arrays have no address on the current device");
    }
    return bl_attention_decode(q, k_cache, v_cache, cu_q, ctx_len, block_table, max_pages, reqs, n, n_splits,
                               scratch, counters, out, H, KV, dh, page_size, window, scale, stream);
}
