// Fused kernels for steps with few rows (decode): a layer's small kernels each cost a chain of dependent
// trips to global memory, so the norm in front of a matrix product and the rotation and cache write behind
// the q/k/v product are folded into the product itself.
//
//   norm -> product -> epilogue, in one launch:
//     rows of the 32-bit residual stream are RMS-normalised (statistics in 32-bit, src/math.br:18-36) into a
//     bfloat16 tile in shared memory; W streams once from global memory straight into tensor-core registers
//     exactly as in gemm_skinny.cu (16-byte loads, k slots dealt as they lie, 8 warps taking 32-wide k chunks
//     in turn, partial sums added in warp order); the epilogue is one of
//       PLAIN   out = acc (+ bias), 32-bit                                  (the output head on the final norm)
//       SWIGLU  out = silu(gate) * up, bfloat16                              (src/math.br:246-261)
//       QKV     split of the joined q/k/v row, rotation of q and k by position (pairs (j, j + head/2) or (2j, 2j + 1),
//               src/math.br:128-157), k and v written into the request's pages, q written out in bfloat16
//               (src/math_gpu.br:2428-2488, 4008-4076 do split + rotation + append in one dispatch, too).
//     For QKV the 16 rows of W that a block owns are 8 dimensions of one head and their partners in the rotation
//     (j + head/2, or 2j + 1 beside 2j), so both halves of every rotation pair end up in the same thread.
#include "common.cuh"
#include "api.h"

namespace {

constexpr int WARPS = 8;
constexpr int MODE_PLAIN = 0, MODE_SWIGLU = 1, MODE_QKV = 2;

struct FusedParams {
    const float* x; const int* row_idx; const void* norm_w; int norm_w_dtype; float eps;
    const __nv_bfloat16* w; const void* bias; int bias_dtype;
    void* out;                        // PLAIN: float [M, N]; SWIGLU: bfloat16 [M, N]; QKV: bfloat16 q [M, H * dh]
    int M, N, K, m_groups;
    // QKV only
    const int* positions; const int* tok_req; const int* block_table; int max_pages;
    const float* inv_freq; float mscale;
    __nv_bfloat16* k_cache; __nv_bfloat16* v_cache; int H, KV, dh, page_size, pair_layout;
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 ld16(const __nv_bfloat16* p, bool ok) {
    return ok ? __ldg(reinterpret_cast<const uint4*>(p)) : make_uint4(0u, 0u, 0u, 0u);
}

template <int MT, int MODE>
__global__ void __launch_bounds__(WARPS * 32, MT == 1 ? (MODE == MODE_SWIGLU ? 3 : 2) : 1)
fused_norm_gemm_kernel(const FusedParams p) {
    constexpr bool GLU = MODE == MODE_SWIGLU;
    constexpr int TOK = MT * 8;
    constexpr int UNROLL = (GLU || MT > 2) ? 2 : 4;    // fewer registers where two matrices stream: three blocks fit an SM
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int K = p.K, XROW = K + 8;
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);                       // [TOK][K + 8]
    float* red = reinterpret_cast<float*>(smem_raw + (((size_t)TOK * XROW * 2 + 15) & ~(size_t)15));   // [GLU?2:1][WARPS][16][TOK + 1]
    float* nws = red + (size_t)(GLU ? 2 : 1) * WARPS * 16 * (TOK + 1);                    // [K] norm weights, 32-bit
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int tile = blockIdx.x / p.m_groups;
    const int m0 = (blockIdx.x % p.m_groups) * TOK;
    // which rows of W are this block's 16 MMA rows
    int r_lo, r_hi, hh = 0, jt = 0;
    if (MODE == MODE_QKV) {
        const int tiles_per_head = p.dh / 16;
        hh = tile / tiles_per_head; jt = tile % tiles_per_head;
        if (p.pair_layout == BL_PAIRS_INTERLEAVED) { r_lo = hh * p.dh + 2 * (jt * 8 + g); r_hi = r_lo + 1; }
        else { r_lo = hh * p.dh + jt * 8 + g; r_hi = r_lo + p.dh / 2; }
    } else {
        r_lo = tile * 16 + g;
        r_hi = r_lo + 8;
    }
    const int n_rows = MODE == MODE_QKV ? (p.H + 2 * p.KV) * p.dh : p.N;
    const bool lo_ok = r_lo < n_rows, hi_ok = r_hi < n_rows;
    const __nv_bfloat16* w_lo = p.w + (size_t)r_lo * K;
    const __nv_bfloat16* w_hi = p.w + (size_t)r_hi * K;
    const __nv_bfloat16* u_lo = p.w + (size_t)(p.N + r_lo) * K;
    const __nv_bfloat16* u_hi = p.w + (size_t)(p.N + r_hi) * K;

    uint4 a_lo[UNROLL], a_hi[UNROLL], g_lo[GLU ? UNROLL : 1], g_hi[GLU ? UNROLL : 1];
    auto fetch = [&](int kc0) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = kc0 + u * WARPS * 32 + 8 * t;
            const bool k_ok = k < K;
            a_lo[u] = ld16(w_lo + k, lo_ok && k_ok);
            a_hi[u] = ld16(w_hi + k, hi_ok && k_ok);
            if (GLU) { g_lo[u] = ld16(u_lo + k, lo_ok && k_ok); g_hi[u] = ld16(u_hi + k, hi_ok && k_ok); }
        }
    };
    bl_pdl_trigger();
    fetch(warp * 32);                                  // W is on its way while the kernel before this one finishes
    {
        const size_t rows_total = MODE == MODE_SWIGLU ? (size_t)2 * p.N : (size_t)n_rows;
        const bool inter = MODE == MODE_QKV && p.pair_layout == BL_PAIRS_INTERLEAVED;    // 16 neighbouring rows, like a plain tile
        const size_t first = MODE == MODE_QKV ? (size_t)hh * p.dh + jt * (inter ? 16 : 8) : (size_t)tile * 16;
        const int span = MODE == MODE_QKV && !inter ? 8 : 16;
        bl_prefetch_rows_l2(p.w, first, span, (size_t)K * 2, rows_total);
        if (MODE == MODE_QKV && !inter) bl_prefetch_rows_l2(p.w, first + p.dh / 2, 8, (size_t)K * 2, rows_total);
        if (MODE == MODE_SWIGLU) bl_prefetch_rows_l2(p.w, (size_t)p.N + first, 16, (size_t)K * 2, rows_total);
    }
    // everything that no earlier kernel of the step writes is fetched before the wait: the norm's weights, and for
    // the q/k/v epilogue each thread's bias pair, position, page and rotation
    for (int k = threadIdx.x; k < K; k += WARPS * 32) nws[k] = bl_load_any(p.norm_w, p.norm_w_dtype, k);
    float e_b0 = 0.f, e_b1 = 0.f, e_cs = 1.f, e_sn = 0.f;
    int e_pos = 0, e_page = -1;
    if (MODE == MODE_QKV && threadIdx.x < 8 * TOK) {
        const int c = threadIdx.x % 8, m = m0 + threadIdx.x / 8;
        if (m < p.M) {
            const bool inter = p.pair_layout == BL_PAIRS_INTERLEAVED;
            const int row_lo = hh * p.dh + (inter ? 2 * (jt * 8 + c) : jt * 8 + c), row_hi = inter ? row_lo + 1 : row_lo + p.dh / 2;
            if (p.bias) { e_b0 = bl_load_any(p.bias, p.bias_dtype, row_lo); e_b1 = bl_load_any(p.bias, p.bias_dtype, row_hi); }
            e_pos = p.positions[m];
            if (hh < p.H + p.KV) {
                const float angle = (float)e_pos * p.inv_freq[jt * 8 + c];
                e_cs = cosf(angle) * p.mscale; e_sn = sinf(angle) * p.mscale;
            }
            if (hh >= p.H && p.k_cache != nullptr)
                e_page = p.block_table[(size_t)p.tok_req[m] * p.max_pages + e_pos / p.page_size];
        }
    }
    bl_pdl_wait();                                     // from here on the residual stream may be read

    __syncthreads();                                   // the norm weights are in shared memory
    // normalise this block's rows into shared memory: warp w takes rows w, w + 8, ...
    constexpr int NB = 8;                              // 16-byte words per lane that hold a row of up to 1,024 values
    if (MT > 1 && K <= NB * 128) {
        // A warp's MT rows at once: all their words are on their way before the first sum is taken (one trip to L2
        // for the warp instead of one per row: at 64 rows a block's norm took 4 us of the kernel's 8). Each row's
        // arithmetic is what the loop below does for it, in the same order.
        float4 v[MT][NB];
#pragma unroll
        for (int r = 0; r < MT; ++r) {
            const int m = m0 + warp + r * WARPS;
            const float* src = p.x + (size_t)(m < p.M ? (p.row_idx ? p.row_idx[m] : m) : 0) * K;
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                const int k = j * 128 + lane * 4;
                v[r][j] = (m < p.M && k < K) ? *reinterpret_cast<const float4*>(src + k) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
#pragma unroll
        for (int r = 0; r < MT; ++r) {
            const int i = warp + r * WARPS, m = m0 + i;
            __nv_bfloat16* dst = xs + (size_t)i * XROW;
            if (m >= p.M) {
                for (int k = lane * 4; k < K; k += 128) *reinterpret_cast<uint2*>(dst + k) = make_uint2(0u, 0u);
                continue;
            }
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < NB; ++j) { ss += v[r][j].x * v[r][j].x; ss += v[r][j].y * v[r][j].y; ss += v[r][j].z * v[r][j].z; ss += v[r][j].w * v[r][j].w; }
            ss = bl_warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)K + p.eps);
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                const int k = j * 128 + lane * 4;
                if (k >= K) continue;
                const float4 nw = *reinterpret_cast<const float4*>(nws + k);
                __nv_bfloat162 lo = __floats2bfloat162_rn(v[r][j].x * inv * nw.x, v[r][j].y * inv * nw.y);
                __nv_bfloat162 hi = __floats2bfloat162_rn(v[r][j].z * inv * nw.z, v[r][j].w * inv * nw.w);
                uint2 pk;
                pk.x = *reinterpret_cast<unsigned*>(&lo); pk.y = *reinterpret_cast<unsigned*>(&hi);
                *reinterpret_cast<uint2*>(dst + k) = pk;
            }
        }
    } else
    for (int i = warp; i < TOK; i += WARPS) {
        const int m = m0 + i;
        __nv_bfloat16* dst = xs + (size_t)i * XROW;
        if (m >= p.M) {
            for (int k = lane * 4; k < K; k += 128) *reinterpret_cast<uint2*>(dst + k) = make_uint2(0u, 0u);
            continue;
        }
        // The row is read in batches of NB 16-byte words per lane, all on their way at once; a row of up to
        // NB * 128 values stays in registers between the sum of squares and the scaling.
        const float* src = p.x + (size_t)(p.row_idx ? p.row_idx[m] : m) * K;
        float4 v[NB];
        auto load_batch = [&](int k0) {
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                const int k = k0 + j * 128 + lane * 4;
                v[j] = k < K ? *reinterpret_cast<const float4*>(src + k) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        };
        const bool single = K <= NB * 128;
        float ss = 0.f;
        for (int k0 = 0; k0 < K; k0 += NB * 128) {
            load_batch(k0);
#pragma unroll
            for (int j = 0; j < NB; ++j) { ss += v[j].x * v[j].x; ss += v[j].y * v[j].y; ss += v[j].z * v[j].z; ss += v[j].w * v[j].w; }
        }
        ss = bl_warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)K + p.eps);
        for (int k0 = 0; k0 < K; k0 += NB * 128) {
            if (!single) load_batch(k0);
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                const int k = k0 + j * 128 + lane * 4;
                if (k >= K) continue;
                const float4 nw = *reinterpret_cast<const float4*>(nws + k);
                __nv_bfloat162 lo = __floats2bfloat162_rn(v[j].x * inv * nw.x, v[j].y * inv * nw.y);
                __nv_bfloat162 hi = __floats2bfloat162_rn(v[j].z * inv * nw.z, v[j].w * inv * nw.w);
                uint2 pk;
                pk.x = *reinterpret_cast<unsigned*>(&lo); pk.y = *reinterpret_cast<unsigned*>(&hi);
                *reinterpret_cast<uint2*>(dst + k) = pk;
            }
        }
    }
    __syncthreads();

    float acc[MT][4], acu[GLU ? MT : 1][4];
#pragma unroll
    for (int j = 0; j < MT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) { acc[j][i] = 0.f; if (GLU) acu[j][i] = 0.f; }
    // warp-uniform loop bounds: the MMA needs all 32 lanes
    for (int kc0 = warp * 32; kc0 < K; kc0 += UNROLL * WARPS * 32) {
        uint4 b[UNROLL][MT];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = kc0 + u * WARPS * 32 + 8 * t;
#pragma unroll
            for (int j = 0; j < MT; ++j)
                b[u][j] = k < K ? *reinterpret_cast<const uint4*>(xs + (size_t)(8 * j + g) * XROW + k) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
            for (int j = 0; j < MT; ++j) {
                mma_bf16(acc[j], a_lo[u].x, a_hi[u].x, a_lo[u].y, a_hi[u].y, b[u][j].x, b[u][j].y);
                mma_bf16(acc[j], a_lo[u].z, a_hi[u].z, a_lo[u].w, a_hi[u].w, b[u][j].z, b[u][j].w);
                if (GLU) {
                    mma_bf16(acu[j], g_lo[u].x, g_hi[u].x, g_lo[u].y, g_hi[u].y, b[u][j].x, b[u][j].y);
                    mma_bf16(acu[j], g_lo[u].z, g_hi[u].z, g_lo[u].w, g_hi[u].w, b[u][j].z, b[u][j].w);
                }
            }
        }
        const int next = kc0 + UNROLL * WARPS * 32;
        if (next < K) fetch(next);
    }
    // c0, c1: (MMA row g, tokens 2t, 2t+1); c2, c3: (MMA row g + 8, same tokens)
    constexpr int RT = TOK + 1;
#pragma unroll
    for (int j = 0; j < MT; ++j) {
        float* r0 = red + ((size_t)warp * 16 + g) * RT + 8 * j + 2 * t;
        float* r1 = red + ((size_t)warp * 16 + g + 8) * RT + 8 * j + 2 * t;
        r0[0] = acc[j][0]; r0[1] = acc[j][1]; r1[0] = acc[j][2]; r1[1] = acc[j][3];
        if (GLU) {
            float* s0 = r0 + (size_t)WARPS * 16 * RT; float* s1 = r1 + (size_t)WARPS * 16 * RT;
            s0[0] = acu[j][0]; s0[1] = acu[j][1]; s1[0] = acu[j][2]; s1[1] = acu[j][3];
        }
    }
    __syncthreads();
    auto total = [&](int plane, int row, int tok) {
        float v = 0.f;
#pragma unroll
        for (int wp = 0; wp < WARPS; ++wp) v += red[((size_t)plane * WARPS * 16 + wp * 16 + row) * RT + tok];
        return v;
    };
    if (MODE == MODE_QKV) {
        // one thread per (dimension pair c, token): both halves of the pair; its constants are in registers
        const int half = p.dh / 2;
        if (threadIdx.x < 8 * TOK) {
            const int c = threadIdx.x % 8, tok = threadIdx.x / 8, m = m0 + tok;
            if (m < p.M) {
                const float v0 = total(0, c, tok) + e_b0, v1 = total(0, c + 8, tok) + e_b1;
                const bool inter = p.pair_layout == BL_PAIRS_INTERLEAVED;
                const int d0 = inter ? 2 * (jt * 8 + c) : jt * 8 + c, d1 = inter ? d0 + 1 : d0 + half;
                const float y0 = v0 * e_cs - v1 * e_sn, y1 = v0 * e_sn + v1 * e_cs;     // cos 1, sin 0 for value heads
                if (hh < p.H) {
                    __nv_bfloat16* q = reinterpret_cast<__nv_bfloat16*>(p.out) + ((size_t)m * p.H + hh) * p.dh;
                    q[d0] = __float2bfloat16_rn(y0); q[d1] = __float2bfloat16_rn(y1);
                } else if (e_page >= 0) {                     // a page < 0 is never scheduled; keep memory safe anyway
                    const bool is_k = hh < p.H + p.KV;
                    const int kvh = is_k ? hh - p.H : hh - p.H - p.KV;
                    __nv_bfloat16* dst = (is_k ? p.k_cache : p.v_cache) +
                        (((size_t)e_page * p.KV + kvh) * p.page_size + e_pos % p.page_size) * p.dh;
                    dst[d0] = __float2bfloat16_rn(y0); dst[d1] = __float2bfloat16_rn(y1);
                }
            }
        }
    } else {
        for (int i = threadIdx.x; i < 16 * TOK; i += WARPS * 32) {
            const int c = i % 16, tok = i / 16;
            const int n = tile * 16 + c, m = m0 + tok;
            if (n >= p.N || m >= p.M) continue;
            float v = total(0, c, tok);
            if (GLU) {
                const float u = total(1, c, tok);
                reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.N + n] = __float2bfloat16_rn(bl_silu(v) * u);
            } else {
                if (p.bias) v += bl_load_any(p.bias, p.bias_dtype, n);
                reinterpret_cast<float*>(p.out)[(size_t)m * p.N + n] = v;
            }
        }
    }
}

size_t smem_bytes(int mt, int K, bool glu) {
    const size_t tok = (size_t)mt * 8;
    const size_t xs = (tok * (K + 8) * 2 + 15) & ~(size_t)15;
    return xs + (glu ? 2 : 1) * (size_t)WARPS * 16 * (tok + 1) * sizeof(float) + (size_t)K * sizeof(float);
}
constexpr size_t SMEM_LIMIT = 200 * 1024;

template <int MT, int MODE>
int launch(const FusedParams& p, int tiles, cudaStream_t s) {
    static size_t configured = 0;
    const size_t bytes = smem_bytes(MT, p.K, MODE == MODE_SWIGLU);
    if (bytes > configured) {
        BL_CUDA(cudaFuncSetAttribute(fused_norm_gemm_kernel<MT, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_LIMIT));
        configured = SMEM_LIMIT;
    }
    BL_CUDA(bl_launch_dependent(fused_norm_gemm_kernel<MT, MODE>, dim3(tiles * p.m_groups), dim3(WARPS * 32), bytes, s, p));
    BL_CHECK_LAUNCH("bl_norm_gemm");
    return 0;
}

template <int MODE>
int dispatch(FusedParams& p, int tiles, cudaStream_t s) {
    // the largest row group whose normalised rows fit shared memory
    int mt = p.M <= 8 ? 1 : p.M <= 16 ? 2 : 4;
    while (mt > 1 && smem_bytes(mt, p.K, MODE == MODE_SWIGLU) > SMEM_LIMIT) mt /= 2;
    if (smem_bytes(mt, p.K, MODE == MODE_SWIGLU) > SMEM_LIMIT)
        BL_FAIL("bl_norm_gemm: rows of %d values do not fit shared memory; run the norm and the product separately", p.K);
    p.m_groups = (p.M + mt * 8 - 1) / (mt * 8);
    if (mt == 1) return launch<1, MODE>(p, tiles, s);
    if (mt == 2) return launch<2, MODE>(p, tiles, s);
    return launch<4, MODE>(p, tiles, s);
}

int check_common(const char* who, const void* x, const void* w, int M, int K, int norm_w_dtype) {
    if (K <= 0 || K % 8 != 0) BL_FAIL("%s: K=%d must be a positive multiple of 8", who, K);
    if (((uintptr_t)x | (uintptr_t)w) & 15) BL_FAIL("%s: x and W must be 16-byte aligned", who);
    if (norm_w_dtype != BL_F32 && norm_w_dtype != BL_BF16) BL_FAIL("%s: unknown norm weight dtype %d", who, norm_w_dtype);
    if (M > 4096) BL_FAIL("%s: %d rows; this kernel is for steps with few rows", who, M);
    return 0;
}

}  // namespace

// Can the fused kernels take rows of K values? (shared memory for at least 8 normalised rows)
extern "C" int bl_norm_gemm_supported(int K) {
    return K > 0 && K % 8 == 0 && smem_bytes(1, K, true) <= SMEM_LIMIT;
}

// out = epilogue(rmsnorm(x[row_idx]) . W^T): epilogue BL_EPI_NONE / BL_EPI_BIAS (float32 out [M, N]) or
// BL_EPI_SWIGLU (bfloat16 out [M, N], W with 2N rows). x: float32 rows of K values; W bfloat16.
extern "C" int bl_norm_gemm(const float* x, const int* row_idx, const void* norm_w, int norm_w_dtype, float eps,
                            const void* w, const void* bias, int bias_dtype, void* out, int M, int N, int K,
                            int epilogue, void* stream) {
    if (M <= 0) return 0;
    if (N <= 0) BL_FAIL("bl_norm_gemm: bad N=%d", N);
    if (check_common("bl_norm_gemm", x, w, M, K, norm_w_dtype)) return 1;
    FusedParams p = {};
    p.x = x; p.row_idx = row_idx; p.norm_w = norm_w; p.norm_w_dtype = norm_w_dtype; p.eps = eps;
    p.w = (const __nv_bfloat16*)w; p.out = out; p.M = M; p.N = N; p.K = K;
    const int tiles = (N + 15) / 16;
    if (epilogue == BL_EPI_SWIGLU) return dispatch<MODE_SWIGLU>(p, tiles, (cudaStream_t)stream);
    if (epilogue == BL_EPI_BIAS) {
        if (bias == nullptr || (bias_dtype != BL_F32 && bias_dtype != BL_BF16)) BL_FAIL("bl_norm_gemm: bias epilogue needs a float32 or bfloat16 bias");
        p.bias = bias; p.bias_dtype = bias_dtype;
    } else if (epilogue != BL_EPI_NONE) {
        BL_FAIL("bl_norm_gemm: epilogue %d is not built here", epilogue);
    }
    return dispatch<MODE_PLAIN>(p, tiles, (cudaStream_t)stream);
}

// q, k, v = rmsnorm(x) . Wqkv^T (+ bias); q and k rotated by position; k, v written to the pages of each token's
// request (k_cache / v_cache may be null: q only). Every dimension of a head rotates (n_rot = head size).
extern "C" int bl_norm_qkv_rope(const float* x, const void* norm_w, int norm_w_dtype, float eps, const void* w_qkv,
                                const void* bias, int bias_dtype, const int* positions, const int* tok_req,
                                const int* block_table, int max_pages, const float* inv_freq, float mscale,
                                void* q_out, void* k_cache, void* v_cache, int M, int K, int H, int KV, int dh,
                                int page_size, int pair_layout, void* stream) {
    if (M <= 0) return 0;
    if (pair_layout != BL_PAIRS_HALVES && pair_layout != BL_PAIRS_INTERLEAVED)
        BL_FAIL("bl_norm_qkv_rope: unknown pair layout %d (0: (j, j + head/2), 1: (2j, 2j + 1))", pair_layout);
    if (check_common("bl_norm_qkv_rope", x, w_qkv, M, K, norm_w_dtype)) return 1;
    if (H <= 0 || KV <= 0 || dh <= 0 || dh % 16 != 0) BL_FAIL("bl_norm_qkv_rope: head size %d must be a multiple of 16", dh);
    if (page_size <= 0 || max_pages <= 0) BL_FAIL("bl_norm_qkv_rope: bad page size or table width");
    if ((k_cache == nullptr) != (v_cache == nullptr)) BL_FAIL("bl_norm_qkv_rope: key and value cache must both be given or both be null");
    if (bias != nullptr && bias_dtype != BL_F32 && bias_dtype != BL_BF16) BL_FAIL("bl_norm_qkv_rope: unknown bias dtype %d", bias_dtype);
    FusedParams p = {};
    p.x = x; p.norm_w = norm_w; p.norm_w_dtype = norm_w_dtype; p.eps = eps; p.w = (const __nv_bfloat16*)w_qkv;
    p.bias = bias; p.bias_dtype = bias_dtype; p.out = q_out; p.M = M; p.N = (H + 2 * KV) * dh; p.K = K;
    p.positions = positions; p.tok_req = tok_req; p.block_table = block_table; p.max_pages = max_pages;
    p.inv_freq = inv_freq; p.mscale = mscale; p.k_cache = (__nv_bfloat16*)k_cache; p.v_cache = (__nv_bfloat16*)v_cache;
    p.H = H; p.KV = KV; p.dh = dh; p.page_size = page_size; p.pair_layout = pair_layout;
    const int heads = k_cache ? H + 2 * KV : H;
    return dispatch<MODE_QKV>(p, heads * (dh / 16), (cudaStream_t)stream);
}
