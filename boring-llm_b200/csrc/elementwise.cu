// Embedding gather, RMSNorm, rotary positions with the paged cache write, arg-max.
// Formulas follow the reference's CPU math: rms_norm (src/math.br:18-36), rope_apply_at
// (src/math.br:128-157); the reference's GPU counterparts are rms_norm_gpu (src/math_gpu.br:2163-2191),
// split_and_rope_qkv_gpu (:2428-2488) and prepare_qkv_decode_slice (:4008-4076).
#include "common.cuh"
#include "api.h"
#include <string.h>

static thread_local char g_error[1024] = "";

void bl_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

extern "C" const char* bl_last_error(void) { return g_error; }

static bool g_pdl = true;
bool bl_pdl_enabled() { return g_pdl; }
// 0 switches programmatic dependent launch off for the kernels that use it (for measurements); default on.
extern "C" void bl_set_dependent_launch(int on) { g_pdl = on != 0; }

extern "C" int bl_device_check(void) {
    int dev = 0;
    BL_CUDA(cudaGetDevice(&dev));
    cudaDeviceProp prop;
    BL_CUDA(cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10)
        BL_FAIL("this library is built for sm_100a (compute capability 10.x); device %d is %d.%d",
                dev, prop.major, prop.minor);
    return 0;
}

// ---------------------------------------------------------------------------------------------
template <typename TT>
__global__ void embed_kernel(const TT* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ out, int d) {
    bl_pdl_trigger();
    bl_pdl_wait();
    const int t = blockIdx.x;
    const size_t row = (size_t)ids[t] * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) out[(size_t)t * d + i] = bl_load(table + row + i);
}

extern "C" int bl_embed(const void* table, int table_dtype, const int* ids, float* out,
                        int T, int d, int vocab, void* stream) {
    if (T <= 0) return 0;
    if (d <= 0 || vocab <= 0) BL_FAIL("bl_embed: bad sizes d=%d vocab=%d", d, vocab);
    cudaStream_t s = (cudaStream_t)stream;
    if (table_dtype == BL_F32)
        BL_CUDA(bl_launch_dependent(embed_kernel<float>, dim3(T), dim3(128), 0, s, (const float*)table, ids, out, d));
    else if (table_dtype == BL_BF16)
        BL_CUDA(bl_launch_dependent(embed_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, s, (const __nv_bfloat16*)table, ids, out, d));
    else
        BL_FAIL("bl_embed: unknown table dtype %d", table_dtype);
    BL_CHECK_LAUNCH("bl_embed");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// One block of 128 threads per row. The sum of squares is reduced in a fixed order that depends
// only on d, so a row's result does not depend on how many rows the call has.
template <typename TY>
__global__ void rmsnorm_kernel(const float* x /* written by the kernel before: no read-only cache */,
                               const int* __restrict__ row_idx,
                               const void* __restrict__ w, int w_dtype, TY* __restrict__ y,
                               int d, float eps) {
    bl_pdl_trigger();
    bl_pdl_wait();
    const int r = blockIdx.x;
    const size_t src = (size_t)(row_idx ? row_idx[r] : r) * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) { float v = x[src + i]; ss += v * v; }
    ss = bl_warp_sum(ss);
    __shared__ float part[4];
    __shared__ float inv_s;
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = (part[0] + part[1]) + (part[2] + part[3]);
        inv_s = 1.0f / sqrtf(tot / (float)d + eps);
    }
    __syncthreads();
    const float inv = inv_s;
    for (int i = threadIdx.x; i < d; i += blockDim.x)
        bl_store(y + (size_t)r * d + i, x[src + i] * inv * bl_load_any(w, w_dtype, i));
}

// The same with one warp per row and 16-byte loads, for widths that are a multiple of 4: a row of up to 1,024
// values stays in registers between the sum of squares and the scaling; nothing is shared between warps, so
// there is no barrier. A lane adds its squares in index order and the warp's sum is a fixed butterfly: the
// result of a row depends only on d.
constexpr int NORM_ROWS_PER_BLOCK = 2;      // small blocks: a few hundred rows still spread over every SM
template <typename TY>
__global__ void __launch_bounds__(32 * NORM_ROWS_PER_BLOCK)
rmsnorm_rows_kernel(const float* x /* written by the kernel before: no read-only cache */,
                    const int* __restrict__ row_idx, const void* __restrict__ w, int w_dtype, TY* __restrict__ y,
                    int rows, int d, float eps) {
    bl_pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * NORM_ROWS_PER_BLOCK + (threadIdx.x >> 5);
    constexpr int NB = 8;
    // the norm's weights do not depend on the kernel before: a row of up to NB * 128 values has them in registers
    // before the wait
    const bool single = d <= NB * 128;
    float4 wv[NB];
    if (single) {
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            const int k = j * 128 + lane * 4;
            wv[j] = k < d ? make_float4(bl_load_any(w, w_dtype, k), bl_load_any(w, w_dtype, k + 1), bl_load_any(w, w_dtype, k + 2),
                                        bl_load_any(w, w_dtype, k + 3)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    bl_pdl_wait();
    if (r >= rows) return;
    const float* src = x + (size_t)(row_idx ? row_idx[r] : r) * d;
    float4 v[NB];
    auto load_batch = [&](int k0) {
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            const int k = k0 + j * 128 + lane * 4;
            v[j] = k < d ? *reinterpret_cast<const float4*>(src + k) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    float ss = 0.f;
    for (int k0 = 0; k0 < d; k0 += NB * 128) {
        load_batch(k0);
#pragma unroll
        for (int j = 0; j < NB; ++j) { ss += v[j].x * v[j].x; ss += v[j].y * v[j].y; ss += v[j].z * v[j].z; ss += v[j].w * v[j].w; }
    }
    ss = bl_warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    TY* dst = y + (size_t)r * d;
    for (int k0 = 0; k0 < d; k0 += NB * 128) {
        if (!single) load_batch(k0);
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            const int k = k0 + j * 128 + lane * 4;
            if (k >= d) continue;
            const float4 ww = single ? wv[j] : make_float4(bl_load_any(w, w_dtype, k), bl_load_any(w, w_dtype, k + 1),
                                                              bl_load_any(w, w_dtype, k + 2), bl_load_any(w, w_dtype, k + 3));
            const float o0 = v[j].x * inv * ww.x, o1 = v[j].y * inv * ww.y;
            const float o2 = v[j].z * inv * ww.z, o3 = v[j].w * inv * ww.w;
            if (sizeof(TY) == 4) {
                *reinterpret_cast<float4*>(dst + k) = make_float4(o0, o1, o2, o3);
            } else {
                __nv_bfloat162 lo = __floats2bfloat162_rn(o0, o1), hi = __floats2bfloat162_rn(o2, o3);
                uint2 pk;
                pk.x = *reinterpret_cast<unsigned*>(&lo); pk.y = *reinterpret_cast<unsigned*>(&hi);
                *reinterpret_cast<uint2*>(dst + k) = pk;
            }
        }
    }
}

extern "C" int bl_rmsnorm(const float* x, const int* row_idx, const void* w, int w_dtype, void* y,
                          int y_dtype, int rows, int d, float eps, void* stream) {
    if (rows <= 0) return 0;
    if (d <= 0) BL_FAIL("bl_rmsnorm: bad width %d", d);
    if (w_dtype != BL_F32 && w_dtype != BL_BF16) BL_FAIL("bl_rmsnorm: unknown weight dtype %d", w_dtype);
    if (y_dtype != BL_F32 && y_dtype != BL_BF16) BL_FAIL("bl_rmsnorm: unknown output dtype %d", y_dtype);
    cudaStream_t s = (cudaStream_t)stream;
    const bool wide = d % 4 == 0 && (((uintptr_t)x | (uintptr_t)y) & 15) == 0;      // 16-byte loads and stores of whole rows
    if (wide && y_dtype == BL_F32)
        BL_CUDA(bl_launch_dependent(rmsnorm_rows_kernel<float>, dim3((rows + NORM_ROWS_PER_BLOCK - 1) / NORM_ROWS_PER_BLOCK), dim3(32 * NORM_ROWS_PER_BLOCK), 0, s, x, row_idx, w, w_dtype, (float*)y, rows, d, eps));
    else if (wide)
        BL_CUDA(bl_launch_dependent(rmsnorm_rows_kernel<__nv_bfloat16>, dim3((rows + NORM_ROWS_PER_BLOCK - 1) / NORM_ROWS_PER_BLOCK), dim3(32 * NORM_ROWS_PER_BLOCK), 0, s, x, row_idx, w, w_dtype, (__nv_bfloat16*)y, rows, d, eps));
    else if (y_dtype == BL_F32)
        BL_CUDA(bl_launch_dependent(rmsnorm_kernel<float>, dim3(rows), dim3(128), 0, s, x, row_idx, w, w_dtype, (float*)y, d, eps));
    else
        BL_CUDA(bl_launch_dependent(rmsnorm_kernel<__nv_bfloat16>, dim3(rows), dim3(128), 0, s, x, row_idx, w, w_dtype, (__nv_bfloat16*)y, d, eps));
    BL_CHECK_LAUNCH("bl_rmsnorm");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// One block per token. Work items: (head, pair) for q and k heads, then the v elements.
// four values as the output type: one 16-byte (float) or 8-byte (bfloat16) store
__device__ __forceinline__ void bl_store4(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void bl_store4(__nv_bfloat16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 pk;
    pk.x = *reinterpret_cast<unsigned*>(&lo); pk.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = pk;
}

// VEC: every head is rotated in full (rot_half = head size / 2, a multiple of 4) and the buffers are 16-byte
// aligned: a work item is four neighbouring pairs of a head, read and written with one vector access each.
template <typename TT, bool VEC>
__global__ void rope_kv_write_kernel(const float* qkv /* written by the kernel before */, const int* __restrict__ positions,
                                     const int* __restrict__ tok_req, const int* __restrict__ block_table,
                                     int max_pages, const float* __restrict__ inv_freq, int rot_half,
                                     float mscale, TT* __restrict__ q_out, TT* __restrict__ k_cache,
                                     TT* __restrict__ v_cache, int H, int KV, int dh, int page_size, int pair_layout) {
    bl_pdl_trigger();
    bl_pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = dh / 2;
    const int width = (H + 2 * KV) * dh;
    const float* row = qkv + (size_t)t * width;
    size_t page_base = 0;
    bool write = k_cache != nullptr;
    if (write) {
        const int page = block_table[(size_t)tok_req[t] * max_pages + pos / page_size];
        if (page < 0) write = false;       // the host never schedules this; keep memory safe anyway
        page_base = ((size_t)(page < 0 ? 0 : page) * KV) * page_size * dh + (size_t)(pos % page_size) * dh;
    }
    // the rotation of pair j is the same for every head of the token: worked out once, into shared memory
    extern __shared__ __align__(16) float cs_sn[];                     // [rot_half] cos, then [rot_half] sin
    for (int j = threadIdx.x; j < rot_half; j += blockDim.x) {
        const float angle = (float)pos * inv_freq[j];
        cs_sn[j] = cosf(angle) * mscale;
        cs_sn[rot_half + j] = sinf(angle) * mscale;
    }
    __syncthreads();
    if (VEC) {
        const int groups = half / 4;                     // groups of four pairs per head
        for (int it = threadIdx.x; it < (H + KV) * groups; it += blockDim.x) {
            const int head = it / groups, j = (it % groups) * 4;
            const float* src = row + (size_t)head * dh;
            const float4 x0 = *reinterpret_cast<const float4*>(src + j), x1 = *reinterpret_cast<const float4*>(src + j + half);
            const float4 c = *reinterpret_cast<const float4*>(cs_sn + j), sn = *reinterpret_cast<const float4*>(cs_sn + half + j);
            TT* dst = head < H ? q_out + (size_t)t * H * dh + (size_t)head * dh
                               : k_cache + page_base + (size_t)(head - H) * page_size * dh;
            if (head < H || write) {
                bl_store4(dst + j, x0.x * c.x - x1.x * sn.x, x0.y * c.y - x1.y * sn.y, x0.z * c.z - x1.z * sn.z, x0.w * c.w - x1.w * sn.w);
                bl_store4(dst + j + half, x0.x * sn.x + x1.x * c.x, x0.y * sn.y + x1.y * c.y, x0.z * sn.z + x1.z * c.z, x0.w * sn.w + x1.w * c.w);
            }
        }
        if (write) {
            const float* vsrc = row + (size_t)(H + KV) * dh;
            for (int it = threadIdx.x; it < KV * dh / 4; it += blockDim.x) {
                const int head = (it * 4) / dh, i = (it * 4) % dh;
                const float4 v = *reinterpret_cast<const float4*>(vsrc + it * 4);
                bl_store4(v_cache + page_base + (size_t)head * page_size * dh + i, v.x, v.y, v.z, v.w);
            }
        }
        return;
    }
    const int n_rot_items = (H + KV) * half;
    for (int it = threadIdx.x; it < n_rot_items; it += blockDim.x) {
        const int head = it / half, j = it % half;
        const float* src = row + (size_t)head * dh;      // q heads first, then k heads: same row layout
        int i0, i1;
        float c = 1.f, s = 0.f;
        if (j < rot_half) {
            if (pair_layout == BL_PAIRS_INTERLEAVED) { i0 = 2 * j; i1 = 2 * j + 1; }
            else { i0 = j; i1 = j + rot_half; }
            c = cs_sn[j];
            s = cs_sn[rot_half + j];
        } else {                                         // dimensions past the rotated ones pass through
            i0 = 2 * j; i1 = 2 * j + 1;
        }
        const float x0 = src[i0], x1 = src[i1];
        const float y0 = x0 * c - x1 * s, y1 = x0 * s + x1 * c;
        if (head < H) {
            TT* dst = q_out + (size_t)t * H * dh + (size_t)head * dh;
            bl_store(dst + i0, y0); bl_store(dst + i1, y1);
        } else if (write) {
            TT* dst = k_cache + page_base + (size_t)(head - H) * page_size * dh;
            bl_store(dst + i0, y0); bl_store(dst + i1, y1);
        }
    }
    if (write) {
        const float* vsrc = row + (size_t)(H + KV) * dh;
        for (int it = threadIdx.x; it < KV * dh; it += blockDim.x) {
            const int head = it / dh, i = it % dh;
            bl_store(v_cache + page_base + (size_t)head * page_size * dh + i, vsrc[it]);
        }
    }
}

extern "C" int bl_rope_kv_write(const float* qkv, const int* positions, const int* tok_req,
                                const int* block_table, int max_pages, const float* inv_freq,
                                int rot_half, float mscale, void* q_out, void* k_cache, void* v_cache,
                                int dtype, int T, int H, int KV, int dh, int page_size, int pair_layout, void* stream) {
    if (T <= 0) return 0;
    if (pair_layout != BL_PAIRS_HALVES && pair_layout != BL_PAIRS_INTERLEAVED)
        BL_FAIL("bl_rope_kv_write: unknown pair layout %d (0: (j, j + n_rot/2), 1: (2j, 2j + 1))", pair_layout);
    if (H <= 0 || KV <= 0 || dh <= 0 || dh % 2 != 0 || page_size <= 0 || max_pages <= 0)
        BL_FAIL("bl_rope_kv_write: bad sizes H=%d KV=%d head=%d page=%d max_pages=%d", H, KV, dh, page_size, max_pages);
    if (rot_half < 0 || rot_half > dh / 2) BL_FAIL("bl_rope_kv_write: %d rotated pairs do not fit a head of %d", rot_half, dh);
    if ((k_cache == nullptr) != (v_cache == nullptr)) BL_FAIL("bl_rope_kv_write: key and value cache must both be given or both be null");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t elem = dtype == BL_F32 ? 4 : 2;
    const bool vec = pair_layout == BL_PAIRS_HALVES && rot_half * 2 == dh && rot_half % 4 == 0 && ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)inv_freq & 3) == 0 &&
                     ((uintptr_t)q_out % (4 * elem)) == 0 && ((uintptr_t)k_cache % (4 * elem)) == 0 && ((uintptr_t)v_cache % (4 * elem)) == 0;
    const size_t smem = (size_t)rot_half * 8;
#define BL_ROPE(TT, VEC) BL_CUDA(bl_launch_dependent(rope_kv_write_kernel<TT, VEC>, dim3(T), dim3(128), smem, s, qkv, positions, tok_req, \
        block_table, max_pages, inv_freq, rot_half, mscale, (TT*)q_out, (TT*)k_cache, (TT*)v_cache, H, KV, dh, page_size, pair_layout))
    if (dtype == BL_F32) { if (vec) BL_ROPE(float, true); else BL_ROPE(float, false); }
    else if (dtype == BL_BF16) { if (vec) BL_ROPE(__nv_bfloat16, true); else BL_ROPE(__nv_bfloat16, false); }
    else BL_FAIL("bl_rope_kv_write: unknown dtype %d", dtype);
#undef BL_ROPE
    BL_CHECK_LAUNCH("bl_rope_kv_write");
    return 0;
}

// The rotation of every token of a step, once for all layers: cs[t, j] = cos(pos_t * inv_freq_j) * mscale and
// sn[t, j] = sin(...) * mscale, with the same 32-bit formulas as the kernels that rotate on the fly.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq, int rot_half,
                                  float mscale, float* __restrict__ cs, float* __restrict__ sn, int T) {
    bl_pdl_trigger();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * rot_half) return;
    const int t = i / rot_half, j = i % rot_half;
    const float angle = (float)positions[t] * inv_freq[j];
    cs[i] = cosf(angle) * mscale;
    sn[i] = sinf(angle) * mscale;
}

extern "C" int bl_rope_table(const int* positions, const float* inv_freq, int rot_half, float mscale, float* cs,
                             float* sn, int T, void* stream) {
    if (T <= 0 || rot_half <= 0) return 0;
    const int n = T * rot_half;
    BL_CUDA(bl_launch_dependent(rope_table_kernel, dim3((n + 255) / 256), dim3(256), 0, (cudaStream_t)stream, positions,
                                inv_freq, rot_half, mscale, cs, sn, T));
    BL_CHECK_LAUNCH("bl_rope_table");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// First maximum wins, as sample_greedy (src/sampling.br:239-249: strict '>').
__global__ void argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab) {
    const float* row = logits + (size_t)blockIdx.x * vocab;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (idx == 0x7fffffff || v > best) { best = v; idx = i; }
    }
    __shared__ float sv[256];
    __shared__ int si[256];
    sv[threadIdx.x] = best; si[threadIdx.x] = idx;
    __syncthreads();
    for (int o = blockDim.x / 2; o > 0; o >>= 1) {
        if (threadIdx.x < o) {
            const float v2 = sv[threadIdx.x + o]; const int i2 = si[threadIdx.x + o];
            if (i2 != 0x7fffffff && (si[threadIdx.x] == 0x7fffffff || v2 > sv[threadIdx.x] ||
                                     (v2 == sv[threadIdx.x] && i2 < si[threadIdx.x]))) {
                sv[threadIdx.x] = v2; si[threadIdx.x] = i2;
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) out[blockIdx.x] = si[0];
}

extern "C" int bl_argmax(const float* logits, int* out_ids, int rows, int vocab, void* stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) BL_FAIL("bl_argmax: bad vocabulary %d", vocab);
    argmax_kernel<<<rows, 256, 0, (cudaStream_t)stream>>>(logits, out_ids, vocab);
    BL_CHECK_LAUNCH("bl_argmax");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// A time stamp between two kernels of a stream (or of a captured graph): one thread writes the GPU's
// nanosecond timer. Launched the ordinary way, so it starts when everything before it has finished; the
// differences between successive stamps are the durations of the kernels in between, in place, with the
// memory state that the real step leaves. Role: the reference's marginal-cost decode profiler
// (tools/profile_decode_marginal.py, src/model.br:1697-1701), which also measures stages inside the running step.
__global__ void stamp_kernel(unsigned long long* buf, int slot) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    buf[slot] = t;
}

extern "C" int bl_stamp(unsigned long long* buf, int slot, void* stream) {
    stamp_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(buf, slot);
    BL_CHECK_LAUNCH("bl_stamp");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// x[r, :] += v for every row: the bias of a projection whose product is added into the 32-bit residual stream
// (the product kernels' residual epilogue adds the product; the bias is added once, by this kernel, before it:
// the reference adds a linear layer's bias after its product, src/math.br:84-93, and the sum of three terms does
// not depend on that order beyond rounding).
__global__ void add_row_vector_kernel(float* x, const void* __restrict__ v, int v_dtype, int rows, int d) {
    bl_pdl_trigger();
    bl_pdl_wait();
    const size_t n = (size_t)rows * d;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        x[i] += bl_load_any(v, v_dtype, i % d);
}

extern "C" int bl_add_row_vector(float* x, const void* v, int v_dtype, int rows, int d, void* stream) {
    if (rows <= 0) return 0;
    if (d <= 0) BL_FAIL("bl_add_row_vector: bad width %d", d);
    if (v_dtype != BL_F32 && v_dtype != BL_BF16) BL_FAIL("bl_add_row_vector: unknown dtype %d", v_dtype);
    const size_t n = (size_t)rows * d;
    const int blocks = (int)((n + 255) / 256 < 1184 ? (n + 255) / 256 : 1184);
    BL_CUDA(bl_launch_dependent(add_row_vector_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, x, v, v_dtype, rows, d));
    BL_CHECK_LAUNCH("bl_add_row_vector");
    return 0;
}
