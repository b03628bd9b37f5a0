// Plain paged causal grouped-query attention: one warp per (token, head), keys in ascending position,
// softmax in its online form with 32-bit statistics. Formulas: gqa_attention_ext (src/math.br:304-359):
// kv head = head / (H / KV), score = dot * scale (scale after the dot), causal with the reference's
// `causal_offset` (src/math_gpu.br:3044-3047), window: key j is seen while j + window > position
// (src/math.br:327-328); online form as FlashAttnKernel (src/math_gpu.br:3224-3287).
// A (token, head) is computed the same way whatever else is in the batch: its chunks of 32 keys start
// at its first visible key. This is the 32-bit path's attention and the twin of the fast kernels.
#include "common.cuh"
#include "api.h"

namespace {

constexpr int MAX_DH = 256;
constexpr int WARPS = 4;

template <typename TT>
__global__ void __launch_bounds__(WARPS * 32)
attention_plain_kernel(const TT* __restrict__ q, const TT* __restrict__ kc, const TT* __restrict__ vc,
                       const int* __restrict__ tok_req, const int* __restrict__ cu_q,
                       const int* __restrict__ ctx_len, const int* __restrict__ block_table, int max_pages,
                       TT* __restrict__ out, int T, int H, int KV, int dh, int page_size, int window,
                       float scale) {
    __shared__ float qs[WARPS][MAX_DH];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.x * WARPS + warp;
    if (item >= T * H) return;                 // whole warps leave together; no block-wide barrier below
    const int t = item / H, h = item % H;
    const int r = tok_req[t];
    const int q_len = cu_q[r + 1] - cu_q[r];
    const int pos = ctx_len[r] - q_len + (t - cu_q[r]);
    const int kvh = h / (H / KV);
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const TT* qrow = q + ((size_t)t * H + h) * dh;
    for (int d = lane; d < dh; d += 32) qs[warp][d] = bl_load(qrow + d);
    __syncwarp();
    const int* bt = block_table + (size_t)r * max_pages;
    const size_t head_off = (size_t)kvh * page_size * dh;
    const size_t page_stride = (size_t)KV * page_size * dh;
    float m = -INFINITY, l = 0.f;
    float acc[MAX_DH / 32];
#pragma unroll
    for (int i = 0; i < MAX_DH / 32; ++i) acc[i] = 0.f;
    for (int base = lo; base <= pos; base += 32) {
        const int j = base + lane;
        const bool valid = j <= pos;
        float s = -INFINITY;
        if (valid) {
            const int page = bt[j / page_size];
            const TT* krow = kc + (size_t)page * page_stride + head_off + (size_t)(j % page_size) * dh;
            float dot = 0.f;
            for (int d = 0; d < dh; ++d) dot = fmaf(qs[warp][d], bl_load(krow + d), dot);
            s = dot * scale;
        }
        const float m_new = fmaxf(m, bl_warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.f;
        const float alpha = expf(m - m_new);           // first chunk: exp(-inf) = 0
        l = l * alpha + bl_warp_sum(p);
#pragma unroll
        for (int i = 0; i < MAX_DH / 32; ++i) acc[i] *= alpha;
        const int n = min(32, pos - base + 1);
        for (int jj = 0; jj < n; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int key = base + jj;
            const int page = bt[key / page_size];
            const TT* vrow = vc + (size_t)page * page_stride + head_off + (size_t)(key % page_size) * dh;
#pragma unroll
            for (int i = 0; i < MAX_DH / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < dh) acc[i] = fmaf(pj, bl_load(vrow + d), acc[i]);
            }
        }
        m = m_new;
    }
    TT* orow = out + ((size_t)t * H + h) * dh;
    const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int i = 0; i < MAX_DH / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < dh) bl_store(orow + d, acc[i] * inv);
    }
}

}  // namespace

extern "C" int bl_attention_plain(const void* q, const void* k_cache, const void* v_cache, int dtype,
                                  const int* tok_req, const int* cu_q, const int* ctx_len,
                                  const int* block_table, int max_pages, void* out, int T, int H, int KV,
                                  int dh, int page_size, int window, float scale, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || KV <= 0 || H % KV != 0) BL_FAIL("bl_attention_plain: %d heads cannot share %d key/value heads", H, KV);
    if (dh <= 0 || dh > MAX_DH) BL_FAIL("bl_attention_plain: head size %d is outside 1..%d", dh, MAX_DH);
    if (page_size <= 0 || max_pages <= 0 || window < 0) BL_FAIL("bl_attention_plain: bad page size, table width or window");
    cudaStream_t s = (cudaStream_t)stream;
    const int blocks = (T * H + WARPS - 1) / WARPS;
    if (dtype == BL_F32)
        attention_plain_kernel<float><<<blocks, WARPS * 32, 0, s>>>((const float*)q, (const float*)k_cache,
            (const float*)v_cache, tok_req, cu_q, ctx_len, block_table, max_pages, (float*)out, T, H, KV, dh,
            page_size, window, scale);
    else if (dtype == BL_BF16)
        attention_plain_kernel<__nv_bfloat16><<<blocks, WARPS * 32, 0, s>>>((const __nv_bfloat16*)q,
            (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, tok_req, cu_q, ctx_len, block_table,
            max_pages, (__nv_bfloat16*)out, T, H, KV, dh, page_size, window, scale);
    else
        BL_FAIL("bl_attention_plain: unknown dtype %d", dtype);
    BL_CHECK_LAUNCH("bl_attention_plain");
    return 0;
}
