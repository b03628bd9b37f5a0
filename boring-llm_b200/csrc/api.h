// C interface of the kernel library. Every function returns 0 on success; otherwise
// bl_last_error() describes what was refused or what failed. Pointers are device pointers
// unless a comment says otherwise; `stream` is a cudaStream_t.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* bl_last_error(void);
int bl_device_check(void);   // 0 when the current device can run this library (compute capability 10.x)

// out[t, :] = table[ids[t], :] as 32-bit floats (the residual stream).
int bl_embed(const void* table, int table_dtype, const int* ids, float* out,
             int T, int d, int vocab, void* stream);

// y[r, :] = x[row_idx ? row_idx[r] : r, :] / sqrt(mean(x^2) + eps) * w, statistics in 32-bit.
int bl_rmsnorm(const float* x, const int* row_idx, const void* w, int w_dtype, void* y, int y_dtype,
               int rows, int d, float eps, void* stream);

// Plain matrix product on CUDA cores, 32-bit accumulation in ascending k for every output element:
// out[M, N] = epilogue(x[M, K] . W[N, K]^T). For BL_EPI_SWIGLU W has 2N rows (gate, then up).
int bl_gemm_plain(const void* x, int x_dtype, const void* w, int w_dtype, const void* bias, int bias_dtype,
                  void* out, int out_dtype, int M, int N, int K, int epilogue, void* stream);

// Splits rows of joined [q | k | v] projections, rotates q and k by position (inside each head, pair j is
// (j, j + n_rot/2) for pair_layout 0 and (2j, 2j + 1) for pair_layout 1; angle = float(position) * inv_freq[j],
// cos and sin times mscale) and writes k and v into the pages of the token's request. k_cache/v_cache may be
// null: then only q is produced.
int bl_rope_kv_write(const float* qkv, const int* positions, const int* tok_req, const int* block_table,
                     int max_pages, const float* inv_freq, int rot_half, float mscale,
                     void* q_out, void* k_cache, void* v_cache, int dtype,
                     int T, int H, int KV, int dh, int page_size, int pair_layout, void* stream);

// Plain paged causal attention: one warp per (token, head), keys visited in ascending position.
// Token t of request r = tok_req[t] stands at position ctx_len[r] - (cu_q[r+1] - cu_q[r]) + (t - cu_q[r])
// and sees keys j <= position with j + window > position (window 0: all of them).
int bl_attention_plain(const void* q, const void* k_cache, const void* v_cache, int dtype,
                       const int* tok_req, const int* cu_q, const int* ctx_len, const int* block_table,
                       int max_pages, void* out, int T, int H, int KV, int dh, int page_size,
                       int window, float scale, void* stream);

// x[r, :] += v[:] for every row of the 32-bit residual stream (the bias of a projection that adds into it).
int bl_add_row_vector(float* x, const void* v, int v_dtype, int rows, int d, void* stream);

// out_ids[r] = index of the first maximum of logits[r, :].
int bl_argmax(const float* logits, int* out_ids, int rows, int vocab, void* stream);

// One token per row: greedy where temperature[r] <= 0, else temperature sampling with the optional
// top_k (0: off), top_p (>= 1: off) and min_p (0: off) cuts over candidates in descending logit order;
// uniform[r] in [0, 1) is the row's random number (unused by greedy rows).
int bl_sample(const float* logits, int rows, int vocab, const float* temperature, const int* top_k,
              const float* top_p, const float* min_p, const float* uniform, int* out_ids, void* stream);

// logits[r, t] is divided by penalty[r] when positive, multiplied otherwise, for each token t in
// tokens[offsets[r] .. offsets[r+1]) (the host lists each distinct token once).
int bl_repeat_penalty(float* logits, int rows, int vocab, const int* tokens, const int* offsets,
                      const float* penalty, void* stream);

// Matrix product for few rows (decode): bfloat16 x[M, K] and W[N, K] read once from global memory straight
// into tensor-core registers. K must be a multiple of 8, x and W 16-byte aligned. Same epilogues as bl_gemm_plain.
int bl_gemm_skinny(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int out_dtype,
                   int M, int N, int K, int epilogue, void* stream);
int bl_gemm_skinny_norm_parts(int N);
int bl_gemm_skinny_residual_norm(const void* x, const void* w, void* out, int M, int N, int K, const void* norm_w,
                                 int norm_w_dtype, void* hw, float* ss, void* stream);
int bl_gemm_skinny_scaled(const void* hw, const void* w, const void* bias, int bias_dtype, void* out, int out_dtype,
                          int M, int N, int K, int epilogue, const float* ss, int parts, float eps, void* stream);

// Tensor-core paged attention (bfloat16, pages of 16 tokens, head sizes 16/32/48/64/96/128).
int bl_attention_mma_supported(int dh, int page_size);
// Prefill shape: tiles[n_tiles][2] = (request, first token of a 64-token tile within the request's new tokens).
int bl_attention_prefill(const void* q, const void* k_cache, const void* v_cache, const int* cu_q,
                         const int* ctx_len, const int* block_table, int max_pages, const int* tiles, int n_tiles,
                         void* out, int H, int KV, int dh, int page_size, int window, float scale, void* stream);
// The same on tcgen05 tensor cores with TMA-fed tiles and scores and outputs in tensor memory (attention_tcgen05.cu):
// head size 64 and pages of 16 only. tiles[n_tiles][2] = (request, first token of a 128-row tile). T: rows of
// q and out; n_pages: pages in k_cache / v_cache. *status = 0 unless a block gave up on a bounded wait since the last
// call (synchronises the device).
int bl_attention_prefill_tc_supported(int dh, int page_size);
int bl_attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache, const int* cu_q,
                            const int* ctx_len, const int* block_table, int max_pages, const int* tiles, int n_tiles,
                            void* out, int T, int n_pages, int H, int KV, int dh, int page_size, int window, float scale,
                            void* stream);
int bl_attention_prefill_tc_status(int* status);
// Blocks of bl_attention_decode that the current device holds at once for this head size (0: not built).
int bl_attention_decode_resident_blocks(int dh);
// Decode shape: reqs[n] = requests with one new token; their keys are cut into n_splits slices. With scratch == null
// (up to 16 slices) the slices of a request are the blocks of one thread-block cluster and merge their partial results
// through distributed shared memory; with scratch (up to 256 slices) the last block to finish merges them from
// scratch: bl_attention_decode_scratch_floats(n, H, dh, n_splits) floats (none for one slice).
long long bl_attention_decode_scratch_floats(int n, int H, int dh, int n_splits);
// counters: n * KV * ceil((H / KV) / 16) ints that are zero at the call and zero again when it is done.
int bl_attention_decode(const void* q, const void* k_cache, const void* v_cache, const int* cu_q,
                        const int* ctx_len, const int* block_table, int max_pages, const int* reqs, int n,
                        int n_splits, float* scratch, int* counters, void* out, int H, int KV, int dh, int page_size,
                        int window, float scale, void* stream);

// The decode shape with TMA-fed rings (attention_decode.cu): head sizes 64 and 128, pages of 16, 1..16 slices that are
// the blocks of one cluster; the MMAs' columns are the query heads of a key/value head (8 or 16 a block). n_pages:
// pages in k_cache / v_cache. early != 0: the launch may start under its predecessor's tail (programmatic dependent
// launch). *status = 0 unless a warp gave up on a bounded wait since the last call (synchronises
// the device). resident_blocks: blocks the device holds at once for this head size and heads per key/value head.
int bl_attention_decode_tma_supported(int dh, int page_size);
int bl_attention_decode_tma_resident_blocks(int dh, int heads_per_kv);
// Clusters of `cluster` blocks that the device runs at once for this shape (0: cannot be launched).
int bl_attention_decode_tma_max_clusters(int dh, int heads_per_kv, int cluster);
int bl_attention_decode_tma(const void* q, const void* k_cache, const void* v_cache, int n_pages, const int* cu_q,
                            const int* ctx_len, const int* block_table, int max_pages, const int* reqs, int n,
                            int n_splits, void* out, int H, int KV, int dh, int page_size, int window, float scale,
                            int early, void* stream);
int bl_attention_decode_tma_status(int* status);

// cs[t, j] = cos(positions[t] * inv_freq[j]) * mscale, sn likewise, j < rot_half: the rotation of a step's tokens,
// worked out once for all layers.
int bl_rope_table(const int* positions, const float* inv_freq, int rot_half, float mscale, float* cs, float* sn, int T,
                  void* stream);
// The joined q/k/v product on pairs of SMs (gemm_tcgen05_pair.cu) with bias, rotation (pairs j, j + dh / 2; cs, sn:
// [M, dh / 2] from bl_rope_table) and the writes of q and of k and v into the pages of each token's request folded
// into its epilogue. Head size 64 or 128, pages of 16; null caches: nothing is cached; bias may be null.
int bl_gemm_tc_pair_qkv_rope_supported(int H, int KV, int dh, int page_size, int K);
// ss != null: x holds rows whose RMS norm is pending (bl_gemm_tc_pair_residual_norm); row m of the product is scaled
// by 1 / sqrt(sum(ss[m, :parts]) * inv_dim + eps) before the bias.
int bl_gemm_tc_pair_qkv_rope(const void* x, const void* w, const void* bias, int bias_dtype, int M, int K,
                             const int* tok_req, const int* positions, const int* block_table, int max_pages,
                             const float* cs, const float* sn, void* q_out, void* k_cache, void* v_cache,
                             int H, int KV, int dh, int page_size, const float* ss, int parts, float inv_dim, float eps,
                             void* stream);
// An RMS norm between two products without a pass of its own: the product that adds into the 32-bit residual stream
// also writes hw = bfloat16(out * norm_w) and per-row sums of squares by tile (ss[M, bl_gemm_tc_pair_norm_parts(M, N)]);
// the products that read the normed rows take hw and scale their accumulator rows by the row's 1 / sqrt(mean + eps).
int bl_gemm_tc_pair_norm_parts(int M, int N);
int bl_gemm_tc_pair_residual_norm(const void* x, const void* w, void* out, int M, int N, int K, const void* norm_w,
                                  int norm_w_dtype, void* hw, float* ss, void* stream);
int bl_gemm_tc_pair_swiglu_scaled(const void* hw, const void* w, void* out, int M, int N, int K, const float* ss,
                                  int parts, float inv_dim, float eps, void* stream);

// Matrix product for many rows (prefill) on tcgen05 tensor cores with TMA-fed shared-memory tiles and the
// accumulator in tensor memory. bfloat16 x[M, K] and W[N, K]; K a multiple of 8, x and W 16-byte aligned.
int bl_gemm_tc(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int out_dtype,
               int M, int N, int K, int epilogue, void* stream);
// *status = 0 unless a block of bl_gemm_tc gave up on a bounded wait since the last call (synchronises the device).
int bl_gemm_tc_status(int* status);

// Few rows (up to 64) times very many columns (an output head), no epilogue: W is the M side of tcgen05.mma and
// streams through a deep TMA ring once, x stays in shared memory, blocks are persistent (gemm_tcgen05_cols.cu).
int bl_gemm_tc_cols_supported(int M, int N, int K);
int bl_gemm_tc_cols(const void* x, const void* w, void* out, int out_dtype, int M, int N, int K, void* stream);
int bl_gemm_tc_cols_status(int* status);

// Fused kernels for steps with few rows (decode_fused.cu): the RMS norm in front of a product, and the split,
// rotation and cache write behind the q/k/v product, folded into the product.
int bl_norm_gemm_supported(int K);
int bl_norm_gemm(const float* x, const int* row_idx, const void* norm_w, int norm_w_dtype, float eps,
                 const void* w, const void* bias, int bias_dtype, void* out, int M, int N, int K,
                 int epilogue, void* stream);
int bl_norm_qkv_rope(const float* x, const void* norm_w, int norm_w_dtype, float eps, const void* w_qkv,
                     const void* bias, int bias_dtype, const int* positions, const int* tok_req,
                     const int* block_table, int max_pages, const float* inv_freq, float mscale,
                     void* q_out, void* k_cache, void* v_cache, int M, int K, int H, int KV, int dh,
                     int page_size, int pair_layout, void* stream);
// Programmatic dependent launch for the small kernels of a step (on by default): 0 launches them the ordinary way.
void bl_set_dependent_launch(int on);

// Writes the GPU's nanosecond timer to buf[slot] once everything before it on the stream has finished.
int bl_stamp(unsigned long long* buf, int slot, void* stream);

// The same product on pairs of SMs (tcgen05 cta_group::2, clusters of two blocks, 256 x 256 tiles): twice the
// arithmetic per byte loaded into shared memory. Same contract as bl_gemm_tc.
int bl_gemm_tc_pair(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int out_dtype,
                    int M, int N, int K, int epilogue, void* stream);
int bl_gemm_tc_pair_status(int* status);

// The same product for shapes with few output tiles: a cluster of up to eight blocks shares a tile of 128 rows and
// cuts K among its blocks; the partial tiles are added up in block order through distributed shared memory
// (gemm_tcgen05_splitk.cu). Same contract as bl_gemm_tc. bl_gemm_tc_splitk_split: how many blocks would share a tile
// (1: K is not cut, the kernel has nothing over bl_gemm_tc).
int bl_gemm_tc_splitk_split(int M, int N, int K, int epilogue);
int bl_gemm_tc_splitk(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int out_dtype,
                      int M, int N, int K, int epilogue, void* stream);
int bl_gemm_tc_splitk_status(int* status);

#ifdef __cplusplus
}
#endif
