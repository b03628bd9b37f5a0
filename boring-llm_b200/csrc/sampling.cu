// Sampling on the device: greedy, and temperature with top-k, top-p and min-p, in the reference's
// semantics (src/sampling.br:490-607, 742-760): candidates ranked in DESCENDING logit order (ties by
// ascending token id), an untempered softmax over the candidates for the top-p and min-p prefix cuts,
// temperature applied last as w = exp((l - l_first) / T), and the first candidate whose running sum
// reaches u * sum(w) is chosen. The uniform number u comes from the host's xorshift64 generator
// (src/sampling.br:42-54), one draw per sampled token; greedy rows consume none (:496-497).
//
// Nothing is sorted. Every step above is "a prefix of the descending order up to a running weight",
// so one primitive serves them all: a radix select over the order-preserving 32-bit image of the
// logits, four passes of 256 buckets, where the buckets hold summed WEIGHTS instead of counts. Weights
// are summed as 64-bit fixed point (2^-40 of the largest weight), so sums do not depend on the order
// in which threads add them and a row's token is the same on every run.
#include "common.cuh"
#include "api.h"

namespace {

constexpr int THREADS = 1024;
constexpr float FIXED_ONE = 1099511627776.0f;   // 2^40

struct Cut { unsigned key; int idx; };           // members: key > cut.key, or key == cut.key and idx <= cut.idx

__device__ __forceinline__ unsigned sort_key(float f) {
    if (f != f) return 0u;                       // NaN ranks last
    const unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct RowCtx {
    const float* row; int vocab; float lmax; float temperature; float min_p; Cut cut;
};

__device__ __forceinline__ bool is_member(const RowCtx& c, float l, unsigned key, int idx) {
    if (!(key > c.cut.key || (key == c.cut.key && idx <= c.cut.idx))) return false;
    if (c.min_p > 0.f && !(expf(l - c.lmax) >= c.min_p)) return false;     // probs[i] >= probs[0] * min_p
    return true;
}

// mode 0: count; 1: exp(l - lmax) (untempered softmax numerator); 2: exp((l - lmax) / T)
__device__ __forceinline__ unsigned long long weight_of(const RowCtx& c, float l, int mode) {
    if (mode == 0) return 1ull;
    const float w = mode == 1 ? expf(l - c.lmax) : expf((l - c.lmax) / c.temperature);
    return __float2ull_rn(w * FIXED_ONE);
}

__device__ unsigned long long block_sum_weights(const RowCtx& c, int mode, unsigned long long* sh_acc) {
    if (threadIdx.x == 0) *sh_acc = 0ull;
    __syncthreads();
    unsigned long long local = 0ull;
    for (int i = threadIdx.x; i < c.vocab; i += THREADS) {
        const float l = c.row[i];
        if (is_member(c, l, sort_key(l), i)) local += weight_of(c, l, mode);
    }
    if (local) atomicAdd(sh_acc, local);
    __syncthreads();
    const unsigned long long r = *sh_acc;
    __syncthreads();
    return r;
}

// The first member, in descending (logit, then ascending id) order, at which the running weight
// reaches `target`. Returns it as a Cut (its key and id).
__device__ Cut select_prefix(const RowCtx& c, int mode, unsigned long long target,
                             unsigned long long* hist, unsigned* sh_u, unsigned long long* sh_t, int* sh_cnt) {
    unsigned prefix = 0;
    for (int pass = 3; pass >= 0; --pass) {
        const int shift = pass * 8;
        for (int b = threadIdx.x; b < 256; b += THREADS) hist[b] = 0ull;
        __syncthreads();
        for (int i = threadIdx.x; i < c.vocab; i += THREADS) {
            const float l = c.row[i];
            const unsigned key = sort_key(l);
            if (pass < 3 && (key >> (shift + 8)) != prefix) continue;
            if (!is_member(c, l, key, i)) continue;
            const unsigned long long w = weight_of(c, l, mode);
            if (w) atomicAdd(&hist[(key >> shift) & 255u], w);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long cum = 0ull;
            int chosen = -1, last = -1;
            for (int b = 255; b >= 0; --b) {
                if (hist[b] == 0ull) continue;
                last = b;
                if (cum + hist[b] >= target) { chosen = b; break; }
                cum += hist[b];
            }
            if (chosen < 0) {                     // target beyond the total (rounding): take the last member
                chosen = last < 0 ? 0 : last;
                cum = last < 0 ? 0ull : cum - hist[last];
            }
            *sh_t = target > cum ? target - cum : 0ull;
            *sh_u = (prefix << 8) | (unsigned)chosen;
        }
        __syncthreads();
        prefix = *sh_u;
        target = *sh_t;
        __syncthreads();
    }
    // `prefix` is the key of the chosen logit value; members with that exact value share one weight and
    // are taken in ascending id: the tie_rank-th of them is the answer (nearly always the only one).
    const int chunk = (c.vocab + THREADS - 1) / THREADS;
    const int begin = threadIdx.x * chunk, end = min(c.vocab, begin + chunk);
    int cnt = 0;
    unsigned long long w_tie = 0ull;
    for (int i = begin; i < end; ++i) {
        const float l = c.row[i];
        const unsigned key = sort_key(l);
        if (key == prefix && is_member(c, l, key, i)) { ++cnt; w_tie = weight_of(c, l, mode); }
    }
    sh_cnt[threadIdx.x] = cnt;
    if (cnt) *sh_t = w_tie;                       // every tie has the same weight; any writer will do
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned long long w = *sh_t;
        long long rank = (w == 0ull || target == 0ull) ? 1 : (long long)((target + w - 1ull) / w);
        long long total = 0;
        for (int t = 0; t < THREADS; ++t) total += sh_cnt[t];
        if (rank > total) rank = total;
        if (rank < 1) rank = 1;
        int owner = 0;
        long long before = 0;
        for (int t = 0; t < THREADS; ++t) {
            if (before + sh_cnt[t] >= rank) { owner = t; break; }
            before += sh_cnt[t];
        }
        sh_u[0] = (unsigned)owner;
        sh_u[1] = (unsigned)(rank - before);
    }
    __syncthreads();
    const int owner = (int)sh_u[0];
    const int local_rank = (int)sh_u[1];
    __syncthreads();
    if (threadIdx.x == owner) {
        int seen = 0, found = c.vocab - 1;
        for (int i = begin; i < end; ++i) {
            const float l = c.row[i];
            const unsigned key = sort_key(l);
            if (key == prefix && is_member(c, l, key, i) && ++seen == local_rank) { found = i; break; }
        }
        sh_u[2] = (unsigned)found;
    }
    __syncthreads();
    Cut r;
    r.key = prefix;
    r.idx = (int)sh_u[2];
    __syncthreads();
    return r;
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* logits /* written by the kernel before */, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
              const float* __restrict__ uniform, int* __restrict__ out_ids) {
    __shared__ unsigned long long hist[256];
    __shared__ unsigned long long sh_t, sh_acc;
    __shared__ unsigned sh_u[4];
    __shared__ int sh_cnt[THREADS];
    __shared__ float red_v[THREADS / 32];
    __shared__ int red_i[THREADS / 32];
    bl_pdl_trigger();
    bl_pdl_wait();
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * vocab;
    // the first maximum (lowest id among equals): the greedy token and the softmax's reference point
    float best = -INFINITY;
    int bidx = 0x7fffffff;
    if ((vocab & 3) == 0 && ((uintptr_t)row & 15) == 0) {          // 16-byte loads, four in flight per thread
        const float4* row4 = reinterpret_cast<const float4*>(row);
        const int n4 = vocab >> 2;
        for (int i0 = threadIdx.x; i0 < n4; i0 += 4 * THREADS) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * THREADS;
                v[u] = i < n4 ? row4[i] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {                           // ascending ids within the thread: the first maximum stays
                const int i = (i0 + u * THREADS) * 4;
                if (i >= vocab) break;
                if (bidx == 0x7fffffff || v[u].x > best) { best = v[u].x; bidx = i; }
                if (v[u].y > best) { best = v[u].y; bidx = i + 1; }
                if (v[u].z > best) { best = v[u].z; bidx = i + 2; }
                if (v[u].w > best) { best = v[u].w; bidx = i + 3; }
            }
        }
    } else {
        for (int i = threadIdx.x; i < vocab; i += THREADS) {
            const float v = row[i];
            if (bidx == 0x7fffffff || v > best) { best = v; bidx = i; }
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float v2 = __shfl_xor_sync(0xffffffffu, best, o);
        const int i2 = __shfl_xor_sync(0xffffffffu, bidx, o);
        if (i2 != 0x7fffffff && (bidx == 0x7fffffff || v2 > best || (v2 == best && i2 < bidx))) { best = v2; bidx = i2; }
    }
    if ((threadIdx.x & 31) == 0) { red_v[threadIdx.x >> 5] = best; red_i[threadIdx.x >> 5] = bidx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < THREADS / 32; ++w) {
            const float v2 = red_v[w]; const int i2 = red_i[w];
            if (i2 != 0x7fffffff && (red_i[0] == 0x7fffffff || v2 > red_v[0] || (v2 == red_v[0] && i2 < red_i[0]))) {
                red_v[0] = v2; red_i[0] = i2;
            }
        }
    }
    __syncthreads();
    const float lmax = red_v[0];
    const int greedy = red_i[0];
    const float T = temperature[r];
    if (!(T > 0.f)) {                              // temperature <= 0: greedy (src/sampling.br:496-497)
        if (threadIdx.x == 0) out_ids[r] = greedy;
        return;
    }
    RowCtx c;
    c.row = row; c.vocab = vocab; c.lmax = lmax; c.temperature = T; c.min_p = 0.f;
    c.cut.key = 0u; c.cut.idx = 0x7fffffff;
    const int k = top_k[r];
    if (k > 0 && k < vocab)                        // rank_candidates keeps the k largest (:280-371)
        c.cut = select_prefix(c, 0, (unsigned long long)k, hist, sh_u, &sh_t, sh_cnt);
    const float p = top_p[r];
    if (p < 1.0f) {                                // smallest prefix whose probability reaches top_p (:531-541)
        const unsigned long long Z = block_sum_weights(c, 1, &sh_acc);
        double tgt = ceil((double)p * (double)Z);
        if (tgt < 1.0) tgt = 1.0;
        c.cut = select_prefix(c, 1, (unsigned long long)tgt, hist, sh_u, &sh_t, sh_cnt);
    }
    const float mp = min_p[r];
    if (mp > 0.f) c.min_p = mp;                    // keep while probs[i] >= probs[0] * min_p (:546-551)
    const unsigned long long W = block_sum_weights(c, 2, &sh_acc);
    const double tgt = ceil((double)uniform[r] * (double)W);
    const Cut chosen = select_prefix(c, 2, (unsigned long long)tgt, hist, sh_u, &sh_t, sh_cnt);
    if (threadIdx.x == 0) out_ids[r] = chosen.idx;
}

// Repeat penalty over a window of earlier tokens, once per distinct token (src/sampling.br:56-88):
// a positive logit is divided by the penalty, any other multiplied by it.
__global__ void repeat_penalty_kernel(float* __restrict__ logits, int vocab, const int* __restrict__ tokens,
                                      const int* __restrict__ offsets, const float* __restrict__ penalty) {
    const int r = blockIdx.x;
    const float pen = penalty[r];
    if (pen == 1.0f) return;
    float* row = logits + (size_t)r * vocab;
    for (int i = offsets[r] + threadIdx.x; i < offsets[r + 1]; i += blockDim.x) {
        const int tok = tokens[i];
        if (tok < 0 || tok >= vocab) continue;
        const float v = row[tok];
        row[tok] = v > 0.f ? v / pen : v * pen;
    }
}

}  // namespace

extern "C" int bl_sample(const float* logits, int rows, int vocab, const float* temperature, const int* top_k,
                         const float* top_p, const float* min_p, const float* uniform, int* out_ids,
                         void* stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) BL_FAIL("bl_sample: bad vocabulary %d", vocab);
    BL_CUDA(bl_launch_dependent(sample_kernel, dim3(rows), dim3(THREADS), 0, (cudaStream_t)stream, logits, vocab,
                                temperature, top_k, top_p, min_p, uniform, out_ids));
    BL_CHECK_LAUNCH("bl_sample");
    return 0;
}

extern "C" int bl_repeat_penalty(float* logits, int rows, int vocab, const int* tokens, const int* offsets,
                                 const float* penalty, void* stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) BL_FAIL("bl_repeat_penalty: bad vocabulary %d", vocab);
    repeat_penalty_kernel<<<rows, 128, 0, (cudaStream_t)stream>>>(logits, vocab, tokens, offsets, penalty);
    BL_CHECK_LAUNCH("bl_repeat_penalty");
    return 0;
}
