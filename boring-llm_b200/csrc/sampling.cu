// Sampling on the device: greedy, and temperature with top-k, top-p and min-p, in the reference's
// semantics (src/sampling.br:490-607, 742-760): candidates ranked in DESCENDING logit order (ties by
// ascending token id), an untempered softmax over the candidates for the top-p and min-p prefix cuts,
// temperature applied last as w = exp((l - l_first) / T), and the first candidate whose running sum
// reaches u * sum(w) is chosen. The uniform number u comes from the host's xorshift64 generator
// (src/sampling.br:42-54), one draw per sampled token; greedy rows consume none (:496-497).
//
// Every step above is "a prefix of the descending order up to a running weight" (a count for top-k, the
// untempered softmax numerator for top-p, the tempered one for the draw). The row is never sorted as a whole, and
// its elements are not added into shared-memory histograms on the common path (152,000 atomic additions by one SM
// cost tens of microseconds a pass):
//   1. the eight blocks of a cluster share the row. Each scans its share for the maximum (the greedy token, and
//      the softmax's reference point) and hands its candidate, and the largest logit of each of its warps, to all
//      the others through distributed shared memory; greedy rows are done here;
//   2. the c-th largest of the cluster's 256 warp maxima is a bound with at least c logits above it (c = k for
//      top-k, else 256, which leaves about a thousand); every block works out the same bound. In one more pass over
//      its share a block sends the logits that reach the bound to the first block (an atomic counter and a store in
//      that block's shared memory) and sums the share's weights in registers (64-bit fixed point, no atomics). The
//      first block then holds the head of the row's descending order and the row's totals, and does the rest alone;
//   3. a list of up to 1,024 candidates (a top-k's, a peaked row's) is sorted once (logit descending, id ascending);
//      top-k, top-p, min-p and the draw are then running sums over a prefix of it, and a cut is a shorter prefix;
//   4. a step over a longer list: the members' weights are added into 2,048 buckets that are
//      linear in (maximum - logit), a scan finds the bucket in which the running weight reaches the target, that
//      bucket's few candidates are sorted (logit descending, id ascending) and a scan of their weights finds the
//      candidate, which becomes the members' new end. The totals of a step that looks at all of the row come from 2.
// Only when a running sum does not reach its target inside the list (a flat row, a top-k above 256) does a step
// walk the row itself, the same way: one pass to fill the buckets, one to copy the bucket's candidates. A bucket
// too full for shared memory (thousands of equal logits) is resolved by a radix select over the floats' bits, four
// passes of 256 buckets.
// Weights are summed as 64-bit fixed point (2^-40 of the largest weight), so sums do not depend on the order in
// which threads add them and a row's token is the same on every run. A weight below 2^-41 of the largest counts
// as zero: candidates that far down cannot be drawn.
#include "common.cuh"
#include "api.h"

namespace {

constexpr int THREADS = 1024;
constexpr int NB = 2048;                         // buckets linear in (maximum - logit); the last takes what lies further, and NaN
constexpr int CAP = 4096;                        // candidates that shared memory holds
constexpr int SORT_MAX = 1024;                   // lists up to this length are sorted once (a bitonic sort of 1,024: 55 stages)
constexpr int SCAN_BLOCKS = 8;                   // blocks of a cluster that share the scan for the maximum
constexpr float FIXED_ONE = 1099511627776.0f;    // 2^40
constexpr float ZERO_BELOW = 28.5f;              // exp(-28.5) * 2^40 < 1/2: weights this far below the largest are 0

struct Cut { unsigned key; int idx; };           // members: key > cut.key, or key == cut.key and idx <= cut.idx

__device__ __forceinline__ unsigned sort_key(float f) {
    if (f != f) return 0u;                       // NaN ranks last
    const unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float from_key(unsigned k) {
    return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k);      // key 0 gives back a NaN
}
// (logit descending, id ascending) as one ascending 64-bit number
__device__ __forceinline__ unsigned long long item_of(unsigned key, int idx) {
    return ((unsigned long long)(~key) << 32) | (unsigned)idx;
}

struct RowCtx {
    const float* row; int vocab; float lmax; float temperature; float min_p; Cut cut;
    float range, per_range;                      // the buckets cover (maximum - logit) in [0, range)
    int only_bucket;                             // radix fallback: only candidates of this bucket (-1: all)
};

__device__ __forceinline__ int bucket_of(const RowCtx& c, float l) {
    const float d = c.lmax - l;
    if (!(d < c.range)) return NB - 1;           // further down, or NaN
    return min(NB - 2, (int)(d * c.per_range));
}

__device__ __forceinline__ bool is_member(const RowCtx& c, float l, unsigned key, int idx) {
    if (!(key > c.cut.key || (key == c.cut.key && idx <= c.cut.idx))) return false;
    if (c.min_p > 0.f && !(expf(l - c.lmax) >= c.min_p)) return false;     // probs[i] >= probs[0] * min_p
    if (c.only_bucket >= 0 && bucket_of(c, l) != c.only_bucket) return false;
    return true;
}

// mode 0: count; 1: exp(l - lmax) (untempered softmax numerator); 2: exp((l - lmax) / T)
__device__ __forceinline__ unsigned long long weight_of(const RowCtx& c, float l, int mode) {
    if (mode == 0) return 1ull;
    const float w = mode == 1 ? expf(l - c.lmax) : expf((l - c.lmax) / c.temperature);
    return __float2ull_rn(w * FIXED_ONE);
}

struct Shared {
    unsigned long long hist_w[NB];
    unsigned hist_c[NB];
    unsigned long long items[CAP];              // the head of the row's descending order, unsorted
    unsigned long long sel[CAP];                // the candidates of one bucket, sorted
    unsigned long long scan[CAP];
    unsigned long long warp_tot[32];
    unsigned long long sh_t, sh_acc;
    unsigned long long hist256[256];
    int found;
    unsigned n_items;
    unsigned sh_u[4];
    float red_v[32]; int red_i[32];
    float cl_v[SCAN_BLOCKS]; int cl_i[SCAN_BLOCKS];          // every block's candidate for the maximum (in every block)
    unsigned long long cl_sum[SCAN_BLOCKS][3];               // first block: the blocks' sums of weights
    unsigned cl_wmax[SCAN_BLOCKS * (THREADS / 32)];          // the largest key of every warp of the cluster (in every block)
    unsigned bound;
    int sh_cnt[THREADS];
};

// distributed shared memory: the address of `local` in block `rank` of the cluster, and stores to it
__device__ __forceinline__ uint32_t in_block(const void* local, unsigned rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_remote(uint32_t addr, unsigned v) { asm volatile("st.shared::cluster.u32 [%0], %1;" :: "r"(addr), "r"(v) : "memory"); }
__device__ __forceinline__ void st_remote(uint32_t addr, unsigned long long v) { asm volatile("st.shared::cluster.u64 [%0], %1;" :: "r"(addr), "l"(v) : "memory"); }
__device__ __forceinline__ unsigned add_remote(uint32_t addr, unsigned v) {
    unsigned old;
    asm volatile("atom.shared::cluster.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(addr), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// the sum of v over the block (every thread gets it)
__device__ unsigned long long block_sum(unsigned long long v, Shared& S) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) S.warp_tot[threadIdx.x >> 5] = v;
    __syncthreads();
    unsigned long long t = 0ull;
#pragma unroll
    for (int w = 0; w < THREADS / 32; ++w) t += S.warp_tot[w];
    __syncthreads();
    return t;
}

// a[0, n) becomes its running sum (n <= 4 * THREADS); returns the total
__device__ unsigned long long block_scan(unsigned long long* a, int n, Shared& S) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int per = (n + THREADS - 1) / THREADS;
    const int j0 = threadIdx.x * per;
    unsigned long long v[4], run = 0ull;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        if (q < per && j0 + q < n) run += a[j0 + q];
        v[q] = run;
    }
    unsigned long long incl = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    if (lane == 31) S.warp_tot[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        unsigned long long w = S.warp_tot[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long up = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += up;
        }
        S.warp_tot[lane] = w;
    }
    __syncthreads();
    const unsigned long long before = (incl - run) + (warp > 0 ? S.warp_tot[warp - 1] : 0ull);
#pragma unroll
    for (int q = 0; q < 4; ++q)
        if (q < per && j0 + q < n) a[j0 + q] = v[q] + before;
    const unsigned long long total = S.warp_tot[31];
    __syncthreads();
    return total;
}

// The first j with a[j] >= target in a running sum a[0, n); n - 1 when the target lies beyond the total.
__device__ int first_at_least(const unsigned long long* a, int n, unsigned long long target, Shared& S) {
    if (threadIdx.x == 0) S.found = n - 1;
    __syncthreads();
    for (int j = threadIdx.x; j < n; j += THREADS)
        if (a[j] >= target && (j == 0 || a[j - 1] < target)) S.found = j;
    __syncthreads();
    const int r = S.found;
    __syncthreads();
    return r;
}

// Ascending bitonic sort of items[0, m), m a power of two. Up to 64 entries are one warp's work (no block barrier).
__device__ void block_sort(unsigned long long* items, int m) {
    if (m <= 64) {
        if (threadIdx.x < 32) {
            for (int k = 2; k <= m; k <<= 1) {
                for (int j = k >> 1; j > 0; j >>= 1) {
                    const int t = threadIdx.x;
                    if (t < (m >> 1)) {
                        const int i = ((t & ~(j - 1)) << 1) | (t & (j - 1));
                        const int p = i | j;
                        const bool up = (i & k) == 0;
                        const unsigned long long a = items[i], b = items[p];
                        if ((a > b) == up) { items[i] = b; items[p] = a; }
                    }
                    __syncwarp();
                }
            }
        }
        __syncthreads();
        return;
    }
    for (int k = 2; k <= m; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int t = threadIdx.x; t < (m >> 1); t += THREADS) {
                const int i = ((t & ~(j - 1)) << 1) | (t & (j - 1));      // the lower index of the pair
                const int p = i | j;
                const bool up = (i & k) == 0;
                const unsigned long long a = items[i], b = items[p];
                if ((a > b) == up) { items[i] = b; items[p] = a; }
            }
            __syncthreads();
        }
    }
}

// Radix select over the floats' bits (the fallback for a bucket that shared memory cannot hold): the first member,
// in descending (logit, then ascending id) order, at which the running weight reaches `target`.
__device__ Cut radix_select(const RowCtx& c, int mode, unsigned long long target, Shared& S) {
    unsigned long long* hist = S.hist256;
    unsigned* sh_u = S.sh_u;
    unsigned long long* sh_t = &S.sh_t;
    int* sh_cnt = S.sh_cnt;
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

// How a step names its target: a count, or a fraction of the step's own total weight.
struct Target { bool fraction; double value; bool at_least_one; };

__device__ unsigned long long target_of(const Target& t, unsigned long long total) {
    if (!t.fraction) return (unsigned long long)t.value;
    double tgt = ceil(t.value * (double)total);
    if (t.at_least_one && tgt < 1.0) tgt = 1.0;
    return (unsigned long long)tgt;
}

// A step over a SORTED list (logit descending, id ascending) whose first n entries are the members, or head them:
// the position at which the running weight reaches the target; -1 when the list only heads a longer order (of total
// weight `outside` >= 0) and the target lies beyond it.
__device__ int sorted_step(const RowCtx& c, int mode, const Target& t, int n, long long outside, Shared& S) {
    for (int j = threadIdx.x; j < n; j += THREADS)
        S.scan[j] = weight_of(c, from_key(~(unsigned)(S.items[j] >> 32)), mode);
    __syncthreads();
    const unsigned long long own = block_scan(S.scan, n, S);
    const unsigned long long target = target_of(t, outside < 0 ? own : (unsigned long long)outside);
    if (outside >= 0 && target > own) return -1;
    return first_at_least(S.scan, n, target, S);
}

// One step (top-k, top-p or the draw): the member at which the running weight of the members, in descending order,
// reaches the target; it is the members' new end (or the drawn token). LIST: the members are looked for in the list
// of n_src candidates in shared memory, else in the whole row. `outside` < 0: what is walked holds every member and a
// fractional target is a fraction of its own total. Else the list is the head of a longer order whose total weight is
// `outside`, and *reached is false when the target lies beyond the list.
template <bool LIST>
__device__ Cut step(const RowCtx& c0, int mode, const Target& t, int n_src, long long outside, bool* reached, Shared& S) {
    RowCtx c = c0;
    Cut none; none.key = 0u; none.idx = 0x7fffffff;
    *reached = true;
    const int n_walk = LIST ? n_src : c.vocab;
    auto element = [&](int i, float& l, unsigned& key, int& idx) {
        if (LIST) { const unsigned long long it = S.items[i]; key = ~(unsigned)(it >> 32); idx = (int)(unsigned)it; l = from_key(key); }
        else { l = c.row[i]; key = sort_key(l); idx = i; }
    };
    for (int b = threadIdx.x; b < NB; b += THREADS) { S.hist_w[b] = 0ull; S.hist_c[b] = 0u; }
    __syncthreads();
    for (int i = threadIdx.x; i < n_walk; i += THREADS) {
        float l; unsigned key; int idx;
        element(i, l, key, idx);
        if (!is_member(c, l, key, idx)) continue;
        const int b = bucket_of(c, l);
        const unsigned long long w = weight_of(c, l, mode);
        if (w) atomicAdd(&S.hist_w[b], w);
        atomicAdd(&S.hist_c[b], 1u);
    }
    __syncthreads();
    const unsigned long long own = block_scan(S.hist_w, NB, S);           // hist_w is now its running sum
    const unsigned long long target = target_of(t, outside < 0 ? own : (unsigned long long)outside);
    if (outside >= 0 && target > own) { *reached = false; return none; }
    int bstar = first_at_least(S.hist_w, NB, target, S);
    if (S.hist_w[bstar] < target) {
        // a target beyond the total (rounding) ends at the last member: the last bucket that holds any
        if (threadIdx.x == 0) S.found = 0;
        __syncthreads();
        for (int b = threadIdx.x; b < NB; b += THREADS) if (S.hist_c[b]) atomicMax(&S.found, b);
        __syncthreads();
        bstar = S.found;
        __syncthreads();
    }
    const unsigned long long before = bstar > 0 ? S.hist_w[bstar - 1] : 0ull;
    const unsigned in_bucket = S.hist_c[bstar];
    const unsigned long long local_target = target > before ? target - before : 0ull;
    __syncthreads();
    if (in_bucket > (unsigned)CAP) {
        // (only a walk of the row can meet this) too many for shared memory, say a row of equal logits: the radix
        // select, inside this bucket
        c.only_bucket = bstar;
        return radix_select(c, mode, local_target, S);
    }
    if (threadIdx.x == 0) S.n_items = 0u;
    __syncthreads();
    for (int i = threadIdx.x; i < n_walk; i += THREADS) {
        float l; unsigned key; int idx;
        element(i, l, key, idx);
        if (is_member(c, l, key, idx) && bucket_of(c, l) == bstar) S.sel[atomicAdd(&S.n_items, 1u)] = item_of(key, idx);
    }
    __syncthreads();
    const int n = (int)S.n_items;
    int m = 1;
    while (m < n) m <<= 1;
    for (int j = n + threadIdx.x; j < m; j += THREADS) S.sel[j] = ~0ull;
    __syncthreads();
    block_sort(S.sel, m);
    for (int j = threadIdx.x; j < n; j += THREADS)
        S.scan[j] = weight_of(c, from_key(~(unsigned)(S.sel[j] >> 32)), mode);
    __syncthreads();
    block_scan(S.scan, n, S);
    const int pos = first_at_least(S.scan, n, local_target, S);
    Cut r;
    r.key = ~(unsigned)(S.sel[pos] >> 32);
    r.idx = (int)(unsigned)S.sel[pos];
    __syncthreads();
    return r;
}

__device__ __forceinline__ void better(float& best, int& bidx, float v2, int i2) {
    if (i2 != 0x7fffffff && (bidx == 0x7fffffff || v2 > best || (v2 == best && i2 < bidx))) { best = v2; bidx = i2; }
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* logits /* written by the kernel before */, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
              const float* __restrict__ uniform, int* __restrict__ out_ids) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Shared& S = *reinterpret_cast<Shared*>(smem_raw);
    bl_pdl_trigger();
    bl_pdl_wait();
    const int r = blockIdx.y;
    const int part = blockIdx.x, parts = gridDim.x;     // the blocks of a cluster share the row
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* row = logits + (size_t)r * vocab;
    // ---- 1. the first maximum (lowest id among equals): the greedy token and the softmax's reference point --------
    float best = -INFINITY;
    int bidx = 0x7fffffff;
    const int share = (((vocab + parts - 1) / parts) + 3) & ~3;
    const int i_begin = min(vocab, part * share), i_end = min(vocab, i_begin + share);
    if ((vocab & 3) == 0 && ((uintptr_t)row & 15) == 0) {          // 16-byte loads
        const float4* row4 = reinterpret_cast<const float4*>(row);
        for (int i4 = (i_begin >> 2) + threadIdx.x; i4 < (i_end >> 2); i4 += THREADS) {
            const float4 v = row4[i4];
            const int i = i4 * 4;                                    // ascending ids within the thread: the first maximum stays
            if (bidx == 0x7fffffff || v.x > best) { best = v.x; bidx = i; }
            if (v.y > best) { best = v.y; bidx = i + 1; }
            if (v.z > best) { best = v.z; bidx = i + 2; }
            if (v.w > best) { best = v.w; bidx = i + 3; }
        }
    } else {
        for (int i = i_begin + threadIdx.x; i < i_end; i += THREADS) {
            const float v = row[i];
            if (bidx == 0x7fffffff || v > best) { best = v; bidx = i; }
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float v2 = __shfl_xor_sync(0xffffffffu, best, o);
        const int i2 = __shfl_xor_sync(0xffffffffu, bidx, o);
        better(best, bidx, v2, i2);
    }
    if (lane == 0) { S.red_v[warp] = best; S.red_i[warp] = bidx; }
    // (this warp's largest logit, for every block of the cluster: see step 3)
    if (lane < parts) st_remote(in_block(&S.cl_wmax[part * (THREADS / 32) + warp], lane), bidx == 0x7fffffff ? 0u : sort_key(best));
    if (threadIdx.x == 0) S.n_items = 0u;
    __syncthreads();
    if (threadIdx.x == 0)
        for (int w = 1; w < THREADS / 32; ++w) better(S.red_v[0], S.red_i[0], S.red_v[w], S.red_i[w]);
    __syncthreads();
    if (threadIdx.x < parts) {                    // this block's candidate goes to every block of the cluster
        st_remote(in_block(&S.cl_v[part], threadIdx.x), __float_as_uint(S.red_v[0]));
        st_remote(in_block(&S.cl_i[part], threadIdx.x), (unsigned)S.red_i[0]);
    }
    if (parts > 1) cluster_sync_all(); else __syncthreads();
    float lmax = S.cl_v[0];
    int greedy = S.cl_i[0];
    for (int b = 1; b < parts; ++b) better(lmax, greedy, S.cl_v[b], S.cl_i[b]);
    const float T = temperature[r];
    if (!(T > 0.f)) {                              // temperature <= 0: greedy (src/sampling.br:496-497)
        if (part == 0 && threadIdx.x == 0) out_ids[r] = greedy;
        return;                                    // (every block of the cluster takes this way or none)
    }
    RowCtx c;
    c.row = row; c.vocab = vocab; c.lmax = lmax; c.temperature = T; c.min_p = 0.f;
    c.cut.key = 0u; c.cut.idx = 0x7fffffff;
    c.range = ZERO_BELOW * fmaxf(1.0f, T);
    c.per_range = (float)(NB - 1) / c.range;
    c.only_bucket = -1;
    const int k = top_k[r];
    const float p = top_p[r], mp = min_p[r];
    const bool cut_k = k > 0 && k < vocab;
    // ---- 2. the head of the descending order, and this block's share of the row's totals, in one pass --------------------
    // The c-th largest of the cluster's warp maxima is a bound that at least c logits reach (every block works out the
    // same one); what reaches it goes to the first block's list.
    const int n_max = parts * (THREADS / 32);      // warp maxima of the cluster
    const bool k_in_list = cut_k && k <= n_max;    // the k largest are sure to be in the list
    {
        const int c_th = k_in_list ? k : n_max;
        if (threadIdx.x < n_max) {
            const unsigned long long mine = item_of(S.cl_wmax[threadIdx.x], threadIdx.x);
            int smaller = 0;
            for (int j = 0; j < n_max; ++j) smaller += item_of(S.cl_wmax[j], j) < mine ? 1 : 0;
            if (smaller == c_th - 1) S.bound = S.cl_wmax[threadIdx.x];
        }
        __syncthreads();
        const unsigned bound = S.bound;
        const uint32_t counter = in_block(&S.n_items, 0), list = in_block(&S.items[0], 0);
        unsigned long long z1 = 0ull, w2 = 0ull, w2m = 0ull;
        const bool sums = !cut_k;                  // after a top-k every later total is one over the members found then
        for (int i = i_begin + threadIdx.x; i < i_end; i += THREADS) {
            const float l = row[i];
            const unsigned key = sort_key(l);
            if (key >= bound) {
                const unsigned at = add_remote(counter, 1u);
                if (at < (unsigned)CAP) st_remote(list + at * 8u, item_of(key, i));
            }
            if (sums) {
                if (p < 1.0f) z1 += weight_of(c, l, 1);
                const unsigned long long w = weight_of(c, l, 2);
                w2 += w;
                if (mp > 0.f && expf(l - lmax) >= mp) w2m += w;
            }
        }
        if (sums) {
            z1 = block_sum(z1, S); w2 = block_sum(w2, S); w2m = block_sum(w2m, S);
        }
        if (threadIdx.x == 0) {
            st_remote(in_block(&S.cl_sum[part][0], 0), z1);
            st_remote(in_block(&S.cl_sum[part][1], 0), w2);
            st_remote(in_block(&S.cl_sum[part][2], 0), w2m);
        }
    }
    if (parts > 1) cluster_sync_all(); else __syncthreads();
    if (part != 0) return;                        // (nothing of this block's shared memory is read by another)
    unsigned long long Z1 = 0ull, W2 = 0ull, W2M = 0ull;
    for (int b = 0; b < parts; ++b) { Z1 += S.cl_sum[b][0]; W2 += S.cl_sum[b][1]; W2M += S.cl_sum[b][2]; }
    bool have_list = S.n_items <= (unsigned)CAP;   // else the bound let too many through (equal logits): the steps walk the row
    int n_list = have_list ? (int)S.n_items : 0;
    bool complete = false;                         // the list holds every member
    bool reached;
    __syncthreads();
    // A short list (a top-k's, a peaked row's) is sorted once; its steps are then running sums over a prefix of it, and a
    // cut is a shorter prefix. A long one stays unsorted: its steps bucket it (step<true>).
    const bool sorted = have_list && n_list <= SORT_MAX;
    if (sorted) {
        int m = 1;
        while (m < n_list) m <<= 1;
        for (int j = n_list + threadIdx.x; j < m; j += THREADS) S.items[j] = ~0ull;
        __syncthreads();
        block_sort(S.items, m);
    }
    auto end_of_list = [&]() { Cut e; e.key = ~(unsigned)(S.items[n_list - 1] >> 32); e.idx = (int)(unsigned)S.items[n_list - 1]; return e; };
    // ---- 4. the cuts and the draw ----------------------------------------------------------------------------------------
    if (cut_k) {                                   // rank_candidates keeps the k largest (:280-371)
        Target t; t.fraction = false; t.value = (double)k; t.at_least_one = false;
        if (have_list && n_list >= k) {
            if (sorted) { n_list = k; c.cut = end_of_list(); }
            else c.cut = step<true>(c, 0, t, n_list, -1, &reached, S);
            complete = true;
        } else { c.cut = step<false>(c, 0, t, 0, -1, &reached, S); have_list = false; }
    }
    if (p < 1.0f) {                                // smallest prefix whose probability reaches top_p (:531-541)
        Target t; t.fraction = true; t.value = (double)p; t.at_least_one = true;
        reached = false;
        Cut cut;
        if (have_list && sorted) {
            const int pos = sorted_step(c, 1, t, n_list, complete ? -1ll : (long long)Z1, S);
            if (pos >= 0) { n_list = pos + 1; cut = end_of_list(); reached = true; }
        } else if (have_list) {
            cut = step<true>(c, 1, t, n_list, complete ? -1ll : (long long)Z1, &reached, S);
        }
        if (reached) { c.cut = cut; complete = true; }
        else { c.cut = step<false>(c, 1, t, 0, -1, &reached, S); have_list = false; }
    }
    if (mp > 0.f) {                                // keep while probs[i] >= probs[0] * min_p (:546-551)
        c.min_p = mp;
        if (have_list && (sorted || !complete)) {
            // the first candidate of the list that fails the test: everything behind it fails too, in the list and beyond
            if (threadIdx.x == 0) S.found = n_list;
            __syncthreads();
            for (int j = threadIdx.x; j < n_list; j += THREADS)
                if (!(expf(from_key(~(unsigned)(S.items[j] >> 32)) - lmax) >= mp)) atomicMin(&S.found, j);
            __syncthreads();
            const int first_out = S.found;
            __syncthreads();
            if (first_out < n_list) {
                complete = true;
                if (sorted) { n_list = max(1, first_out); c.cut = end_of_list(); }
            }
        }
    }
    Target t; t.fraction = true; t.value = (double)uniform[r]; t.at_least_one = false;
    reached = false;
    Cut drawn;
    if (have_list && sorted) {
        const int pos = sorted_step(c, 2, t, n_list, complete ? -1ll : (long long)(mp > 0.f ? W2M : W2), S);
        if (pos >= 0) { drawn.key = 0u; drawn.idx = (int)(unsigned)S.items[pos]; reached = true; }
    } else if (have_list) {
        drawn = step<true>(c, 2, t, n_list, complete ? -1ll : (long long)(mp > 0.f ? W2M : W2), &reached, S);
    }
    if (!reached) drawn = step<false>(c, 2, t, 0, -1, &reached, S);
    if (threadIdx.x == 0) out_ids[r] = drawn.idx;
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
    static bool configured = false;
    if (!configured) {
        BL_CUDA(cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Shared)));
        configured = true;
    }
    if (rows > 65535) BL_FAIL("bl_sample: %d rows are more than a launch takes (65,535)", rows);
    // the blocks of a cluster share a row: eight of them while that fills the device in one round, fewer for many rows
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        BL_CUDA(cudaGetDevice(&dev));
        BL_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    }
    int parts = SCAN_BLOCKS;
    while (parts > 1 && rows * parts > sms) parts >>= 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(parts, rows); cfg.blockDim = dim3(THREADS); cfg.dynamicSmemBytes = sizeof(Shared);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = bl_pdl_enabled() ? 1 : 0;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = parts; attr[1].val.clusterDim.y = 1; attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 2;
    BL_CUDA(cudaLaunchKernelEx(&cfg, sample_kernel, logits, vocab, temperature, top_k, top_p, min_p, uniform, out_ids));
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
