// Matrix product for few rows (decode steps, short portions): out[M, N] = epilogue(x[M, K] . W[N, K]^T) with
// M up to a few dozen tokens. The step is bound by reading W once from HBM, so W goes straight from global
// memory into tensor-core registers with 16-byte loads and never touches shared memory: the product is
// computed transposed (rows of W are the MMA's M dimension, tokens its N dimension of 8), and because a dot
// product does not care about the order of its terms, each thread's 8 contiguous k values are dealt to the
// MMA's k slots as they lie; x is read with the same dealing. A block of 8 warps owns 16 output columns;
// the warps take 32-wide k chunks in turn and their partial sums are added in warp order, so a token's
// result does not depend on what else is in the batch.
// Role in the reference: the seq = 1 "warp-broadcast" matvec, one warp per output row
// (WarpBroadcastKernel, src/math_gpu.br:1038-1106); formula y = x . W^T (src/math.br:66-82).
#include "common.cuh"
#include "api.h"
#include <mma.h>

namespace {

constexpr int COLS = 16;          // output columns (rows of W) per block

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld16(const __nv_bfloat16* p, bool ok) {
    return ok ? __ldg(reinterpret_cast<const uint4*>(p)) : make_uint4(0u, 0u, 0u, 0u);
}

// An RMS norm shared between two products without a pass of its own (few rows: decode steps).
// The product that adds into the residual stream (residual epilogue) also writes, for the norm that reads the stream
// next, hw = bfloat16(stream * norm weight) and, per row and block of 16 columns, the sum of the squares of the new
// stream (ss_out[row][block]). A product that takes hw as its x (ss_in set) multiplies each row of its result by
// 1 / sqrt(sum(ss_in[row][:]) / dim + eps): the row's scale commutes with the product. Statistics and scale in 32-bit,
// the partial sums added in a fixed order.
struct SkinnyLink {
    const void* norm_w; int norm_w_dtype; __nv_bfloat16* hw; float* ss_out;      // producer
    const float* ss_in; int parts_in; float inv_dim, eps;                         // consumer
};

// SPLIT 2: two neighbouring blocks (a cluster) share 16 columns and cut K in two; the second hands its sums to the first
// through distributed shared memory, and the first adds them to its own (always in this order) before the epilogue.
// For a long K on few column blocks (a down projection at decode time: 56 blocks would leave most SMs idle, and each
// of the 56 would pull its 155 KB of W and all of x through one SM's port to L2).
// MT: groups of 8 tokens handled by one block (M tile = 8 * MT). NW: warps per block (8, or 16 for long K).
// DEEP: two batches of loads in flight per warp (few blocks, each short: hide the trips to memory); without it one
// batch and half the registers, so that twice as many blocks fit an SM (many blocks: HBM throughput is what counts).
template <int MT, int EPI, typename TO, int NW, bool DEEP, int SPLIT = 1>
__global__ void __launch_bounds__(NW * 32, DEEP ? (EPI == BL_EPI_SWIGLU && MT == 2 ? 2 : 1) : (NW == 8 ? 4 : 2))
gemm_skinny_kernel(const __nv_bfloat16* x /* written by the kernel before: no read-only cache */,
                   const __nv_bfloat16* __restrict__ w,
                   const void* __restrict__ bias, int bias_dtype, TO* out,
                   int M, int N, int K, int m_groups, const SkinnyLink lk) {
    constexpr bool GLU = EPI == BL_EPI_SWIGLU;
    constexpr int TOK = MT * 8;
    __shared__ float red[GLU ? 2 : 1][NW][COLS][TOK + 1];
    __shared__ float row_scale[TOK];
    __shared__ float peer_sums[SPLIT == 2 ? COLS * TOK : 1];      // the second block's sums, written by it into the first
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int tile = blockIdx.x / SPLIT, part = SPLIT == 2 ? (int)(blockIdx.x % SPLIT) : 0;   // (a cluster is SPLIT neighbouring blocks)
    const int n0 = (tile / m_groups) * COLS;
    const int m0 = (tile % m_groups) * TOK;
    // this block's share of K: whole 32-wide chunks
    const int k_cut = SPLIT == 2 ? ((K / 2 + 31) / 32) * 32 : K;
    const int k_begin = part == 0 ? 0 : k_cut, k_end = part == 0 ? min(K, k_cut) : K;
    float acc[MT][4], acu[GLU ? MT : 1][4];
#pragma unroll
    for (int j = 0; j < MT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) { acc[j][i] = 0.f; if (GLU) acu[j][i] = 0.f; }
    const int r_lo = n0 + g, r_hi = n0 + g + 8;
    const bool lo_ok = r_lo < N, hi_ok = r_hi < N;
    const __nv_bfloat16* w_lo = w + (size_t)r_lo * K;
    const __nv_bfloat16* w_hi = w + (size_t)r_hi * K;
    const __nv_bfloat16* u_lo = w + (size_t)(N + r_lo) * K;      // up rows follow the N gate rows
    const __nv_bfloat16* u_hi = w + (size_t)(N + r_hi) * K;
    // The loop bounds are the same for every lane of a warp (the MMA needs all 32 lanes); a lane whose 8 values
    // lie past K loads zeros. Loads go out in batches of UNROLL chunks, and the next batch is on its way while
    // the current one is multiplied: a trip to L2 costs far more than the arithmetic of a batch. The first
    // batch of W, and the whole slice of W as an L2 prefetch, are issued before the kernel waits for its
    // predecessor, since W does not depend on it.
    constexpr int UNROLL = (GLU || MT > 2 || (MT == 2 && NW == 16)) ? 2 : 4;   // (16 warps of 128 registers: two groups of tokens leave room for two loads a batch)
    constexpr int STEP = UNROLL * NW * 32;
    struct Batch { uint4 a_lo[UNROLL], a_hi[UNROLL], g_lo[GLU ? UNROLL : 1], g_hi[GLU ? UNROLL : 1], b[UNROLL][MT]; };
    auto fetch_w = [&](Batch& bt, int kc0) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = kc0 + u * NW * 32 + 8 * t;
            const bool k_ok = k < k_end;
            bt.a_lo[u] = ld16(w_lo + k, lo_ok && k_ok);
            bt.a_hi[u] = ld16(w_hi + k, hi_ok && k_ok);
            if (GLU) { bt.g_lo[u] = ld16(u_lo + k, lo_ok && k_ok); bt.g_hi[u] = ld16(u_hi + k, hi_ok && k_ok); }
        }
    };
    auto fetch_x = [&](Batch& bt, int kc0) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = kc0 + u * NW * 32 + 8 * t;
#pragma unroll
            for (int j = 0; j < MT; ++j) {
                const int tok = m0 + 8 * j + g;
                bt.b[u][j] = (tok < M && k < k_end) ? *reinterpret_cast<const uint4*>(x + (size_t)tok * K + k)
                                                    : make_uint4(0u, 0u, 0u, 0u);
            }
        }
    };
    auto multiply = [&](const Batch& bt) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
            for (int j = 0; j < MT; ++j) {
                mma_bf16(acc[j], bt.a_lo[u].x, bt.a_hi[u].x, bt.a_lo[u].y, bt.a_hi[u].y, bt.b[u][j].x, bt.b[u][j].y);
                mma_bf16(acc[j], bt.a_lo[u].z, bt.a_hi[u].z, bt.a_lo[u].w, bt.a_hi[u].w, bt.b[u][j].z, bt.b[u][j].w);
                if (GLU) {
                    mma_bf16(acu[j], bt.g_lo[u].x, bt.g_hi[u].x, bt.g_lo[u].y, bt.g_hi[u].y, bt.b[u][j].x, bt.b[u][j].y);
                    mma_bf16(acu[j], bt.g_lo[u].z, bt.g_hi[u].z, bt.g_lo[u].w, bt.g_hi[u].w, bt.b[u][j].z, bt.b[u][j].w);
                }
            }
        }
    };
    Batch b0;
    Batch b1;        // used only when DEEP
    bl_pdl_trigger();
    fetch_w(b0, k_begin + warp * 32);
    if (SPLIT == 2) {
        // this block's half of the 16 rows of W: the 128-byte lines of k_begin .. k_end of each row
        const int lines = ((k_end - k_begin) * 2 + 127) / 128;
        for (int i = threadIdx.x; i < COLS * lines; i += NW * 32) {
            const int r = n0 + i / lines;
            if (r < N) bl_prefetch_l2(reinterpret_cast<const char*>(w + (size_t)r * K + k_begin) + (size_t)(i % lines) * 128);
        }
    } else {
        bl_prefetch_rows_l2(w, n0, COLS, (size_t)K * 2, (size_t)(GLU ? 2 * N : N));
        if (GLU) bl_prefetch_rows_l2(w, (size_t)N + n0, COLS, (size_t)K * 2, (size_t)2 * N);
    }
    // this thread's output element and, for the bias epilogue, its bias
    const int e_c = threadIdx.x % COLS, e_tok = threadIdx.x / COLS;
    const int e_n = n0 + e_c, e_m = m0 + e_tok;
    const bool e_ok = threadIdx.x < COLS * TOK && e_n < N && e_m < M && part == 0;
    float e_add = 0.f;
    if (EPI == BL_EPI_BIAS && e_ok) e_add = bl_load_any(bias, bias_dtype, e_n);
    const bool begins_norm = EPI == BL_EPI_RESIDUAL && lk.hw != nullptr;
    float e_nw = 0.f;                                             // the next norm's weight of this thread's column
    if (begins_norm && e_ok) e_nw = bl_load_any(lk.norm_w, lk.norm_w_dtype, e_n);
    bl_pdl_wait();
    if (EPI == BL_EPI_RESIDUAL && e_ok) e_add = bl_load(out + (size_t)e_m * N + e_n);   // on its way during the product
    fetch_x(b0, k_begin + warp * 32);
    if (lk.ss_in != nullptr) {
        // the scale of each of this block's rows, while the product's operands are on their way: warp w adds up the
        // partial sums of rows w, w + NW, ... (a lane its share in ascending order, then the warp's fixed tree)
        for (int i = warp; i < TOK; i += NW) {
            const int m = m0 + i;
            float sum = 0.f;
            if (m < M)
                for (int q = lane; q < lk.parts_in; q += 32) sum += lk.ss_in[(size_t)m * lk.parts_in + q];
            sum = bl_warp_sum(sum);
            if (lane == 0) row_scale[i] = 1.0f / sqrtf(sum * lk.inv_dim + lk.eps);
        }
    }
    // two batches per trip of the loop, so that the buffers keep their names (and their registers)
    if (DEEP) {
        for (int kc0 = k_begin + warp * 32; kc0 < k_end; kc0 += 2 * STEP) {
            const bool more1 = kc0 + STEP < k_end;
            if (more1) { fetch_w(b1, kc0 + STEP); fetch_x(b1, kc0 + STEP); }
            multiply(b0);
            if (!more1) break;
            if (kc0 + 2 * STEP < k_end) { fetch_w(b0, kc0 + 2 * STEP); fetch_x(b0, kc0 + 2 * STEP); }
            multiply(b1);
        }
    } else {
        for (int kc0 = k_begin + warp * 32; kc0 < k_end; kc0 += STEP) {
            multiply(b0);
            if (kc0 + STEP < k_end) { fetch_w(b0, kc0 + STEP); fetch_x(b0, kc0 + STEP); }
        }
    }
    // c0, c1: (column g, tokens 2t, 2t+1); c2, c3: (column g + 8, tokens 2t, 2t+1)
#pragma unroll
    for (int j = 0; j < MT; ++j) {
        red[0][warp][g][8 * j + 2 * t] = acc[j][0];     red[0][warp][g][8 * j + 2 * t + 1] = acc[j][1];
        red[0][warp][g + 8][8 * j + 2 * t] = acc[j][2]; red[0][warp][g + 8][8 * j + 2 * t + 1] = acc[j][3];
        if (GLU) {
            red[1][warp][g][8 * j + 2 * t] = acu[j][0];     red[1][warp][g][8 * j + 2 * t + 1] = acu[j][1];
            red[1][warp][g + 8][8 * j + 2 * t] = acu[j][2]; red[1][warp][g + 8][8 * j + 2 * t + 1] = acu[j][3];
        }
    }
    __syncthreads();
    if (SPLIT == 2) {
        // the second block adds up its warps' sums and stores them into the first block's shared memory; both meet
        // at the cluster's barrier (release / acquire), after which the first reads them
        static_assert(SPLIT == 1 || !GLU, "the split kernel has one matrix per column");
        if (part == 1) {
            uint32_t remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(peer_sums)), "r"(0u));
            for (int i = threadIdx.x; i < COLS * TOK; i += NW * 32) {
                float v = 0.f;
#pragma unroll
                for (int wp = 0; wp < NW; ++wp) v += red[0][wp][i % COLS][i / COLS];
                asm volatile("st.shared::cluster.f32 [%0], %1;" :: "r"(remote + 4u * (uint32_t)i), "f"(v) : "memory");
            }
        }
        asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (part == 1) return;
    }
    // the first COLS * TOK threads each own one output element (their residual or bias is already in a register)
    // (every lane of a warp makes the same number of trips: COLS * TOK is a multiple of 32)
    for (int i = threadIdx.x; i < COLS * TOK; i += NW * 32) {
        const int c = i % COLS, tok = i / COLS;
        const int n = n0 + c, m = m0 + tok;
        const bool valid = n < N && m < M;
        float v = 0.f, u = 0.f;
        if (valid) {
#pragma unroll
            for (int wp = 0; wp < NW; ++wp) { v += red[0][wp][c][tok]; if (GLU) u += red[1][wp][c][tok]; }
            if (SPLIT == 2) v += peer_sums[i];
            if (lk.ss_in != nullptr) { const float r = row_scale[tok]; v *= r; if (GLU) u *= r; }
            TO* dst = out + (size_t)m * N + n;
            if (EPI == BL_EPI_BIAS || EPI == BL_EPI_RESIDUAL) v += (i == threadIdx.x) ? e_add : (EPI == BL_EPI_BIAS ? bl_load_any(bias, bias_dtype, n) : bl_load(dst));
            if (GLU) v = bl_silu(v) * u;
            bl_store(dst, v);
        }
        if (begins_norm) {                                        // (the same for the whole block)
            // a token's 16 columns lie in 16 neighbouring lanes: their squares are added there, always in this order
            float sq = valid ? v * v : 0.f;
#pragma unroll
            for (int o = 8; o; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            if (valid) lk.hw[(size_t)m * N + n] = __float2bfloat16_rn(v * ((i == threadIdx.x) ? e_nw : bl_load_any(lk.norm_w, lk.norm_w_dtype, n)));
            if (c == 0 && m < M) lk.ss_out[(size_t)m * (gridDim.x / SPLIT / m_groups) + tile / m_groups] = sq;
        }
    }
}

// The same product for very many columns (an output head): one warp owns 16 columns over the whole of K, so
// nothing is summed across warps and no barrier is met; a warp streams its rows of W with two batches of
// 16-byte loads in flight from start to end. Blocks of 8 warps cover 128 columns.
template <int MT, int EPI, typename TO>
__global__ void __launch_bounds__(256, MT <= 2 ? 2 : 1)
gemm_skinny_cols_kernel(const __nv_bfloat16* x /* written by the kernel before: no read-only cache */,
                        const __nv_bfloat16* __restrict__ w,
                        const void* __restrict__ bias, int bias_dtype, TO* out,
                        int M, int N, int K, int m_groups) {
    static_assert(EPI != BL_EPI_SWIGLU, "two matrices per column: use the 16-column kernel");
    constexpr int TOK = MT * 8;
    constexpr int UNROLL = MT == 1 ? 4 : 2;
    constexpr int STEP = UNROLL * 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = ((blockIdx.x / m_groups) * 8 + warp) * COLS;
    const int m0 = (blockIdx.x % m_groups) * TOK;
    float acc[MT][4];
#pragma unroll
    for (int j = 0; j < MT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
    const int r_lo = n0 + g, r_hi = n0 + g + 8;
    const bool lo_ok = r_lo < N, hi_ok = r_hi < N;
    const __nv_bfloat16* w_lo = w + (size_t)r_lo * K;
    const __nv_bfloat16* w_hi = w + (size_t)r_hi * K;
    struct Batch { uint4 a_lo[UNROLL], a_hi[UNROLL], b[UNROLL][MT]; };
    auto fetch_w = [&](Batch& bt, int kc0) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = kc0 + u * 32 + 8 * t;
            bt.a_lo[u] = ld16(w_lo + k, lo_ok && k < K);
            bt.a_hi[u] = ld16(w_hi + k, hi_ok && k < K);
        }
    };
    auto fetch_x = [&](Batch& bt, int kc0) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = kc0 + u * 32 + 8 * t;
#pragma unroll
            for (int j = 0; j < MT; ++j) {
                const int tok = m0 + 8 * j + g;
                bt.b[u][j] = (tok < M && k < K) ? *reinterpret_cast<const uint4*>(x + (size_t)tok * K + k)
                                                : make_uint4(0u, 0u, 0u, 0u);
            }
        }
    };
    auto multiply = [&](const Batch& bt) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
            for (int j = 0; j < MT; ++j) {
                mma_bf16(acc[j], bt.a_lo[u].x, bt.a_hi[u].x, bt.a_lo[u].y, bt.a_hi[u].y, bt.b[u][j].x, bt.b[u][j].y);
                mma_bf16(acc[j], bt.a_lo[u].z, bt.a_hi[u].z, bt.a_lo[u].w, bt.a_hi[u].w, bt.b[u][j].z, bt.b[u][j].w);
            }
        }
    };
    Batch b0, b1;
    bl_pdl_trigger();
    fetch_w(b0, 0);
    float e_lo = 0.f, e_hi = 0.f;
    if (EPI == BL_EPI_BIAS) {
        if (lo_ok) e_lo = bl_load_any(bias, bias_dtype, r_lo);
        if (hi_ok) e_hi = bl_load_any(bias, bias_dtype, r_hi);
    }
    bl_pdl_wait();
    fetch_x(b0, 0);
    // the loop bounds are the same for every lane (the MMA needs all 32); two batches per trip keep the buffers' names
    for (int kc0 = 0; kc0 < K; kc0 += 2 * STEP) {
        const bool more1 = kc0 + STEP < K;
        if (more1) { fetch_w(b1, kc0 + STEP); fetch_x(b1, kc0 + STEP); }
        multiply(b0);
        if (!more1) break;
        if (kc0 + 2 * STEP < K) { fetch_w(b0, kc0 + 2 * STEP); fetch_x(b0, kc0 + 2 * STEP); }
        multiply(b1);
    }
    // c0, c1: (column g, tokens 2t, 2t+1); c2, c3: (column g + 8, tokens 2t, 2t+1)
#pragma unroll
    for (int j = 0; j < MT; ++j) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int m = m0 + 8 * j + 2 * t + (i & 1);
            const bool hi = i >= 2;
            if (m >= M || !(hi ? hi_ok : lo_ok)) continue;
            TO* dst = out + (size_t)m * N + (hi ? r_hi : r_lo);
            float v = acc[j][i];
            if (EPI == BL_EPI_BIAS) v += hi ? e_hi : e_lo;
            if (EPI == BL_EPI_RESIDUAL) v += bl_load(dst);
            bl_store(dst, v);
        }
    }
}

template <int MT, typename TO>
int launch_cols(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int M, int N, int K,
                int epi, cudaStream_t s) {
    const int m_groups = (M + MT * 8 - 1) / (MT * 8);
    const int blocks = ((N + 8 * COLS - 1) / (8 * COLS)) * m_groups;
#define BL_GO(E) BL_CUDA(bl_launch_dependent(gemm_skinny_cols_kernel<MT, E, TO>, dim3(blocks), dim3(256), 0, s, \
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, bias, bias_dtype, (TO*)out, M, N, K, m_groups))
    switch (epi) {
        case BL_EPI_NONE: BL_GO(BL_EPI_NONE); break;
        case BL_EPI_BIAS: BL_GO(BL_EPI_BIAS); break;
        case BL_EPI_RESIDUAL: BL_GO(BL_EPI_RESIDUAL); break;
        default: BL_FAIL("bl_gemm_skinny: the column kernel has no epilogue %d", epi);
    }
#undef BL_GO
    return 0;
}

template <int MT, typename TO, int NW, bool DEEP>
int launch_nw(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int M, int N, int K,
              int epi, const SkinnyLink& lk, cudaStream_t s) {
    const int m_groups = (M + MT * 8 - 1) / (MT * 8);
    const int blocks = ((N + COLS - 1) / COLS) * m_groups;
#define BL_GO(E) BL_CUDA(bl_launch_dependent(gemm_skinny_kernel<MT, E, TO, NW, DEEP>, dim3(blocks), dim3(NW * 32), 0, s, \
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, bias, bias_dtype, (TO*)out, M, N, K, m_groups, lk))
    switch (epi) {
        case BL_EPI_NONE: BL_GO(BL_EPI_NONE); break;
        case BL_EPI_BIAS: BL_GO(BL_EPI_BIAS); break;
        case BL_EPI_RESIDUAL: BL_GO(BL_EPI_RESIDUAL); break;
        case BL_EPI_SWIGLU: BL_GO(BL_EPI_SWIGLU); break;
        default: BL_FAIL("bl_gemm_skinny: unknown epilogue %d", epi);
    }
#undef BL_GO
    return 0;
}

// The long-K kernel (16 warps, one or two groups of 8 tokens) with K cut over the two blocks of a cluster.
template <int MT, typename TO>
int launch_split(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int M, int N, int K,
                 int epi, const SkinnyLink& lk, cudaStream_t s) {
    const int blocks = (N + COLS - 1) / COLS;
#define BL_GO(E) BL_CUDA(bl_launch_dependent_clusters(gemm_skinny_kernel<MT, E, TO, 16, true, 2>, dim3(2 * blocks), dim3(16 * 32), 0, s, 2u, \
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, bias, bias_dtype, (TO*)out, M, N, K, 1, lk))
    switch (epi) {
        case BL_EPI_NONE: BL_GO(BL_EPI_NONE); break;
        case BL_EPI_BIAS: BL_GO(BL_EPI_BIAS); break;
        case BL_EPI_RESIDUAL: BL_GO(BL_EPI_RESIDUAL); break;
        default: BL_FAIL("bl_gemm_skinny: the kernel that cuts K over two blocks has no epilogue %d", epi);
    }
#undef BL_GO
    return 0;
}

int sm_count() {
    static int sms = 0;                                          // (of the current device at the first call)
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
    }
    return sms;
}

// Long rows of W are cut over 16 warps instead of 8: fewer trips to memory one after the other per warp.
template <int MT, typename TO>
int launch(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int M, int N, int K,
           int epi, const SkinnyLink& lk, cudaStream_t s) {
    const int m_groups = (M + MT * 8 - 1) / (MT * 8);
    const int blocks = ((N + COLS - 1) / COLS) * m_groups;
    const bool linked = lk.hw != nullptr || lk.ss_in != nullptr;
    // the choice depends on N alone, so that a row's result is the same whatever else is in the batch
    if ((N + COLS - 1) / COLS > 4 * 148 && epi != BL_EPI_SWIGLU) {
        if (linked) BL_FAIL("bl_gemm_skinny_linked: %d columns run on the kernel of whole warps per column block, which shares no norm", N);
        return launch_cols<MT, TO>(x, w, bias, bias_dtype, out, M, N, K, epi, s);
    }
    if (blocks > 4 * 148) return launch_nw<MT, TO, 8, false>(x, w, bias, bias_dtype, out, M, N, K, epi, lk, s);
    // (this choice, too, depends on N and K alone)
    if (K >= 2048 && MT <= 2 && epi != BL_EPI_SWIGLU && 2 * blocks <= sm_count()) return launch_split<(MT <= 2 ? MT : 1), TO>(x, w, bias, bias_dtype, out, M, N, K, epi, lk, s);
    if (K >= 2048 && MT == 1 && epi != BL_EPI_SWIGLU) return launch_nw<1, TO, 16, true>(x, w, bias, bias_dtype, out, M, N, K, epi, lk, s);
    return launch_nw<MT, TO, 8, true>(x, w, bias, bias_dtype, out, M, N, K, epi, lk, s);
}

}  // namespace

namespace {

int run(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int out_dtype, int M, int N, int K,
        int epilogue, const SkinnyLink& lk, void* stream) {
    if (M <= 0) return 0;
    if (N <= 0 || K <= 0) BL_FAIL("bl_gemm_skinny: bad sizes N=%d K=%d", N, K);
    if (K % 8 != 0) BL_FAIL("bl_gemm_skinny: K=%d is not a multiple of 8 (use the plain kernel)", K);
    if (((uintptr_t)x | (uintptr_t)w) & 15) BL_FAIL("bl_gemm_skinny: x and W must be 16-byte aligned");
    if (epilogue == BL_EPI_BIAS && (bias == nullptr || (bias_dtype != BL_F32 && bias_dtype != BL_BF16)))
        BL_FAIL("bl_gemm_skinny: bias epilogue needs a float32 or bfloat16 bias");
    if (epilogue == BL_EPI_RESIDUAL && out_dtype != BL_F32)
        BL_FAIL("bl_gemm_skinny: the residual stream is 32-bit; output dtype must be float32");
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == BL_F32) {
        if (M <= 8) return launch<1, float>(x, w, bias, bias_dtype, out, M, N, K, epilogue, lk, s);
        if (M <= 16) return launch<2, float>(x, w, bias, bias_dtype, out, M, N, K, epilogue, lk, s);
        return launch<4, float>(x, w, bias, bias_dtype, out, M, N, K, epilogue, lk, s);
    }
    if (out_dtype == BL_BF16) {
        if (M <= 8) return launch<1, __nv_bfloat16>(x, w, bias, bias_dtype, out, M, N, K, epilogue, lk, s);
        if (M <= 16) return launch<2, __nv_bfloat16>(x, w, bias, bias_dtype, out, M, N, K, epilogue, lk, s);
        return launch<4, __nv_bfloat16>(x, w, bias, bias_dtype, out, M, N, K, epilogue, lk, s);
    }
    BL_FAIL("bl_gemm_skinny: unknown output dtype %d", out_dtype);
}

}  // namespace

// bfloat16 x and W; K a multiple of 8 and both base addresses 16-byte aligned (16-byte loads); any M, N.
// Meant for M up to a few dozen: W is read once per 32 tokens.
extern "C" int bl_gemm_skinny(const void* x, const void* w, const void* bias, int bias_dtype, void* out,
                              int out_dtype, int M, int N, int K, int epilogue, void* stream) {
    return run(x, w, bias, bias_dtype, out, out_dtype, M, N, K, epilogue, SkinnyLink{}, stream);
}

// Partial sums of squares per row that the linked residual product writes: one per block of 16 columns.
extern "C" int bl_gemm_skinny_norm_parts(int N) { return (N + COLS - 1) / COLS; }

// out += x . W^T (32-bit residual stream, in place) and, for the RMS norm with weight norm_w that reads out next:
// hw[M, N] = bfloat16(out * norm_w), ss[M, parts] = sums of squares of the new rows by block of 16 columns
// (parts = bl_gemm_skinny_norm_parts(N)).
extern "C" int bl_gemm_skinny_residual_norm(const void* x, const void* w, void* out, int M, int N, int K,
                                            const void* norm_w, int norm_w_dtype, void* hw, float* ss, void* stream) {
    if (norm_w == nullptr || hw == nullptr || ss == nullptr || (norm_w_dtype != BL_F32 && norm_w_dtype != BL_BF16))
        BL_FAIL("bl_gemm_skinny_residual_norm: needs a float32 or bfloat16 norm weight, hw and ss");
    SkinnyLink lk = {};
    lk.norm_w = norm_w; lk.norm_w_dtype = norm_w_dtype; lk.hw = (__nv_bfloat16*)hw; lk.ss_out = ss;
    return run(x, w, nullptr, 0, out, BL_F32, M, N, K, BL_EPI_RESIDUAL, lk, stream);
}

// out = epilogue(r * (hw . W^T)) with r[m] = 1 / sqrt(sum(ss[m][:]) / K + eps): the product of rows whose RMS norm
// the linked residual product left pending. Epilogues: none, bias, SwiGLU.
extern "C" int bl_gemm_skinny_scaled(const void* hw, const void* w, const void* bias, int bias_dtype, void* out,
                                     int out_dtype, int M, int N, int K, int epilogue, const float* ss, int parts,
                                     float eps, void* stream) {
    if (ss == nullptr || parts <= 0) BL_FAIL("bl_gemm_skinny_scaled: needs the rows' partial sums of squares");
    if (epilogue == BL_EPI_RESIDUAL) BL_FAIL("bl_gemm_skinny_scaled: the residual epilogue takes no pending norm");
    SkinnyLink lk = {};
    lk.ss_in = ss; lk.parts_in = parts; lk.inv_dim = 1.0f / (float)K; lk.eps = eps;
    return run(hw, w, bias, bias_dtype, out, out_dtype, M, N, K, epilogue, lk, stream);
}
