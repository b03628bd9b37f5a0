// Plain matrix product on CUDA cores: out = epilogue(x . W^T), W stored (outputs x inputs) row-major
// as in the reference's `linear` (src/math.br:66-82) and its tiled GPU kernel LinearKernel
// (src/math_gpu.br:82-135). Every output element accumulates its products in ascending k in one
// 32-bit accumulator, whatever the number of rows, so results do not depend on how a batch is cut.
// This is the whole-model 32-bit path's product and the twin that the tensor-core kernels are
// checked against.
#include "common.cuh"
#include "api.h"

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

template <typename TX, typename TW, typename TO, int EPI>
__global__ void __launch_bounds__(256)
gemm_plain_kernel(const TX* __restrict__ x, const TW* __restrict__ w, const void* __restrict__ bias,
                  int bias_dtype, TO* __restrict__ out, int M, int N, int K) {
    __shared__ float xs[TK][TM + 1];
    __shared__ float ws[TK][TN + 1];
    __shared__ float us[EPI == BL_EPI_SWIGLU ? TK : 1][TN + 1];
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;   // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4] = {};
    float acu[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += TK) {
        for (int i = threadIdx.x; i < TM * TK; i += 256) {
            const int r = i / TK, c = i % TK;
            const int m = m0 + r, k = k0 + c;
            xs[c][r] = (m < M && k < K) ? bl_load(x + (size_t)m * K + k) : 0.f;
        }
        for (int i = threadIdx.x; i < TN * TK; i += 256) {
            const int r = i / TK, c = i % TK;
            const int n = n0 + r, k = k0 + c;
            const bool ok = n < N && k < K;
            ws[c][r] = ok ? bl_load(w + (size_t)n * K + k) : 0.f;
            if (EPI == BL_EPI_SWIGLU) us[c][r] = ok ? bl_load(w + (size_t)(N + n) * K + k) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TK; ++k) {
            float a[4], b[4], u[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[k][tx * 4 + j];
            if (EPI == BL_EPI_SWIGLU) {
#pragma unroll
                for (int j = 0; j < 4; ++j) u[j] = us[k][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                    if (EPI == BL_EPI_SWIGLU) acu[i][j] = fmaf(a[i], u[j], acu[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            TO* dst = out + (size_t)m * N + n;
            float v = acc[i][j];
            if (EPI == BL_EPI_BIAS) v += bl_load_any(bias, bias_dtype, n);
            if (EPI == BL_EPI_RESIDUAL) v += bl_load(dst);
            if (EPI == BL_EPI_SWIGLU) v = bl_silu(v) * acu[i][j];
            bl_store(dst, v);
        }
    }
}

template <typename TX, typename TW, typename TO>
int launch_epi(const void* x, const void* w, const void* bias, int bias_dtype, void* out,
               int M, int N, int K, int epi, cudaStream_t s) {
    dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
#define BL_GO(E) gemm_plain_kernel<TX, TW, TO, E><<<grid, 256, 0, s>>>( \
        (const TX*)x, (const TW*)w, bias, bias_dtype, (TO*)out, M, N, K)
    switch (epi) {
        case BL_EPI_NONE: BL_GO(BL_EPI_NONE); break;
        case BL_EPI_BIAS: BL_GO(BL_EPI_BIAS); break;
        case BL_EPI_RESIDUAL: BL_GO(BL_EPI_RESIDUAL); break;
        case BL_EPI_SWIGLU: BL_GO(BL_EPI_SWIGLU); break;
        default: BL_FAIL("bl_gemm_plain: unknown epilogue %d", epi);
    }
#undef BL_GO
    BL_CHECK_LAUNCH("bl_gemm_plain");
    return 0;
}

template <typename TX, typename TW>
int launch_out(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int out_dtype,
               int M, int N, int K, int epi, cudaStream_t s) {
    if (out_dtype == BL_F32) return launch_epi<TX, TW, float>(x, w, bias, bias_dtype, out, M, N, K, epi, s);
    if (out_dtype == BL_BF16) {
        if (epi == BL_EPI_RESIDUAL) BL_FAIL("bl_gemm_plain: the residual stream is 32-bit; output dtype must be float32");
        return launch_epi<TX, TW, __nv_bfloat16>(x, w, bias, bias_dtype, out, M, N, K, epi, s);
    }
    BL_FAIL("bl_gemm_plain: unknown output dtype %d", out_dtype);
}

}  // namespace

extern "C" int bl_gemm_plain(const void* x, int x_dtype, const void* w, int w_dtype, const void* bias,
                             int bias_dtype, void* out, int out_dtype, int M, int N, int K, int epilogue,
                             void* stream) {
    if (M <= 0) return 0;
    if (N <= 0 || K <= 0) BL_FAIL("bl_gemm_plain: bad sizes N=%d K=%d", N, K);
    if (epilogue == BL_EPI_BIAS && bias == nullptr) BL_FAIL("bl_gemm_plain: bias epilogue without a bias");
    if (epilogue == BL_EPI_BIAS && bias_dtype != BL_F32 && bias_dtype != BL_BF16)
        BL_FAIL("bl_gemm_plain: unknown bias dtype %d", bias_dtype);
    cudaStream_t s = (cudaStream_t)stream;
    if (x_dtype == BL_F32 && w_dtype == BL_F32)
        return launch_out<float, float>(x, w, bias, bias_dtype, out, out_dtype, M, N, K, epilogue, s);
    if (x_dtype == BL_BF16 && w_dtype == BL_BF16)
        return launch_out<__nv_bfloat16, __nv_bfloat16>(x, w, bias, bias_dtype, out, out_dtype, M, N, K, epilogue, s);
    if (x_dtype == BL_F32 && w_dtype == BL_BF16)
        return launch_out<float, __nv_bfloat16>(x, w, bias, bias_dtype, out, out_dtype, M, N, K, epilogue, s);
    BL_FAIL("bl_gemm_plain: unsupported input dtypes x=%d w=%d", x_dtype, w_dtype);
}
