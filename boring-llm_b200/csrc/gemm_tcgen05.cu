// Matrix product for many rows (prefill) on the fifth-generation tensor cores:
// out[M, N] = epilogue(x[M, K] . W[N, K]^T), bfloat16 operands, 32-bit accumulation in tensor memory.
//
// One block computes one 128 x 128 tile of the output. A single thread feeds a three-stage ring of
// shared-memory tiles with TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast: every block fetches
// its own tiles; rows and k past the matrices' edges arrive as zeros), a single thread of another warp
// issues tcgen05.mma (M 128, N 128, K 16; four per 64-wide k block) on those tiles in place, and
// tcgen05.commit hands each stage back to the loader and, after the last k block, the accumulator to the
// epilogue. All four warps then read their 32 lanes of the accumulator with tcgen05.ld and apply the
// epilogue (bias, residual add into the 32-bit stream, or SwiGLU over a tile whose first 64 columns are
// gate rows of W and last 64 the matching up rows). Two blocks fit an SM (96 KB of stages, 128 of 512
// tensor-memory columns each), so one block's epilogue overlaps the other's main loop.
//
// The kernel takes part in programmatic dependent launch: barriers and the first ring of W before the wait, tensor
// memory, x and out after it.
// Every wait on an mbarrier is bounded: when a bound runs out the block records a code in a status word,
// drains its own copies, frees its tensor memory and returns; bl_gemm_tc_status() reports it on the host.
// Role in the reference: the compiler's "native" tensor schedule for prefill matmuls
// (kernel.tensors.linear, src/math_gpu.br:1998-2030; boring.toml:8-26); formula y = x . W^T (src/math.br:66-82).
#include "tcgen05.cuh"

namespace {

constexpr const char* WHO = "bl_gemm_tc";

constexpr int BM = 128, BN = 128, BK = 64;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
// Stages of the ring: three, so that two blocks share an SM, where a launch has more blocks than SMs; six where it
// has fewer (a block then has an SM to itself, and three 32 KB stages in flight against a microsecond of latency
// are 100 GB/s: gate/up of a 64-row decode step, 76 blocks that each stream 344 KB, took 9 us).
constexpr int STAGES_SHARED = 3, STAGES_ALONE = 6;
constexpr int smem_bytes(int stages) { return stages * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */; }
constexpr int TMEM_COLS = 128;
constexpr uint32_t WAIT_LIMIT = 1u << 22;

__device__ int g_status = 0;      // 0 = fine; else the code of the first wait that ran out

// Bounded wait. Returns false when the bound ran out or another thread of the block has given up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* give_up, int code) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if (*give_up) return false;
    }
    *give_up = 1;
    atomicCAS(&g_status, 0, code);
    return false;
}

// kind::f16 instruction descriptor: D 32-bit, A and B bfloat16 and K-major, N >> 3 at bit 17, M >> 4 at bit 24.
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

template <int EPI, typename TO, int STAGES>
__global__ void __launch_bounds__(128)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const void* __restrict__ bias, int bias_dtype, TO* __restrict__ out, int M, int N, int K) {
    constexpr bool GLU = EPI == BL_EPI_SWIGLU;
    extern __shared__ unsigned char smem_raw[];
    if (threadIdx.x == 0) { tma_prefetch_map(&map_a); tma_prefetch_map(&map_b); }
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;              // tiles need 1024-byte alignment
    unsigned char* aligned = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + STAGES * STAGE_BYTES;                         // full[S], empty[S], accum
    volatile int* give_up = reinterpret_cast<volatile int*>(aligned + STAGES * STAGE_BYTES + 128);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(aligned + STAGES * STAGE_BYTES + 136);
    const uint32_t full0 = bars, empty0 = bars + 8 * STAGES, accum = bars + 16 * STAGES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tile = blockIdx.x, m0 = blockIdx.y * BM;
    const int n0 = n_tile * (GLU ? BN / 2 : BN);                              // first output column of the tile
    const int kblocks = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        *give_up = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // W does not depend on the kernel before this one: the loader starts W for the first ring of k blocks before the
    // dependent-launch wait (the stage's barrier expects x and W together; x follows after the wait)
    auto load_w = [&](int s, int kb) {
        const uint32_t b_dst = base + s * STAGE_BYTES + A_BYTES;
        if (GLU) {                                                              // 64 gate rows, then the 64 up rows that match
            tma_load_2d(b_dst, &map_b, full0 + 8 * s, kb * BK, n0);
            tma_load_2d(b_dst + B_BYTES / 2, &map_b, full0 + 8 * s, kb * BK, N + n0);
        } else {
            tma_load_2d(b_dst, &map_b, full0 + 8 * s, kb * BK, n0);
        }
    };
    int early = 0;
    if (warp == 0 && lane == 0) {
        for (; early < STAGES && early < kblocks; ++early) {
            mbar_expect_tx(full0 + 8 * early, STAGE_BYTES);
            load_w(early, early);
        }
    }
    __syncwarp();
    bl_pdl_wait();                                                              // x, out and the SM's tensor memory belong to the predecessor until here
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(smem_u32((const void*)tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    bl_pdl_trigger();                                                           // the next kernel may start its preamble (it waits before it touches data)

    if (warp == 0 && lane == 0) {
        // loader: wait until the MMAs that read a stage are done, then refill it
        int issued = early;
        for (int kb = 0; kb < kblocks; ++kb) {
            const int s = kb % STAGES;
            if (kb >= STAGES && !mbar_wait(empty0 + 8 * s, ((kb / STAGES) & 1) ^ 1, give_up, 1)) break;
            if (kb >= early) {
                mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                load_w(s, kb);
            }
            tma_load_2d(base + s * STAGE_BYTES, &map_a, full0 + 8 * s, kb * BK, m0);
            issued = kb + 1;
        }
        if (*give_up)                                                           // let our own copies land before leaving
            for (int kb = max(0, issued - STAGES); kb < issued; ++kb)
                mbar_wait(full0 + 8 * (kb % STAGES), (kb / STAGES) & 1, give_up, 0);
    } else if (warp == 1 && lane == 0) {
        // issuer: four K = 16 MMAs per stage; the accumulator starts from zero at the first of them
        for (int kb = 0; kb < kblocks; ++kb) {
            const int s = kb % STAGES;
            if (!mbar_wait(full0 + 8 * s, (kb / STAGES) & 1, give_up, 2)) break;
            fence_after_sync();
            const uint64_t a_desc = smem_desc(base + s * STAGE_BYTES);
            const uint64_t b_desc = smem_desc(base + s * STAGE_BYTES + A_BYTES);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)                                   // 32 bytes along K inside the swizzled row
                umma_bf16(tmem, a_desc + 2 * k, b_desc + 2 * k, IDESC, (kb | k) != 0);
            umma_commit(empty0 + 8 * s);
        }
        umma_commit(accum);
    }
    __syncwarp();
    const bool ready = mbar_wait(accum, 0, give_up, 3);
    fence_after_sync();
    if (ready && !*give_up) {
        // A thread of tcgen05.ld holds 32 consecutive columns of ONE row; written out like that, every store
        // instruction of a warp would touch 32 different rows. So each warp passes its 32 x 32 chunk through a
        // padded tile of shared memory (the stages are free by now) and writes it out four rows at a time,
        // 128 contiguous bytes per row, with 16-byte accesses.
        constexpr int PITCH = 36;                                               // floats per staged row (16-byte aligned, conflict-free)
        float* tile = reinterpret_cast<float*>(aligned) + warp * 32 * PITCH;
        const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
        const int r_sub = lane >> 3, c4 = (lane & 7) * 4;                       // this lane's row (of four) and column quad when writing out
        const bool vec_ok = (N % 4) == 0;
        constexpr int CHUNKS = GLU ? 2 : BN / 32;
#pragma unroll 1
        for (int c = 0; c < CHUNKS; ++c) {
            uint32_t r[32];
            tmem_ld32(lane_addr + c * 32, r);
            if (GLU) {
                uint32_t u[32];
                tmem_ld32(lane_addr + 64 + c * 32, u);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(bl_silu_fast(__uint_as_float(r[j])) * __uint_as_float(u[j]));
            } else {
                tmem_ld_wait();
            }
#pragma unroll
            for (int j = 0; j < 8; ++j)
                *reinterpret_cast<uint4*>(tile + lane * PITCH + 4 * j) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
            __syncwarp();
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const int row = it * 4 + r_sub;
                const int m = m0 + warp * 32 + row;
                const int n = n0 + c * 32 + c4;
                if (m >= M || n >= N) continue;
                float4 v = *reinterpret_cast<const float4*>(tile + row * PITCH + c4);
                TO* dst = out + (size_t)m * N + n;
                if (vec_ok && n + 3 < N) {
                    if (EPI == BL_EPI_BIAS) {
                        v.x += bl_load_any(bias, bias_dtype, n); v.y += bl_load_any(bias, bias_dtype, n + 1);
                        v.z += bl_load_any(bias, bias_dtype, n + 2); v.w += bl_load_any(bias, bias_dtype, n + 3);
                    }
                    if (sizeof(TO) == 4) {
                        if (EPI == BL_EPI_RESIDUAL) {
                            const float4 o = *reinterpret_cast<const float4*>(dst);
                            v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                        }
                        *reinterpret_cast<float4*>(dst) = v;
                    } else {
                        __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
                        uint2 pk;
                        pk.x = *reinterpret_cast<unsigned*>(&lo); pk.y = *reinterpret_cast<unsigned*>(&hi);
                        *reinterpret_cast<uint2*>(dst) = pk;
                    }
                } else {
                    const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (n + j >= N) break;
                        float x1 = e[j];
                        if (EPI == BL_EPI_BIAS) x1 += bl_load_any(bias, bias_dtype, n + j);
                        if (EPI == BL_EPI_RESIDUAL) x1 += bl_load(dst + j);
                        bl_store(dst + j, x1);
                    }
                }
            }
            __syncwarp();
        }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(TMEM_COLS) : "memory");
    }
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

template <int EPI, typename TO, int STAGES>
int launch_stages(const CUtensorMap& a, const CUtensorMap& b, const void* bias, int bias_dtype, void* out, int M, int N, int K,
                  dim3 grid, cudaStream_t s) {
    static bool configured = false;
    if (!configured) {
        BL_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<EPI, TO, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(STAGES)));
        configured = true;
    }
    // a block waits (griddepcontrol.wait) before it allocates tensor memory or touches x and out, so it may be launched
    // while its predecessor still runs
    BL_CUDA(bl_launch_dependent(gemm_tc_kernel<EPI, TO, STAGES>, grid, dim3(128), (size_t)smem_bytes(STAGES), s, a, b, bias, bias_dtype, (TO*)out, M, N, K));
    BL_CHECK_LAUNCH("bl_gemm_tc");
    return 0;
}

template <int EPI, typename TO>
int launch(const CUtensorMap& a, const CUtensorMap& b, const void* bias, int bias_dtype, void* out, int M, int N, int K,
           cudaStream_t s) {
    const int cols_per_tile = EPI == BL_EPI_SWIGLU ? BN / 2 : BN;
    dim3 grid((N + cols_per_tile - 1) / cols_per_tile, (M + BM - 1) / BM);
    // (the sums of a tile do not depend on the depth of the ring)
    if ((long long)grid.x * grid.y <= sm_count()) return launch_stages<EPI, TO, STAGES_ALONE>(a, b, bias, bias_dtype, out, M, N, K, grid, s);
    return launch_stages<EPI, TO, STAGES_SHARED>(a, b, bias, bias_dtype, out, M, N, K, grid, s);
}

}  // namespace

// bfloat16 x[M, K] and W[N, K] (2N rows for BL_EPI_SWIGLU); K a multiple of 8, both 16-byte aligned.
extern "C" int bl_gemm_tc(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int out_dtype,
                          int M, int N, int K, int epilogue, void* stream) {
    if (M <= 0) return 0;
    if (N <= 0 || K <= 0) BL_FAIL("bl_gemm_tc: bad sizes N=%d K=%d", N, K);
    if (K % 8 != 0) BL_FAIL("bl_gemm_tc: K=%d is not a multiple of 8 (TMA rows must be 16-byte multiples)", K);
    if (((uintptr_t)x | (uintptr_t)w) & 15) BL_FAIL("bl_gemm_tc: x and W must be 16-byte aligned");
    if (epilogue == BL_EPI_BIAS && (bias == nullptr || (bias_dtype != BL_F32 && bias_dtype != BL_BF16)))
        BL_FAIL("bl_gemm_tc: bias epilogue needs a float32 or bfloat16 bias");
    const bool glu = epilogue == BL_EPI_SWIGLU;
    CUtensorMap a, b;
    if (bl_make_map_bf16(WHO, &a, x, M, K, BM, BK)) return 1;
    if (bl_make_map_bf16(WHO, &b, w, glu ? 2 * N : N, K, glu ? BN / 2 : BN, BK)) return 1;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == BL_F32) {
        switch (epilogue) {
            case BL_EPI_NONE: return launch<BL_EPI_NONE, float>(a, b, bias, bias_dtype, out, M, N, K, s);
            case BL_EPI_BIAS: return launch<BL_EPI_BIAS, float>(a, b, bias, bias_dtype, out, M, N, K, s);
            case BL_EPI_RESIDUAL: return launch<BL_EPI_RESIDUAL, float>(a, b, bias, bias_dtype, out, M, N, K, s);
            case BL_EPI_SWIGLU: return launch<BL_EPI_SWIGLU, float>(a, b, bias, bias_dtype, out, M, N, K, s);
        }
    } else if (out_dtype == BL_BF16) {
        switch (epilogue) {
            case BL_EPI_NONE: return launch<BL_EPI_NONE, __nv_bfloat16>(a, b, bias, bias_dtype, out, M, N, K, s);
            case BL_EPI_BIAS: return launch<BL_EPI_BIAS, __nv_bfloat16>(a, b, bias, bias_dtype, out, M, N, K, s);
            case BL_EPI_SWIGLU: return launch<BL_EPI_SWIGLU, __nv_bfloat16>(a, b, bias, bias_dtype, out, M, N, K, s);
            case BL_EPI_RESIDUAL: BL_FAIL("bl_gemm_tc: the residual stream is 32-bit; output dtype must be float32");
        }
    } else {
        BL_FAIL("bl_gemm_tc: unknown output dtype %d", out_dtype);
    }
    BL_FAIL("bl_gemm_tc: unknown epilogue %d", epilogue);
}

// Reads and clears the status word: 0 when no block has given up on a wait since the last call
// (1 loader, 2 issuer, 3 epilogue). Synchronises the device.
extern "C" int bl_gemm_tc_status(int* status) {
    int v = 0, zero = 0;
    BL_CUDA(cudaMemcpyFromSymbol(&v, g_status, sizeof(int)));
    if (v != 0) BL_CUDA(cudaMemcpyToSymbol(g_status, &zero, sizeof(int)));
    *status = v;
    return 0;
}
