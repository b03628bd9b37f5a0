// Matrix product for FEW rows and VERY MANY columns (an output head at decode time) on the fifth-generation tensor
// cores: out[M, N] = x[M, K] . W[N, K]^T with M up to 64, bfloat16 operands, 32-bit accumulation in tensor memory.
//
// The roles of the operands are swapped: 128 rows of W are the M side of tcgen05.mma and the (padded) rows of x its
// N side, so a tile of the accumulator is 128 columns of the output x NT tokens and every byte of W passes through
// shared memory exactly once, as a TMA box of 128 rows x 64 k (16 KB, 128-byte swizzle). The kernel is bound by
// HBM, so everything serves the stream of W:
//   - blocks are persistent (one per SM) and walk the 128-column tiles t, t + blocks, ...;
//   - x is copied into shared memory once per block and stays there (NT rows x K);
//   - the ring of W stages is as deep as shared memory allows (up to ten stages, 160 KB in flight per SM), and its
//     first round is requested BEFORE the dependent-launch wait: W does not depend on the kernel before;
//   - the accumulator is double buffered in tensor memory, so the four epilogue warps write tile t (lane r of
//     tensor memory is output column n0 + r: a warp's store of one token's 32 columns is one 128-byte line) while
//     tile t + 1 is multiplied.
// One thread issues the copies, one the MMAs. Every wait on an mbarrier is bounded; when a bound runs out the block
// records a code in a status word, lets its own copies land, frees its tensor memory and returns.
// Formula y = x . W^T (src/math.br:66-82); role in the reference: the output projection of forward_step
// (src/model.br:1360-1362).
#include "tcgen05.cuh"

namespace {

constexpr const char* WHO = "bl_gemm_tc_cols";

constexpr int BN = 128;                 // output columns (rows of W) per tile
constexpr int BK = 64;
constexpr int W_BYTES = BN * BK * 2;    // one stage
constexpr int MAX_STAGES = 10;
constexpr int THREADS = 192;            // warp 0: copies, warp 1: MMAs, warps 2..5: epilogue
constexpr uint32_t WAIT_LIMIT = 1u << 22;
constexpr int SMEM_LIMIT = 227 * 1024;

__device__ int g_status3 = 0;           // 0 = fine; else the code of the first wait that ran out

// Bounded wait. False when the bound ran out or another thread of the block has given up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* give_up, int code) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if (*give_up) return false;
    }
    *give_up = 1;
    atomicCAS(&g_status3, 0, code);
    return false;
}
// Bounded wait that does not look at the give-up flag (a block that has given up waits for its own copies).
__device__ __forceinline__ void mbar_wait_plain(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return;
    }
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}

// kind::f16: D 32-bit, A and B bfloat16 and K-major, N >> 3 at bit 17, M >> 4 at bit 24
constexpr uint32_t idesc_for(int nt) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(nt >> 3) << 17) | ((uint32_t)(BN >> 4) << 24);
}

// shared memory: [x: kblocks tiles of NT x 64][ring: stages x 16 KB][barriers]
template <int NT, typename TO>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_cols_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    TO* __restrict__ out, int M, int N, int K, int stages) {
    constexpr int X_TILE = NT * BK * 2;                                       // one k block of x
    constexpr int TMEM_COLS = NT <= 32 ? 64 : 128;                            // two accumulators of NT columns
    extern __shared__ __align__(1024) unsigned char smem[];
    if (threadIdx.x == 0) { tma_prefetch_map(&map_x); tma_prefetch_map(&map_w); }
    const uint32_t base = smem_u32(smem);
    const int kblocks = (K + BK - 1) / BK;
    const int x_bytes = kblocks * X_TILE;                                     // a multiple of 1024 (NT >= 16)
    const uint32_t ring = base + x_bytes;
    const int bars_off = x_bytes + stages * W_BYTES;
    const uint32_t bars = base + bars_off;
    const uint32_t full0 = bars, empty0 = bars + 8 * MAX_STAGES, full_x = bars + 16 * MAX_STAGES,
                   acc_full0 = full_x + 8, acc_empty0 = acc_full0 + 16;
    volatile int* give_up = reinterpret_cast<volatile int*>(smem + bars_off + 16 * MAX_STAGES + 48);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + bars_off + 16 * MAX_STAGES + 56);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = (N + BN - 1) / BN;
    const int my_tiles = blockIdx.x < n_tiles ? (n_tiles - 1 - blockIdx.x) / gridDim.x + 1 : 0;
    const int total = my_tiles * kblocks;                                     // k blocks of W this block streams

    if (threadIdx.x == 0) {
        *give_up = (base & 1023u) ? 1 : 0;                                    // the swizzled tiles need 1024-byte alignment
        if (base & 1023u) atomicCAS(&g_status3, 0, 9);
        for (int s = 0; s < stages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(full_x, 1);
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full0 + 8 * b, 1); mbar_init(acc_empty0 + 8 * b, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // W does not depend on the kernel before this one: the first round of the ring is requested before the wait
    int early = 0;
    if (warp == 0 && lane == 0 && !*give_up) {
        for (; early < stages && early < total; ++early) {
            const int t = blockIdx.x + (early / kblocks) * gridDim.x, kb = early % kblocks;
            mbar_expect_tx(full0 + 8 * early, W_BYTES);
            tma_load_2d(ring + early * W_BYTES, &map_w, full0 + 8 * early, kb * BK, t * BN);
        }
    }
    __syncwarp();
    bl_pdl_wait();                                                            // x, out and the SM's tensor memory belong to the predecessor until here
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(smem_u32((const void*)tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    bl_pdl_trigger();

    if (warp == 0) {
        if (lane == 0 && !*give_up) {
            // x: every k block as its own swizzled tile (rows past M arrive as zeros)
            mbar_expect_tx(full_x, (uint32_t)x_bytes);
            for (int kb = 0; kb < kblocks; ++kb) tma_load_2d(base + kb * X_TILE, &map_x, full_x, kb * BK, 0);
            int issued = early;
            for (int it = early; it < total; ++it) {
                const int s = it % stages;
                if (!mbar_wait(empty0 + 8 * s, ((it / stages) & 1) ^ 1, give_up, 1)) break;
                const int t = blockIdx.x + (it / kblocks) * gridDim.x, kb = it % kblocks;
                mbar_expect_tx(full0 + 8 * s, W_BYTES);
                tma_load_2d(ring + s * W_BYTES, &map_w, full0 + 8 * s, kb * BK, t * BN);
                issued = it + 1;
            }
            if (*give_up && !(base & 1023u)) {                                 // let our own copies land before leaving
                mbar_wait_plain(full_x, 0);
                for (int it = issued > stages ? issued - stages : 0; it < issued; ++it)
                    mbar_wait_plain(full0 + 8 * (it % stages), (uint32_t)((it / stages) & 1));
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && !*give_up && my_tiles > 0) {
            bool ok = mbar_wait(full_x, 0, give_up, 2);
            int it = 0;
            for (int local = 0; ok && local < my_tiles; ++local) {
                const int buf = local & 1;
                // the epilogue warps must have drained this accumulator buffer (its first two uses find it free)
                if (local >= 2 && !mbar_wait(acc_empty0 + 8 * buf, ((local / 2) & 1) ^ 1, give_up, 4)) break;
                fence_after_sync();
                const uint32_t d_tmem = tmem + buf * NT;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % stages;
                    if (!mbar_wait(full0 + 8 * s, (it / stages) & 1, give_up, 3)) { ok = false; break; }
                    fence_after_sync();
                    const uint64_t a_desc = smem_desc(ring + s * W_BYTES);     // 128 rows of W: the M side
                    const uint64_t b_desc = smem_desc(base + kb * X_TILE);     // NT rows of x: the N side
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)                          // 32 bytes along K inside the swizzled row
                        umma_bf16(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc_for(NT), (kb | k) != 0);
                    umma_commit(empty0 + 8 * s);
                }
                if (!ok) break;
                umma_commit(acc_full0 + 8 * buf);
            }
        }
    } else {
        // epilogue: lane r of tensor memory is output column n0 + r, its NT columns are the tokens
        const int q = warp & 3;                                               // the 32 lanes this warp may read
        bool ok = true;
        for (int local = 0; local < my_tiles; ++local) {
            const int buf = local & 1;
            const int n = (blockIdx.x + local * gridDim.x) * BN + q * 32 + lane;
            ok = mbar_wait(acc_full0 + 8 * buf, (local / 2) & 1, give_up, 5) && ok;
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            fence_after_sync();
            const uint32_t taddr = tmem + buf * NT + ((uint32_t)(q * 32) << 16);
#pragma unroll
            for (int c = 0; c < NT / 16; ++c) {
                uint32_t r[16];
                tmem_ld16(taddr + c * 16, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int m = c * 16 + j;
                    if (m < M && n < N) bl_store(out + (size_t)m * N + n, __uint_as_float(r[j]));
                }
            }
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
        }
    }
    __syncwarp();
    fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 1;
    }
    return n;
}

// stages of the ring of W that fit beside x (0: it does not fit)
int stages_for(int nt, int K) {
    const int kblocks = (K + BK - 1) / BK;
    const int left = SMEM_LIMIT - kblocks * nt * BK * 2 - 256;
    int s = left / W_BYTES;
    return s > MAX_STAGES ? MAX_STAGES : (s >= 3 ? s : 0);
}

template <int NT, typename TO>
int launch(const void* x, const void* w, void* out, int M, int N, int K, cudaStream_t s) {
    const int stages = stages_for(NT, K);
    const int kblocks = (K + BK - 1) / BK;
    const int bytes = kblocks * NT * BK * 2 + stages * W_BYTES + 256;
    static bool configured = false;
    if (!configured) {
        BL_CUDA(cudaFuncSetAttribute(gemm_tc_cols_kernel<NT, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT));
        configured = true;
    }
    CUtensorMap mx, mw;
    if (bl_make_map_bf16(WHO, &mx, x, M, K, NT, BK)) return 1;
    if (bl_make_map_bf16(WHO, &mw, w, N, K, BN, BK)) return 1;
    const int n_tiles = (N + BN - 1) / BN;
    const int blocks = n_tiles < sm_count() ? n_tiles : sm_count();
    BL_CUDA(bl_launch_dependent(gemm_tc_cols_kernel<NT, TO>, dim3(blocks), dim3(THREADS), (size_t)bytes, s, mx, mw, (TO*)out, M, N, K, stages));
    BL_CHECK_LAUNCH("bl_gemm_tc_cols");
    return 0;
}

}  // namespace

// Whether bl_gemm_tc_cols takes these sizes: up to 64 rows, K a multiple of 8, and x beside at least three stages
// of W in shared memory.
extern "C" int bl_gemm_tc_cols_supported(int M, int N, int K) {
    return M >= 1 && M <= 64 && N >= 1 && K >= 8 && K % 8 == 0 && stages_for(M <= 16 ? 16 : (M <= 32 ? 32 : 64), K) > 0;
}

// bfloat16 x[M, K] (M <= 64) and W[N, K], both 16-byte aligned; out[M, N] float32 or bfloat16; no epilogue.
extern "C" int bl_gemm_tc_cols(const void* x, const void* w, void* out, int out_dtype, int M, int N, int K, void* stream) {
    if (M <= 0) return 0;
    if (!bl_gemm_tc_cols_supported(M, N, K))
        BL_FAIL("bl_gemm_tc_cols: M=%d N=%d K=%d is not built (up to 64 rows, K a multiple of 8, x must fit shared memory beside the ring)", M, N, K);
    if (((uintptr_t)x | (uintptr_t)w) & 15) BL_FAIL("bl_gemm_tc_cols: x and W must be 16-byte aligned");
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == BL_F32)
        return M <= 16 ? launch<16, float>(x, w, out, M, N, K, s)
             : M <= 32 ? launch<32, float>(x, w, out, M, N, K, s) : launch<64, float>(x, w, out, M, N, K, s);
    if (out_dtype == BL_BF16)
        return M <= 16 ? launch<16, __nv_bfloat16>(x, w, out, M, N, K, s)
             : M <= 32 ? launch<32, __nv_bfloat16>(x, w, out, M, N, K, s) : launch<64, __nv_bfloat16>(x, w, out, M, N, K, s);
    BL_FAIL("bl_gemm_tc_cols: unknown output dtype %d", out_dtype);
}

// Reads and clears the status word: 0 when no block has given up on a wait since the last call (1 loader, 2 x,
// 3 issuer, 4 accumulator free, 5 epilogue, 9 shared memory not 1024-byte aligned). Synchronises the device.
extern "C" int bl_gemm_tc_cols_status(int* status) {
    int v = 0, zero = 0;
    BL_CUDA(cudaMemcpyFromSymbol(&v, g_status3, sizeof(int)));
    if (v != 0) BL_CUDA(cudaMemcpyToSymbol(g_status3, &zero, sizeof(int)));
    *status = v;
    return 0;
}
