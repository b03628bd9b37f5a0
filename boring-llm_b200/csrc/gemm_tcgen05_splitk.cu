// Matrix product for shapes with few output tiles (a few dozen to a few hundred rows of x, or a narrow W) on the
// fifth-generation tensor cores: out[M, N] = epilogue(x[M, K] . W[N, K]^T), bfloat16 operands, 32-bit accumulation.
//
// A product of 512 rows by 896 columns has 28 tiles of 128 x 128: with one block a tile, four fifths of the SMs
// would idle while each busy one walks all of K alone, and the launch lasts as long as that walk whatever M is. Here
// a CLUSTER of up to eight blocks shares one tile of 128 rows x BN columns and cuts K among its blocks: each block
// streams its slice of x and W through a deep TMA ring (no multicast: every block fetches its own tiles) into
// tcgen05.mma with the accumulator in tensor memory, writes its partial tile into its own shared memory, and after a
// cluster barrier every block adds up a band of the tile's rows over all blocks' partial tiles, read through
// distributed shared memory in block order (the sum of an output element is the same whichever block adds it), applies
// the epilogue (bias, residual add into the 32-bit stream, or SwiGLU over a tile whose first BN/2 columns are gate
// rows of W and last BN/2 the matching up rows) and writes its band. The partial sums never touch global memory.
//
// The kernel takes part in programmatic dependent launch: barriers and the first ring of W before the wait, tensor
// memory, x and out after it. Every wait on an mbarrier is bounded: when a bound runs out the block records a code
// in a status word and stops computing, but still meets its cluster at both cluster barriers (they are hardware
// barriers: every block of the cluster arrives), frees its tensor memory and returns; bl_gemm_tc_splitk_status()
// reports it on the host and the launch's results are invalid.
// Role in the reference: the tiled linear kernels for mid-sized sequence counts (TiledLinearKernel,
// src/math_gpu.br:837-1036); formula y = x . W^T (src/math.br:66-82).
#include "tcgen05.cuh"

namespace {

constexpr const char* WHO = "bl_gemm_tc_splitk";

constexpr int BM = 128, BK = 64;
constexpr int A_BYTES = BM * BK * 2;
constexpr int RING_BYTES = 192 * 1024;                   // 8 stages of 24 KB (BN 64) or 6 of 32 KB (BN 128)
constexpr int SMEM_BYTES = RING_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
constexpr int MAX_STAGES = 8;
constexpr int MAX_SPLIT = 8;                             // the portable cluster size
constexpr uint32_t WAIT_LIMIT = 1u << 22;

__device__ int g_status_sk = 0;    // 0 = fine; else the code of the first wait that ran out

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* give_up, int code) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if (*give_up) return false;
    }
    *give_up = 1;
    atomicCAS(&g_status_sk, 0, code);
    return false;
}

__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the address of `local` (an address in this block's shared memory) in the shared memory of block `rank` of the cluster
__device__ __forceinline__ uint32_t peer_smem(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ float4 ld_cluster4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}

template <int EPI, typename TO, int BN>
__global__ void __launch_bounds__(128, 1)
gemm_tc_splitk_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const void* __restrict__ bias, int bias_dtype, TO* __restrict__ out, int M, int N, int K) {
    constexpr bool GLU = EPI == BL_EPI_SWIGLU;
    constexpr int B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES, STAGES = RING_BYTES / STAGE_BYTES;
    constexpr int PITCH = BN + 4;                                              // floats per row of the partial tile
    static_assert(STAGES <= MAX_STAGES && BM * PITCH * 4 <= RING_BYTES, "the partial tile reuses the ring");
    // kind::f16 instruction descriptor: D 32-bit, A and B bfloat16 and K-major, N >> 3 at bit 17, M >> 4 at bit 24
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    extern __shared__ unsigned char smem_raw[];
    if (threadIdx.x == 0) { tma_prefetch_map(&map_a); tma_prefetch_map(&map_b); }
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;              // tiles need 1024-byte alignment
    unsigned char* aligned = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + RING_BYTES;                                   // full[S], empty[S], accum
    volatile int* give_up = reinterpret_cast<volatile int*>(aligned + RING_BYTES + 192);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(aligned + RING_BYTES + 200);
    const uint32_t full0 = bars, empty0 = bars + 8 * MAX_STAGES, accum = bars + 16 * MAX_STAGES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t rank, split;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(split));
    const int n_tile = blockIdx.y, m0 = blockIdx.z * BM;
    const int n0 = n_tile * (GLU ? BN / 2 : BN);                              // first output column of the tile
    const int kblocks = (K + BK - 1) / BK;
    const int kb0 = (int)((long long)rank * kblocks / split), kb1 = (int)((long long)(rank + 1) * kblocks / split);
    const int nkb = kb1 - kb0;                                                 // this block's share of K (the host keeps it >= 1)

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
        if (GLU) {                                                              // BN/2 gate rows, then the BN/2 up rows that match
            tma_load_2d(b_dst, &map_b, full0 + 8 * s, kb * BK, n0);
            tma_load_2d(b_dst + B_BYTES / 2, &map_b, full0 + 8 * s, kb * BK, N + n0);
        } else {
            tma_load_2d(b_dst, &map_b, full0 + 8 * s, kb * BK, n0);
        }
    };
    int early = 0;
    if (warp == 0 && lane == 0) {
        for (; early < STAGES && early < nkb; ++early) {
            mbar_expect_tx(full0 + 8 * early, STAGE_BYTES);
            load_w(early, kb0 + early);
        }
    }
    __syncwarp();
    bl_pdl_wait();                                                              // x, out and the SM's tensor memory belong to the predecessor until here
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(smem_u32((const void*)tmem_slot)), "r"(BN) : "memory");
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
        for (int j = 0; j < nkb; ++j) {
            const int s = j % STAGES;
            if (j >= STAGES && !mbar_wait(empty0 + 8 * s, ((j / STAGES) & 1) ^ 1, give_up, 1)) break;
            if (j >= early) {
                mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                load_w(s, kb0 + j);
            }
            tma_load_2d(base + s * STAGE_BYTES, &map_a, full0 + 8 * s, (kb0 + j) * BK, m0);
            issued = j + 1;
        }
        if (*give_up)                                                           // let our own copies land before the ring is reused
            for (int j = max(0, issued - STAGES); j < issued; ++j)
                mbar_wait(full0 + 8 * (j % STAGES), (j / STAGES) & 1, give_up, 0);
    } else if (warp == 1 && lane == 0) {
        // issuer: four K = 16 MMAs per stage; the accumulator starts from zero at the first of them
        for (int j = 0; j < nkb; ++j) {
            const int s = j % STAGES;
            if (!mbar_wait(full0 + 8 * s, (j / STAGES) & 1, give_up, 2)) break;
            fence_after_sync();
            const uint64_t a_desc = smem_desc(base + s * STAGE_BYTES);
            const uint64_t b_desc = smem_desc(base + s * STAGE_BYTES + A_BYTES);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)                                   // 32 bytes along K inside the swizzled row
                umma_bf16(tmem, a_desc + 2 * k, b_desc + 2 * k, IDESC, (j | k) != 0);
            umma_commit(empty0 + 8 * s);
        }
        umma_commit(accum);
    }
    __syncwarp();
    const bool ready = mbar_wait(accum, 0, give_up, 3);
    fence_after_sync();
    // every copy into the ring has been consumed by an MMA that has completed: the ring is free for the partial tile
    float* part = reinterpret_cast<float*>(aligned);                            // [128][PITCH]
    if (ready && !*give_up) {
        const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
        float* mine = part + (size_t)(warp * 32 + lane) * PITCH;                // thread = row of the tile
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(lane_addr + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 8; ++j)
                *reinterpret_cast<uint4*>(mine + c * 32 + 4 * j) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        }
    }
    fence_before_sync();
    cluster_sync();                                                             // every block's partial tile is written and visible
    {
        // this block's band of the tile's valid rows: sums over the blocks in block order, epilogue, store
        const int rows_valid = min(BM, M - m0);
        const int r0 = (int)((long long)rank * rows_valid / split), r1 = (int)((long long)(rank + 1) * rows_valid / split);
        constexpr int OUT_COLS = GLU ? BN / 2 : BN;
        constexpr int Q = OUT_COLS / 4;                                         // column quads of a row
        const uint32_t part_u32 = smem_u32(part);
        uint32_t peers[MAX_SPLIT];
#pragma unroll
        for (int pr = 0; pr < MAX_SPLIT; ++pr) peers[pr] = peer_smem(part_u32, (uint32_t)pr < split ? (uint32_t)pr : rank);
        const bool vec_ok = (N % 4) == 0;
        for (int it = threadIdx.x; it < (r1 - r0) * Q; it += 128) {
            const int row = r0 + it / Q, c4 = (it % Q) * 4;
            const uint32_t off = (uint32_t)((row * PITCH + c4) * 4);
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f), u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int pr = 0; pr < MAX_SPLIT; ++pr) {
                if ((uint32_t)pr >= split) break;
                const float4 a = ld_cluster4(peers[pr] + off);
                v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
                if (GLU) {
                    const float4 b = ld_cluster4(peers[pr] + off + (BN / 2) * 4);
                    u.x += b.x; u.y += b.y; u.z += b.z; u.w += b.w;
                }
            }
            if (GLU) {
                v.x = bl_silu_fast(v.x) * u.x; v.y = bl_silu_fast(v.y) * u.y;
                v.z = bl_silu_fast(v.z) * u.z; v.w = bl_silu_fast(v.w) * u.w;
            }
            const int m = m0 + row, n = n0 + c4;
            if (n >= N) continue;
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
    }
    cluster_sync();                                                             // no block leaves while another may still read its partial tile
    if (warp == 0) {
        fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(BN) : "memory");
    }
}

int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
    }
    return n;
}

// How many blocks share a tile: the largest cluster (at most eight blocks, at most one per k block) of which the
// device holds as many at once as there are tiles. Clusters live inside one GPC, so fewer of them fit than SMs divided
// by their size; a launch that needs a second round of clusters takes twice as long. 1 when even single blocks need
// several rounds.
template <int EPI, typename TO, int BN>
int choose_split(int tiles, int kblocks) {
    static int active[MAX_SPLIT + 1] = {};                                  // clusters of each size that run at once (0: not asked yet)
    static bool sized = false;
    if (!sized) {                                                               // the query counts the shared memory the launch will ask for
        if (cudaFuncSetAttribute(gemm_tc_splitk_kernel<EPI, TO, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) {
            (void)cudaGetLastError();
            return 1;
        }
        sized = true;
    }
    int best = 1;
    for (int sp = 2; sp <= MAX_SPLIT && sp <= kblocks; ++sp) {
        if (active[sp] == 0) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(sp, sm_count(), 1);
            cfg.blockDim = dim3(128);
            cfg.dynamicSmemBytes = SMEM_BYTES;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = sp; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr; cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_splitk_kernel<EPI, TO, BN>, &cfg) != cudaSuccess || n <= 0) {
                (void)cudaGetLastError();
                n = -1;                                                         // this size cannot be launched here
            }
            active[sp] = n;
        }
        if (active[sp] >= tiles) best = sp;
    }
    return best;
}

template <int EPI, typename TO, int BN>
int launch(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int M, int N, int K, cudaStream_t s) {
    static bool configured = false;
    if (!configured) {
        BL_CUDA(cudaFuncSetAttribute(gemm_tc_splitk_kernel<EPI, TO, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        BL_CUDA(bl_same_carveout(gemm_tc_splitk_kernel<EPI, TO, BN>));
        configured = true;
    }
    const bool glu = EPI == BL_EPI_SWIGLU;
    CUtensorMap a, b;
    if (bl_make_map_bf16(WHO, &a, x, M, K, BM, BK)) return 1;
    if (bl_make_map_bf16(WHO, &b, w, glu ? 2 * N : N, K, glu ? BN / 2 : BN, BK)) return 1;
    const int cols = glu ? BN / 2 : BN;
    const int n_tiles = (N + cols - 1) / cols, m_tiles = (M + BM - 1) / BM, kblocks = (K + BK - 1) / BK;
    if (n_tiles > 65535 || m_tiles > 65535) BL_FAIL("bl_gemm_tc_splitk: %d x %d tiles are more than a launch takes", m_tiles, n_tiles);
    const int split = choose_split<EPI, TO, BN>(n_tiles * m_tiles, kblocks);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(split, n_tiles, m_tiles);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = split; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    // a block waits (griddepcontrol.wait) before it allocates tensor memory or touches x and out, so it may be launched
    // while its predecessor still runs
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = bl_pdl_enabled() ? 1 : 0;
    cfg.attrs = attr; cfg.numAttrs = 2;
    BL_CUDA(cudaLaunchKernelEx(&cfg, gemm_tc_splitk_kernel<EPI, TO, BN>, a, b, bias, bias_dtype, (TO*)out, M, N, K));
    BL_CHECK_LAUNCH("bl_gemm_tc_splitk");
    return 0;
}

template <int BN>
int tiles_of(int M, int N, bool glu) {
    const int cols = glu ? BN / 2 : BN;
    return ((N + cols - 1) / cols) * ((M + BM - 1) / BM);
}

// Tiles of 64 or of 128 columns: whichever keeps more blocks busy in one round (128 on a tie: x is fetched by fewer).
// *blocks gets that number of blocks, *split the blocks per tile.
template <int EPI, typename TO>
int plan(int M, int N, int K, int* blocks, int* split) {
    const bool glu = EPI == BL_EPI_SWIGLU;
    const int kblocks = (K + BK - 1) / BK;
    const int t64 = tiles_of<64>(M, N, glu), t128 = tiles_of<128>(M, N, glu);
    const int s64 = choose_split<EPI, TO, 64>(t64, kblocks), s128 = choose_split<EPI, TO, 128>(t128, kblocks);
    const bool narrow = (long long)t64 * s64 > (long long)t128 * s128 && t64 <= sm_count();
    *blocks = narrow ? t64 * s64 : t128 * s128;
    *split = narrow ? s64 : s128;
    return narrow ? 64 : 128;
}

template <int EPI, typename TO>
int launch_any(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int M, int N, int K, cudaStream_t s) {
    int blocks, split;
    if (plan<EPI, TO>(M, N, K, &blocks, &split) == 64) return launch<EPI, TO, 64>(x, w, bias, bias_dtype, out, M, N, K, s);
    return launch<EPI, TO, 128>(x, w, bias, bias_dtype, out, M, N, K, s);
}

}  // namespace

// How many blocks share each output tile for this product (1: K is not cut, the kernel has nothing over one block a
// tile). More than 1 means that the tiles are few enough for clusters of that size to run all at once.
extern "C" int bl_gemm_tc_splitk_split(int M, int N, int K, int epilogue) {
    if (M <= 0 || N <= 0 || K <= 0) return 1;
    int blocks = 0, split = 1;
    if (epilogue == BL_EPI_SWIGLU) plan<BL_EPI_SWIGLU, __nv_bfloat16>(M, N, K, &blocks, &split);
    else plan<BL_EPI_NONE, float>(M, N, K, &blocks, &split);
    return split;
}

// bfloat16 x[M, K] and W[N, K] (2N rows for BL_EPI_SWIGLU); K a multiple of 8, both 16-byte aligned.
extern "C" int bl_gemm_tc_splitk(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int out_dtype,
                                 int M, int N, int K, int epilogue, void* stream) {
    if (M <= 0) return 0;
    if (N <= 0 || K <= 0) BL_FAIL("bl_gemm_tc_splitk: bad sizes N=%d K=%d", N, K);
    if (K % 8 != 0) BL_FAIL("bl_gemm_tc_splitk: K=%d is not a multiple of 8 (TMA rows must be 16-byte multiples)", K);
    if (((uintptr_t)x | (uintptr_t)w) & 15) BL_FAIL("bl_gemm_tc_splitk: x and W must be 16-byte aligned");
    if (epilogue == BL_EPI_BIAS && (bias == nullptr || (bias_dtype != BL_F32 && bias_dtype != BL_BF16)))
        BL_FAIL("bl_gemm_tc_splitk: bias epilogue needs a float32 or bfloat16 bias");
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == BL_F32) {
        switch (epilogue) {
            case BL_EPI_NONE: return launch_any<BL_EPI_NONE, float>(x, w, bias, bias_dtype, out, M, N, K, s);
            case BL_EPI_BIAS: return launch_any<BL_EPI_BIAS, float>(x, w, bias, bias_dtype, out, M, N, K, s);
            case BL_EPI_RESIDUAL: return launch_any<BL_EPI_RESIDUAL, float>(x, w, bias, bias_dtype, out, M, N, K, s);
            case BL_EPI_SWIGLU: return launch_any<BL_EPI_SWIGLU, float>(x, w, bias, bias_dtype, out, M, N, K, s);
        }
    } else if (out_dtype == BL_BF16) {
        switch (epilogue) {
            case BL_EPI_NONE: return launch_any<BL_EPI_NONE, __nv_bfloat16>(x, w, bias, bias_dtype, out, M, N, K, s);
            case BL_EPI_BIAS: return launch_any<BL_EPI_BIAS, __nv_bfloat16>(x, w, bias, bias_dtype, out, M, N, K, s);
            case BL_EPI_SWIGLU: return launch_any<BL_EPI_SWIGLU, __nv_bfloat16>(x, w, bias, bias_dtype, out, M, N, K, s);
            case BL_EPI_RESIDUAL: BL_FAIL("bl_gemm_tc_splitk: the residual stream is 32-bit; output dtype must be float32");
        }
    } else {
        BL_FAIL("bl_gemm_tc_splitk: unknown output dtype %d", out_dtype);
    }
    BL_FAIL("bl_gemm_tc_splitk: unknown epilogue %d", epilogue);
}

// Reads and clears the status word: 0 when no block has given up on a wait since the last call
// (1 loader, 2 issuer, 3 epilogue). Synchronises the device.
extern "C" int bl_gemm_tc_splitk_status(int* status) {
    int v = 0, zero = 0;
    BL_CUDA(cudaMemcpyFromSymbol(&v, g_status_sk, sizeof(int)));
    if (v != 0) BL_CUDA(cudaMemcpyToSymbol(g_status_sk, &zero, sizeof(int)));
    *status = v;
    return 0;
}
