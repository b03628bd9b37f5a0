// Shared helpers of the engine's CUDA sources: storage types, error reporting, warp reductions.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

// Storage type codes of the C interface.
#define BL_F32 0
#define BL_BF16 1

// Epilogues of the matrix products.
#define BL_EPI_NONE 0      // out = acc
#define BL_EPI_BIAS 1      // out = acc + bias[n]
#define BL_EPI_RESIDUAL 2  // out (32-bit, in place) = out + acc
#define BL_EPI_SWIGLU 3    // out[m, n] = silu(acc_gate[m, n]) * acc_up[m, n]; W holds gate rows then up rows

// Which two dimensions of a head a rotary position encoding turns together (src/math.br:128-157, its `neox` argument).
#define BL_PAIRS_HALVES 0        // pair j = (j, j + n_rot / 2)
#define BL_PAIRS_INTERLEAVED 1   // pair j = (2j, 2j + 1)

void bl_set_error(const char* fmt, ...);

#define BL_FAIL(...) do { bl_set_error(__VA_ARGS__); return 1; } while (0)
#define BL_CHECK_LAUNCH(name) do { cudaError_t e_ = cudaGetLastError(); \
    if (e_ != cudaSuccess) BL_FAIL("%s: launch failed: %s", name, cudaGetErrorString(e_)); } while (0)
#define BL_CUDA(call) do { cudaError_t e_ = (call); \
    if (e_ != cudaSuccess) BL_FAIL("%s failed: %s", #call, cudaGetErrorString(e_)); } while (0)

__device__ __forceinline__ float bl_load(const float* p) { return *p; }
__device__ __forceinline__ float bl_load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void bl_store(float* p, float v) { *p = v; }
__device__ __forceinline__ void bl_store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// Reads element i of an array whose storage type is known only at run time (small vectors:
// norm weights, biases; a tensor stored in 32-bit stays 32-bit beside bfloat16 matrices).
__device__ __forceinline__ float bl_load_any(const void* p, int dtype, size_t i) {
    return dtype == BL_F32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}

__device__ __forceinline__ float bl_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float bl_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// x / (1 + exp(-x)), as src/math.br:232-233.
__device__ __forceinline__ float bl_silu(float x) { return x / (1.0f + expf(-x)); }
// The same with the hardware's exp2 and reciprocal units (relative error around 1e-6): for epilogues whose result
// is rounded to bfloat16 (2^-9) anyway and that evaluate it millions of times per step.
__device__ __forceinline__ float bl_silu_fast(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

// Programmatic dependent launch. A kernel launched with bl_launch_dependent() may start while its predecessor
// on the stream is still running; whatever it does before bl_pdl_wait() must touch only data that no earlier
// kernel of the step writes (weights, the step's index arrays). bl_pdl_wait() returns once the predecessor has
// completed and its writes are visible. bl_pdl_trigger() lets the successor be scheduled as soon as every block
// of this kernel has issued it. Both are no-ops in a kernel that was launched the ordinary way.
__device__ __forceinline__ void bl_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void bl_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Asks for the 128-byte line at `p` to be brought into L2 (no register, no wait).
__device__ __forceinline__ void bl_prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" :: "l"(p)); }

// Brings rows [row0, row0 + n_rows) of a row-major matrix with `row_bytes` per row into L2, spread over the
// block's threads. Used before bl_pdl_wait() so that a kernel's weights stream from HBM while its
// predecessor is still running.
__device__ __forceinline__ void bl_prefetch_rows_l2(const void* base, size_t row0, int n_rows, size_t row_bytes,
                                                    size_t rows_total) {
    const int lines_per_row = (int)((row_bytes + 127) / 128);
    for (int i = threadIdx.x; i < n_rows * lines_per_row; i += blockDim.x) {
        const size_t r = row0 + i / lines_per_row;
        if (r < rows_total)
            bl_prefetch_l2(reinterpret_cast<const char*>(base) + r * row_bytes + (size_t)(i % lines_per_row) * 128);
    }
}

bool bl_pdl_enabled();

// The small kernels of a step all ask for the same split of an SM's memory between shared memory and L1.
// Kernels that want different splits cannot share an SM, so a chain of them would drain the SMs at every
// boundary and could never overlap under programmatic dependent launch. Set once per kernel.
template <typename... KArgs>
cudaError_t bl_same_carveout(void (*kernel)(KArgs...)) {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
}

template <typename... KArgs, typename... Args>
cudaError_t bl_launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                Args... args) {
    // one look-up per launch in a small table of kernels that already carry the carveout preference
    static thread_local const void* seen[64];
    static thread_local int n_seen = 0;
    bool known = false;
    for (int i = 0; i < n_seen; ++i) if (seen[i] == (const void*)kernel) { known = true; break; }
    if (!known) {
        cudaError_t e = bl_same_carveout(kernel);
        if (e != cudaSuccess) return e;
        if (n_seen < 64) seen[n_seen++] = (const void*)kernel;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = bl_pdl_enabled() ? 1 : 0;
    cfg.attrs = &attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same for a kernel whose neighbouring blocks form clusters of `cluster_x` (grid.x a multiple of it).
template <typename... KArgs, typename... Args>
cudaError_t bl_launch_dependent_clusters(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                         unsigned cluster_x, Args... args) {
    static thread_local const void* seen[16];
    static thread_local int n_seen = 0;
    bool known = false;
    for (int i = 0; i < n_seen; ++i) if (seen[i] == (const void*)kernel) { known = true; break; }
    if (!known) {
        cudaError_t e = bl_same_carveout(kernel);
        if (e != cudaSuccess) return e;
        if (n_seen < 16) seen[n_seen++] = (const void*)kernel;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = bl_pdl_enabled() ? 1 : 0;
    attrs[1].id = cudaLaunchAttributeClusterDimension;
    attrs[1].val.clusterDim.x = cluster_x; attrs[1].val.clusterDim.y = 1; attrs[1].val.clusterDim.z = 1;
    cfg.attrs = attrs; cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
