// Shared helpers of the kernel library: element types, warp and block reductions, the
// status convention of the exported launchers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// Every exported launcher returns 0 on success, a cudaError_t if the launch failed, or one
// of the library's own codes below.  bc_last_error() gives the text.
#define BC_OK 0
#define BC_ERR_ARG 10001       // sizes or pointers the kernel refuses
#define BC_ERR_DRIVER 10002    // a driver entry point could not be had
#define BC_ERR_LIMIT 10003     // larger than a stated maximum

// Tokens held by one page of the key/value cache.
#define BC_PAGE 64

void bc_set_error(const char* fmt, ...);
extern "C" int bc_sm_count();   // streaming multiprocessors of the current device

#define BC_CHECK_ARG(cond, ...)        \
    do {                               \
        if (!(cond)) {                 \
            bc_set_error(__VA_ARGS__); \
            return BC_ERR_ARG;         \
        }                              \
    } while (0)

#define BC_LAUNCH_STATUS()                                            \
    do {                                                              \
        cudaError_t e_ = cudaGetLastError();                          \
        if (e_ != cudaSuccess) {                                      \
            bc_set_error("%s: %s", __func__, cudaGetErrorString(e_)); \
            return (int)e_;                                           \
        }                                                             \
        return BC_OK;                                                 \
    } while (0)

typedef __nv_bfloat16 bf16;

// Programmatic dependent launch: a kernel launched with the attribute may start while its
// predecessor in the stream is still draining.  Everything before pdl_wait() (set-up, and
// loads of weights, which no kernel writes) then overlaps the predecessor's tail; pdl_wait()
// returns once the predecessor has completed and its writes are visible.  Every kernel of
// this library waits before it touches anything another kernel produced or still reads.
// Without the attribute both calls do nothing.
extern int g_bc_pdl;
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <class... KArgs, class... Args>
static inline cudaError_t bc_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_bc_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The same for a grid of thread-block clusters of `cluster` blocks each (the grid must be a
// multiple of it in every dimension): the blocks of a cluster run at the same time and may
// read one another's shared memory.
template <class... KArgs, class... Args>
static inline cudaError_t bc_launch_clustered(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, dim3 cluster,
                                              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster.x;
    attr[0].val.clusterDim.y = cluster.y;
    attr[0].val.clusterDim.z = cluster.z;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_bc_pdl ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <class T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds
// 32 floats of shared memory.  The order of the additions is fixed by the thread layout.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = lane < warps ? scratch[lane] : 0.0f;
    return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = lane < warps ? scratch[lane] : -INFINITY;
    return warp_max(t);
}
