// Shared device helpers for the sm_100a kernels of this library.
//
// Activation type T is float (the true 32-bit path) or __nv_bfloat16 (serving).
// rnd<T>(x) rounds a float to T's precision and returns it as float: the identity for
// float, round-to-nearest-even for bfloat16.  The kernels place it exactly where the
// reference rounds (engine/kernels/torch_ref.py:16-29).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define THN_API extern "C" __attribute__((visibility("default")))

enum ThnDtype { THN_F32 = 0, THN_BF16 = 1 };

// Error codes returned by the launchers (0 = ok, 1..999 = cudaError_t of the launch).
enum ThnStatus {
    THN_OK = 0,
    THN_BAD_ARGUMENT = 1001,
    THN_UNSUPPORTED = 1002,
};

// Bits set by kernels in the caller's device error word.
enum ThnDeviceError {
    THN_ERR_TOKEN_RANGE = 1,     // a token id outside [0, vocab)
    THN_ERR_PAGE_UNMAPPED = 2,   // a cache position whose page is not mapped
    THN_ERR_POSITION_RANGE = 4,  // a position beyond the rotary table
    THN_ERR_WAIT_TIMEOUT = 8,    // a bounded wait on a barrier gave up
};

void thn_set_error(const char* fmt, ...);

#define THN_CHECK_ARG(cond, ...)              \
    do {                                      \
        if (!(cond)) {                        \
            thn_set_error(__VA_ARGS__);       \
            return THN_BAD_ARGUMENT;          \
        }                                     \
    } while (0)

#define THN_UNSUPPORTED_IF(cond, ...)         \
    do {                                      \
        if (cond) {                           \
            thn_set_error(__VA_ARGS__);       \
            return THN_UNSUPPORTED;           \
        }                                     \
    } while (0)

static inline int thn_launch_status(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        thn_set_error("%s: launch failed: %s", what, cudaGetErrorString(e));
        return (int)e;
    }
    return THN_OK;
}

// Programmatic dependent launch.  Every kernel of this library says at its start that the
// next kernel in the stream may be scheduled (pdl_launch_dependents), and waits for the
// kernels before it to finish (pdl_wait) before it reads anything they wrote or writes
// anything at all.  What a kernel does between the two must depend on nothing but constant
// data (weights): it runs while the previous kernel is still at work.  Without the launch
// attribute both are no-ops.  Neither is a spin: the wait is the hardware's own.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

extern int g_thn_pdl;   // 1: launch with programmatic stream serialization (elementwise.cu)

template <typename... Params, typename... Args>
inline void thn_launch(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = g_thn_pdl ? 1 : 0;
    cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);   // the caller reads cudaGetLastError
}

// The same with the blocks grouped into thread-block clusters of the given shape.
template <typename... Params, typename... Args>
inline void thn_launch_cluster(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                               dim3 cluster, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = cluster.x;
    attribute[0].val.clusterDim.y = cluster.y;
    attribute[0].val.clusterDim.z = cluster.z;
    attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = g_thn_pdl ? 2 : 1;
    cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);   // the caller reads cudaGetLastError
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T> __device__ __forceinline__ float rnd(float v) { return to_f32<T>(from_f32<T>(v)); }

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

// Sum over a block of up to 1024 threads; every thread gets the result.  The order of
// additions depends only on blockDim, never on the data or the grid.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        const int n_warps = (blockDim.x + 31) >> 5;
        float t = lane < n_warps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Geometry of one cache entry: pages of page_size tokens; inside a page K then V, each
// [n_kv][page_size][head_dim].
struct PagedKV {
    const void* base;      // first byte of this entry's pool
    const int* block_table;  // [max_slots][bt_stride] physical page of (slot, logical page), -1 = unmapped
    int bt_stride;
    int n_kv;
    int page_size;
    int head_dim;
};

__device__ __forceinline__ long long kv_offset(const PagedKV& kv, int page, int which, int kvh, int in_page) {
    return ((((long long)page * 2 + which) * kv.n_kv + kvh) * kv.page_size + in_page) * (long long)kv.head_dim;
}
