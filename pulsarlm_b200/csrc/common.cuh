// Shared declarations of the kernel library: dtype codes, error reporting, loads
// and stores that go through fp32, and block reductions.
//
// Every entry point is `extern "C" int pl_<name>(..., cudaStream_t stream)`, takes
// raw device pointers, launches on `stream`, never synchronises and never
// allocates. It returns 0, or a non-zero code after storing a message that
// `pl_last_error()` returns (sizes it refuses, a failed launch).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#define PL_API extern "C" __attribute__((visibility("default")))

enum pl_dtype : int { PL_F32 = 0, PL_BF16 = 1 };

// Stores a printf-style message for pl_last_error() and returns `code`.
int pl_fail(int code, const char* format, ...);

#define PL_REQUIRE(cond, ...)                     \
    do {                                          \
        if (!(cond)) {                            \
            return pl_fail(2, __VA_ARGS__);       \
        }                                         \
    } while (0)

#define PL_CHECK_LAUNCH(name)                                                         \
    do {                                                                              \
        cudaError_t pl_err_ = cudaGetLastError();                                     \
        if (pl_err_ != cudaSuccess) {                                                 \
            return pl_fail(3, "%s: launch failed: %s", name, cudaGetErrorString(pl_err_)); \
        }                                                                             \
    } while (0)

// Overlap of consecutive kernels in a stream (programmatic dependent launch).
//
// A kernel launched through pl_launch_overlapped may become resident while its
// predecessor in the stream still runs. It calls pl_grid_trigger() at its top (its
// own successor may then be made resident as soon as all of this grid's CTAs are)
// and pl_grid_wait() before it first reads or writes anything that another kernel
// writes or reads: the wait returns when every earlier kernel of the stream has
// finished and its writes are visible. What a kernel does before the wait (barrier
// set-up, tensor-memory allocation, loads of weights, which no kernel writes)
// overlaps the predecessor's tail. Every kernel launched this way executes the wait
// in every thread that touches global memory, so completion stays in stream order.
// Without the launch attribute both calls do nothing.
__device__ __forceinline__ void pl_grid_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pl_grid_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// 1 unless pl_set_overlap(0) was called.
int pl_overlap_enabled();

template <typename... Params, typename... Args>
cudaError_t pl_launch_overlapped(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = pl_overlap_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

// Dispatch on a dtype code: binds `scalar_t` to float or __nv_bfloat16.
#define PL_DISPATCH_DTYPE(code, name, ...)                                  \
    do {                                                                    \
        if ((code) == PL_F32) {                                             \
            using scalar_t = float;                                         \
            __VA_ARGS__                                                     \
        } else if ((code) == PL_BF16) {                                     \
            using scalar_t = __nv_bfloat16;                                 \
            __VA_ARGS__                                                     \
        } else {                                                            \
            return pl_fail(2, "%s: unknown dtype code %d", name, (code));   \
        }                                                                   \
    } while (0)

__device__ __forceinline__ float pl_load(const float* p) { return *p; }
__device__ __forceinline__ float pl_load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void pl_store(float* p, float v) { *p = v; }
__device__ __forceinline__ void pl_store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// Four elements at a time.
struct alignas(8) bf16x4 {
    __nv_bfloat162 lo, hi;
};
__device__ __forceinline__ float4 pl_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 pl_load4(const __nv_bfloat16* p) {
    const bf16x4 v = *reinterpret_cast<const bf16x4*>(p);
    const float2 a = __bfloat1622float2(v.lo), b = __bfloat1622float2(v.hi);
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void pl_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void pl_store4(__nv_bfloat16* p, float4 v) {
    bf16x4 o;
    o.lo = __floats2bfloat162_rn(v.x, v.y);
    o.hi = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<bf16x4*>(p) = o;
}

__device__ __forceinline__ float pl_warp_sum(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        v += __shfl_xor_sync(0xffffffffu, v, offset);
    }
    return v;
}

__device__ __forceinline__ float pl_warp_max(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
    }
    return v;
}

// Sum over a block of up to 1024 threads; `scratch` holds 32 floats. Every thread
// gets the result. The order of additions is fixed by the block size alone.
__device__ __forceinline__ float pl_block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = pl_warp_sum(v);
    __syncthreads();
    if (lane == 0) {
        scratch[warp] = v;
    }
    __syncthreads();
    const int warps = (blockDim.x + 31) >> 5;
    float total = lane < warps ? scratch[lane] : 0.0f;
    return pl_warp_sum(total);
}

__device__ __forceinline__ float pl_block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = pl_warp_max(v);
    __syncthreads();
    if (lane == 0) {
        scratch[warp] = v;
    }
    __syncthreads();
    const int warps = (blockDim.x + 31) >> 5;
    float total = lane < warps ? scratch[lane] : -INFINITY;
    return pl_warp_max(total);
}
