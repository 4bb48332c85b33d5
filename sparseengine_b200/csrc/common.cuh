// Shared device helpers for the sparseengine_b200 kernels (sm_100a).
//
// Conventions of every exported launcher (extern "C", prefix se_):
//   * pointers are raw device pointers, sizes are explicit integer arguments;
//   * `dtype` selects the activation type: 0 = float32, 1 = bfloat16;
//   * the last argument is the CUDA stream; the return value is a cudaError_t as int
//     (0 = success), or a negative SE_ERR_* code for an argument the kernel refuses.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define SE_ERR_UNSUPPORTED (-2)   // a size this kernel does not take
#define SE_ERR_ARGUMENT (-3)      // an inconsistent argument

#define SE_DTYPE_F32 0
#define SE_DTYPE_BF16 1

#define SE_LAUNCH_CHECK() return (int)cudaGetLastError()

#define SE_DISPATCH_DTYPE(dtype, T, ...)                         \
    if ((dtype) == SE_DTYPE_F32) { using T = float; __VA_ARGS__; } \
    else if ((dtype) == SE_DTYPE_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else return SE_ERR_ARGUMENT;

namespace se {

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Round a 32-bit value to the activation type and return it as 32-bit again.
template <typename T> __device__ __forceinline__ float round_act(float v) { return to_float<T>(from_float<T>(v)); }

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

// Sum over the whole block; every thread gets the result. `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__host__ __device__ __forceinline__ int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Programmatic dependent launch.  A kernel started with `launch_dependent` may begin while the
// kernel before it in the stream still runs, as soon as every block of that kernel has called
// `grid_dependency_trigger` (or has ended).  What it does before `grid_dependency_wait` may
// only read what no kernel of the step writes (weights): the wait returns when the kernel
// before it has ended and its writes can be seen.  A kernel that is launched the ordinary
// way starts after everything before it, so the two calls cost it nothing.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_trigger() {
#ifndef SE_NO_TRIGGER
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}

// SE_NO_PDL=name,name,... launches the named kernels the ordinary way (a tuning aid; names are
// the tags at the launch sites).
static inline bool pdl_enabled(const char* tag) {
    const char* v = ::getenv("SE_NO_PDL");
    return !(v != nullptr && ::strstr(v, tag) != nullptr);
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent_if(bool dependent, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                       cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependent ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
// launch_dependent("tag", kernel, grid, block, smem, stream, args...)
#define SE_LAUNCH_DEPENDENT(tag, ...) \
    ([&] { static const bool on = se::pdl_enabled(tag); return se::launch_dependent_if(on, __VA_ARGS__); }())
// the same, as a dependent only if `cond` holds (else the ordinary way: after everything before it)
#define SE_LAUNCH_DEPENDENT_IF(cond, tag, ...) \
    ([&] { static const bool on = se::pdl_enabled(tag); return se::launch_dependent_if(on && (cond), __VA_ARGS__); }())

// Codes a kernel writes into the library's error word (one int per device, 0 = fine; the
// first failure stays).  1..19: a bounded wait on a barrier ran out (the number names the
// waiting role).  From 20: an index a kernel was given points outside what it may touch; the
// access is skipped and the code names the kernel.
#define SE_CODE_BAD_PAGE_QK_PREP 21
#define SE_CODE_BAD_PAGE_ATTN_PLAIN 22
#define SE_CODE_BAD_PAGE_ATTN_DECODE 23
#define SE_CODE_BAD_PAGE_ATTN_PREFILL 24
#define SE_CODE_BAD_PAGE_ATTN_PREFILL_TC 25
#define SE_CODE_BAD_TABLE_UPDATE 26

// True if block-table entry `page` names a page of a pool of `num_pages`; otherwise the code
// goes to the error word (if there is one) and the caller leaves the page alone.
__device__ __forceinline__ bool page_in_pool(int page, int num_pages, int* error, int code) {
    if ((unsigned)page < (unsigned)num_pages) return true;
    if (error != nullptr) atomicCAS(error, 0, code);
    return false;
}

// Eight consecutive elements as 32-bit values, with 16-byte loads; `p` must be 16-byte
// aligned (float32 takes two such loads).
__device__ __forceinline__ void load8(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* v) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void store8(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float* v) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
}
template <typename T> __device__ __forceinline__ bool aligned8(const T* p) {
    return (reinterpret_cast<uintptr_t>(p) & 15) == 0;
}

}  // namespace se
