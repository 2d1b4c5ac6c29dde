// Shared helpers for the sm_100a kernels: dtype codes, conversions, 16-byte loads,
// block reductions with a fixed order, and the error channel of the C entry points.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define ZI_EXPORT extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python side (zedinfer_b200/ops/_lib.py)
#define ZI_F32 0
#define ZI_BF16 1

typedef __nv_bfloat16 bf16;

// ---- error channel -------------------------------------------------------------------
// Every entry point returns 0 on success.  On failure it returns non-zero and leaves a
// message that zi_last_error() of the same library returns.
static thread_local char zi_error_buf[512];

static inline int zi_fail(const char* fmt, ...) __attribute__((format(printf, 1, 2)));
#include <stdarg.h>
static inline int zi_fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(zi_error_buf, sizeof(zi_error_buf), fmt, ap);
    va_end(ap);
    return 1;
}

static inline int zi_check_launch(const char* what) {
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        cudaGetLastError();
        return zi_fail("%s: launch failed: %s", what, cudaGetErrorString(e));
    }
    return 0;
}

#define ZI_DEFINE_LAST_ERROR(libname)                                            \
    ZI_EXPORT const char* zi_last_error_##libname() { return zi_error_buf; }

// ---- conversions ----------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// Load 8 consecutive elements (16-byte aligned for bf16, 32-byte for float) as floats.
__device__ __forceinline__ void load8(const float* p, float* out) {
    float4 a = *reinterpret_cast<const float4*>(p);
    float4 b = *reinterpret_cast<const float4*>(p + 4);
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
    out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, float* out) {
    uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 f = __bfloat1622float2(h[i]);
        out[2 * i] = f.x;
        out[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void store8(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(bf16* p, const float* v) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
}

// ---- reductions with a fixed order -----------------------------------------------------
// The order of additions depends only on the block size, never on the data or the grid,
// so a row's result is the same whatever else is in the batch.
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
// Block sum; `scratch` holds at least 32 floats of shared memory.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : 0.0f;
    r = warp_sum(r);
    return r;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}

// ---- programmatic dependent launch -------------------------------------------------------
// Kernels of a step run back to back on one stream, each reading what the one before wrote.
// Launched with zi_launch they may start while their predecessor is still draining: everything a
// kernel does before pdl_wait() (index arithmetic, loads of weights, which no kernel of the step
// writes) overlaps with the predecessor's tail; pdl_wait() returns once the predecessor has
// finished and its writes are visible.  Every kernel launched this way calls pdl_wait() before it
// touches anything another kernel of the step produces or still reads, and pdl_launch_dependents()
// to let its own successor be scheduled early.
//
// Measured on the 1.5B decode step the overlap bought about 3 % while costing the cached read path for
// activations, so it is compiled out unless ZI_PDL=1 is defined: pdl_wait / pdl_trigger_* are then empty,
// ld_dep is an ordinary load and zi_launch sets no attribute.
#ifndef ZI_PDL
#define ZI_PDL 0
#endif
__device__ __forceinline__ void pdl_wait() {
#if ZI_PDL
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
#endif
}
__device__ __forceinline__ void pdl_launch_dependents() {
#if ZI_PDL
    asm volatile("griddepcontrol.launch_dependents;\n" ::);
#endif
}
// Where a kernel lets its successor be scheduled: at its start (ZI_PDL_TRIGGER=0), once its main loads are
// issued (1, the default), or never before it ends (2).
#ifndef ZI_PDL_TRIGGER
#define ZI_PDL_TRIGGER 1
#endif
__device__ __forceinline__ void pdl_trigger_early() { if (ZI_PDL_TRIGGER == 0) pdl_launch_dependents(); }
__device__ __forceinline__ void pdl_trigger_late() { if (ZI_PDL_TRIGGER == 1) pdl_launch_dependents(); }

// Data that the predecessor wrote must be read with coherent loads after pdl_wait(): a load through the
// read-only (non-coherent) path, which the compiler picks for `const __restrict__` pointers, may return what
// the cache held before the predecessor's write, because this kernel was launched before that write.
// ld_dep() loads through L2 only.
#if ZI_PDL
__device__ __forceinline__ float ld_dep(const float* p) { return __ldcg(p); }
__device__ __forceinline__ int ld_dep(const int* p) { return __ldcg(p); }
__device__ __forceinline__ bf16 ld_dep(const bf16* p) {
    return __ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short*>(p)));
}
__device__ __forceinline__ uint4 ld_dep16(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
#else
__device__ __forceinline__ float ld_dep(const float* p) { return *p; }
__device__ __forceinline__ int ld_dep(const int* p) { return *p; }
__device__ __forceinline__ bf16 ld_dep(const bf16* p) { return *p; }
__device__ __forceinline__ uint4 ld_dep16(const void* p) { return *reinterpret_cast<const uint4*>(p); }
#endif
// Data written by other blocks of the *same* kernel (split sums, chunk partials) is always read through L2.
__device__ __forceinline__ float ld_l2(const float* p) { return __ldcg(p); }
template <typename T> __device__ __forceinline__ float ld_dep_f32(const T* p) { return to_f32<T>(ld_dep(p)); }

// ZEDINFER_NO_PDL=1 launches the same kernels without the attribute (plain stream order); griddepcontrol
// instructions are then no-ops.
#ifndef ZI_PDL_BIT
#define ZI_PDL_BIT 1
#endif
static inline bool zi_pdl_enabled() {
    static int enabled = -1;
    if (enabled < 0) {
        const char* e = getenv("ZEDINFER_NO_PDL");
        enabled = (e && e[0] == '1') ? 0 : 1;
        const char* m = getenv("ZEDINFER_PDL_MASK");          // experiments: bit per library
        if (enabled && m) enabled = (atoi(m) & ZI_PDL_BIT) ? 1 : 0;
    }
    return enabled == 1;
}

template <typename... KArgs, typename... Args>
static inline cudaError_t zi_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args&&... args) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (ZI_PDL && zi_pdl_enabled()) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Dispatch a dtype code to a type.  Usage: ZI_DISPATCH(code, T, { kernel<T><<<...>>>(...); })
#define ZI_DISPATCH(code, T, ...)                        \
    do {                                                 \
        if ((code) == ZI_F32) { typedef float T; __VA_ARGS__ }        \
        else if ((code) == ZI_BF16) { typedef bf16 T; __VA_ARGS__ }   \
        else return zi_fail("unknown dtype code %d", (int)(code));    \
    } while (0)
