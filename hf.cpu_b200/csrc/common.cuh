// Shared helpers of the CUDA sources: element types, loads/stores in float, status reporting.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "hfb200.h"

#define HFB_TRACE_CAP 32768ull

namespace hfb {

// Records the message `hfb_last_error()` returns; returns `code` so callers can `return fail(...)`.
int fail(int code, const char *fmt, ...);

inline int check_launch(const char *what)
{
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(HFB_ECUDA, "%s: %s", what, cudaGetErrorString(e));
    return HFB_OK;
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Load element i of an array whose element type is only known at run time (HFB_F32 / HFB_BF16).
__device__ __forceinline__ float load_any(const void *p, int dt, size_t i)
{
    return dt == HFB_F32 ? ((const float *)p)[i] : __bfloat162float(((const __nv_bfloat16 *)p)[i]);
}

__device__ __forceinline__ void store_any(void *p, int dt, size_t i, float v)
{
    if (dt == HFB_F32) ((float *)p)[i] = v;
    else ((__nv_bfloat16 *)p)[i] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Programmatic dependent launch.  Every kernel of the forward pass is launched so that it may start while the
// kernel before it is still running; it does what needs none of that kernel's results (set-up, and in the
// products the first loads of the weights), then waits for the predecessor to finish, then lets its own
// successor start, so that one kernel runs ahead (two behind a short kernel: see pdl_entry below).
//
// A build with -DHFB_TRACE (developers only) logs, from thread 0 of block 0 of each kernel, the time the block
// started and the time its wait for the predecessor returned; `hfb_trace_take` reads the log.
#ifdef HFB_TRACE
static __device__ unsigned long long *g_trace_ptr = nullptr;          // [0] = count, then (id << 8 | kind, time) pairs
__device__ __forceinline__ void trace_log(int id, int kind)
{
    unsigned long long *log = g_trace_ptr;
    if (log && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        unsigned long long i = atomicAdd(log, 1ull);
        if (i < HFB_TRACE_CAP) { log[2 + 2 * i] = ((unsigned long long)id << 8) | (unsigned)kind; log[3 + 2 * i] = t; }
    }
}
// (developers) a value of the caller's instead of the time, from thread 0 of block 0
__device__ __forceinline__ void trace_put(int kind, unsigned long long value)
{
    unsigned long long *log = g_trace_ptr;
    if (log && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
        unsigned long long i = atomicAdd(log, 1ull);
        if (i < HFB_TRACE_CAP) { log[2 + 2 * i] = (unsigned)kind; log[3 + 2 * i] = value; }
    }
}
// (developers) the time, from thread 0 of whichever block calls it
__device__ __forceinline__ void trace_any(int kind)
{
    unsigned long long *log = g_trace_ptr;
    if (log && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        unsigned long long i = atomicAdd(log, 1ull);
        if (i < HFB_TRACE_CAP) { log[2 + 2 * i] = (unsigned)kind; log[3 + 2 * i] = t; }
    }
}
// (developers) "ready" from the calling thread of block 0, for kernels whose thread 0 does not wait for the predecessor
__device__ __forceinline__ void trace_ready_here()
{
    unsigned long long *log = g_trace_ptr;
    if (log && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        unsigned long long i = atomicAdd(log, 1ull);
        if (i < HFB_TRACE_CAP) { log[2 + 2 * i] = 1ull; log[3 + 2 * i] = t; }
    }
}
void trace_register(void (*setter)(void *));
static void trace_set_ptr(void *p) { cudaMemcpyToSymbol(g_trace_ptr, &p, sizeof p); }
namespace { struct TraceRegistration { TraceRegistration() { trace_register(trace_set_ptr); } } g_trace_registration; }
#define HFB_TRACE_ENTRY(id) trace_log(id, 0)
#define HFB_TRACE_READY() trace_log(0, 1)
#define HFB_TRACE_MARK(k) trace_log(0, k)
#define HFB_TRACE_ANY(k) trace_any(k)
#define HFB_TRACE_READY_HERE() trace_ready_here()
#else
#define HFB_TRACE_READY_HERE()
#define HFB_TRACE_ANY(k)
#define HFB_TRACE_ENTRY(id)
#define HFB_TRACE_READY()
#define HFB_TRACE_MARK(k)
#endif
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); HFB_TRACE_READY(); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_sync() { pdl_wait(); pdl_trigger(); }
// The short kernels between the products (norms, sums of split-K partials, rotation, embedding, arg-max) release their
// successor when they start, not when their own wait returns: the product behind a short kernel is then resident a
// few microseconds earlier and its weight tiles are on their way while the short kernel still waits and works (a
// successor's blocks are placed only when all of this kernel's have started, so they never take their place; what a
// kernel does before its wait depends on nothing the kernels in front write).  Batch 8: 3.098 -> 3.055 ms a step.  The
// products and the attention kernels release at their wait: released at entry too, the step was slower.
__device__ __forceinline__ void pdl_entry() { pdl_trigger(); }
__device__ __forceinline__ void pdl_sync_small() { pdl_wait(); }

// One rotation pair (src/model.c:587-601): products and sums each rounded to float32 on their own, so that every kernel
// that rotates gives the same bits (the compiler is free to contract a * c - b * s into a fused multiply-add in one
// place and not in another).
__device__ __forceinline__ void rope_pair(float a, float b, float c, float s, float &lo, float &hi)
{
    lo = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
    hi = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
}

// Index of the current device (0 where it cannot be told), for what is remembered per device.
inline int current_device()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    return dev;
}

bool pdl_enabled();          // HFB_PDL != 0

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline int check_pdl_launch(cudaError_t e, const char *what)
{
    if (e != cudaSuccess) return fail(HFB_ECUDA, "%s: %s", what, cudaGetErrorString(e));
    return check_launch(what);
}

inline bool valid_dt(int dt) { return dt == HFB_F32 || dt == HFB_BF16; }

}  // namespace hfb
