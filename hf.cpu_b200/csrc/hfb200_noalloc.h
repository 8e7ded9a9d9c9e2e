/* hfb200_noalloc.h - one entry point that allocates nothing.
 *
 * This has no counterpart in the reference (ebowh/hf.cpu is a CPU program and never meets the question).
 *
 * Who it is for: code that may launch work on a GPU but may not ask the driver for memory.  Typical cases
 * are a plugin that runs inside a host application whose allocator owns all device memory and forbids
 * cudaMalloc from other code, a caller inside a region where allocation would stall or is not permitted
 * (a real-time loop, a signal-safe path), or an embedder that links this library without PyTorch and so has
 * no caching allocator to lend us a workspace.  The regular entry point, hfb_linear_tc, needs the caller
 * to pass a float32 workspace for its split-K partial sums; such callers have none to give.
 *
 * hfb_linear_tc_noalloc computes the same product, out[M,N] (=|+=) a[M,K] . w[N,K]^T (+ bias), for bfloat16
 * a and w on the tensor cores, and keeps the split-K partial sums in a fixed array that is part of the
 * library image: HFB_NOALLOC_SCRATCH_BYTES (8 MiB) of device memory on every GPU that loads the library,
 * held until the process exits.  The caller still owns and passes a, w, bias and out.
 *
 *  - Sizes: the partial sums take splits * M * N floats, where splits is what hfb_linear_tc would choose
 *    (at most one work item per SM, M <= 128 only).  If that exceeds the array the call fails with
 *    HFB_ERANGE and a message naming both numbers; nothing is launched.  Other argument rules are those of
 *    hfb_linear_tc (K a multiple of 8; a, w, out and the bias 16-byte aligned, else HFB_ENOTSUP).
 *  - First call on a device: looks up the array's device address (cudaGetSymbolAddress, with that device
 *    current), asks for the SM count and opts the kernel in to its shared memory; all three are remembered
 *    per device.  Make this first call before any stream capture begins, and from one thread: the per-device
 *    records are filled without a lock, so two threads must not make their first call on the same device at
 *    the same time (later calls only read them).
 *  - It calls no cudaMalloc / cudaFree and no allocating library routine, on any call.  Where the CUDA runtime
 *    loads modules lazily, the first use of the library's kernels is what places its image, this array
 *    included, on the device: the 8 MiB appear then, once, not per call, and the amount of free device memory
 *    is the same before and after every later call.
 *  - Every call uses the same array and finds the previous call's numbers in it.  Nothing in it has to
 *    start at zero: each split overwrites its whole [M, N] slice before the reduction reads it.  For the
 *    same reason two calls whose kernels may run at the same time on one GPU (different streams, or several
 *    host threads) race on the array: keep calls on one stream, or order them yourself.
 *  - As with hfb_linear_tc, the kernel may start while the kernel in front of it on the stream still runs and
 *    reads `w` before it waits for that kernel: `w` must be complete before the kernel in front is launched.
 */
#ifndef HFB200_NOALLOC_H
#define HFB200_NOALLOC_H

#include "hfb200.h"

#ifdef __cplusplus
extern "C" {
#endif

#define HFB_NOALLOC_SCRATCH_BYTES (8u << 20)

int hfb_linear_tc_noalloc(const void *a, const void *w, const void *bias, int bias_dt, void *out, int out_dt,
                          int accumulate, int M, int N, int K, hfb_stream s);

#ifdef __cplusplus
}
#endif
#endif
