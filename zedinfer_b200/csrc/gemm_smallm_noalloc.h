// zi_gemm_smallm_noalloc: the decode-step matrix product of gemm_smallm.cu for callers that must not
// allocate device memory.  It has no counterpart in tianyuxbear/zedinfer; it exists for embedders of this
// library.
//
// Who needs it.  zi_gemm_smallm takes its split-K scratch (partial sums and arrival counters) from the
// caller, and the Python side gets that scratch from torch's allocator.  Some callers cannot do that at the
// moment they need the product: code that runs between cudaStreamBeginCapture and cudaStreamEndCapture
// (cudaMalloc is not permitted while a stream is being captured), hosts that sized every device buffer up
// front and gave the rest of the GPU to a cache pool so that a late cudaMalloc may simply fail, and plug-ins
// that are handed raw pointers and a stream by an engine they do not own and have no allocator to ask.
//
// What it does instead.  The scratch is a file-scope `static __device__ __align__(256)` array inside the
// library (ZI_NOALLOC_SCRATCH_BYTES = 514 KiB; every GPU that loads the library holds it until the process
// exits).  The first call on a device looks the array's device address up with cudaGetSymbolAddress and
// remembers it per device; make that first call outside any stream capture.  The entry point calls no
// cudaMalloc, no cudaFree and no library routine that allocates.
//
// When the array is used.  Narrow outputs with a long K are cut into K ranges, one thread block each.  Where
// the ranges of a column tile can be launched as one thread-block cluster, their sums meet in distributed
// shared memory and the array is only cleared; where such a cluster cannot be launched, or after
// zi_gemm_smallm_noalloc_reduction(1), every range writes its sums to the array, counts itself there, and the
// block that arrives last adds them in range order.  The two ways give the same bits.
//
// Limits.  At most 16 rows of X, K a multiple of 32, operands 16-byte aligned (as zi_gemm_smallm).  A shape
// that is cut into `ksplit` ranges (zi_gemm_smallm_ksplit(N, K, 0) > 1) is refused with an error unless
//     ksplit * 16 * N <= ZI_NOALLOC_PART_FLOATS (131,072)   and   ceil(N / 16) <= ZI_NOALLOC_COUNTER_INTS (512).
// That holds for the down projections of the 1.5B- and 7B-class layers (98,304 and 114,688 floats); N = 4,704
// with K = 4,096 (150,528 floats) is an example of a shape that is refused.  Shapes that are not cut need no
// scratch and are never refused for it.
//
// Sharing.  All calls on a device use the same array, which still holds what the previous call left.  The
// arrival counters are cleared on the stream before every launch; the partial sums are overwritten before
// they are read.  Two calls that may overlap on the GPU (different streams, or graphs replayed
// concurrently) race on the array: keep calls on one device in stream order.
#pragma once
#include <cuda_runtime.h>

#define ZI_NOALLOC_PART_FLOATS 131072               /* partial sums: ksplit * 16 * N floats of a call must fit */
#define ZI_NOALLOC_COUNTER_INTS 512                 /* arrival counters: one per 16 output columns */
#define ZI_NOALLOC_SCRATCH_BYTES (ZI_NOALLOC_PART_FLOATS * 4 + ZI_NOALLOC_COUNTER_INTS * 4)

#ifdef __cplusplus
extern "C" {
#endif
// C[M,N] = X[M,K] . W[N,K]^T (+ bias[N]); bfloat16 operands, c_dtype 0 = float32 / 1 = bfloat16 output; leading
// dimensions in elements.  Returns 0, or non-zero with a message from zi_last_error_gemm_smallm().
int zi_gemm_smallm_noalloc(const void* X, const void* W, const void* bias, void* C, int c_dtype, int M, int N, int K,
                           long long ldx, long long ldw, long long ldc, cudaStream_t stream);
// through_array != 0: the sums of the K ranges always pass through the built-in array (see above); 0: only where a
// cluster cannot be launched (default).  Returns the previous setting.
int zi_gemm_smallm_noalloc_reduction(int through_array);
#ifdef __cplusplus
}
#endif
