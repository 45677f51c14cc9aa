// Column reduction without any allocation.  This entry point has no counterpart in the reference
// project; it exists for callers of this library that are not allowed to allocate device memory.
//
// Who that is: code that runs where cudaMalloc is forbidden or unavailable - a host thread inside
// a real-time or signal-like context, a plug-in loaded into a process whose memory pool is owned
// and sized by someone else (an inference server with a fixed arena), or a caller that hands
// this library raw pointers and must be sure no hidden allocation can fail or fragment its pool
// in the middle of a step.  The ordinary entry point, dmb_col_reduce_acc, needs the caller to
// bring `nsplit * d` floats of scratch; this one brings its own.
//
// What it computes is the same:  out[col] += sum over rows of dy[row][col] * x[row][col] * rstd[row]
// (x == NULL: the plain column sum of dy).  The caller still passes every input and the output.
//
// The scratch is a fixed array of DMB_NOALLOC_MAX_SPLIT * DMB_NOALLOC_MAX_COLS floats (2 MiB) that
// is part of the library image: every GPU that loads the library holds it until the process exits.
// Limits and rules:
//   * at most DMB_NOALLOC_MAX_COLS columns; a wider input is refused with DMB_NOALLOC_E_SIZE and a
//     message from dmb_noalloc_last_error().  Any number of rows >= 1.
//   * the first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//     that device current).  Make that first call outside of any stream capture.
//   * the function itself calls no cudaMalloc, cudaFree or other allocating routine.
//   * all calls on one GPU share the one array.  It keeps whatever the last call left in it; that
//     is harmless, because each call overwrites every entry it later reads.  Two calls that can
//     run at the same time on one GPU (different streams, different host threads) race on it: keep
//     calls on a device ordered, e.g. on one stream.
#pragma once
#include <cuda_runtime.h>

#define DMB_NOALLOC_MAX_SPLIT 64
#define DMB_NOALLOC_MAX_COLS 8192
#define DMB_NOALLOC_MAX_DEVICES 64
#define DMB_NOALLOC_E_SIZE (-3)
#define DMB_NOALLOC_E_DEVICE (-4)

#ifdef __cplusplus
extern "C" {
#endif

// dy: [rows, d] bf16 (dy_f32 = 0) or fp32 (dy_f32 = 1), row-contiguous; x: [rows, *] bf16 with row
// stride xs elements, or NULL; rstd: [rows] fp32 (ignored when x is NULL); out: [d] fp32,
// accumulated into.  Returns 0, a negative DMB_NOALLOC_E_* code, or a positive CUDA error code.
int dmb_col_reduce_acc_noalloc(const void* dy, int dy_f32, const void* x, long long xs, const float* rstd,
                               float* out, int rows, int d, cudaStream_t st);

// Text of the calling host thread's last refusal by dmb_col_reduce_acc_noalloc ("" if its last call was
// accepted).  The buffer is per host thread; the pointer stays valid for that thread's lifetime.
const char* dmb_noalloc_last_error();

// The ordinary entry point, with caller-provided scratch of nsplit * d floats.
int dmb_col_reduce_acc(const void* dy, int dy_f32, const void* x, long long xs, const float* rstd,
                       float* partial, int nsplit, float* out, int rows, int d, cudaStream_t st);

#ifdef __cplusplus
}
#endif
