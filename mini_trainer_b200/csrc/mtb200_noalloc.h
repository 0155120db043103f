// Allocation-free entry points of libmtb200_cuda.so.
//
// This header has no counterpart in the reference project: the reference is pure Python and
// every buffer it touches comes from PyTorch's allocator.
//
// Who needs this: code that may not allocate device memory at the moment it wants to run one
// of this library's kernels. Examples are a plugin called from inside another framework's
// memory plan (every byte of device memory already handed out, the framework's allocator not
// reachable from C), a real-time or signal-handler-like path where cudaMalloc's implicit
// device synchronisation is not acceptable, and plain C callers that have no tensor library at
// hand to create a workspace. The regular entry points take their workspace from the caller;
// the one below carries its own.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest number of columns mtb200_colsum_noalloc accepts. The built-in workspace is
// 32 x MTB200_COLSUM_NOALLOC_MAX_N floats = 2 MiB of device memory, reserved on every GPU that
// loads the library for as long as the process lives.
#define MTB200_COLSUM_NOALLOC_MAX_N 16384

// out[N] (bf16) = column sums of the row-major bf16 matrix x[T, N] (leading dimension ld, in
// elements). Same result as mtb200_colsum, but the fp32 partial-sum workspace is a fixed array
// inside the library instead of a caller-provided buffer, and the call performs no cudaMalloc,
// cudaFree or any other allocating call.
//
// * N must be even and at most MTB200_COLSUM_NOALLOC_MAX_N; a larger N returns -11 and launches
//   nothing. Other argument errors return -10, a failed workspace lookup -12, a launch error -5.
// * The first call on each device looks up the workspace's device address
//   (cudaGetSymbolAddress, with that device current). Make that first call before starting any
//   stream capture on that device. The address is cached per device for the life of the process;
//   after cudaDeviceReset it is stale, so do not reset a device between calls. Two threads making
//   the first call on a device at once both look the address up and store the same value.
// * All calls on a device share the one workspace. Each call overwrites the part it uses before
//   reading it, so stale contents never leak into a result, but two calls whose kernels overlap on
//   the GPU (different streams) race on it: keep calls on one stream or order them with events.
int mtb200_colsum_noalloc(const void* x, long long ld, void* out, int T, int N, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
