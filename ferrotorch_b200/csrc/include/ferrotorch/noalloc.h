// Allocation-free entry points of libft_kernels.so.
//
// This header has no counterpart in the reference framework: the reference allocates a fresh buffer per
// operation (ferrotorch-gpu/src/pool.rs, allocator.rs) and offers no way to run a kernel without touching
// an allocator.
//
// Who needs this: callers that must not, or cannot, allocate device memory where they call the kernel -
// a serving loop that may not risk the implicit device synchronisation of cudaMalloc/cudaFree, a plug-in that
// was handed a fixed set of buffers by its host application, or a process whose device memory pool is owned
// by another runtime. For them the scratch memory that the ordinary launcher takes from the caller lives in a
// fixed `static __device__` array inside the library image instead.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// RMSNorm backward with built-in scratch.
//
//   dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) [+ dres],   dw = sum_rows dy * xhat
//
// x, dy, dx, dres (optional): bf16 [rows, d];  w: bf16 [d];  rstd: f32 [rows] saved by the forward pass;
// dw_bf16 (bf16 [d]) and dw_f32 (f32 [d]) receive dw - either may be null; accumulate != 0 adds to them.
// All pointers are device pointers owned by the caller. The same arithmetic as ft_rmsnorm_bwd, with the
// per-CTA partial sums of dw kept in a 148 x 8192 float array (4.6 MiB) that every GPU loading the library
// holds until the process exits.
//
// Limits and rules:
//  * d must be a multiple of 8 and at most ft_rmsnorm_bwd_noalloc_max_d() (8192); a larger d is rejected
//    with FT_ERR_TOO_LARGE (-4) and a message on stderr, before anything is launched.
//  * The call performs no cudaMalloc, no cudaFree and calls no allocating library routine.
//  * `stream` must be a stream of the device that is current in the calling thread (the built-in array that is used is that device's);
//    a stream of another device is refused with FT_ERR_ARG (-1).
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
//    device current) and caches it; make that first call outside any stream capture.
//  * All calls on a device share the one array. Its contents after a call are that call's partial sums;
//    nothing has to start at zero, because every slot that is read is written first by the same call. Two calls
//    whose kernels overlap on the GPU (different streams, no ordering between them) race on the array and
//    produce wrong dw: order them with events or keep them on one stream.
// Returns 0 on success, a negative FtError code for a refused argument, or a positive CUDA error code.
int ft_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* dy, const float* rstd, const void* dres, void* dx,
                           void* dw_bf16, float* dw_f32, int accumulate, int rows, int d, cudaStream_t stream);

// Largest hidden size the built-in scratch covers.
int ft_rmsnorm_bwd_noalloc_max_d(void);

#ifdef __cplusplus
}
#endif
