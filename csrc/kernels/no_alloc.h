// Allocation-free entry point of the CUDA library.
//
// This entry point has no counterpart in the reference.  It exists for callers
// that are not allowed to allocate device memory at the moment they need the
// op: code running inside a memory-planned region whose pools are frozen, a
// host application that owns the whole GPU heap and hands out none of it, or a
// step loop that must stay free of allocator calls so its timing and its memory
// high-water mark are reproducible.  The regular entry point
// (`ft_rmsnorm_bwd`) asks its caller for a scratch buffer of
// `ft_rmsnorm_bwd_parts() * H` floats, which the Python binding obtains from
// the framework's caching allocator on every call; the variant below keeps that
// scratch in a fixed array inside the library instead.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest hidden size the built-in scratch array is dimensioned for.  The array
// holds FT_RMSNORM_NOALLOC_PARTS * FT_RMSNORM_NOALLOC_MAX_H floats (9.25 MiB)
// and is resident on every GPU that loads the library, until the process exits.
#define FT_RMSNORM_NOALLOC_MAX_H 8192
#define FT_RMSNORM_NOALLOC_PARTS 296

// Backward of RMSNorm, same math and argument meaning as `ft_rmsnorm_bwd`, minus
// the scratch argument:
//   x, dy, dx : [rows, H]   w, dw : [H]   inv_rms : [rows] (saved by the forward)
//   dt        : 1 = bf16, 2 = fp16
// The caller passes every input and output; the function calls no cudaMalloc,
// cudaFree or any other allocating routine.
//
// Returns 0 on success, -2 if H is not a multiple of 8, -3 if H exceeds
// FT_RMSNORM_NOALLOC_MAX_H (use `ft_rmsnorm_bwd` with your own scratch then),
// -1 for an unsupported dtype, -4 if the current device's index is 64 or more
// (the per-device address table has 64 entries), or a positive CUDA error code.
//
// Set-up: the first call on each device looks up the device address of the
// scratch array (one `cudaGetSymbolAddress` with that device current) and caches
// it.  Make that first call before any CUDA stream capture on the device.  With
// lazy module loading that look-up is also what brings the 9.25 MiB array into
// being on the device, so a caller whose memory is about to be frozen should make
// one warm-up call (any small shape) before it freezes its pools.
//
// Threads: two host threads that make the first call on a device at the same time
// both look the address up and both store the same value, which is harmless; the
// function takes no lock.
//
// Sharing: all calls on one device use the same array, and it keeps whatever the
// previous call left in it.  Each call overwrites every scratch element it later
// reads, so nothing needs clearing between calls, but two calls that may overlap
// on the GPU (different streams without an ordering between them) race on the
// array and must be serialised by the caller.
int ft_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* dy, const float* inv_rms,
                           void* dx, void* dw, int64_t rows, int H, int dt, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
