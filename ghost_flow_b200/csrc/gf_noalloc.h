// RMSNorm backward for callers that are not allowed to allocate device memory.
//
// This entry point has no counterpart in the reference; it exists only in this library.
//
// Who needs it: code that runs where a device allocation is impossible or forbidden, for example
// a plug-in called from inside another framework's memory plan (the host owns every byte and hands
// out only the input and output buffers), a real-time or serving loop that must never block in the
// allocator, or a C program that links this library without any tensor library to provide workspaces.
// The regular entry point, gf_rmsnorm_bwd, needs the caller to bring a scratch buffer for the
// per-block partial sums of the weight gradient. This variant keeps that scratch inside the library,
// in a fixed device array that is part of the loaded module, so the caller passes inputs and outputs only.
//
// Limits and rules
//  * D (row length) must be a multiple of 8 and at most GF_NOALLOC_MAX_D; T (rows) is unlimited.
//    Larger D is rejected with GFH_TOO_LARGE and a message on stderr; nothing is launched.
//  * x, w, dy, dres and dx must be 16-byte aligned (rows move as 16-byte vectors), rstd 4-byte, dw 2-byte aligned.
//    A call with a null, misaligned or otherwise invalid argument returns GFH_BAD_ARG before it touches the device:
//    nothing is launched and the calling thread's current device is left alone.
//  * The scratch array takes GF_NOALLOC_MAX_PARTS * GF_NOALLOC_MAX_D * 4 bytes (about 4.6 MiB) on every
//    GPU that loads the library, from load until the process exits.
//  * The first call on each device looks up the device address of that array (one runtime query, no
//    allocation). Make that first call outside any stream capture, with the device current.
//  * Every call on a device uses the same array. The kernels overwrite every partial they later read,
//    so no clearing is needed between calls, but the array keeps the last call's partial sums, and two
//    calls that overlap on the GPU (different streams, or different host threads) race on it and give
//    wrong weight gradients. Serialise calls per device.
//  * No cudaMalloc, cudaFree or allocating library routine is called on any path.
#pragma once

#define GF_NOALLOC_MAX_D 8192
#define GF_NOALLOC_MAX_PARTS 148

#ifdef __cplusplus
extern "C" {
#endif

// x, w, dy, dres (may be null), dx, dw: bf16 device pointers; rstd: fp32 [T] from the forward pass.
// dw receives the weight gradient (accumulate != 0 adds to what is already there).
// Returns 0 on success, a negative gf::HostErr code otherwise.
__attribute__((visibility("default"))) int gf_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* dy,
                                                                   const float* rstd, const void* dres, void* dx,
                                                                   void* dw, int T, int D, int accumulate,
                                                                   void* stream);

#ifdef __cplusplus
}
#endif
