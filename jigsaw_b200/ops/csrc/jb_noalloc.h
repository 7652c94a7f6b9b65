// Allocation-free entry point of the kernel library.
//
// This entry point has no counterpart in the reference library (which owns no device code
// and no allocator of its own); it exists for callers that are not allowed to allocate
// device memory at the point where they need the result: code running inside a memory pool
// that must not grow, a latency-critical loop that bans cudaMalloc because it synchronises
// the device, or a host application that hands this library a fixed amount of device memory.
//
// jb_conv3x3_c64_wgrad_noalloc computes the same weight / bias gradient as
// jb_conv3x3_c64_wgrad, but the per-CTA partial sums it needs as scratch live in a static
// device array that is part of the library image (JB_NOALLOC_WGRAD_SCRATCH_BYTES bytes on
// every GPU that loads the library, for the life of the process).  The caller passes only
// inputs and outputs.
//
//  * Limits: NB * H * W <= JB_NOALLOC_WGRAD_MAX_PIXELS and W <= 65534; larger problems are
//    refused with return code -5 and a message on stderr.  At most
//    JB_NOALLOC_WGRAD_MAX_CTAS thread blocks run, so big tiles are slower than through the
//    allocating entry point.
//  * The first call on a device looks up the device address of the scratch array (one
//    cudaGetSymbolAddress, no allocation; host threads making that first call at the same
//    time take turns).  Make that first call outside any stream capture.
//  * check_status != 0 reads the status word back and synchronises the stream; on a stream
//    that is being captured the call is refused with -8 before anything is enqueued.
//  * All calls share the one scratch array and it keeps the previous call's contents; the
//    entry point clears the one word that must start at zero (its status word).  Two calls
//    that overlap on the GPU (different streams, no ordering between them) race on the
//    scratch and give wrong results: order them.
//  * Nothing in this path calls cudaMalloc, cudaFree or an allocating library routine.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define JB_NOALLOC_WGRAD_MAX_CTAS 32
/* one block of partial sums (5 x 128 x 64 floats) per thread block: 5 MiB; the source file checks
   this against the kernel's own constant */
#define JB_NOALLOC_WGRAD_SCRATCH_BYTES (JB_NOALLOC_WGRAD_MAX_CTAS * 5 * 128 * 64 * 4)
#define JB_NOALLOC_WGRAD_MAX_PIXELS (4096LL * 4096LL)

// x_padded : [NB][H+2][W+2][64] bf16 input of the layer, halo border filled (or zero)
// gy_padded: [NB][H+2][W+2][64] bf16 gradient of the layer output (interior is read)
// gw       : [64][64][3][3] fp32 out, weight gradient in the torch layout
// gb       : [64] fp32 out, bias gradient (may be null)
// Returns 0 on success; -5 if the problem exceeds the limits; other negative codes if the
// launch could not be set up; 1 if a bounded wait inside the kernel timed out (the outputs
// are then undefined).  The result is ready when `stream` reaches this point; the return
// code 1 is only reported when `check_status` is non-zero, which synchronises the stream.
int jb_conv3x3_c64_wgrad_noalloc(const void* x_padded, const void* gy_padded, float* gw, float* gb, int NB, int H,
                                 int W, int check_status, void* stream);

#ifdef __cplusplus
}
#endif
