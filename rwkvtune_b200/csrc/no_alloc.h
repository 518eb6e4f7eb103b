// Allocation-free LayerNorm backward.
//
// This entry point has no counterpart in the reference project.  It exists for callers that
// are not allowed to allocate device memory at the point where they need the kernel: code
// running inside a memory-pool callback or an allocator hook, host callbacks enqueued on a
// stream, real-time inference loops with a frozen memory plan, and embedders that hand this
// library a fixed arena and forbid cudaMalloc / cudaFree (and therefore any torch allocation)
// afterwards.  The ordinary entry point `rwkv_layer_norm_backward` needs a caller-provided
// scratch buffer for per-block partial sums; the variant below keeps that scratch inside the
// library, in one file-scope device array.
//
// Limits and rules:
//   * Scratch capacity is RWKV_NOALLOC_LN_SCRATCH_FLOATS floats (1 MiB).  A call needs
//     ceil(rows / strip) * 2 * C floats; larger requests return RWKV_ERR_TOO_LARGE (3) and launch
//     nothing.  Every GPU that loads the library holds this 1 MiB until the process exits.
//   * The first call on each device looks up the device address of the array (a host-side
//     symbol is not a device pointer) with that device current.  That first call should be made
//     before any stream capture begins.
//   * All calls on a device share the array and it keeps the previous call's contents.  Nothing
//     in it has to start at zero: every slot that is read was written earlier in the same call.
//     Two calls whose kernels overlap on the GPU (different streams, no dependency) race on it;
//     serialise them.
//   * No cudaMalloc, cudaFree or allocating library routine is called on any path.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define RWKV_NOALLOC_LN_SCRATCH_FLOATS (256 * 1024)

// dy, x: bf16 [rows, C]; mean, rstd: fp32 [rows] (saved by the forward); ln_w: fp32 [C].
// Outputs: dx bf16 [rows, C]; dw, db fp32 [C] (sums over all rows).
// `strip` = rows handled per thread block (>= 1).  Returns 0 on success.
int rwkv_layer_norm_backward_noalloc(const void* dy, const void* x, const void* mean, const void* rstd,
                                     const void* ln_w, void* dx, void* dw, void* db, int rows, int C, int strip,
                                     void* stream);

#ifdef __cplusplus
}
#endif
