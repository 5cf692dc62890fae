// Allocation-free entry point of the block-scaled FP8 GEMM.  This entry point has no counterpart in the
// reference project; it exists for callers of this library that are not in a position to allocate
// device memory:
//
//   * code that runs while a stream is being captured into a CUDA graph, or inside a latency-critical serving
//     loop, where cudaMalloc / cudaFree are either illegal or synchronize the whole device;
//   * hosts that hand the library a fixed memory budget (for example a server that has already given all free
//     HBM to KV pages and expert slots) and want a guarantee that a call cannot fail or stall on allocation;
//   * language bindings without an allocator of their own, which can pass only the buffers they already hold.
//
// The split-K scratch (fp32 partial tiles, per-tile arrival counters and the kernel status word) that the regular
// entry point mfq_fp8_gemm() takes from the caller lives here in one file-scope device array of
// MFQ_NOALLOC_SCRATCH_BYTES inside the library.  Every GPU that loads the library reserves that array until the
// process exits.  The caller still passes inputs and outputs.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

// Capacity of the built-in scratch.  A call needs
//   splits * ceil(N/128) * ceil(M/token_tile) * token_tile * 128 * 4  bytes of partial tiles (<= 8 MiB) and
//   ceil(N/128) * ceil(M/token_tile)  counters (<= 4096);
// a larger problem is rejected with MFQ_NOALLOC_TOO_LARGE (use mfq_fp8_gemm with your own buffers, or fewer splits).
#define MFQ_NOALLOC_PARTIAL_BYTES (8u << 20)
#define MFQ_NOALLOC_MAX_TILES 4096
#define MFQ_NOALLOC_SCRATCH_BYTES (MFQ_NOALLOC_PARTIAL_BYTES + MFQ_NOALLOC_MAX_TILES * 4 + 256)

#define MFQ_NOALLOC_OK 0
#define MFQ_NOALLOC_BAD_ARGUMENT (-1)
#define MFQ_NOALLOC_TOO_LARGE (-20)   // the problem does not fit the built-in scratch
#define MFQ_NOALLOC_SETUP_FAILED (-21)  // the device address of the scratch could not be obtained

// out[M, N] (bf16) = (x * x_scale[:, None]) @ (w * blockscale(w_scale))^T (+ residual), same maths and same kernel
// as mfq_fp8_gemm().  x: [M, K] E4M3, w: [N, K] E4M3, w_scale: [ceil(N/128), K/128] fp32, x_scale: [M] fp32,
// K % 128 == 0, token_tile in {16, 32, 64, 128}, splits >= 1 (clamped to K/128).
//
// Allocation: none.  No cudaMalloc, cudaFree or allocating library routine is called, here or in the kernel.
//
// First call on a device: looks up the device address of the scratch array and opts the kernel into its large
// dynamic shared memory (both once per device, with that device current) before launching.  Make that first call
// outside of any stream capture.
//
// Sharing: all calls on a device use the same scratch, which keeps whatever the previous call left there.  The
// counters and the status word are cleared on `stream` at the start of every call; the partial tiles need no
// clearing because every element that is read has been written by the same call.  Two calls that overlap in time
// on one GPU (different streams, or different host threads) race on the scratch and give wrong results: serialize
// them on one stream.
//
// Returns MFQ_NOALLOC_OK when the work has been queued on `stream`, a negative code otherwise (a one-line reason
// is also written to stderr).
int mfq_fp8_gemm_noalloc(const void* w, const float* w_scale, const void* x, const float* x_scale, void* out,
                         const void* residual, int M, int N, int K, int token_tile, int splits, cudaStream_t stream);

// The kernel's waits are bounded; one that runs out (a protocol fault, never expected) leaves a non-zero code in the
// status word inside the scratch instead of hanging, and the output of that call is then incomplete.  This reads the
// word left by the calls queued so far on `stream` of the current device: it waits for `stream`, copies the word to
// *status_out (0 = every call completed normally; 1 producer, 2 tensor-core issuer, 3 epilogue wait ran out) and
// allocates nothing.  The word is cleared at the start of every mfq_fp8_gemm_noalloc call, so read it after the call
// you care about and before the next one.
int mfq_fp8_gemm_noalloc_status(int* status_out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
