// Entry point for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project: it exists for embedders of this
// library who run where cudaMalloc is off limits: inside a host process that has handed the whole
// device heap to its own pool, in a real-time loop where an allocation may stall on the driver,
// or after start-up in a service whose memory budget is fixed and audited. Such callers still own
// their inputs and outputs; what they cannot provide is the sampling kernel's work area
// (rows x vocabulary floats for the probabilities). Here that work area is a fixed array inside
// the library's own device image.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// The most floats (rows * vocab) one call may need: 2 Mi floats = 8 MiB, held on every GPU that
// loads the library until the process exits. At a vocabulary of 128,256 that is 16 rows a call.
#define GI_SAMPLE_NO_ALLOC_MAX_FLOATS (2 * 1024 * 1024)

// Same result as gi_sample (one token id per row of logits [rows, vocab] under temperature,
// top-k and top-p, with the caller's uniform number per row), but without a scratch argument.
//   * A row whose temperature is <= 0 (greedy) is left alone: out[row] keeps the value the caller
//     put there. As with gi_sample, write the row's argmax into out (gi_argmax) before this call if
//     greedy rows are mixed with sampled ones; a row that is never written is not a token id.
//   * Allocates nothing: no cudaMalloc, cudaFree or allocating library call, on any call.
//   * The first call on a device looks up the device address of the built-in work area (with that
//     device current) and remembers it; make that first call before any stream capture begins.
//     The address is remembered for the life of the process: after cudaDeviceReset() it is stale,
//     so a process that resets the device must not call this entry point afterwards.
//   * rows * vocab above GI_SAMPLE_NO_ALLOC_MAX_FLOATS is refused with an error (non-zero return,
//     message from gi_last_error()), never truncated.
//   * All calls on a device share the one work area, which keeps what the last call left there.
//     Nothing in it has to start at zero (every probability is written before it is read), but two
//     calls whose kernels overlap on the GPU (different streams, no ordering) race on it: order them.
int gi_sample_no_alloc(const float* logits, int rows, int vocab, const float* temperature, const int* top_k,
                       const float* top_p, const float* uniform, int* out, void* stream);

#ifdef __cplusplus
}
#endif
