// Entry point for callers that are not allowed to allocate device memory.
//
// This has no counterpart in the reference implementation; it is an addition of this library.
//
// Who needs it: code that runs where cudaMalloc is off limits -- inside a latency-critical serving
// loop whose memory budget was fixed at start-up, under a host framework that owns the whole device
// heap, or in a plug-in that is only handed input and output buffers.  The regular sampler
// (smc_sample_or_score) wants a caller-provided scratch buffer for its per-chunk partial results;
// such callers have nowhere to get one from.
//
// smc_sample_or_score_static() is the same fused Gumbel-max sampler / log-probability scorer, but its
// scratch lives in a fixed array inside the library (SMC_STATIC_SAMPLE_MAX_ROWS rows, 256 KiB of
// device memory held by every GPU that loads the library, until the process exits).
//
//  * Limit: rows <= SMC_STATIC_SAMPLE_MAX_ROWS.  Larger requests are refused with
//    SMC_STATIC_ERR_TOO_LARGE and a message in smc_no_alloc_last_error(); nothing is launched.
//  * The first call on each device looks up the device address of the scratch array (one
//    cudaGetSymbolAddress call, with that device current).  Make that first call outside any CUDA
//    stream capture.
//  * It never calls cudaMalloc, cudaFree or any allocating library routine.
//  * All calls share the one array and it keeps whatever the last call left in it.  The sampler
//    overwrites every entry it later reads, so nothing needs clearing between calls -- but two calls
//    that may run at the same time on the GPU (different streams, no dependency) race on it.
//    Serialise them.
//  * Inputs and outputs are passed exactly as for smc_sample_or_score.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SMC_STATIC_SAMPLE_MAX_ROWS 256
#define SMC_STATIC_ERR_TOO_LARGE (-90)
#define SMC_STATIC_ERR_SETUP (-91)
#define SMC_STATIC_ERR_ARG (-92)

// logits: fp32 [splits, rows (pitch row_stride), V]; tokens_in: per row, >= 0 scores that token, < 0 samples
// (null = sample every row); outputs tok_out / logp_out / logz_out: [rows] (logz_out may be null).
// Returns 0 on success, a negative SMC_STATIC_ERR_* code when refused, or a positive cudaError_t.
int smc_sample_or_score_static(const float* logits, int splits, long long split_stride, long long row_stride, int rows,
                               int V, float temperature, float alpha, float softcap, const int* tokens_in,
                               unsigned long long seed, const long long* cycle_counter, int call_id, int* tok_out,
                               float* logp_out, float* logz_out, cudaStream_t stream);

// Human-readable reason for the last refusal on this thread ("" if none).
const char* smc_no_alloc_last_error(void);

#ifdef __cplusplus
}
#endif
