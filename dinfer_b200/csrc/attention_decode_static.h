// dinfer_attention_decode_static: the split-key decode attention for callers that cannot allocate.
//
// This entry point has no counterpart in the reference engine (rayze-ai/dinfer); it exists for
// embedders of this library whose code runs where device allocation is off limits: a host process
// that hands this library a fixed memory budget and forbids it to grow, a plug-in that may not touch
// the host application's allocator (torch's caching allocator included), or a latency-critical loop
// in which a cudaMalloc, which may synchronise the whole device, is not acceptable.
//
// The split-key kernel needs scratch: f32 partial sums per (request, head, split) and one arrival
// counter per (request, kv head).  The regular entry point (dinfer_attention_decode) takes that
// scratch from the caller.  This one keeps it in a fixed array inside the library's device image
// (DINFER_DECODE_STATIC_SCRATCH_BYTES, held by every GPU that loads the library until the process
// exits) and therefore calls no cudaMalloc, cudaFree or any allocating routine.
//
// Rules for the caller
//   * Sizes: B*H*splits*(D+2) floats must fit DINFER_DECODE_STATIC_FLOATS and B*Hkv counters must fit
//     DINFER_DECODE_STATIC_COUNTERS; otherwise the call is refused (DINFER_BAD_ARGUMENT, text from
//     dinfer_last_error) and nothing is launched.  Every argument is checked before anything is
//     queued on the stream.
//   * First call on a device: looks the array's device address up (cudaGetSymbolAddress, once per
//     device, with that device current; host threads may race to it, a lock orders them).  Make this
//     first call before any stream capture begins.
//   * All calls share the one array and it keeps what the last call left.  The counters are cleared
//     on the caller's stream before every launch (cudaMemsetAsync, no allocation), the partial sums
//     are fully rewritten before they are read.  Two calls that overlap on the GPU (different
//     streams without ordering) race on the array: order them.
//   * Inputs, outputs and every other argument are exactly those of dinfer_attention_decode.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define DINFER_DECODE_STATIC_SCRATCH_BYTES (8u << 20)                      /* 8 MiB per GPU */
#define DINFER_DECODE_STATIC_COUNTERS 16384                                 /* ints at the array's end */
#define DINFER_DECODE_STATIC_FLOATS ((DINFER_DECODE_STATIC_SCRATCH_BYTES / 4) - DINFER_DECODE_STATIC_COUNTERS)

#ifdef __cplusplus
extern "C" {
#endif
__attribute__((visibility("default")))
int dinfer_attention_decode_static(const void* q, int64_t ldq, void* out, int64_t ldo, const void* cache,
                                   const int* block_table, int max_blocks, const int* cu_seqlens,
                                   const int* seq_lens, int B, int H, int Hkv, int D, int block_size,
                                   float scale, int window, int splits, cudaStream_t stream);
#ifdef __cplusplus
}
#endif
