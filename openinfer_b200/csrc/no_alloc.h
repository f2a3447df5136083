// Entry point for callers that cannot allocate device memory.
//
// This has no counterpart in the reference engine: there every kernel's scratch comes from the
// process's own allocator (pegainfer-sample/src/lib.rs:58-121 sizes a SampleScratch up front).
//
// Who needs it. A host program may give all free device memory to one pool of its own at start-up
// (a KV-cache pool does exactly that), after which cudaMalloc simply fails; a serving loop may
// forbid allocation on its hot path because cudaMalloc and cudaFree synchronise the whole device;
// and a caller that reaches this library through the plain C ABI from another language has no
// torch allocator to lend us. For them the two-stage argmax is offered with its scratch inside the
// library image: a file-scope device array that every GPU loading the library carries until the
// process exits.
//
// Limits (checked; larger calls are refused with OI_ERR_TOO_LARGE and a message):
//   rows * ceil(vocab / 4096) <= OI_ARGMAX_NOALLOC_MAX_PARTIALS (16384 partial results, 128 KiB
//   of device memory in all, e.g. 256 rows of a 262144-entry vocabulary).
//
// Contract.
//   * The caller passes input and output; nothing is allocated or freed, here or in any library
//     routine called from here.
//   * The first call on a device looks the array's device address up (cudaGetSymbolAddress, with
//     that device current) and remembers it per device. Make that first call outside any stream
//     capture.
//   * All calls share the one array. It keeps what the last call left; this kernel pair overwrites
//     every partial result it later reads, so nothing has to be cleared between calls. Two calls
//     that overlap on the GPU (different streams, no ordering between them) race on the array and
//     may both return wrong indices: order them.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define OI_ARGMAX_NOALLOC_MAX_PARTIALS 16384

// out[r] = index of the largest of logits[r, 0..vocab) (lowest index on ties), r < rows.
// logits: float32, row r at logits + r * row_stride. stream: a cudaStream_t (may be null).
// Returns 0, or an error code; oi_last_error() gives the message.
int oi_argmax_noalloc(int* out, const float* logits, int rows, int vocab, long long row_stride, void* stream);

#ifdef __cplusplus
}
#endif
