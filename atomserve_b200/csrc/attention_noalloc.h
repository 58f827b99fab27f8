// Paged attention with split keys for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference engine (aneesh-sathe/atomserve): there
// every kernel wrapper allocates its partial results with the framework's allocator
// (atomserve/kernels.py:667-676). It exists for hosts that embed these kernels through the C
// ABI and must not, or cannot, call cudaMalloc around them: a serving process that handed the
// whole GPU to its own weight and cache pools at start-up and treats any later allocation as
// a fault; a latency-bound loop for which cudaMalloc's implicit device synchronisation is too
// dear; a foreign runtime that passes raw pointers and a stream and has no allocator to lend.
//
//   int asb_paged_attention_static_scratch(... same arguments as asb_paged_attention,
//                                           without the three scratch pointers ...)
//
// Same computation and bit-for-bit the same results as asb_paged_attention (attention_simt.cu): the general
// paged grouped-query attention kernel with the keys cut into NP partitions and a reduction
// that merges them. The difference is only where the partial results (max, sum, accumulator
// per token, head and partition) live: in a fixed array inside the library instead of buffers
// from the caller. The caller still passes q, the caches, the tables and the output.
//
// Limits and rules
//   * The array holds ASB_STATIC_SCRATCH_FLOATS float32 values (4 Mi = 16 MiB). Every GPU
//     that loads the library holds those 16 MiB until the process exits, used or not.
//     A call with NP > 1 needs num_tokens * H * NP * (hd + 2) of them; a call that needs more
//     is refused with an error message (asb_last_error) and launches nothing. A call with
//     NP == 1 has no partial results: it never touches the array and has no such limit.
//     H and NP must lie in 1..65535 and hd in 1..256, as for asb_paged_attention.
//   * The first call on each device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current) and remembers it. Make that first call
//     before any stream capture begins on that device.
//   * Nothing in the array has to start at zero: every slot the reduction reads is written by
//     the same call's partition kernel first. The array keeps the last call's contents.
//   * All calls on a device share the one array. Two calls whose kernels can overlap on the
//     GPU (different streams without an ordering between them) race on it; keep such calls on
//     one stream or order them with events.
//   * It calls no cudaMalloc, cudaFree or other allocating routine.
#pragma once

#include <cuda_runtime.h>

#define ASB_STATIC_SCRATCH_FLOATS (4u * 1024u * 1024u)

#ifdef __cplusplus
extern "C" {
#endif

int asb_paged_attention_static_scratch(void* out, const void* q, const void* k_cache,
                                       const void* v_cache, const int* block_tables,
                                       const int* req_q_start, const int* req_pos_start,
                                       int num_tokens, int R, int H, int KV, int hd, int bs,
                                       int table_width, int window, int PS, int NP, float scale,
                                       int dtype, cudaStream_t stream);

// The capacity above, for callers that size their batches against it.
unsigned int asb_static_scratch_floats(void);

#ifdef __cplusplus
}
#endif
