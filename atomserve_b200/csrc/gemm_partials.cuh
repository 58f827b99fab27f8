// The float32 partial sums that the tensor-core GEMM leaves in its workspace when it cuts K
// (few tokens, swapped operands), and how a kernel that consumes the product reads them
// directly: the consumer adds a tile's slots up itself, which saves the reduction kernel and a
// round trip of the result through memory.
//
// The flattened sequence of (tile, K block) pairs is cut into `blocks` equal contiguous
// ranges, one per thread block of the GEMM. Tile t (weight rows 128 t .. 128 t + 127) gets one
// slot from each block whose range touches it, in block order; slot s of tile t holds
// [bn tokens][128 weight rows] floats at ws + ((t * max_slots + s) * bn + token) * 128 + row.
#pragma once

#include <cuda_runtime.h>

#include <type_traits>

namespace asb {

constexpr int kPartialRows = 128;  // weight rows per tile

struct PartialSums {
  const float* ws;  // null: there are no partial sums, the product is in memory as usual
  int max_slots, bn, kb_per_tile, num_tiles, blocks;
};

// First flattened K block of block c's range when `total` K blocks are cut into `parts` ranges.
__host__ __device__ __forceinline__ long long range_begin(long long total, int parts, int c) {
  return total * c / parts;
}

// The block whose range holds flattened K block `pos` (the largest c with range_begin(c) <= pos).
__host__ __device__ __forceinline__ int block_of(long long total, int parts, long long pos) {
  int c = (int)(pos * parts / total);
  if (c >= parts) c = parts - 1;
  while (c + 1 < parts && range_begin(total, parts, c + 1) <= pos) ++c;
  while (c > 0 && range_begin(total, parts, c) > pos) --c;
  return c;
}

// Number of slots that hold a part of tile `tile`'s sum.
__device__ __forceinline__ int partial_slots(const PartialSums& p, int tile) {
  const long long total = (long long)p.num_tiles * p.kb_per_tile;
  const long long begin = (long long)tile * p.kb_per_tile;
  return block_of(total, p.blocks, begin + p.kb_per_tile - 1) - block_of(total, p.blocks, begin) + 1;
}

// Sum over the slots, in slot order from 0.f (the order of the GEMM's own reduction kernel), of
// N consecutive output columns col.. (inside one tile) of one token. N is 1, 2, 4 or 8. The loads
// of four slots are issued together, so that their latencies overlap.
template <int N>
__device__ __forceinline__ void partial_sum(const PartialSums& p, int token, int col, int slots, float (&out)[N]) {
  constexpr int V = N >= 4 ? 4 : N;  // floats per load
  constexpr int L = N / V;           // loads per slot
  using Vec = typename std::conditional<V == 4, float4, typename std::conditional<V == 2, float2, float>::type>::type;
  const int tile = col / kPartialRows, row = col % kPartialRows;
  const float* at = p.ws + (((size_t)tile * p.max_slots) * p.bn + token) * kPartialRows + row;
  const size_t stride = (size_t)p.bn * kPartialRows;
#pragma unroll
  for (int k = 0; k < N; ++k) out[k] = 0.f;
  for (int s0 = 0; s0 < slots; s0 += 4) {
    Vec v[4][L];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (s0 + u < slots) {
#pragma unroll
        for (int l = 0; l < L; ++l) v[u][l] = *reinterpret_cast<const Vec*>(at + (s0 + u) * stride + l * V);
      }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (s0 + u < slots) {
#pragma unroll
        for (int l = 0; l < L; ++l) {
          const float* f = reinterpret_cast<const float*>(&v[u][l]);
#pragma unroll
          for (int k = 0; k < V; ++k) out[l * V + k] += f[k];
        }
      }
  }
}

}  // namespace asb
