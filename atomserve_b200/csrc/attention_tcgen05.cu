// Paged grouped-query attention for prompt portions on the fifth-generation tensor cores:
// bfloat16, head size 128, both products (Q K^T and P V) issued as tcgen05.mma with the scores
// and the output accumulator in tensor memory, operands brought in by TMA straight from the
// cache pages. It serves the same requests as the mma.sync prefill kernel of attention_mma.cu
// (portions of more than 8 tokens) where its shape rules hold; the math is the same: causal and
// window masks from absolute positions, softmax in float32, one rounding of the output
// (atomserve/model.py:199-232).
//
// One block per (request, tile of QT query tokens, kv head). Its 128 rows are the (token, head)
// pairs of the tile, QT = 128 / G tokens (rounded down) times the G query heads of the kv head, loaded as one
// 3-D TMA box of q [T, H, hd]. Keys are visited in tiles of 64 at absolute multiples of 64.
//
//   warp 0     TMA: the Q tile once, then per key tile the pages of K named by the block table,
//              each page as two boxes (the two 64-element halves of the head).
//   warp 7     TMA: the pages of V, through a ring of stages of its own.
//   warp 1     MMA: S[b] = Q K^T into score buffer b = tile & 1 (two buffers, so the next tile's
//              scores are computed while this tile's softmax runs).
//   warp 6     MMA: O += P V once the softmax has written P, which is the product's A operand in
//              tensor memory. V is consumed as an MN-major operand: its rows in shared memory are
//              keys, exactly as the pages hold them. (A thread of its own, because issuing the
//              next tile's Q K^T would hold this product back.)
//   warps 2-5  softmax: thread r owns row r (a TMEM lane), so row maxima and sums need no
//              shuffles. It reads its scores once, rescales its row of O in tensor memory only when
//              the maximum moved by more than a factor of 256, writes P as bfloat16 over the first
//              half of the tile's score columns (a row's keys packed two to a column), and at the
//              end stores O / sum. A score buffer is free for the tile after next when the P V
//              that read its P has completed.
//
// Shared memory: Q 32 KB, two stages of K and three of V, 16 KB each: 112 KB, so that two blocks
// share an SM and one's softmax overlaps the other's MMAs. Tensor memory: two score buffers of 64
// columns and the output accumulator of 128, 256 columns a block. All barrier waits are bounded;
// a wait that runs out sets *status and the roles wind down to the final barrier.
#include "tcgen05.cuh"

namespace {

using namespace asb::t5;

constexpr int kThreads = 256;
constexpr int HD = 128;
constexpr int kRows = 128;
constexpr int kKeys = 64;                         // keys per tile
constexpr int kBlockBytes = kRows * 64 * 2;       // one [128 rows][64 elements] swizzled block: 16 KB
constexpr int kQBytes = 2 * kBlockBytes;          // Q: the two 64-element halves of the head
constexpr int kKVBlockBytes = kKeys * 64 * 2;     // one [kKeys rows][64 elements] block: 8 KB
constexpr int kKVBytes = 2 * kKVBlockBytes;       // K or V of a tile: two halves of the head
// A block's shared memory stays under 113 KB, so that two blocks share an SM: while one block's
// softmax runs, the other's MMAs do (one block per SM with deeper rings left the tensor cores
// waiting on the softmax-to-MMA hand-offs: 112 us against 103 us at 2,048 tokens, 334 against
// 296 us at 4,096). Q K^T runs a tile ahead of the softmax, hence two stages of keys; a tile's
// values are requested when the P V three tiles before has completed.
constexpr int kKStages = 2;                       // key tiles in flight
constexpr int kVStages = 3;                       // value tiles in flight
static_assert(kKStages >= 2, "Q K^T of the next tile is issued while this tile's keys are still in use");
constexpr int kSmem = kQBytes + (kKStages + kVStages) * kKVBytes + 256;  // tiles, then barriers
constexpr int kBarriers = 7 + 2 * (kKStages + kVStages);
constexpr uint32_t kTmemCols = 256;               // two score buffers of kKeys columns, 128 of output
constexpr int kShortRows = 8;

struct AttnParams {
  __nv_bfloat16* out;        // [T, H, HD]
  const int* block_tables;   // [R, table_width]
  const int* req_q_start;    // [R + 1]
  const int* req_pos_start;  // [R]
  int* status;
  int T, R, H, KV, bs, table_width;
  int G, QT;                 // query heads per kv head, tokens per tile (128 / G)
  int window;
  float scale_log2;          // softmax scale times log2(e)
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(kThreads, 2)
prefill_attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                 const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];  // the swizzled tiles need this alignment
  const uint32_t base = smem_u32(smem_raw);
  unsigned char* aligned = smem_raw;
  const uint32_t q_smem = base;
  auto k_smem = [&](int s) { return base + kQBytes + (uint32_t)s * kKVBytes; };
  auto v_smem = [&](int s) { return base + kQBytes + (uint32_t)(kKStages + s) * kKVBytes; };
  const uint32_t bars = base + kQBytes + (kKStages + kVStages) * kKVBytes;
  const uint32_t q_full = bars;
  auto s_full = [&](int b) { return bars + 8u * (1 + b); };
  auto p_full = [&](int b) { return bars + 8u * (3 + b); };   // P written over score buffer b
  auto pv_done = [&](int b) { return bars + 8u * (5 + b); };  // the P V that read score buffer b's P has completed
  auto k_full = [&](int s) { return bars + 8u * (7 + s); };
  auto k_empty = [&](int s) { return bars + 8u * (7 + kKStages + s); };
  auto v_full = [&](int s) { return bars + 8u * (7 + 2 * kKStages + s); };
  auto v_empty = [&](int s) { return bars + 8u * (7 + 2 * kKStages + kVStages + s); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(aligned + kQBytes + (kKStages + kVStages) * kKVBytes + 8 * kBarriers);
  static_assert(8 * kBarriers + 4 <= 256, "the barriers and the tensor-memory slot have 256 bytes");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // The 1 KB beyond the tiles holds the alignment padding and, after it, the barriers.
  if (base & 1023u) {  // the launch did not honour the declared alignment
    if (threadIdx.x == 0) atomicExch(p.status, 19);
    return;
  }

  // Which request and tile of its tokens? Only requests with more than kShortRows tokens count.
  // Blocks are numbered kv head fastest: the hardware hands blocks out in the order of their
  // numbers, so every kv head's block of a request's last tile (the one that sees the most keys)
  // starts before any block of an earlier tile. (Numbered tile fastest, the long blocks of the
  // last kv heads started when half the kernel's time had passed: 64.8 us at 2,048 tokens.)
  int tile = blockIdx.x / p.KV, r = 0, q_len = 0;
  for (; r < p.R; ++r) {
    q_len = p.req_q_start[r + 1] - p.req_q_start[r];
    if (q_len <= kShortRows) continue;
    const int tiles = (q_len + p.QT - 1) / p.QT;
    if (tile < tiles) {
      tile = tiles - 1 - tile;  // late tiles see the most keys: start them first
      break;
    }
    tile -= tiles;
  }
  if (r >= p.R) return;  // the whole block leaves before any barrier or allocation
  const int q0 = tile * p.QT;
  const int nq = min(p.QT, q_len - q0);
  const int row0 = p.req_q_start[r] + q0;
  const int pos0 = p.req_pos_start[r] + q0;
  const int kvh = blockIdx.x % p.KV;
  const int head0 = kvh * p.G;
  const int* table = p.block_tables + (size_t)r * p.table_width;
  const int key_lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int key_hi = pos0 + nq;  // exclusive
  const int kt_begin = (key_lo / kKeys) * kKeys;
  const int num_tiles = (key_hi - kt_begin + kKeys - 1) / kKeys;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kKStages; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(k_empty(s), 1);
    }
    for (int s = 0; s < kVStages; ++s) {
      mbar_init(v_full(s), 1);
      mbar_init(v_empty(s), 1);
    }
    mbar_init(s_full(0), 1);
    mbar_init(s_full(1), 1);
    mbar_init(p_full(0), 4);  // one arrival per softmax warp
    mbar_init(p_full(1), 4);
    mbar_init(pv_done(0), 1);
    mbar_init(pv_done(1), 1);
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc(smem_u32((const void*)tmem_slot), kTmemCols);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  auto tmem_s = [&](int j) { return tmem_base + (uint32_t)(j & 1) * kKeys; };  // two score buffers
  const uint32_t tmem_o = tmem_base + 2 * kKeys;
  asb::pdl_wait();
  asb::pdl_launch_dependents();

  if (warp == 0 || warp == 7) {
    // Warp 0 brings the keys, warp 7 the values, each through a ring of its own: a tile's keys
    // are done with when its Q K^T has completed, a tile before its values are (after P V), and
    // the next tile but one's keys are then requested that much earlier. (With keys and values in
    // one ring, a tile's loads could only start when the P V of the tile two before had completed,
    // and their latency, 1,500 to 2,000 cycles from L2, lay on the block's chain.)
    // The whole warp looks up the pages of a key tile (one page per lane, the loads in flight
    // together); lane 0 waits for the stage, and the lanes issue the tile's TMA loads together.
    const bool keys = warp == 0;
    if (keys && lane == 0) {
      // the box is QT tokens by G heads: 128 rows when G divides 128, fewer otherwise (the rows
      // after them are padding: never real, masked out, stored nowhere)
      mbar_expect_tx(q_full, (uint32_t)(2 * p.QT * p.G * 128));
      tma_load_3d(q_smem, &map_q, q_full, 0, head0, row0);
      tma_load_3d(q_smem + kBlockBytes, &map_q, q_full, 64, head0, row0);
    }
    const int box_rows = min(p.bs, kKeys);        // rows one TMA box brings (the tensor maps' box)
    const int boxes_per_tile = kKeys / box_rows;  // at most 8
    const int last_page = (key_hi - 1) / p.bs;    // the last page this request certainly holds
    const int fallback = table[last_page];
    bool ok = true;
    const int ring = keys ? kKStages : kVStages;
    for (int j = 0; j < num_tiles; ++j) {
      const int s = j % ring;
      // pages beyond the request's end, or released by the window, are masked out anyway: read a
      // page the request holds, so that shared memory never holds non-finite values
      int row_y = 0;
      if (lane < boxes_per_tile) {
        const int key = kt_begin + j * kKeys + lane * box_rows;
        int blk = table[min(key / p.bs, last_page)];
        if (blk < 0) blk = fallback;
        row_y = (blk * p.KV + kvh) * p.bs + key % p.bs;
      }
      int ok_i = 1;
      if (lane == 0) {
        const uint32_t parity = (((uint32_t)j / ring) & 1u) ^ 1u;
        ok_i = mbar_wait(keys ? k_empty(s) : v_empty(s), parity, p.status, keys ? 11 : 21) ? 1 : 0;
        if (ok_i) mbar_expect_tx(keys ? k_full(s) : v_full(s), kKVBytes);
      }
      ok = __shfl_sync(0xffffffffu, ok_i, 0) != 0;
      if (!ok) break;
      // one box per lane pair: box i's two copies (the two halves of the head) go out from lanes
      // 2i and 2i + 1 in one instruction instead of one after another from a single lane
      {
        const int i = lane >> 1, which = lane & 1;
        const int y = __shfl_sync(0xffffffffu, row_y, i);
        if (i < boxes_per_tile) {
          const uint32_t off = (uint32_t)(i * box_rows) * 128u + (uint32_t)which * kKVBlockBytes;
          if (keys) tma_load_2d(k_smem(s) + off, &map_k, k_full(s), which * 64, y);
          else tma_load_2d(v_smem(s) + off, &map_v, v_full(s), which * 64, y);
        }
      }
    }
  } else if (warp == 1) {
    // Q K^T, one tile ahead of the softmax. (Issuing a tcgen05.mma takes its thread 60-80 cycles
    // whatever its shape, so the two products have a thread each: warp 6 issues P V.)
    if (lane == 0) {
      constexpr uint32_t idesc_qk = instr_desc_bf16(kRows, kKeys, false);
      auto issue_qk = [&](int j) {
        const int s = j % kKStages;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {  // 16 head elements per MMA: 32 bytes along the swizzled row
          const uint32_t in_row = (uint32_t)(ks % 4) * 32u;
          umma_bf16(tmem_s(j), desc_k_major(q_smem + (uint32_t)(ks / 4) * kBlockBytes + in_row, 1024),
                    desc_k_major(k_smem(s) + (uint32_t)(ks / 4) * kKVBlockBytes + in_row, 1024), idesc_qk,
                    (uint32_t)(ks != 0));
        }
        umma_commit(s_full(j & 1));
        umma_commit(k_empty(s));  // the keys' stage, once this product has read it
      };
      bool ok = mbar_wait(q_full, 0, p.status, 12);
      if (ok) ok = mbar_wait(k_full(0), 0, p.status, 13);
      if (ok) {
        fence_after_sync();
        issue_qk(0);
      }
      for (int j = 0; j + 1 < num_tiles && ok; ++j) {
        ok = mbar_wait(k_full((j + 1) % kKStages), ((uint32_t)(j + 1) / kKStages) & 1u, p.status, 14);
        // score buffer (j + 1) & 1 held tile j - 1's scores and then its P, the buffer's use number
        // (j - 1) / 2: has that tile's P V read it?
        if (ok && j >= 1) ok = mbar_wait(pv_done((j + 1) & 1), ((uint32_t)(j - 1) >> 1) & 1u, p.status, 18);
        if (!ok) break;
        fence_after_sync();
        issue_qk(j + 1);
      }
    }
  } else if (warp == 6) {
    // O += P V as soon as the softmax has written a tile's P
    if (lane == 0) {
      constexpr uint32_t idesc_pv = instr_desc_bf16(kRows, HD, true);
      bool ok = true;
      for (int j = 0; j < num_tiles && ok; ++j) {
        ok = mbar_wait(v_full(j % kVStages), ((uint32_t)j / kVStages) & 1u, p.status, 22);
        if (ok) ok = mbar_wait(p_full(j & 1), ((uint32_t)j >> 1) & 1u, p.status, 15);
        if (!ok) break;
        fence_after_sync();
        const int s = j % kVStages;
#pragma unroll
        for (int ks = 0; ks < kKeys / 16; ++ks) {  // 16 keys per MMA: eight 32-bit columns of P
          // V: rows are keys (128 bytes each), 8-key groups 1024 bytes apart, head halves one block apart
          const uint64_t b = desc_mn_major(v_smem(s) + (uint32_t)ks * 2048u, kKVBlockBytes, 1024);
          umma_bf16_a_tmem(tmem_o, tmem_s(j) + (uint32_t)ks * 8u, b, idesc_pv, (uint32_t)((j | ks) != 0));
        }
        umma_commit(pv_done(j & 1));
        umma_commit(v_empty(s));
      }
    }
  } else {
    // Softmax and epilogue: thread `row` of the block owns TMEM lane `row`.
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int qi = row / p.G;
    const bool real = qi < nq;
    const int pos = real ? pos0 + qi : -1;  // padding rows see nothing
    const int row_lo = p.window > 0 ? max(key_lo, pos - p.window + 1) : key_lo;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const bool real_block = nq * p.G == kRows;  // no padding rows in this block
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    uint32_t scores_there = 0;  // lane 0: the answer to an early question about this tile's scores
    for (int j = 0; j < num_tiles && ok; ++j) {
      const int kt0 = kt_begin + j * kKeys;
      int ok_i = 1;
      // (Q K^T runs a tile or two ahead, so the scores are usually there; asking takes a thread
      // a few hundred cycles even then, which is why lane 0 asked during the previous tile.)
      if (lane == 0 && !scores_there) ok_i = mbar_wait(s_full(j & 1), ((uint32_t)j >> 1) & 1u, p.status, 16) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok_i, 0) != 0;
      if (!ok) break;
      fence_after_sync();
      // The row's 128 raw scores, read from tensor memory once (four loads in flight, one wait)
      // and kept in registers. Tiles strictly inside every row's view (below the diagonal,
      // inside the window) need no mask.
      const bool inside = kt0 + kKeys <= pos0 + 1 && kt0 >= key_lo && real_block &&
                          (p.window <= 0 || kt0 > pos0 + nq - 1 - p.window);
      uint32_t raw[kKeys];
#pragma unroll
      for (int c = 0; c < kKeys; c += 32) tmem_ld32_nowait(tmem_s(j) + lane_addr + (uint32_t)c, raw + c);
      tmem_ld_wait();
      // (eight running maxima, so that no comparison waits for the one before it)
      float part_max[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) part_max[u] = -INFINITY;
      if (inside) {
#pragma unroll
        for (int i = 0; i < kKeys; ++i) part_max[i & 7] = fmaxf(part_max[i & 7], __uint_as_float(raw[i]));
      } else {
#pragma unroll
        for (int i = 0; i < kKeys; ++i) {
          const int key = kt0 + i;
          if (!(key <= pos && key >= row_lo)) raw[i] = 0xff800000u;  // -inf
          part_max[i & 7] = fmaxf(part_max[i & 7], __uint_as_float(raw[i]));
        }
      }
      const float raw_max = fmaxf(fmaxf(fmaxf(part_max[0], part_max[1]), fmaxf(part_max[2], part_max[3])),
                                  fmaxf(fmaxf(part_max[4], part_max[5]), fmaxf(part_max[6], part_max[7])));
      const float tile_max = raw_max * p.scale_log2;  // the scale is positive
      // The running maximum moves only when the new one exceeds it by more than 8 (a factor of
      // 256 in the probabilities, harmless in float32 sums and bfloat16 operands); otherwise the
      // older maximum stays and neither the sum nor the accumulator needs rescaling.
      float corr = 1.f;
      if (tile_max > m + 8.f || (m == -INFINITY && tile_max > -INFINITY)) {  // a row that has still seen nothing stays as it is
        const float m_new = fmaxf(m, tile_max);
        const float m_ref = m_new == -INFINITY ? 0.f : m_new;  // a row that has seen nothing yet
        corr = fast_exp2(m - m_ref);  // 0 when m was -inf
        m = m_new;
        l *= corr;
      }
      const float m_use = m == -INFINITY ? 0.f : m;
      if (lane == 0) scores_there = j + 1 < num_tiles ? mbar_try(s_full((j + 1) & 1), ((uint32_t)(j + 1) >> 1) & 1u) : 0u;
      if (j > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
        // rescale this row of O: the previous P V (tile j - 1) must have completed
        if (lane == 0) ok_i = mbar_wait(pv_done((j - 1) & 1), ((uint32_t)(j - 1) >> 1) & 1u, p.status, 17) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok_i, 0) != 0;
        if (!ok) break;
        fence_after_sync();
#pragma unroll 1
        for (int c = 0; c < HD; c += 32) {
          uint32_t oraw[32];
          tmem_ld32(tmem_o + lane_addr + (uint32_t)c, oraw);
#pragma unroll
          for (int i = 0; i < 32; ++i) oraw[i] = __float_as_uint(__uint_as_float(oraw[i]) * corr);
          tmem_st32(tmem_o + lane_addr + (uint32_t)c, oraw);
        }
        tmem_st_wait();
      }
      // probabilities exp2(score * scale - max), their sum, and P as bfloat16 over the first half
      // of the tile's score columns, a row's keys packed two to a column: the A operand of P V
      // (a masked score is -inf and gives 0)
      const float neg_m = -m_use;
      uint32_t packed[kKeys / 2];
      float part_sum[4] = {0.f, 0.f, 0.f, 0.f};  // the tile's sum in four strands, added to the row's at the end
#pragma unroll
      for (int i = 0; i < kKeys; i += 2) {
        const float a = fast_exp2(fmaf(__uint_as_float(raw[i]), p.scale_log2, neg_m));
        const float b = fast_exp2(fmaf(__uint_as_float(raw[i + 1]), p.scale_log2, neg_m));
        part_sum[(i >> 1) & 3] += a + b;
        __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        packed[i >> 1] = *reinterpret_cast<uint32_t*>(&v);
      }
      l += (part_sum[0] + part_sum[1]) + (part_sum[2] + part_sum[3]);
      tmem_st32(tmem_s(j) + lane_addr, packed);
      tmem_st_wait();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full(j & 1));
    }
    // epilogue: O / sum, rounded once
    if (ok) {
      int ok_i = 1;
      if (lane == 0) ok_i = mbar_wait(pv_done((num_tiles - 1) & 1), ((uint32_t)(num_tiles - 1) >> 1) & 1u, p.status, 18) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok_i, 0) != 0;
    }
    if (ok) {
      fence_after_sync();
      const float inv = real ? 1.f / l : 0.f;
      __nv_bfloat16* o = p.out + ((size_t)(row0 + qi) * p.H + head0 + (row - qi * p.G)) * HD;
#pragma unroll 1
      for (int c = 0; c < HD; c += 32) {
        uint32_t raw[32];
        tmem_ld32(tmem_o + lane_addr + (uint32_t)c, raw);
        if (real) {
          uint4 v[4];
          __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(v);
#pragma unroll
          for (int i = 0; i < 32; i += 2)
            h2[i >> 1] = __floats2bfloat162_rn(__uint_as_float(raw[i]) * inv, __uint_as_float(raw[i + 1]) * inv);
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) *reinterpret_cast<uint4*>(o + c + q4 * 8) = v[q4];
        }
      }
    }
  }

  fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

// 1 if the tcgen05 prefill kernel serves this shape: head size 128, 1 to 16 query heads per kv
// head (a tile is 128 / group tokens, so a group that does not divide 128 leaves a few padding
// rows), pages of 8 to 256 tokens (a power of two).
extern "C" int asb_attention_tcgen05_supported(int hd, int group, int block_size) {
  const bool group_ok = group >= 1 && group <= 16;
  const bool pow2_page = block_size >= 8 && block_size <= 256 && (block_size & (block_size - 1)) == 0;
  return hd == 128 && group_ok && pow2_page ? 1 : 0;
}

// Attention for every request that brings more than 8 tokens in this step (others are left
// untouched for the decode kernel). q, out: [T, H, 128] bfloat16; caches [num_blocks, KV, bs, 128].
extern "C" int asb_prefill_attention_tcgen05(void* out, const void* q, const void* k_cache, const void* v_cache,
                                             const int* block_tables, const int* req_q_start,
                                             const int* req_pos_start, int num_tokens, int R, int H, int KV,
                                             int hd, int bs, int num_blocks, int table_width, int window,
                                             float scale, int* status, cudaStream_t stream) {
  if (num_tokens == 0 || R == 0) return 0;
  if (KV < 1 || H % KV) return asb::fail("prefill_attention_tcgen05: %d heads over %d kv heads", H, KV);
  if (!asb_attention_tcgen05_supported(hd, H / KV, bs))
    return asb::fail("prefill_attention_tcgen05: head_dim %d, group %d, page %d are not served", hd, H / KV, bs);
  if (!status) return asb::fail("prefill_attention_tcgen05: a status word is required");
  AttnParams p;
  p.out = (__nv_bfloat16*)out;
  p.block_tables = block_tables; p.req_q_start = req_q_start; p.req_pos_start = req_pos_start;
  p.status = status;
  p.T = num_tokens; p.R = R; p.H = H; p.KV = KV; p.bs = bs; p.table_width = table_width;
  p.G = H / KV;
  p.QT = kRows / p.G;
  p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;

  alignas(64) CUtensorMap mq, mk, mv;
  {
    const cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)H, (cuuint64_t)num_tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)H * HD * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)p.G, (cuuint32_t)p.QT};
    if (int rc = make_bf16_map(&mq, q, 3, dims, strides, box)) return rc;
  }
  {
    const cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)num_blocks * KV * bs};
    const cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)(bs < kKeys ? bs : kKeys)};
    if (int rc = make_bf16_map(&mk, k_cache, 2, dims, strides, box)) return rc;
    if (int rc = make_bf16_map(&mv, v_cache, 2, dims, strides, box)) return rc;
  }
  auto kern = prefill_attention_tcgen05_kernel;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  if (e != cudaSuccess) return asb::fail("prefill_attention_tcgen05: shared memory %d: %s", kSmem, cudaGetErrorString(e));
  const long long blocks = (long long)((num_tokens + p.QT - 1) / p.QT + R) * KV;
  if (blocks > 0x7fffffffLL) return asb::fail("prefill_attention_tcgen05: %lld blocks exceed the grid", blocks);
  asb::launch(kern, dim3((unsigned)blocks), kThreads, kSmem, stream, mq, mk, mv, p);
  return asb::check_launch("prefill_attention_tcgen05");
}
