// Paged grouped-query attention for bfloat16 on the tensor cores (mma.sync m16n8k16, float32
// accumulation), head sizes 64 and 128. Two kernels share one tile machinery:
//
//   decode   one block per (new token, kv head, key partition). The token's G query heads are
//            the rows of a 16-row tile, so keys and values are read once for all of them. The
//            block's four warps take the keys of each 64-key tile sixteen apiece, keep their own
//            running softmax, and merge at the end. With more than one partition the block
//            writes (max, sum, accumulator) for the reduction kernel of attention_simt.cu.
//            Serves every request that brings at most kShortRows tokens in the step; each of
//            those tokens is its own row with its own context length.
//   prefill  one block per (request, tile of query tokens, kv head): 128 rows = (token, head)
//            pairs, sixteen per warp, all key tiles up to the tile's last position, causal and
//            window masks from absolute positions. Serves the longer portions.
//
// Keys and values come straight from the cache pages through the block table with 16-byte
// cp.async copies into shared memory (two stages), swizzled so that ldmatrix reads are free of
// bank conflicts. Scores, maxima, sums and the output accumulator are float32; probabilities are
// rounded to bfloat16 only as the tensor-core operand of the second product, the output once
// (atomserve/kernels.py:147-334 is the reference's scalar decode kernel; its prefill is a
// library call, atomserve/model.py:225-231).
//
// Key tiles start at absolute multiples of 64 and partitions at multiples of the partition
// size, so what a row computes does not depend on the rest of the batch.
#include "common.cuh"

namespace {

constexpr int kThreads = 128;
constexpr int kKeyTile = 64;
constexpr int kShortRows = 8;  // requests with at most this many new tokens go row by row

struct MmaParams {
  const __nv_bfloat16* q;    // [T, H, HD]
  __nv_bfloat16* out;        // [T, H, HD]
  const __nv_bfloat16* k_cache;  // [num_blocks, KV, bs, HD]
  const __nv_bfloat16* v_cache;
  const int* block_tables;   // [R, table_width]
  const int* req_q_start;    // [R + 1]
  const int* req_pos_start;  // [R]
  float* part_m;             // [T, H, NP]
  float* part_l;
  float* part_acc;           // [T, H, NP, HD]
  int T, R, H, KV, bs, table_width;
  int G, GC, HC;             // heads per kv head, heads per block (<= 16), chunks per kv head
  int QT;                    // prefill: tokens per 128-row tile
  int window, PS, NP;
  int all_single;            // every request brings exactly one token: request = row
  int short_rows;            // > 0: the decode kernel's grid and the partial results count only the rows of
                             // requests with at most kShortRows tokens (a step that also holds longer portions)
  float scale;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Shared-memory tile of `rows` x HD bfloat16, 16-byte chunks XOR-swizzled by the row.
template <int HD>
__device__ __forceinline__ uint32_t tile_offset(int row, int chunk) {
  return (uint32_t)(row * (HD * 2) + ((chunk ^ (row & 7)) << 4));
}

// Copy keys [kt0, kt0 + 64) of one kv head into a tile; rows outside [key_lo, key_hi) are zero.
// A thread copies one 16-byte chunk column of a run of consecutive keys, so that when a run lies
// inside one page (pages of at least that many tokens, a power of two) it looks the page up once.
template <int HD, int NT = kThreads>
__device__ __forceinline__ void load_kv_tile(uint32_t k_tile, uint32_t v_tile, const MmaParams& p,
                                             const int* table, int kvh, int kt0, int key_lo, int key_hi) {
  constexpr int kChunks = HD / 8;                        // 16-byte chunks per row
  constexpr int kRun = kKeyTile / (NT / kChunks);        // consecutive keys per thread
  const int chunk = threadIdx.x % kChunks;
  const int run0 = (threadIdx.x / kChunks) * kRun;
  const int j0 = kt0 + run0;
  const bool one_page = p.bs >= kRun && (p.bs & (p.bs - 1)) == 0;
  size_t page_at = 0;
  if (one_page && j0 < key_hi && j0 + kRun > key_lo) {
    const int blk = table[j0 / p.bs];
    page_at = (((size_t)blk * p.KV + kvh) * p.bs + (j0 & (p.bs - 1))) * HD + chunk * 8;
  }
#pragma unroll
  for (int i = 0; i < kRun; ++i) {
    const int j = j0 + i;
    const bool valid = j >= key_lo && j < key_hi;
    size_t at = 0;
    if (valid) {
      if (one_page) {
        at = page_at + (size_t)i * HD;
      } else {
        const int blk = table[j / p.bs];
        at = (((size_t)blk * p.KV + kvh) * p.bs + (j % p.bs)) * HD + chunk * 8;
      }
    }
    const uint32_t off = tile_offset<HD>(run0 + i, chunk);
    cp_async16(k_tile + off, p.k_cache + at, valid);
    cp_async16(v_tile + off, p.v_cache + at, valid);
  }
}

// One warp: scores of its 16 rows against 16 keys (rows key0.. of the tile) -> s[2][4].
template <int HD>
__device__ __forceinline__ void qk_16keys(float (&s)[2][4], const uint32_t (&qf)[HD / 16][4],
                                          uint32_t k_tile, int key0, int lane, float scale) {
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
  const int krow = key0 + (lane & 7) + ((lane >> 4) << 3);
  const int kchunk = (lane >> 3) & 1;
#pragma unroll
  for (int kc = 0; kc < HD / 16; ++kc) {
    uint32_t b[4];
    ldmatrix_x4(b, k_tile + tile_offset<HD>(krow, kc * 2 + kchunk));
    mma_bf16(s[0], qf[kc], b[0], b[1]);
    mma_bf16(s[1], qf[kc], b[2], b[3]);
  }
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[j][e] *= scale;
}

// One warp: scores of its 16 rows against all 64 keys of a tile. The eight accumulators advance
// together along the head dimension, so eight independent MMA chains are in flight.
template <int HD>
__device__ __forceinline__ void qk_64keys(float (&s)[kKeyTile / 8][4], const uint32_t (&qf)[HD / 16][4],
                                          uint32_t k_tile, int lane, float scale) {
#pragma unroll
  for (int j = 0; j < kKeyTile / 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
  const int krow = (lane & 7) + ((lane >> 4) << 3);
  const int kchunk = (lane >> 3) & 1;
#pragma unroll
  for (int kc = 0; kc < HD / 16; ++kc) {
#pragma unroll
    for (int sub = 0; sub < kKeyTile / 16; ++sub) {
      uint32_t b[4];
      ldmatrix_x4(b, k_tile + tile_offset<HD>(sub * 16 + krow, kc * 2 + kchunk));
      mma_bf16(s[sub * 2], qf[kc], b[0], b[1]);
      mma_bf16(s[sub * 2 + 1], qf[kc], b[2], b[3]);
    }
  }
#pragma unroll
  for (int j = 0; j < kKeyTile / 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[j][e] *= scale;
}

// The same with the Q fragments read from shared memory as they are needed, which frees the
// HD/4 registers that holding them costs (the prefill kernel runs two blocks per SM that way).
template <int HD>
__device__ __forceinline__ void qk_64keys_smem_q(float (&s)[kKeyTile / 8][4], uint32_t q_tile, int q_row0,
                                                 uint32_t k_tile, int lane, float scale) {
#pragma unroll
  for (int j = 0; j < kKeyTile / 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
  const int krow = (lane & 7) + ((lane >> 4) << 3);
  const int kchunk = (lane >> 3) & 1;
  const int qrow = q_row0 + (lane & 7) + (((lane >> 3) & 1) << 3);
  const int qchunk = lane >> 4;
#pragma unroll
  for (int kc = 0; kc < HD / 16; ++kc) {
    uint32_t a[4];
    ldmatrix_x4(a, q_tile + tile_offset<HD>(qrow, kc * 2 + qchunk));
#pragma unroll
    for (int sub = 0; sub < kKeyTile / 16; ++sub) {
      uint32_t b[4];
      ldmatrix_x4(b, k_tile + tile_offset<HD>(sub * 16 + krow, kc * 2 + kchunk));
      mma_bf16(s[sub * 2], a, b[0], b[1]);
      mma_bf16(s[sub * 2 + 1], a, b[2], b[3]);
    }
  }
#pragma unroll
  for (int j = 0; j < kKeyTile / 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[j][e] *= scale;
}

template <int HD>
__device__ __forceinline__ void qk_16keys_smem_q(float (&s)[2][4], uint32_t q_tile, int q_row0, uint32_t k_tile,
                                                 int key0, int lane, float scale) {
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
  const int krow = key0 + (lane & 7) + ((lane >> 4) << 3);
  const int kchunk = (lane >> 3) & 1;
  const int qrow = q_row0 + (lane & 7) + (((lane >> 3) & 1) << 3);
  const int qchunk = lane >> 4;
#pragma unroll
  for (int kc = 0; kc < HD / 16; ++kc) {
    uint32_t a[4], b[4];
    ldmatrix_x4(a, q_tile + tile_offset<HD>(qrow, kc * 2 + qchunk));
    ldmatrix_x4(b, k_tile + tile_offset<HD>(krow, kc * 2 + kchunk));
    mma_bf16(s[0], a, b[0], b[1]);
    mma_bf16(s[1], a, b[2], b[3]);
  }
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[j][e] *= scale;
}

// One warp: acc[HD/8][4] += P (16 rows x 16 keys, as an A fragment) . V (16 keys x HD).
template <int HD>
__device__ __forceinline__ void pv_16keys(float (&acc)[HD / 8][4], const uint32_t (&pf)[4],
                                          uint32_t v_tile, int key0, int lane) {
  const int vrow = key0 + (lane & 7) + (((lane >> 3) & 1) << 3);
  const int vchunk = lane >> 4;
#pragma unroll
  for (int nc = 0; nc < HD / 16; ++nc) {
    uint32_t b[4];
    ldmatrix_x4_trans(b, v_tile + tile_offset<HD>(vrow, nc * 2 + vchunk));
    mma_bf16(acc[nc * 2], pf, b[0], b[1]);
    mma_bf16(acc[nc * 2 + 1], pf, b[2], b[3]);
  }
}

// Load a 16-row Q tile (already in shared memory, swizzled) into A fragments.
template <int HD>
__device__ __forceinline__ void load_q_frags(uint32_t (&qf)[HD / 16][4], uint32_t q_tile, int row0, int lane) {
  const int row = row0 + (lane & 7) + (((lane >> 3) & 1) << 3);
  const int chunk = lane >> 4;
#pragma unroll
  for (int kc = 0; kc < HD / 16; ++kc) ldmatrix_x4(qf[kc], q_tile + tile_offset<HD>(row, kc * 2 + chunk));
}

__device__ __forceinline__ int find_request(const int* req_q_start, int R, int row) {
  int lo = 0, hi = R - 1;  // the last r with req_q_start[r] <= row
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (req_q_start[mid] <= row) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// ---- decode ------------------------------------------------------------------------------------

template <int HD>
__global__ void __launch_bounds__(kThreads)
decode_attention_kernel(const MmaParams p) {
  asb::pdl_wait();  // the stream's previous kernel has completed (programmatic dependent launch)
  asb::pdl_launch_dependents();
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr int kTileBytes = kKeyTile * HD * 2;
  // [K stage 0][K stage 1][V stage 0][V stage 1][Q 16 rows]; the merge reuses the K/V stages
  const uint32_t smem = smem_u32(smem_raw);
  auto k_stage = [&](int i) { return smem + (uint32_t)(i & 1) * kTileBytes; };
  auto v_stage = [&](int i) { return smem + (uint32_t)(2 + (i & 1)) * kTileBytes; };
  const uint32_t q_tile = smem + 4 * kTileBytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int row = blockIdx.x;  // flat token row
  int r;
  if (p.all_single) {
    r = row;
  } else if (p.short_rows > 0) {
    row = asb::nth_short_row(p.req_q_start, p.R, kShortRows, blockIdx.x, &r);
    if (row < 0) return;
  } else {
    r = find_request(p.req_q_start, p.R, row);
    if (p.req_q_start[r + 1] - p.req_q_start[r] > kShortRows) return;  // the prefill kernel's
  }
  const int pos = p.req_pos_start[r] + (row - p.req_q_start[r]);
  const int kvh = blockIdx.y / p.HC;
  const int head0 = kvh * p.G + (blockIdx.y % p.HC) * p.GC;
  const int gc = min(p.GC, kvh * p.G + p.G - head0);

  const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  const int part = lo / p.PS + blockIdx.z;
  const int key_lo = max(lo, part * p.PS);
  const int key_hi = (int)min((long long)pos + 1, (long long)(part + 1) * p.PS);
  const int* table = p.block_tables + (size_t)r * p.table_width;

  // Q: gc heads of this token, zero rows above gc. (The scale is applied to the float32 scores.)
  {
    constexpr int kChunks = HD / 8;
    for (int i = threadIdx.x; i < 16 * kChunks; i += kThreads) {
      const int qr = i / kChunks, c = i % kChunks;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (qr < gc) {
        const __nv_bfloat162* src = reinterpret_cast<const __nv_bfloat162*>(
            p.q + ((size_t)row * p.H + head0 + qr) * HD + c * 8);
        v = *reinterpret_cast<const uint4*>(src);
      }
      *reinterpret_cast<uint4*>(smem_raw + (q_tile - smem) + tile_offset<HD>(qr, c)) = v;
    }
  }

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float acc[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;

  const int kt_begin = (key_lo / kKeyTile) * kKeyTile;
  const int num_tiles = key_hi > key_lo ? (key_hi - kt_begin + kKeyTile - 1) / kKeyTile : 0;
  if (num_tiles > 0) load_kv_tile<HD>(k_stage(0), v_stage(0), p, table, kvh, kt_begin, key_lo, key_hi);
  cp_async_commit();
  __syncthreads();  // Q tile written
  uint32_t qf[HD / 16][4];
  load_q_frags<HD>(qf, q_tile, 0, lane);

  for (int it = 0; it < num_tiles; ++it) {
    const int kt0 = kt_begin + it * kKeyTile;
    if (it + 1 < num_tiles)
      load_kv_tile<HD>(k_stage(it + 1), v_stage(it + 1), p, table, kvh, kt0 + kKeyTile, key_lo, key_hi);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    const int key0 = warp * 16;  // this warp's keys inside the tile
    if (kt0 + key0 < key_hi && kt0 + key0 + 16 > key_lo) {
      float s[2][4];
      qk_16keys<HD>(s, qf, k_stage(it), key0, lane, p.scale);
      // mask by absolute key position; both rows of a thread share the token, hence the mask
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = kt0 + key0 + j * 8 + (lane & 3) * 2 + (e & 1);
          if (key < key_lo || key >= key_hi) s[j][e] = -INFINITY;
        }
      float rmax[2] = {fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1])),
                       fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]))};
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        rmax[h] = fmaxf(rmax[h], __shfl_xor_sync(0xffffffffu, rmax[h], 1));
        rmax[h] = fmaxf(rmax[h], __shfl_xor_sync(0xffffffffu, rmax[h], 2));
      }
      float corr[2], rsum[2] = {0.f, 0.f};
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float m_new = fmaxf(m[h], rmax[h]);  // finite: at least one key of the 16 is visible
        corr[h] = __expf(m[h] - m_new);
        m[h] = m_new;
      }
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pe = __expf(s[j][e] - m[e >> 1]);
          s[j][e] = pe;
          rsum[e >> 1] += pe;
        }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        rsum[h] += __shfl_xor_sync(0xffffffffu, rsum[h], 1);
        rsum[h] += __shfl_xor_sync(0xffffffffu, rsum[h], 2);
        l[h] = l[h] * corr[h] + rsum[h];
      }
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) {
        acc[i][0] *= corr[0]; acc[i][1] *= corr[0];
        acc[i][2] *= corr[1]; acc[i][3] *= corr[1];
      }
      const uint32_t pf[4] = {pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]),
                              pack_bf16(s[1][0], s[1][1]), pack_bf16(s[1][2], s[1][3])};
      pv_16keys<HD>(acc, pf, v_stage(it), key0, lane);
    }
    __syncthreads();  // the stage is free for the load after next
  }
  cp_async_wait<0>();
  __syncthreads();

  // Merge the four warps through shared memory (over the K/V stages): per row max, sum, acc.
  float* mm = reinterpret_cast<float*>(smem_raw);          // [4][16]
  float* ml = mm + 64;                                     // [4][16]
  float* ma = ml + 64;                                     // [4][16][HD]
  {
    const int g = lane >> 2, t = lane & 3;
    if (t == 0) {
      mm[warp * 16 + g] = m[0]; mm[warp * 16 + g + 8] = m[1];
      ml[warp * 16 + g] = l[0]; ml[warp * 16 + g + 8] = l[1];
    }
    // only the rows that are query heads (gc of the 16) are read back
    if (g < gc) {
#pragma unroll
      for (int i = 0; i < HD / 8; ++i)
        *reinterpret_cast<float2*>(ma + ((size_t)(warp * 16 + g) * HD + i * 8 + t * 2)) = make_float2(acc[i][0], acc[i][1]);
    }
    if (g + 8 < gc) {
#pragma unroll
      for (int i = 0; i < HD / 8; ++i)
        *reinterpret_cast<float2*>(ma + ((size_t)(warp * 16 + g + 8) * HD + i * 8 + t * 2)) = make_float2(acc[i][2], acc[i][3]);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < gc * HD; i += kThreads) {
    const int qr = i / HD, col = i - qr * HD;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w)
      if (ml[w * 16 + qr] > 0.f) mx = fmaxf(mx, mm[w * 16 + qr]);
    float a = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w)
      if (ml[w * 16 + qr] > 0.f) {
        const float f = __expf(mm[w * 16 + qr] - mx);
        den += ml[w * 16 + qr] * f;
        a += ma[(size_t)(w * 16 + qr) * HD + col] * f;
      }
    const size_t orow = (size_t)row * p.H + head0 + qr;
    if (p.NP == 1) {
      p.out[orow * HD + col] = __float2bfloat16_rn(a / den);
    } else {
      const size_t prow = p.short_rows > 0 ? (size_t)blockIdx.x * p.H + head0 + qr : orow;
      const size_t at = prow * p.NP + blockIdx.z;
      p.part_acc[at * HD + col] = a;
      if (col == 0) {
        p.part_m[at] = mx;
        p.part_l[at] = den;
      }
    }
  }
}

// ---- prefill -----------------------------------------------------------------------------------

constexpr int kPrefillThreads = 256;  // eight warps of sixteen rows
constexpr int kPrefillRows = 128;

template <int HD>
__global__ void __launch_bounds__(kPrefillThreads, 2)
prefill_attention_kernel(const MmaParams p) {
  asb::pdl_wait();  // the stream's previous kernel has completed (programmatic dependent launch)
  asb::pdl_launch_dependents();
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr int kTileBytes = kKeyTile * HD * 2;
  const uint32_t smem = smem_u32(smem_raw);
  auto k_stage = [&](int i) { return smem + (uint32_t)(i & 1) * kTileBytes; };
  auto v_stage = [&](int i) { return smem + (uint32_t)(2 + (i & 1)) * kTileBytes; };
  const uint32_t q_tile = smem + 4 * kTileBytes;  // 128 rows

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Which request and tile of its tokens? Only requests with more than kShortRows tokens count.
  // (blocks are numbered head chunk fastest, so that every kv head's longest block starts first)
  const int chunks = p.KV * p.HC;
  const int chunk = blockIdx.x % chunks;
  int tile = blockIdx.x / chunks, r = 0, q_len = 0;
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
  if (r >= p.R) return;
  const int q0 = tile * p.QT;
  const int nq = min(p.QT, q_len - q0);
  const int row0 = p.req_q_start[r] + q0;
  const int pos0 = p.req_pos_start[r] + q0;
  const int kvh = chunk / p.HC;
  const int head0 = kvh * p.G + (chunk % p.HC) * p.GC;
  const int gc = min(p.GC, kvh * p.G + p.G - head0);
  const int num_rows = nq * gc;  // tile row rr = qi * gc + g
  const int* table = p.block_tables + (size_t)r * p.table_width;

  const int key_lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int key_hi = pos0 + nq;

  {
    constexpr int kChunks = HD / 8;
    for (int i = threadIdx.x; i < kPrefillRows * kChunks; i += kPrefillThreads) {
      const int rr = i / kChunks, c = i % kChunks;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (rr < num_rows) {
        const int qi = rr / gc, g = rr - qi * gc;
        const __nv_bfloat162* src = reinterpret_cast<const __nv_bfloat162*>(
            p.q + ((size_t)(row0 + qi) * p.H + head0 + g) * HD + c * 8);
        v = *reinterpret_cast<const uint4*>(src);
      }
      *reinterpret_cast<uint4*>(smem_raw + (q_tile - smem) + tile_offset<HD>(rr, c)) = v;
    }
  }

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float acc[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;

  // positions of this thread's two rows (rows warp*16 + g and + 8)
  const int g4 = lane >> 2;
  int qpos[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int rr = warp * 16 + g4 + h * 8;
    qpos[h] = rr < num_rows ? pos0 + rr / gc : -1;  // -1: a padding row, sees nothing
  }
  // keys this warp's rows can see at all
  const int warp_first = warp * 16, warp_last = min(warp * 16 + 15, num_rows - 1);
  const int warp_hi = warp_first < num_rows ? pos0 + warp_last / gc + 1 : 0;
  const int warp_lo = p.window > 0 ? max(0, pos0 + warp_first / gc - p.window + 1) : 0;
  const int warp_min_pos = pos0 + warp_first / gc;            // position of the warp's first row
  const int warp_max_pos = warp_hi - 1;                       // and of its last real row
  const bool warp_full = warp_first + 15 < num_rows;          // no padding rows in this warp

  const int kt_begin = (key_lo / kKeyTile) * kKeyTile;
  const int num_tiles = (key_hi - kt_begin + kKeyTile - 1) / kKeyTile;
  load_kv_tile<HD, kPrefillThreads>(k_stage(0), v_stage(0), p, table, kvh, kt_begin, key_lo, key_hi);
  cp_async_commit();
  __syncthreads();  // the Q tile is in shared memory; fragments are read from it as needed

  for (int it = 0; it < num_tiles; ++it) {
    const int kt0 = kt_begin + it * kKeyTile;
    if (it + 1 < num_tiles)
      load_kv_tile<HD, kPrefillThreads>(k_stage(it + 1), v_stage(it + 1), p, table, kvh, kt0 + kKeyTile, key_lo, key_hi);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    if (kt0 < warp_hi && kt0 + kKeyTile > warp_lo) {
      // Scores of this warp's 16 rows against all 64 keys of the tile, in units of log2(e) so that
      // the exponentials are bare ex2 instructions; 16-key groups no row can see are skipped.
      float s[kKeyTile / 8][4];
      bool live[kKeyTile / 16];
      const bool all_live = kt0 + kKeyTile <= warp_hi && kt0 >= warp_lo;  // uniform in the warp
      if (all_live) {
#pragma unroll
        for (int sub = 0; sub < kKeyTile / 16; ++sub) live[sub] = true;
        qk_64keys_smem_q<HD>(s, q_tile, warp * 16, k_stage(it), lane, p.scale * 1.4426950408889634f);
      } else
#pragma unroll
      for (int sub = 0; sub < kKeyTile / 16; ++sub) {
        live[sub] = kt0 + sub * 16 < warp_hi && kt0 + sub * 16 + 16 > warp_lo;  // uniform in the warp
        if (live[sub]) {
          float part[2][4];
          qk_16keys_smem_q<HD>(part, q_tile, warp * 16, k_stage(it), sub * 16, lane, p.scale * 1.4426950408889634f);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            s[sub * 2][e] = part[0][e];
            s[sub * 2 + 1][e] = part[1][e];
          }
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) s[sub * 2][e] = s[sub * 2 + 1][e] = -INFINITY;
        }
      }
      // Masks are needed only where the tile touches a row's own position, the window's edge or
      // the ends of the key range; tiles strictly inside every row's view skip them.
      const bool inside = warp_full && kt0 + kKeyTile <= warp_min_pos + 1 && kt0 >= key_lo && kt0 + kKeyTile <= key_hi &&
                          (p.window <= 0 || kt0 > warp_max_pos - p.window);
      float rmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < kKeyTile / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (!inside) {
            const int key = kt0 + j * 8 + (lane & 3) * 2 + (e & 1);
            const int qp = qpos[e >> 1];
            const bool visible = key <= qp && key >= key_lo && (p.window <= 0 || key > qp - p.window);
            if (!visible) s[j][e] = -INFINITY;
          }
          rmax[e >> 1] = fmaxf(rmax[e >> 1], s[j][e]);
        }
      float corr[2], rsum[2] = {0.f, 0.f}, m_use[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        rmax[h] = fmaxf(rmax[h], __shfl_xor_sync(0xffffffffu, rmax[h], 1));
        rmax[h] = fmaxf(rmax[h], __shfl_xor_sync(0xffffffffu, rmax[h], 2));
        const float m_new = fmaxf(m[h], rmax[h]);
        // a row that has seen nothing yet keeps max -inf: use 0 in the exponent to avoid inf - inf
        m_use[h] = m_new == -INFINITY ? 0.f : m_new;
        corr[h] = fast_exp2(m[h] - m_use[h]);
        m[h] = m_new;
      }
#pragma unroll
      for (int j = 0; j < kKeyTile / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pe = fast_exp2(s[j][e] - m_use[e >> 1]);
          s[j][e] = pe;
          rsum[e >> 1] += pe;
        }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        rsum[h] += __shfl_xor_sync(0xffffffffu, rsum[h], 1);
        rsum[h] += __shfl_xor_sync(0xffffffffu, rsum[h], 2);
        l[h] = l[h] * corr[h] + rsum[h];
      }
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) {
        acc[i][0] *= corr[0]; acc[i][1] *= corr[0];
        acc[i][2] *= corr[1]; acc[i][3] *= corr[1];
      }
#pragma unroll
      for (int sub = 0; sub < kKeyTile / 16; ++sub) {
        if (!live[sub]) continue;
        const uint32_t pf[4] = {pack_bf16(s[sub * 2][0], s[sub * 2][1]), pack_bf16(s[sub * 2][2], s[sub * 2][3]),
                                pack_bf16(s[sub * 2 + 1][0], s[sub * 2 + 1][1]), pack_bf16(s[sub * 2 + 1][2], s[sub * 2 + 1][3])};
        pv_16keys<HD>(acc, pf, v_stage(it), sub * 16, lane);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  const int t = lane & 3;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int rr = warp * 16 + g4 + h * 8;
    if (rr >= num_rows) continue;
    const int qi = rr / gc, g = rr - qi * gc;
    __nv_bfloat16* o = p.out + ((size_t)(row0 + qi) * p.H + head0 + g) * HD;
    const float inv = 1.f / l[h];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i)
      *reinterpret_cast<__nv_bfloat162*>(o + i * 8 + t * 2) =
          __floats2bfloat162_rn(acc[i][h * 2] * inv, acc[i][h * 2 + 1] * inv);
  }
}

template <int HD>
int launch_mma(const MmaParams& p, int run_decode, int run_prefill, cudaStream_t stream) {
  constexpr int kTileBytes = kKeyTile * HD * 2;
  if (run_decode) {
    const int smem = 4 * kTileBytes + 16 * HD * 2;  // merge scratch (2*64 + 64*HD floats) fits in the stages
    auto kern = decode_attention_kernel<HD>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return asb::fail("decode_attention: %s", cudaGetErrorString(e));
    dim3 grid(p.short_rows > 0 ? p.short_rows : p.T, p.KV * p.HC, p.NP);
    asb::launch(kern, grid, kThreads, smem, stream, p);
    if (int rc = asb::check_launch("decode_attention")) return rc;
  }
  if (run_prefill) {
    const int smem = 4 * kTileBytes + kPrefillRows * HD * 2;
    auto kern = prefill_attention_kernel<HD>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return asb::fail("prefill_attention: %s", cudaGetErrorString(e));
    const long long blocks = (long long)((p.T + p.QT - 1) / p.QT + p.R) * p.KV * p.HC;
    if (blocks > 0x7fffffffLL) return asb::fail("prefill_attention: %lld blocks exceed the grid", blocks);
    asb::launch(kern, dim3((unsigned)blocks), kPrefillThreads, smem, stream, p);
    if (int rc = asb::check_launch("prefill_attention")) return rc;
  }
  return 0;
}

}  // namespace

// How many blocks of the decode kernel the device holds at once (blocks per SM x SMs), which is
// what the caller's choice of key partitions aims to fill evenly; 0 for a head size not served.
extern "C" int asb_decode_attention_resident_blocks(int hd) {
  if (hd != 64 && hd != 128) return 0;
  static int cached[2] = {0, 0};
  int& slot = cached[hd == 128];
  if (slot) return slot;
  int device = 0, sms = 0, per_sm = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
    return 0;
  const int smem = 4 * kKeyTile * hd * 2 + 16 * hd * 2;
  cudaError_t e;
  if (hd == 64) {
    cudaFuncSetAttribute(decode_attention_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_attention_kernel<64>, kThreads, smem);
  } else {
    cudaFuncSetAttribute(decode_attention_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_attention_kernel<128>, kThreads, smem);
  }
  if (e != cudaSuccess || per_sm < 1) return 0;
  return slot = per_sm * sms;
}

// 1 if this (head size, group) is served by the tensor-core kernels.
extern "C" int asb_attention_mma_supported(int hd, int group) {
  return (hd == 64 || hd == 128) && group >= 1 ? 1 : 0;
}

// Rows of requests with at most 8 new tokens go through the decode kernel (`run_decode`), longer
// portions through the prefill kernel (`run_prefill`); the caller says which kinds the step
// holds. Partitions (PS, NP) apply to the decode kernel only, so steps that also hold longer
// portions use NP == 1. With NP > 1 every block writes (max, sum, accumulator) to the scratch
// and the caller runs asb_attention_reduce over it afterwards. (Letting the last block to arrive
// merge the partitions inside this kernel was measured and was slower than the second launch.)
// short_rows > 0 (with run_decode alone): the number of rows of requests with at most 8 tokens in
// a step that also holds longer portions; the decode kernel then starts blocks for those rows
// only, and the scratch is [short_rows, H, NP(, hd)], merged by asb_attention_reduce_short.
extern "C" int asb_paged_attention_mma(void* out, const void* q, const void* k_cache,
                                       const void* v_cache, const int* block_tables,
                                       const int* req_q_start, const int* req_pos_start,
                                       float* part_m, float* part_l, float* part_acc,
                                       int num_tokens, int R, int H, int KV, int hd, int bs,
                                       int table_width, int window, int PS, int NP, float scale,
                                       int run_decode, int run_prefill, int all_single, int short_rows,
                                       cudaStream_t stream) {
  if (num_tokens == 0 || R == 0) return 0;
  if (short_rows < 0 || short_rows > num_tokens || (short_rows > 0 && (run_prefill || all_single)))
    return asb::fail("paged_attention_mma: %d short rows of %d tokens (decode-only launches of mixed steps)", short_rows, num_tokens);
  if (KV < 1 || H % KV) return asb::fail("paged_attention_mma: %d heads over %d kv heads", H, KV);
  if (!asb_attention_mma_supported(hd, H / KV)) return asb::fail("paged_attention_mma: head_dim %d is not 64 or 128", hd);
  if (NP < 1 || PS < kKeyTile || PS % kKeyTile) return asb::fail("paged_attention_mma: partition size %d must be a positive multiple of %d", PS, kKeyTile);
  if (NP > 1 && run_prefill) return asb::fail("paged_attention_mma: key partitions are for decode-only launches");
  if (NP > 1 && (!part_m || !part_l || !part_acc)) return asb::fail("paged_attention_mma: %d partitions need scratch", NP);
  if (NP > 65535) return asb::fail("paged_attention_mma: %d partitions exceed the grid", NP);
  MmaParams p;
  p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out;
  p.k_cache = (const __nv_bfloat16*)k_cache; p.v_cache = (const __nv_bfloat16*)v_cache;
  p.block_tables = block_tables; p.req_q_start = req_q_start; p.req_pos_start = req_pos_start;
  p.part_m = part_m; p.part_l = part_l; p.part_acc = part_acc;
  p.T = num_tokens; p.R = R; p.H = H; p.KV = KV; p.bs = bs; p.table_width = table_width;
  p.G = H / KV;
  p.GC = p.G < 16 ? p.G : 16;
  p.HC = (p.G + p.GC - 1) / p.GC;
  p.QT = kPrefillRows / p.GC;
  if (p.KV * p.HC > 65535) return asb::fail("paged_attention_mma: too many head chunks");
  p.window = window; p.PS = PS; p.NP = NP; p.all_single = all_single; p.short_rows = short_rows; p.scale = scale;
  if (hd == 64) return launch_mma<64>(p, run_decode, run_prefill, stream);
  return launch_mma<128>(p, run_decode, run_prefill, stream);
}
