// Paged grouped-query attention over the cache, for any mix of prompt portions and decoded
// tokens in one launch. This is the general kernel: float32 arithmetic on CUDA cores for both
// element types, any head size up to 256, any number of heads and groups, any page size, an
// optional sliding window. It is the whole of the float32 path and the fallback of the
// bfloat16 path for sizes its tensor-core kernels refuse.
//
// What it computes (atomserve/model.py:199-232 for a portion, :269-289 for single queries;
// the split into partitions follows atomserve/kernels.py:147-334): a query at absolute
// position p of request r attends keys of r at positions j with j <= p (and j > p - window
// when a window is set); softmax(q.k * scale) v with query head h reading kv head h / G.
// Scores, the running maximum and sum, and the accumulator are float32; the output is
// rounded once.
//
// Work split. grid.x walks query tiles: each request's new tokens are cut into tiles of QT
// tokens, and a block finds its (request, tile) by walking the per-request token counts, so no
// tile list has to be built on the host. grid.y is (kv head, chunk of GC of its query heads);
// the QT*GC <= 32 rows of a block share every key and value it loads. grid.z is the key
// partition: partitions are aligned to absolute key positions (multiples of PS), so the value
// computed for a row does not depend on what else is in the batch. With one partition the block
// writes the output; otherwise it writes (max, sum, accumulator) and `attention_reduce` merges.
//
// Keys are visited in tiles of 32 at absolute multiples of 32; lane = key for the scores, lane =
// output column (mod 32) for the weighted sum of values.
#include "common.cuh"

namespace {

constexpr int kWarps = 8;
constexpr int kRowsPerWarp = 4;
constexpr int kMaxRows = kWarps * kRowsPerWarp;  // 32
constexpr int kKeyTile = 32;

struct AttentionParams {
  const void* q;         // [T, H, hd]
  void* out;             // [T, H, hd]
  const void* k_cache;   // [num_blocks, KV, bs, hd]
  const void* v_cache;
  const int* block_tables;   // [R, table_width]
  const int* req_q_start;    // [R + 1] first row of each request in the flat batch
  const int* req_pos_start;  // [R] position of each request's first new token
  float* part_m;             // [T, H, NP]      (NP > 1 only)
  float* part_l;             // [T, H, NP]
  float* part_acc;           // [T, H, NP, hd]
  int R, H, KV, hd, bs, table_width;
  int QT, GC, HC;            // tokens per tile, heads per chunk, chunks per kv head
  int window;                // 0: none
  int PS, NP;                // partition size in keys, number of partitions (grid.z)
  float scale;
};

template <typename T, int EPL>
__global__ void __launch_bounds__(kWarps * 32)
paged_attention_kernel(const AttentionParams p) {
  asb::pdl_wait();  // the stream's previous kernel has completed (programmatic dependent launch)
  asb::pdl_launch_dependents();
  extern __shared__ float smem[];
  const int hd = p.hd;
  const int kstride = hd | 1;  // odd stride: lanes reading one column of 32 keys hit 32 banks
  float* q_s = smem;                          // [32][hd]
  float* k_s = q_s + kMaxRows * hd;           // [32][kstride]
  float* v_s = k_s + kKeyTile * kstride;      // [32][hd]
  __shared__ int block_of_key[kKeyTile];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.H / p.KV;

  // Which request and tile is this block's?
  int tile = blockIdx.x, r = 0, q_len = 0;
  for (; r < p.R; ++r) {
    q_len = p.req_q_start[r + 1] - p.req_q_start[r];
    const int tiles = (q_len + p.QT - 1) / p.QT;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (r == p.R) return;
  const int q0 = tile * p.QT;
  const int nq = min(p.QT, q_len - q0);
  const int row0 = p.req_q_start[r] + q0;      // first flat row of the tile
  const int pos0 = p.req_pos_start[r] + q0;    // position of the tile's first query
  const int kvh = blockIdx.y / p.HC;
  const int head0 = kvh * G + (blockIdx.y % p.HC) * p.GC;
  const int gc = min(p.GC, kvh * G + G - head0);
  const int num_rows = nq * gc;  // row rr = qi * gc + g

  // Keys this block visits.
  const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int hi = pos0 + nq;  // exclusive
  const int part = lo / p.PS + blockIdx.z;
  const int key_lo = max(lo, part * p.PS);
  const int key_hi = (int)min((long long)hi, (long long)(part + 1) * p.PS);

  const T* q = (const T*)p.q;
  for (int i = threadIdx.x; i < num_rows * hd; i += blockDim.x) {
    const int rr = i / hd, e = i - rr * hd;
    const int qi = rr / gc, g = rr - qi * gc;
    q_s[rr * hd + e] = asb::to_float(q[((size_t)(row0 + qi) * p.H + head0 + g) * hd + e]) * p.scale;
  }

  float m[kRowsPerWarp], l[kRowsPerWarp], acc[kRowsPerWarp][EPL];
#pragma unroll
  for (int s = 0; s < kRowsPerWarp; ++s) {
    m[s] = -INFINITY;
    l[s] = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[s][e] = 0.f;
  }

  const T* kc = (const T*)p.k_cache;
  const T* vc = (const T*)p.v_cache;
  const int* table = p.block_tables + (size_t)r * p.table_width;

  for (int kt0 = (key_lo / kKeyTile) * kKeyTile; kt0 < key_hi; kt0 += kKeyTile) {
    __syncthreads();  // previous tile fully consumed (and q_s written, first time round)
    if (threadIdx.x < kKeyTile) {
      const int j = kt0 + threadIdx.x;
      block_of_key[threadIdx.x] = (j >= key_lo && j < key_hi) ? table[j / p.bs] : -1;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kKeyTile * hd; i += blockDim.x) {
      const int jj = i / hd, e = i - jj * hd;
      const int blk = block_of_key[jj];
      float kv = 0.f, vv = 0.f;
      if (blk >= 0) {
        const size_t at = (((size_t)blk * p.KV + kvh) * p.bs + (kt0 + jj) % p.bs) * hd + e;
        kv = asb::to_float(kc[at]);
        vv = asb::to_float(vc[at]);
      }
      k_s[jj * kstride + e] = kv;
      v_s[jj * hd + e] = vv;
    }
    __syncthreads();

    const int j = kt0 + lane;
    const bool in_range = block_of_key[lane] >= 0;
#pragma unroll
    for (int s = 0; s < kRowsPerWarp; ++s) {
      const int rr = warp + s * kWarps;
      if (rr >= num_rows) break;
      const int pq = pos0 + rr / gc;
      const bool visible = in_range && j <= pq && (p.window <= 0 || j > pq - p.window);
      float score = -INFINITY;
      if (visible) {
        const float* qrow = q_s + rr * hd;
        const float* krow = k_s + lane * kstride;
        float d = 0.f;
        for (int e = 0; e < hd; ++e) d = fmaf(qrow[e], krow[e], d);
        score = d;
      }
      const float m_new = fmaxf(m[s], asb::warp_max(score));
      if (m_new == -INFINITY) continue;  // this row sees none of these keys
      const float corr = expf(m[s] - m_new);
      const float pj = visible ? expf(score - m_new) : 0.f;
      l[s] = l[s] * corr + asb::warp_sum(pj);
      m[s] = m_new;
#pragma unroll
      for (int e = 0; e < EPL; ++e) acc[s][e] *= corr;
      for (int jj = 0; jj < kKeyTile; ++jj) {
        const float w = __shfl_sync(0xffffffffu, pj, jj);
        if (w == 0.f) continue;  // uniform across the warp
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
          const int col = e * 32 + lane;
          if (col < hd) acc[s][e] = fmaf(w, v_s[jj * hd + col], acc[s][e]);
        }
      }
    }
  }

  // Results.
#pragma unroll
  for (int s = 0; s < kRowsPerWarp; ++s) {
    const int rr = warp + s * kWarps;
    if (rr >= num_rows) break;
    const int qi = rr / gc, g = rr - qi * gc;
    const size_t row = (size_t)(row0 + qi) * p.H + head0 + g;
    if (p.NP == 1) {
      T* o = (T*)p.out + row * hd;
      const float inv = 1.f / l[s];
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const int col = e * 32 + lane;
        if (col < hd) o[col] = asb::from_float<T>(acc[s][e] * inv);
      }
    } else {
      const size_t at = row * p.NP + blockIdx.z;
      if (lane == 0) {
        p.part_m[at] = m[s];
        p.part_l[at] = l[s];
      }
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const int col = e * 32 + lane;
        if (col < hd) p.part_acc[at * hd + col] = acc[s][e];
      }
    }
  }
}

// Merge the partitions of one (token, head): weights exp(m_p - max m), empty partitions (sum 0)
// are skipped, in ascending order of partition (atomserve/kernels.py:308-334). The weights go
// through shared memory, kReduceChunk partitions at a time, so that the accumulator loads that
// follow are unconditional and several are in flight.
constexpr int kReduceChunk = 64;

// Short: the partial results are those of the short rows only, [short rows, H, NP(, hd)] (a step
// that mixes prompt portions with single tokens); block b merges head b % H of short row b / H
// into that row's place in `out`.
template <typename T, bool Short>
__global__ void attention_reduce_kernel(T* __restrict__ out, const float* __restrict__ part_m,
                                        const float* __restrict__ part_l,
                                        const float* __restrict__ part_acc, int NP, int hd,
                                        const int* __restrict__ req_q_start, int R, int limit, int H) {
  asb::pdl_wait();  // the stream's previous kernel has completed (programmatic dependent launch)
  asb::pdl_launch_dependents();
  __shared__ float weight[kReduceChunk];
  const size_t row = blockIdx.x;
  size_t out_row = row;
  if (Short) {
    int request;
    const int flat = asb::nth_short_row(req_q_start, R, limit, (int)(blockIdx.x / H), &request);
    if (flat < 0) return;
    out_row = (size_t)flat * H + blockIdx.x % H;
  }
  const float* pm = part_m + row * NP;
  const float* pl = part_l + row * NP;
  float mx = -INFINITY;
  for (int i = 0; i < NP; ++i)
    if (pl[i] > 0.f) mx = fmaxf(mx, pm[i]);
  float denom = 0.f;
  for (int i = 0; i < NP; ++i)
    if (pl[i] > 0.f) denom += pl[i] * expf(pm[i] - mx);
  // A row no partition wrote anything for (its sums zeroed by the caller) is not this kernel's:
  // in a step that mixes prompt portions with single tokens, the portions' rows were stored by
  // their own kernel and only the single tokens' rows have partial results.
  if (!(denom > 0.f)) return;
  const int e = threadIdx.x;  // the launch gives hd <= blockDim.x a thread per element, else strides
  float a[2] = {0.f, 0.f};    // up to two elements per thread (head sizes to 512 with 256 threads)
  for (int i0 = 0; i0 < NP; i0 += kReduceChunk) {
    const int n = min(kReduceChunk, NP - i0);
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) weight[i] = pl[i0 + i] > 0.f ? expf(pm[i0 + i] - mx) : -1.f;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int col = e + k * blockDim.x;
      if (col >= hd) break;
      const float* acc = part_acc + (row * NP + i0) * hd + col;
      for (int j0 = 0; j0 < n; j0 += 4) {
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (j0 + u < n) v[u] = acc[(size_t)(j0 + u) * hd];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (j0 + u < n && weight[j0 + u] >= 0.f) a[k] += v[u] * weight[j0 + u];
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int col = e + k * blockDim.x;
    if (col < hd) out[out_row * hd + col] = asb::from_float<T>(a[k] / denom);
  }
}

template <typename T>
int launch(const AttentionParams& p, int num_tokens, cudaStream_t stream) {
  const int epl = (p.hd + 31) / 32;
  const size_t smem = sizeof(float) * ((size_t)kMaxRows * p.hd + kKeyTile * (p.hd | 1) + kKeyTile * p.hd);
  const int tiles = (num_tokens + p.QT - 1) / p.QT + p.R;
  dim3 grid(tiles, p.KV * p.HC, p.NP);
#define ASB_ATTN_CASE(E)                                                                        \
  case E: {                                                                                     \
    auto kern = paged_attention_kernel<T, E>;                                                   \
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (e != cudaSuccess) return asb::fail("paged_attention: shared memory %zu: %s", smem, cudaGetErrorString(e)); \
    asb::launch(kern, grid, kWarps * 32, smem, stream, p);                                               \
    break;                                                                                      \
  }
  switch (epl) {
    ASB_ATTN_CASE(1)
    ASB_ATTN_CASE(2)
    ASB_ATTN_CASE(3)
    ASB_ATTN_CASE(4)
    ASB_ATTN_CASE(5)
    ASB_ATTN_CASE(6)
    ASB_ATTN_CASE(7)
    ASB_ATTN_CASE(8)
    default:
      return asb::fail("paged_attention: head_dim %d exceeds 256", p.hd);
  }
#undef ASB_ATTN_CASE
  if (int rc = asb::check_launch("paged_attention")) return rc;
  if (p.NP > 1) {
    int threads = 32;
    while (threads < p.hd && threads < 256) threads <<= 1;
    asb::launch(attention_reduce_kernel<T, false>, num_tokens * p.H, threads, 0, stream,
        (T*)p.out, p.part_m, p.part_l, p.part_acc, p.NP, p.hd, (const int*)nullptr, 0, 0, 1);
    return asb::check_launch("attention_reduce");
  }
  return 0;
}

}  // namespace

// Merge partition results written by any of the attention kernels: rows = tokens * heads.
extern "C" int asb_attention_reduce(void* out, const float* part_m, const float* part_l,
                                    const float* part_acc, int rows, int NP, int hd, int dtype,
                                    cudaStream_t stream) {
  if (rows == 0) return 0;
  if (hd < 1 || hd > 512) return asb::fail("attention_reduce: head_dim %d not in 1..512", hd);
  int threads = 32;
  while (threads < hd && threads < 256) threads <<= 1;
  ASB_DISPATCH_DTYPE(dtype, T,
                     asb::launch(attention_reduce_kernel<T, false>, rows, threads, 0, stream,
                         (T*)out, part_m, part_l, part_acc, NP, hd, (const int*)nullptr, 0, 0, 1));
  return asb::check_launch("attention_reduce");
}

// The same for partial results that cover only the rows of requests with at most `limit` tokens,
// [short_rows, H, NP(, hd)] in request order: each is merged into its row of out [T, H, hd].
extern "C" int asb_attention_reduce_short(void* out, const float* part_m, const float* part_l,
                                          const float* part_acc, const int* req_q_start, int R, int limit,
                                          int short_rows, int H, int NP, int hd, int dtype, cudaStream_t stream) {
  if (short_rows == 0) return 0;
  if (hd < 1 || hd > 512) return asb::fail("attention_reduce_short: head_dim %d not in 1..512", hd);
  if (!req_q_start || R < 1 || H < 1 || short_rows < 0) return asb::fail("attention_reduce_short: no requests");
  int threads = 32;
  while (threads < hd && threads < 256) threads <<= 1;
  ASB_DISPATCH_DTYPE(dtype, T,
                     asb::launch(attention_reduce_kernel<T, true>, short_rows * H, threads, 0, stream,
                         (T*)out, part_m, part_l, part_acc, NP, hd, req_q_start, R, limit, H));
  return asb::check_launch("attention_reduce_short");
}

// Query tile geometry for G query heads per kv head: GC heads per block, QT tokens per tile.
extern "C" void asb_attention_tile_shape(int G, int* QT, int* GC) {
  *GC = G < kMaxRows ? G : kMaxRows;
  *QT = kMaxRows / *GC;
}

// Float scratch needed when NP > 1: part_m and part_l take T*H*NP floats each, part_acc
// T*H*NP*hd. Every partition slot of every row is written before the reduction reads it.
extern "C" int asb_paged_attention(void* out, const void* q, const void* k_cache,
                                   const void* v_cache, const int* block_tables,
                                   const int* req_q_start, const int* req_pos_start,
                                   float* part_m, float* part_l, float* part_acc,
                                   int num_tokens, int R, int H, int KV, int hd, int bs,
                                   int table_width, int window, int PS, int NP, float scale,
                                   int dtype, cudaStream_t stream) {
  if (num_tokens == 0 || R == 0) return 0;
  if (KV < 1 || H % KV) return asb::fail("paged_attention: %d heads over %d kv heads", H, KV);
  if (hd < 1 || hd > 256) return asb::fail("paged_attention: head_dim %d not in 1..256", hd);
  if (NP < 1 || PS < kKeyTile || PS % kKeyTile) return asb::fail("paged_attention: partition size %d must be a positive multiple of %d", PS, kKeyTile);
  if (NP > 1 && (!part_m || !part_l || !part_acc)) return asb::fail("paged_attention: %d partitions need scratch", NP);
  if (NP > 65535) return asb::fail("paged_attention: %d partitions exceed the grid", NP);
  AttentionParams p;
  p.q = q; p.out = out; p.k_cache = k_cache; p.v_cache = v_cache;
  p.block_tables = block_tables; p.req_q_start = req_q_start; p.req_pos_start = req_pos_start;
  p.part_m = part_m; p.part_l = part_l; p.part_acc = part_acc;
  p.R = R; p.H = H; p.KV = KV; p.hd = hd; p.bs = bs; p.table_width = table_width;
  asb_attention_tile_shape(H / KV, &p.QT, &p.GC);
  p.HC = (H / KV + p.GC - 1) / p.GC;
  if (p.KV * p.HC > 65535) return asb::fail("paged_attention: too many head chunks");
  p.window = window; p.PS = PS; p.NP = NP; p.scale = scale;
  ASB_DISPATCH_DTYPE(dtype, T, return launch<T>(p, num_tokens, stream));
  return 0;
}
