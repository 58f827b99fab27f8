// Sampling on the device, one block per row of float32 logits [B, V].
//
// The rules are the reference sampler's (atomserve/sampler.py:82-129): top-k on the raw
// logits (0 or >= V keeps all; temperature 0 is the single best), divide by the temperature,
// softmax over the kept, top-p drops a token once the probability mass ranked above it has
// reached top_p (the best always stays), then an exponential race: argmax of p_i / E_i with
// E_i ~ Exp(1) picks token i with probability p_i / sum(p). The presence penalty is a
// separate scatter that runs first (atomserve/sampler.py:144-168).
//
// The reference sorts (torch.topk, or its 1024-thread Metal kernel, atomserve/kernels.py:336-435).
// Here nothing is sorted: the k-th largest logit is found by a radix select on order-preserving
// integer keys (four 8-bit digits, counting histograms in shared memory), and the top-p cut
// by the same walk over histograms of probability mass, kept as 64-bit fixed point so that
// the sums do not depend on the order of the atomic additions. Ties at a cut are broken towards
// the lower token id, by a third select over the ids. When top-k leaves at most 1024
// candidates they are compacted into shared memory and the later passes read only those.
//
// Random numbers are Philox-4x32-10 keyed by the row's seed; the counter is (token id, the
// row's draw counter). A seeded request passes its own seed and counts its own draws, so what
// it draws does not depend on its neighbours in the batch (atomserve/sampler.py:123-127).
#include "common.cuh"

namespace {

constexpr int kThreads = 1024;
constexpr int kBins = 256;
constexpr int kHistCopies = 8;
constexpr int kCompact = 1024;

__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // ascending with the float order
}

struct Philox {
  static __device__ __forceinline__ void round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
    c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
  }
  static __device__ __forceinline__ uint32_t draw(uint64_t seed, uint64_t counter, uint32_t index) {
    uint32_t c[4] = {index, (uint32_t)counter, (uint32_t)(counter >> 32), 0x5a17u};
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
    for (int i = 0; i < 10; ++i) {
      round(c, k0, k1);
      k0 += 0x9E3779B9u;
      k1 += 0xBB67AE85u;
    }
    return c[0];
  }
};

// A row as the passes see it: the full logits (id == position) or the compacted candidates.
struct RowView {
  const float* val;
  const int* id;  // null: identity
  int n;
  __device__ __forceinline__ float value(int i) const { return val[i]; }
  __device__ __forceinline__ int token(int i) const { return id ? id[i] : i; }
};

struct Scratch {
  unsigned long long hist[kHistCopies][kBins];
  float red[32];
  int red_i[32];
  unsigned long long bcast[4];
  float cand_val[kCompact];
  int cand_id[kCompact];
  int cand_n;
};

// Calls f(i, value, valid) for every element of the row, the same number of times in every
// thread of the block (valid false: no such element), so that f may use warp-wide ballots. The
// full row is read with 16-byte loads, four in flight per thread; one scalar load per trip would
// leave a row of 150,000 logits bound by the latency of its loads.
template <typename F>
__device__ __forceinline__ void for_each_value(const RowView& row, F f) {
  int done = 0;
  if (row.id == nullptr && ((uintptr_t)row.val & 15) == 0) {
    const float4* v4 = reinterpret_cast<const float4*>(row.val);
    const int n4 = row.n >> 2;
    for (int base = 0; base < n4; base += blockDim.x * 4) {
      float4 x[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int at = base + threadIdx.x + u * blockDim.x;
        x[u] = at < n4 ? v4[at] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int at = base + threadIdx.x + u * blockDim.x;
        const float e[4] = {x[u].x, x[u].y, x[u].z, x[u].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) f(at * 4 + k, e[k], at < n4);
      }
    }
    done = n4 << 2;
  }
  for (int base = done; base < row.n; base += blockDim.x) {
    const int i = base + threadIdx.x;
    const bool valid = i < row.n;
    f(i, valid ? row.value(i) : 0.f, valid);
  }
}

// Descending radix select over 32-bit keys. `item(i, value, key, weight)` says whether element i takes
// part, its key and its non-negative integer weight. Finds the largest key c such that the
// weight of all taking-part elements with key > c is < target <= that weight plus the weight
// of key == c. Returns c, and in `above` the weight strictly above c. (With weight 1 and
// target k this is the k-th largest key.) If the total weight is below target, returns 0 with
// `above` = total: everything is kept.
//
// `last_shift` 16 stops after the two high digits: the result then has its low 16 bits clear and
// names a bin of 65,536 keys, `above` and `equal` counting what lies above and inside it.
//
// A whole row's first digit falls into a handful of bins (sign and exponent of logits that lie
// close together), so lanes of a warp that hit the same bin hand their weight to one of them
// before the atomic addition: up to three such groups a warp, the rest add for themselves.
//
// kUnit: every weight is 1 (a count). A group's weight is then its number of lanes, and the
// histograms are 32-bit, whose shared-memory atomics are native (64-bit ones are not).
template <bool kUnit, typename Item>
__device__ uint32_t radix_select(const RowView& row, Scratch& s, unsigned long long target,
                                 unsigned long long* above, unsigned long long* equal, Item item,
                                 int last_shift = 0) {
  uint32_t prefix = 0, mask = 0;
  unsigned long long acc = 0;
  const int lane = threadIdx.x & 31;
  for (int shift = 24; shift >= last_shift; shift -= 8) {
    for (int i = threadIdx.x; i < kHistCopies * kBins; i += blockDim.x) (&s.hist[0][0])[i] = 0ull;
    __syncthreads();
    unsigned long long* h = s.hist[(threadIdx.x >> 5) % kHistCopies];
    unsigned int* h32 = reinterpret_cast<unsigned int*>(h);  // kUnit: the copy's first 256 words
    for_each_value(row, [&](int i, float v, bool valid) {
      uint32_t key = 0;
      unsigned long long w = 0;
      bool take = valid && item(i, v, key, w) && (key & mask) == prefix && w;
      const uint32_t bin = (key >> shift) & 255u;
      unsigned remaining = __ballot_sync(0xffffffffu, take);
      for (int round = 0; round < 3 && remaining; ++round) {
        const int leader = __ffs(remaining) - 1;
        const uint32_t leader_bin = __shfl_sync(0xffffffffu, bin, leader);
        const bool mine = take && bin == leader_bin;
        const unsigned group = __ballot_sync(0xffffffffu, mine);
        if (kUnit) {
          if (lane == leader) atomicAdd(&h32[leader_bin], (unsigned int)__popc(group));
        } else {
          unsigned long long sum = mine ? w : 0ull;
          if (group & (group - 1))  // more than one lane in the group (the whole warp agrees)
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
          if (lane == leader) atomicAdd(&h[leader_bin], sum);
        }
        if (mine) take = false;
        remaining &= ~group;
      }
      if (take) {
        if (kUnit) atomicAdd(&h32[bin], 1u);
        else atomicAdd(&h[bin], w);
      }
    });
    __syncthreads();
    unsigned long long bin_total = 0;
    if (threadIdx.x < kBins)
      for (int c = 0; c < kHistCopies; ++c)
        bin_total += kUnit ? (unsigned long long)reinterpret_cast<const unsigned int*>(s.hist[c])[threadIdx.x] : s.hist[c][threadIdx.x];
    __syncthreads();  // copy 0's 32-bit words lie where the 64-bit totals are written next
    if (threadIdx.x < kBins) s.hist[0][threadIdx.x] = bin_total;
    __syncthreads();
    if (threadIdx.x < 32) {
      // The first bin, from the top, at which the weight so far reaches the target: lane l walks
      // bins 255 - 8l downwards, after a scan over the lanes has told it the weight above them.
      unsigned long long mine[8], lane_sum = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        mine[j] = s.hist[0][kBins - 1 - (8 * lane + j)];
        lane_sum += mine[j];
      }
      unsigned long long upto = lane_sum;  // inclusive scan over the lanes
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long t = __shfl_up_sync(0xffffffffu, upto, o);
        if (lane >= o) upto += t;
      }
      unsigned long long a = acc + upto - lane_sum;
      int found = -1;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (found < 0) {
          if (a + mine[j] >= target) found = j;
          else a += mine[j];
        }
      const unsigned hit = __ballot_sync(0xffffffffu, found >= 0);
      if (hit == 0u) {
        if (lane == 31) {  // the whole set weighs less than the target
          s.bcast[0] = acc + upto;
          s.bcast[1] = (unsigned long long)(long long)-1;
          s.bcast[3] = 0ull;
        }
      } else if (lane == __ffs(hit) - 1) {
        unsigned long long in_bin = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j == found) in_bin = mine[j];
        s.bcast[0] = a;
        s.bcast[1] = (unsigned long long)(long long)(kBins - 1 - (8 * lane + found));
        s.bcast[3] = in_bin;
      }
    }
    __syncthreads();
    acc = s.bcast[0];
    const long long digit = (long long)s.bcast[1];
    *equal = s.bcast[3];  // after the last digit: the weight of key == result
    __syncthreads();
    if (digit < 0) {  // the whole set weighs less than target
      *above = acc;
      return 0u;
    }
    prefix |= (uint32_t)digit << shift;
    mask |= 255u << shift;
  }
  *above = acc;
  return prefix;
}

// The cut of one stage: keep key > cut_key, and of key == cut_key the tokens with id <= cut_id.
struct Cut {
  uint32_t key;
  int id;
  __device__ __forceinline__ bool keeps(uint32_t k, int token) const {
    return k > key || (k == key && token <= id);
  }
};

// After a select that found `key` with `need` more units wanted among the ties: the id below
// which ties are kept. Unit weights (top-k) keep exactly `need` ties.
template <typename Item>
__device__ Cut cut_with_ties(const RowView& row, Scratch& s, uint32_t key, unsigned long long need,
                             unsigned long long equal, unsigned long long unit, Item item) {
  Cut cut{key, 0x7fffffff};
  if (key == 0u || unit == 0ull) return cut;
  // how many ties are wanted: the smallest t with t * unit >= need
  const unsigned long long want = (need + unit - 1) / unit;
  if (want * unit >= equal) return cut;  // all of them: no pass over the ids
  unsigned long long dummy, dummy2;
  auto by_id = [&](int i, float v, uint32_t& k2, unsigned long long& w2) {
    uint32_t k;
    unsigned long long w;
    if (!item(i, v, k, w) || k != key) return false;
    k2 = ~(uint32_t)row.token(i);  // descending on ~id is ascending on id
    w2 = 1ull;
    return true;
  };
  const uint32_t idk = radix_select<true>(row, s, want, &dummy, &dummy2, by_id);
  if (idk != 0u) cut.id = (int)~idk;
  return cut;
}

__device__ int row_argmax(const RowView& row, Scratch& s, float* best_value) {
  float best = -INFINITY;
  int best_id = 0x7fffffff;
  int done = 0;
  if (row.id == nullptr && ((uintptr_t)row.val & 15) == 0) {
    // the full row: 16-byte loads, four in flight per thread
    const float4* v4 = reinterpret_cast<const float4*>(row.val);
    const int n4 = row.n >> 2;
    for (int i = threadIdx.x; i < n4; i += blockDim.x * 4) {
      float4 x[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int at = i + u * blockDim.x;
        x[u] = at < n4 ? v4[at] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int t0 = (i + u * blockDim.x) * 4;
        const float e[4] = {x[u].x, x[u].y, x[u].z, x[u].w};
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (e[k] > best || (e[k] == best && t0 + k < best_id)) { best = e[k]; best_id = t0 + k; }
      }
    }
    done = n4 << 2;
  }
  for (int i = done + threadIdx.x; i < row.n; i += blockDim.x) {
    const float v = row.value(i);
    const int t = row.token(i);
    if (v > best || (v == best && t < best_id)) { best = v; best_id = t; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_id, o);
    if (ov > best || (ov == best && oi < best_id)) { best = ov; best_id = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) { s.red[warp] = best; s.red_i[warp] = best_id; }
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    best = lane < nw ? s.red[lane] : -INFINITY;
    best_id = lane < nw ? s.red_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_id, o);
      if (ov > best || (ov == best && oi < best_id)) { best = ov; best_id = oi; }
    }
    if (lane == 0) { s.red[0] = best; s.red_i[0] = best_id; }
  }
  __syncthreads();
  const int id = s.red_i[0] == 0x7fffffff ? 0 : s.red_i[0];  // a row of NaN or -inf only
  if (best_value) *best_value = s.red[0];
  __syncthreads();
  return id;
}

// Probability mass of one token as 64-bit fixed point: exp((v - max) / T) * 2^32.
__device__ __forceinline__ unsigned long long mass_of(float v, float vmax, float inv_t) {
  const float w = expf((v - vmax) * inv_t);  // in [0, 1]
  return (unsigned long long)((double)w * 4294967296.0);
}

__global__ void __launch_bounds__(kThreads)
sample_rows_kernel(int* __restrict__ out, const float* __restrict__ logits, int V,
                   const float* __restrict__ temperature, const int* __restrict__ top_k,
                   const float* __restrict__ top_p, const unsigned long long* __restrict__ seed,
                   const unsigned long long* __restrict__ counter) {
  asb::pdl_wait();  // the stream's previous kernel has completed (programmatic dependent launch)
  asb::pdl_launch_dependents();
  __shared__ Scratch s;
  const int b = blockIdx.x;
  RowView row{logits + (size_t)b * V, nullptr, V};
  const float temp = temperature[b];

  float vmax;
  const int best = row_argmax(row, s, &vmax);
  if (!(temp > 0.f)) {  // greedy: the single best, lowest id among equals
    if (threadIdx.x == 0) out[b] = best;
    return;
  }
  const float inv_t = 1.f / temp;

  // top-k
  const int k = top_k[b];
  Cut kcut{0u, 0x7fffffff};
  if (k > 0 && k < V) {
    auto unit = [&](int i, float v, uint32_t& key, unsigned long long& w) {
      key = order_key(v);
      w = 1ull;
      return true;
    };
    unsigned long long above, equal;
    bool early = false;
    if (k <= kCompact) {
      // The two high digits of the k-th largest key: if everything from that bin of 65,536 keys
      // upwards fits the candidate buffer (it holds at least k), gather it now and finish the
      // selection, like all later passes, on the candidates in shared memory.
      // Only keys within four first-digit bins of the largest (a factor of 16 or so below the best
      // logit when it is positive) are counted here, which spares the atomics of nearly the whole
      // row; if fewer than k lie there, `high` comes back 0 and the full selection below runs.
      const uint32_t top_bin = order_key(vmax) >> 24;
      const uint32_t floor_key = top_bin >= 3u ? (top_bin - 3u) << 24 : 0u;
      auto unit_near_top = [&](int i, float v, uint32_t& key, unsigned long long& w) {
        key = order_key(v);
        w = 1ull;
        return key >= floor_key;
      };
      const uint32_t high = radix_select<true>(row, s, (unsigned long long)k, &above, &equal, unit_near_top, 16);
      if (high != 0u && above + equal <= (unsigned long long)kCompact) {
        early = true;
        if (threadIdx.x == 0) s.cand_n = 0;
        __syncthreads();
        for_each_value(row, [&](int i, float v, bool valid) {
          if (valid && order_key(v) >= high) {
            const int at = atomicAdd(&s.cand_n, 1);
            if (at < kCompact) { s.cand_val[at] = v; s.cand_id[at] = i; }
          }
        });
        __syncthreads();
        row = RowView{s.cand_val, s.cand_id, min(s.cand_n, kCompact)};
        const uint32_t key = radix_select<true>(row, s, (unsigned long long)k, &above, &equal, unit);
        kcut = cut_with_ties(row, s, key, (unsigned long long)k - above, equal, 1ull, unit);
      }
    }
    if (!early) {
      const uint32_t key = radix_select<true>(row, s, (unsigned long long)k, &above, &equal, unit);
      kcut = cut_with_ties(row, s, key, (unsigned long long)k - above, equal, 1ull, unit);
      if (k <= kCompact) {  // later passes read the candidates from shared memory
        if (threadIdx.x == 0) s.cand_n = 0;
        __syncthreads();
        for_each_value(row, [&](int i, float v, bool valid) {
          if (valid && kcut.keeps(order_key(v), i)) {
            const int at = atomicAdd(&s.cand_n, 1);
            if (at < kCompact) { s.cand_val[at] = v; s.cand_id[at] = i; }
          }
        });
        __syncthreads();
        row = RowView{s.cand_val, s.cand_id, min(s.cand_n, kCompact)};
        kcut = Cut{0u, 0x7fffffff};
      }
    }
  }

  // total mass of the kept, then the top-p cut
  auto massed = [&](int i, float v, uint32_t& key, unsigned long long& w) {
    key = order_key(v);
    if (!kcut.keeps(key, row.token(i))) return false;
    w = mass_of(v, vmax, inv_t);
    return true;
  };
  unsigned long long total = 0;
  for_each_value(row, [&](int i, float v, bool valid) {
    uint32_t key;
    unsigned long long w;
    if (valid && massed(i, v, key, w)) total += w;
  });
  {
    // integer sum over the block: exact, so independent of the order
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s.hist[0][threadIdx.x >> 5] = total;
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned long long t = 0;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += s.hist[0][w];
      s.bcast[2] = t;
    }
    __syncthreads();
    total = s.bcast[2];
    __syncthreads();
  }

  Cut pcut{0u, 0x7fffffff};
  const float p = top_p[b];
  if (p < 1.f) {
    // keep a token while the mass ranked above it is < p * total: find the first key whose
    // cumulative mass (itself included) exceeds p * total, ties by ascending id
    unsigned long long target = (unsigned long long)ceil((double)p * (double)total);
    if (target < 1ull) target = 1ull;  // the best token always stays
    if (target > total) target = total;
    unsigned long long above, equal;
    const uint32_t key = radix_select<false>(row, s, target, &above, &equal, massed);
    // mass of one tied token (all ties share the key, hence the value)
    unsigned long long unit = mass_of(__uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key), vmax, inv_t);
    pcut = cut_with_ties(row, s, key, target - above, equal, unit, massed);
  }

  // exponential race among the kept
  const unsigned long long sd = seed[b], ctr = counter[b];
  float best_score = -1.f;
  int best_token = 0x7fffffff;
  for_each_value(row, [&](int i, float v, bool valid) {
    if (!valid) return;
    const uint32_t key = order_key(v);
    const int token = row.token(i);
    if (!kcut.keeps(key, token) || !pcut.keeps(key, token)) return;
    const float w = expf((v - vmax) * inv_t);
    const uint32_t bits = Philox::draw(sd, ctr, (uint32_t)token);
    const float u = ((float)(bits >> 8) + 0.5f) * (1.f / 16777216.f);  // (0, 1)
    const float e = fmaxf(-logf(u), 1e-10f);
    const float score = w / e;
    if (score > best_score || (score == best_score && token < best_token)) {
      best_score = score;
      best_token = token;
    }
  });
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float os = __shfl_xor_sync(0xffffffffu, best_score, o);
    const int ot = __shfl_xor_sync(0xffffffffu, best_token, o);
    if (os > best_score || (os == best_score && ot < best_token)) { best_score = os; best_token = ot; }
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) { s.red[threadIdx.x >> 5] = best_score; s.red_i[threadIdx.x >> 5] = best_token; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (s.red[w] > best_score || (s.red[w] == best_score && s.red_i[w] < best_token)) {
        best_score = s.red[w];
        best_token = s.red_i[w];
      }
    out[b] = best_token == 0x7fffffff ? best : best_token;
  }
}

__global__ void argmax_rows_kernel(int* __restrict__ out, const float* __restrict__ logits, int V) {
  asb::pdl_wait();  // the stream's previous kernel has completed (programmatic dependent launch)
  asb::pdl_launch_dependents();
  __shared__ Scratch s;
  RowView row{logits + (size_t)blockIdx.x * V, nullptr, V};
  const int best = row_argmax(row, s, nullptr);
  if (threadIdx.x == 0) out[blockIdx.x] = best;
}

__global__ void presence_penalty_kernel(float* __restrict__ logits, const int* __restrict__ rows,
                                        const int* __restrict__ tokens,
                                        const float* __restrict__ amounts, int n, int V) {
  asb::pdl_wait();  // the stream's previous kernel has completed (programmatic dependent launch)
  asb::pdl_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n && tokens[i] >= 0 && tokens[i] < V) logits[(size_t)rows[i] * V + tokens[i]] -= amounts[i];
}

}  // namespace

extern "C" int asb_argmax_rows(int* out, const float* logits, int B, int V, cudaStream_t stream) {
  if (B == 0) return 0;
  asb::launch(argmax_rows_kernel, B, kThreads, 0, stream, out, logits, V);
  return asb::check_launch("argmax_rows");
}

// Each (row, token) pair must appear once: the penalty is subtracted once per distinct token.
extern "C" int asb_presence_penalty(float* logits, const int* rows, const int* tokens,
                                    const float* amounts, int n, int V, cudaStream_t stream) {
  if (n == 0) return 0;
  asb::launch(presence_penalty_kernel, (n + 255) / 256, 256, 0, stream, logits, rows, tokens, amounts, n, V);
  return asb::check_launch("presence_penalty");
}

extern "C" int asb_sample_rows(int* out, const float* logits, int B, int V,
                               const float* temperature, const int* top_k, const float* top_p,
                               const unsigned long long* seed, const unsigned long long* counter,
                               cudaStream_t stream) {
  if (B == 0) return 0;
  if (V < 1) return asb::fail("sample_rows: vocabulary %d", V);
  asb::launch(sample_rows_kernel, B, kThreads, 0, stream, out, logits, V, temperature, top_k, top_p, seed, counter);
  return asb::check_launch("sample_rows");
}
