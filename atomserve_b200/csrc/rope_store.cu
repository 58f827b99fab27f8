// Fused per-head RMSNorm of q and k, rotary position encoding of both, and the write of k and v
// into their cache pages: one launch per attention layer in place of a dozen elementwise ones
// (atomserve/kernels.py:66-145 is the reference's fused form; atomserve/model.py:326-333 the
// unfused one). All arithmetic is float32 and each value is rounded once, at the store.
//
// One warp owns one (token, head) vector. The vector is staged in shared memory so that the
// rotate-half partner (i, i + rotary_dim/2) can be read whatever the head size.
//
//   qkv          [T, (H + 2*KV) * hd]   rows ordered q heads | k heads | v heads
//   q_out        [T, H, hd]
//   k/v cache    [num_blocks, KV, block_size, hd]  (one cache entry); slot = block*block_size+offset
//   q_gain/k_gain  [hd] float32 or null (no per-head norm)
//   inv_freq     [rotary_dim/2] float32 or null (no rotation); dims >= rotary_dim pass through
//   slots        [T] int32, or null / negative entries: nothing is stored for that token
#include "common.cuh"
#include "gemm_partials.cuh"

namespace {

constexpr int kWarps = 4;
constexpr int kMaxHeadDim = 256;

template <typename T>
__global__ void qk_norm_rope_store_kernel(
    T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
    const T* __restrict__ qkv, const float* __restrict__ q_gain, const float* __restrict__ k_gain,
    const float* __restrict__ inv_freq, const int* __restrict__ positions,
    const int* __restrict__ slots, int H, int KV, int hd, int rotary_dim, int block_size,
    float eps) {
  asb::pdl_wait();  // the stream's previous kernel has completed (programmatic dependent launch)
  asb::pdl_launch_dependents();
  __shared__ float stage[kWarps][kMaxHeadDim];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y * kWarps + warp;
  const int t = blockIdx.x;
  if (head >= H + 2 * KV) return;
  float* s = stage[warp];
  const T* src = qkv + ((size_t)t * (H + 2 * KV) + head) * hd;

  const bool is_q = head < H;
  const bool is_k = !is_q && head < H + KV;
  const int slot = slots ? slots[t] : -1;
  T* dst;
  if (is_q) {
    dst = q_out + ((size_t)t * H + head) * hd;
  } else {
    if (slot < 0) return;
    const int kvh = is_k ? head - H : head - H - KV;
    const size_t block = slot / block_size, off = slot % block_size;
    dst = (is_k ? k_cache : v_cache) + ((block * KV + kvh) * block_size + off) * (size_t)hd;
  }

  if (!is_q && !is_k) {  // v: stored as it is
    for (int e = lane; e < hd; e += 32) dst[e] = src[e];
    return;
  }

  float ss = 0.f;
  for (int e = lane; e < hd; e += 32) {
    const float v = asb::to_float(src[e]);
    s[e] = v;
    ss += v * v;
  }
  const float* gain = is_q ? q_gain : k_gain;
  if (gain) {
    ss = asb::warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)hd + eps);
    for (int e = lane; e < hd; e += 32) s[e] = s[e] * rstd * gain[e];
  }
  __syncwarp();
  const int half = inv_freq ? rotary_dim / 2 : 0;
  const float pos = (float)positions[t];
  for (int i = lane; i < half; i += 32) {
    float sn, cs;
    sincosf(pos * inv_freq[i], &sn, &cs);
    const float a = s[i], b = s[i + half];
    dst[i] = asb::from_float<T>(a * cs - b * sn);
    dst[i + half] = asb::from_float<T>(b * cs + a * sn);
  }
  for (int e = 2 * half + lane; e < hd; e += 32) dst[e] = asb::from_float<T>(s[e]);
}

// Vector form for head sizes 32, 64, 128, 256 with the whole head rotated: each lane holds EPT
// consecutive elements, lanes 0-15 the first half of the head and lanes 16-31 the second, so a
// rotate-half partner is one shuffle away and nothing passes through shared memory. A warp
// takes kHeadsPerWarp heads of one token and computes the token's sines and cosines once: four
// heads when there are many tokens, one when there are few (decoding), where spreading the
// heads over more warps matters more than saving the trigonometry.
//
// qkv may also be given as the partial sums that the tensor-core GEMM left in its workspace
// (ps.ws set, qkv null): each lane then adds its elements' slots up itself and rounds the sums to
// T, as the GEMM's reduction kernel would have, which saves that kernel.
template <typename T, int EPT, int kHeadsPerWarp>
__global__ void qk_norm_rope_store_vec_kernel(
    T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
    const T* __restrict__ qkv, const asb::PartialSums ps, const float* __restrict__ q_gain,
    const float* __restrict__ k_gain, const float* __restrict__ inv_freq, const int* __restrict__ positions,
    const int* __restrict__ slots, int H, int KV, int block_size, float eps) {
  constexpr int hd = EPT * 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int head_first = (blockIdx.y * kWarps + warp) * kHeadsPerWarp;
  const int heads = H + 2 * KV;
  const int e0 = lane * EPT;  // this lane's first element
  // Positions and cache slots were uploaded before the step's first kernel, and the angles depend
  // on nothing else: all of this overlaps the previous kernel's tail. (Read from L2: an SM's L1
  // could still hold these addresses' lines from an earlier step.)
  int slot = -1;
  float cs[EPT], sn[EPT];
  if (head_first < heads) {
    slot = slots ? __ldcg(slots + t) : -1;
    if (inv_freq) {
      const float pos = (float)__ldcg(positions + t);
      const int i0 = (lane & 15) * EPT;
#pragma unroll
      for (int k = 0; k < EPT; ++k) sincosf(pos * inv_freq[i0 + k], &sn[k], &cs[k]);
    }
  }
  asb::pdl_wait();  // the stream's previous kernel has completed (programmatic dependent launch)
  asb::pdl_launch_dependents();
  if (head_first >= heads) return;
  struct alignas(sizeof(T) * EPT > 16 ? 16 : sizeof(T) * EPT) Vec { T v[EPT]; };

  for (int head = head_first; head < min(head_first + kHeadsPerWarp, heads); ++head) {
    const bool is_q = head < H;
    const bool is_k = !is_q && head < H + KV;
    T* dst;
    if (is_q) {
      dst = q_out + ((size_t)t * H + head) * hd;
    } else {
      if (slot < 0) continue;
      const int kvh = is_k ? head - H : head - H - KV;
      const size_t block = slot / block_size, off = slot % block_size;
      dst = (is_k ? k_cache : v_cache) + ((block * KV + kvh) * block_size + off) * (size_t)hd;
    }
    Vec in;
    if (ps.ws) {
      const int col = head * hd + e0;
      const int n = asb::partial_slots(ps, col / asb::kPartialRows);
      float f[EPT];
      asb::partial_sum<EPT>(ps, t, col, n, f);
#pragma unroll
      for (int k = 0; k < EPT; ++k) in.v[k] = asb::from_float<T>(f[k]);
    } else {
      in = *reinterpret_cast<const Vec*>(qkv + ((size_t)t * heads + head) * hd + e0);
    }
    if (!is_q && !is_k) {
      *reinterpret_cast<Vec*>(dst + e0) = in;
      continue;
    }
    float x[EPT];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
      x[k] = asb::to_float(in.v[k]);
      ss += x[k] * x[k];
    }
    const float* gain = is_q ? q_gain : k_gain;
    if (gain) {
      ss = asb::warp_sum(ss);
      const float rstd = rsqrtf(ss / (float)hd + eps);
#pragma unroll
      for (int k = 0; k < EPT; ++k) x[k] = x[k] * rstd * gain[e0 + k];
    }
    Vec o;
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
      float y = x[k];
      if (inv_freq) {
        const float other = __shfl_xor_sync(0xffffffffu, x[k], 16);
        y = lane < 16 ? x[k] * cs[k] - other * sn[k] : x[k] * cs[k] + other * sn[k];
      }
      o.v[k] = asb::from_float<T>(y);
    }
    *reinterpret_cast<Vec*>(dst + e0) = o;
  }
}

// Many tokens, bfloat16: one block per token walks all its heads, hd / 8 lanes per head with one
// 16-byte vector each (a warp holds 256 / hd heads at a time), so that the angles are computed
// once per token and every load and store moves 16 bytes. The rotation partner of a lane is the
// lane hd / 16 further along in its group.
template <int HD>
__global__ void qk_norm_rope_store_wide_kernel(
    __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
    const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ q_gain, const float* __restrict__ k_gain,
    const float* __restrict__ inv_freq, const int* __restrict__ positions, const int* __restrict__ slots,
    int H, int KV, int block_size, float eps) {
  constexpr int kLanes = HD / 8;                 // lanes per head
  constexpr int kHeadsAtOnce = kWarps * 32 / kLanes;
  const int t = blockIdx.x;
  const int sub = threadIdx.x % kLanes;          // this lane's place in its head
  const int e0 = sub * 8;
  const int heads = H + 2 * KV;
  // the lanes of this head: groups of a warp take different branches below (a query head beside a
  // value head), so their shuffles name only their own lanes
  const unsigned group = kLanes == 32 ? 0xffffffffu : ((1u << kLanes) - 1u) << ((threadIdx.x & 31) / kLanes * kLanes);
  // before the wait: what no kernel of the step writes
  const int slot = slots ? __ldcg(slots + t) : -1;
  float cs[8], sn[8], gq[8], gk[8];
  if (inv_freq) {
    const float pos = (float)__ldcg(positions + t);
    const int i0 = (sub % (kLanes / 2)) * 8;
#pragma unroll
    for (int k = 0; k < 8; ++k) sincosf(pos * inv_freq[i0 + k], &sn[k], &cs[k]);
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    gq[k] = q_gain ? q_gain[e0 + k] : 1.f;
    gk[k] = k_gain ? k_gain[e0 + k] : 1.f;
  }
  asb::pdl_wait();  // the stream's previous kernel has completed (programmatic dependent launch)
  asb::pdl_launch_dependents();
  for (int head = threadIdx.x / kLanes; head < heads; head += kHeadsAtOnce) {
    const bool is_q = head < H;
    const bool is_k = !is_q && head < H + KV;
    __nv_bfloat16* dst;
    if (is_q) {
      dst = q_out + ((size_t)t * H + head) * HD;
    } else {
      if (slot < 0) continue;
      const int kvh = is_k ? head - H : head - H - KV;
      const size_t block = slot / block_size, off = slot % block_size;
      dst = (is_k ? k_cache : v_cache) + ((block * KV + kvh) * block_size + off) * (size_t)HD;
    }
    const uint4 raw = *reinterpret_cast<const uint4*>(qkv + ((size_t)t * heads + head) * HD + e0);
    if (!is_q && !is_k) {
      *reinterpret_cast<uint4*>(dst + e0) = raw;
      continue;
    }
    const __nv_bfloat16* in = reinterpret_cast<const __nv_bfloat16*>(&raw);
    float x[8];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      x[k] = __bfloat162float(in[k]);
      ss += x[k] * x[k];
    }
    if (is_q ? q_gain != nullptr : k_gain != nullptr) {
#pragma unroll
      for (int o = kLanes / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(group, ss, o);
      const float rstd = rsqrtf(ss / (float)HD + eps);
#pragma unroll
      for (int k = 0; k < 8; ++k) x[k] = x[k] * rstd * (is_q ? gq[k] : gk[k]);
    }
    uint4 packed;
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(&packed);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float y = x[k];
      if (inv_freq) {
        const float other = __shfl_xor_sync(group, x[k], kLanes / 2);
        y = sub < kLanes / 2 ? x[k] * cs[k] - other * sn[k] : x[k] * cs[k] + other * sn[k];
      }
      o[k] = __float2bfloat16_rn(y);
    }
    *reinterpret_cast<uint4*>(dst + e0) = packed;
  }
}

template <typename T, int EPT>
void launch_vec(T* q_out, T* k_cache, T* v_cache, const T* qkv, const asb::PartialSums& ps, const float* q_gain,
                const float* k_gain, const float* inv_freq, const int* positions, const int* slots,
                int num_tokens, int H, int KV, int block_size, float eps, cudaStream_t stream) {
  if constexpr (sizeof(T) == 2 && EPT >= 2) {  // (EPT 1 is head size 32: four lanes a head; left to the kernel below)
    if (num_tokens >= 256 && !ps.ws) {
      asb::launch(qk_norm_rope_store_wide_kernel<EPT * 32>, num_tokens, kWarps * 32, 0, stream,
                  (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, (const __nv_bfloat16*)qkv,
                  q_gain, k_gain, inv_freq, positions, slots, H, KV, block_size, eps);
      return;
    }
  }
  if (num_tokens >= 256) {
    const int heads_per_block = kWarps * 4;
    dim3 grid(num_tokens, (H + 2 * KV + heads_per_block - 1) / heads_per_block);
    asb::launch(qk_norm_rope_store_vec_kernel<T, EPT, 4>, grid, kWarps * 32, 0, stream, 
        q_out, k_cache, v_cache, qkv, ps, q_gain, k_gain, inv_freq, positions, slots, H, KV, block_size, eps);
  } else {
    dim3 grid(num_tokens, (H + 2 * KV + kWarps - 1) / kWarps);
    asb::launch(qk_norm_rope_store_vec_kernel<T, EPT, 1>, grid, kWarps * 32, 0, stream, 
        q_out, k_cache, v_cache, qkv, ps, q_gain, k_gain, inv_freq, positions, slots, H, KV, block_size, eps);
  }
}

}  // namespace

namespace {
int rope_store(void* q_out, void* k_cache, void* v_cache, const void* qkv, const asb::PartialSums& ps,
               const float* q_gain, const float* k_gain, const float* inv_freq, const int* positions,
               const int* slots, int num_tokens, int H, int KV, int hd, int rotary_dim, int block_size,
               float eps, int dtype, cudaStream_t stream);
}

extern "C" int asb_qk_norm_rope_store(void* q_out, void* k_cache, void* v_cache, const void* qkv,
                                      const float* q_gain, const float* k_gain,
                                      const float* inv_freq, const int* positions,
                                      const int* slots, int num_tokens, int H, int KV, int hd,
                                      int rotary_dim, int block_size, float eps, int dtype,
                                      cudaStream_t stream) {
  const asb::PartialSums none = {nullptr, 0, 0, 0, 0, 0};
  return rope_store(q_out, k_cache, v_cache, qkv, none, q_gain, k_gain, inv_freq, positions, slots, num_tokens,
                    H, KV, hd, rotary_dim, block_size, eps, dtype, stream);
}

// The same with qkv given as the partial sums of asb_gemm_tcgen05 mode 3 on [tokens, K] x
// [(H + 2 KV) hd, K]: bfloat16 only, head sizes 32, 64, 128, 256 with the whole head rotated.
extern "C" int asb_qk_norm_rope_store_partial(void* q_out, void* k_cache, void* v_cache, const float* ws,
                                              int max_slots, int bn, int kb_per_tile, int num_tiles, int blocks,
                                              const float* q_gain, const float* k_gain, const float* inv_freq,
                                              const int* positions, const int* slots, int num_tokens, int H,
                                              int KV, int hd, int rotary_dim, int block_size, float eps,
                                              cudaStream_t stream) {
  if (!ws || ((uintptr_t)ws & 15)) return asb::fail("qk_norm_rope_store_partial: the partial sums must be 16-byte aligned");
  if (num_tokens > bn || num_tiles * asb::kPartialRows < (H + 2 * KV) * hd)
    return asb::fail("qk_norm_rope_store_partial: %d tokens x %d columns do not fit the partial sums (%d x %d)",
                     num_tokens, (H + 2 * KV) * hd, bn, num_tiles * asb::kPartialRows);
  if (!(hd == 32 || hd == 64 || hd == 128 || hd == 256) || (inv_freq && rotary_dim != hd))
    return asb::fail("qk_norm_rope_store_partial: head_dim %d with rotary_dim %d is not taken", hd, rotary_dim);
  const asb::PartialSums ps = {ws, max_slots, bn, kb_per_tile, num_tiles, blocks};
  return rope_store(q_out, k_cache, v_cache, nullptr, ps, q_gain, k_gain, inv_freq, positions, slots, num_tokens,
                    H, KV, hd, rotary_dim, block_size, eps, asb::kBFloat16, stream);
}

namespace {
int rope_store(void* q_out, void* k_cache, void* v_cache, const void* qkv, const asb::PartialSums& ps,
               const float* q_gain, const float* k_gain, const float* inv_freq, const int* positions,
               const int* slots, int num_tokens, int H, int KV, int hd, int rotary_dim, int block_size,
               float eps, int dtype, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (hd < 1 || hd > kMaxHeadDim) return asb::fail("qk_norm_rope_store: head_dim %d not in 1..%d", hd, kMaxHeadDim);
  if (inv_freq && (rotary_dim < 2 || rotary_dim > hd || rotary_dim % 2))
    return asb::fail("qk_norm_rope_store: rotary_dim %d must be even and <= head_dim %d", rotary_dim, hd);
  if (KV > 0 && (!k_cache || !v_cache) && slots) return asb::fail("qk_norm_rope_store: slots given without a cache");
  const bool whole_head = !inv_freq || rotary_dim == hd;
  const bool aligned = ((uintptr_t)q_out % 16 == 0) && ((uintptr_t)qkv % 16 == 0) &&
                       ((uintptr_t)k_cache % 16 == 0) && ((uintptr_t)v_cache % 16 == 0);
  if (whole_head && aligned && (hd == 32 || hd == 64 || hd == 128 || hd == 256)) {
#define ASB_ROPE_VEC(E)                                                                          \
  ASB_DISPATCH_DTYPE(dtype, T,                                                                   \
                     launch_vec<T, E>((T*)q_out, (T*)k_cache, (T*)v_cache, (const T*)qkv, ps, q_gain, \
                                      k_gain, inv_freq, positions, slots, num_tokens, H, KV,     \
                                      block_size, eps, stream))
    if (hd == 32) { ASB_ROPE_VEC(1); }
    else if (hd == 64) { ASB_ROPE_VEC(2); }
    else if (hd == 128) { ASB_ROPE_VEC(4); }
    else { ASB_ROPE_VEC(8); }
#undef ASB_ROPE_VEC
    return asb::check_launch("qk_norm_rope_store");
  }
  if (ps.ws) return asb::fail("qk_norm_rope_store_partial: the pointers must be 16-byte aligned");
  dim3 grid(num_tokens, (H + 2 * KV + kWarps - 1) / kWarps);
  ASB_DISPATCH_DTYPE(dtype, T,
                     asb::launch(qk_norm_rope_store_kernel<T>, grid, kWarps * 32, 0, stream, 
                         (T*)q_out, (T*)k_cache, (T*)v_cache, (const T*)qkv, q_gain, k_gain,
                         inv_freq, positions, slots, H, KV, hd, rotary_dim, block_size, eps));
  return asb::check_launch("qk_norm_rope_store");
}
}  // namespace
