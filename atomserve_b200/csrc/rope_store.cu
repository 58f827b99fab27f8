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

}  // namespace

extern "C" int asb_qk_norm_rope_store(void* q_out, void* k_cache, void* v_cache, const void* qkv,
                                      const float* q_gain, const float* k_gain,
                                      const float* inv_freq, const int* positions,
                                      const int* slots, int num_tokens, int H, int KV, int hd,
                                      int rotary_dim, int block_size, float eps, int dtype,
                                      cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (hd < 1 || hd > kMaxHeadDim) return asb::fail("qk_norm_rope_store: head_dim %d not in 1..%d", hd, kMaxHeadDim);
  if (inv_freq && (rotary_dim < 2 || rotary_dim > hd || rotary_dim % 2))
    return asb::fail("qk_norm_rope_store: rotary_dim %d must be even and <= head_dim %d", rotary_dim, hd);
  if (KV > 0 && (!k_cache || !v_cache) && slots) return asb::fail("qk_norm_rope_store: slots given without a cache");
  dim3 grid(num_tokens, (H + 2 * KV + kWarps - 1) / kWarps);
  ASB_DISPATCH_DTYPE(dtype, T,
                     qk_norm_rope_store_kernel<T><<<grid, kWarps * 32, 0, stream>>>(
                         (T*)q_out, (T*)k_cache, (T*)v_cache, (const T*)qkv, q_gain, k_gain,
                         inv_freq, positions, slots, H, KV, hd, rotary_dim, block_size, eps));
  return asb::check_launch("qk_norm_rope_store");
}
