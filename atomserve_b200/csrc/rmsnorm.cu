// RMSNorm over the last dimension: y = gain * x / sqrt(mean(x^2) + eps), accumulated in
// float32 and rounded once (atomserve/model.py:125-139). Gains are float32 whatever the
// activation type. An optional row list gathers the rows to normalise, which is how the
// final norm runs only on the rows whose logits are wanted (atomserve/model.py:383-384).
//
// Rows whose width is a multiple of a 16-byte vector and fits one vector per thread are read
// once into registers (one 16-byte load per thread); other widths take the strided loop.
#include "common.cuh"
#include "gemm_partials.cuh"

namespace {

template <typename T>
__global__ void rmsnorm_kernel(T* __restrict__ out, const T* __restrict__ x,
                               const float* __restrict__ gain, const int* __restrict__ rows,
                               int width, float eps) {
  asb::pdl_wait();  // the stream's previous kernel has completed (programmatic dependent launch)
  asb::pdl_launch_dependents();
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const T* src = x + (size_t)(rows ? rows[r] : r) * width;
  T* dst = out + (size_t)r * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = asb::to_float(src[i]);
    ss += v * v;
  }
  ss = asb::block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    dst[i] = asb::from_float<T>(asb::to_float(src[i]) * rstd * gain[i]);
}

// One 16-byte vector (VEC elements) per thread; threads beyond the row's vectors only take
// part in the reduction.
template <typename T, int VEC>
__global__ void rmsnorm_vec_kernel(T* __restrict__ out, const T* __restrict__ x,
                                   const float* __restrict__ gain, const int* __restrict__ rows,
                                   int width, float eps) {
  asb::pdl_wait();  // the stream's previous kernel has completed (programmatic dependent launch)
  asb::pdl_launch_dependents();
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const T* src = x + (size_t)(rows ? rows[r] : r) * width;
  T* dst = out + (size_t)r * width;
  const int i = threadIdx.x * VEC;
  const bool active = i < width;
  float v[VEC];
  float ss = 0.f;
  if (active) {
    const uint4 raw = *reinterpret_cast<const uint4*>(src + i);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      v[k] = asb::to_float(e[k]);
      ss += v[k] * v[k];
    }
  }
  ss = asb::block_sum(ss, scratch);
  if (!active) return;
  const float rstd = rsqrtf(ss / (float)width + eps);
  uint4 packed;
  T* o = reinterpret_cast<T*>(&packed);
#pragma unroll
  for (int k = 0; k < VEC; k += 4) {
    const float4 g = *reinterpret_cast<const float4*>(gain + i + k);
    o[k] = asb::from_float<T>(v[k] * rstd * g.x);
    o[k + 1] = asb::from_float<T>(v[k + 1] * rstd * g.y);
    o[k + 2] = asb::from_float<T>(v[k + 2] * rstd * g.z);
    o[k + 3] = asb::from_float<T>(v[k + 3] * rstd * g.w);
  }
  *reinterpret_cast<uint4*>(dst + i) = packed;
}

// sum = (a product left as partial sums by the tensor-core GEMM) + residual, rounded to bfloat16,
// and normed = RMSNorm(sum): the reduction of the partial sums, the residual addition
// (atomserve/model.py:336,360) and the next norm in one kernel. The arithmetic and its order are
// those of the GEMM's own reduction followed by rmsnorm_vec_kernel with the same block size, so
// the results are the same bits. One block per token, eight consecutive columns per thread.
__global__ void partial_add_rmsnorm_kernel(__nv_bfloat16* __restrict__ sum_out, __nv_bfloat16* __restrict__ normed_out,
                                           const asb::PartialSums ps, const __nv_bfloat16* __restrict__ residual,
                                           const float* __restrict__ gain, int width, float eps) {
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int i = threadIdx.x * 8;
  const bool active = i < width;
  // what does not depend on the GEMM comes first: it overlaps the GEMM's tail
  int slots = 0;
  float4 g0 = make_float4(0.f, 0.f, 0.f, 0.f), g1 = g0;
  if (active) {
    slots = asb::partial_slots(ps, i / asb::kPartialRows);
    g0 = *reinterpret_cast<const float4*>(gain + i);
    g1 = *reinterpret_cast<const float4*>(gain + i + 4);
  }
  asb::pdl_wait();  // the GEMM has completed (programmatic dependent launch)
  asb::pdl_launch_dependents();
  float v[8];
  float ss = 0.f;
  if (active) {
    float sum[8];
    asb::partial_sum<8>(ps, t, i, slots, sum);
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (residual) raw = *reinterpret_cast<const uint4*>(residual + (size_t)t * width + i);
    const __nv_bfloat16* r = reinterpret_cast<const __nv_bfloat16*>(&raw);
    uint4 packed;
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(&packed);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float x = sum[k];
      if (residual) x += __bfloat162float(r[k]);
      o[k] = __float2bfloat16_rn(x);
      v[k] = __bfloat162float(o[k]);
      ss += v[k] * v[k];
    }
    *reinterpret_cast<uint4*>(sum_out + (size_t)t * width + i) = packed;
  }
  ss = asb::block_sum(ss, scratch);
  if (!active) return;
  const float rstd = rsqrtf(ss / (float)width + eps);
  const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
  uint4 packed;
  __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(&packed);
#pragma unroll
  for (int k = 0; k < 8; ++k) o[k] = __float2bfloat16_rn(v[k] * rstd * g[k]);
  *reinterpret_cast<uint4*>(normed_out + (size_t)t * width + i) = packed;
}

template <typename T>
int launch(void* out, const void* x, const float* gain, const int* rows, int num_rows, int width,
           float eps, cudaStream_t stream) {
  constexpr int VEC = 16 / sizeof(T);
  const bool aligned = ((uintptr_t)out % 16 == 0) && ((uintptr_t)x % 16 == 0) && ((uintptr_t)gain % 16 == 0);
  if (width % VEC == 0 && width / VEC <= 1024 && aligned) {
    const int threads = ((width / VEC) + 31) / 32 * 32;
    asb::launch(rmsnorm_vec_kernel<T, VEC>, num_rows, threads, 0, stream, (T*)out, (const T*)x, gain, rows, width, eps);
  } else {
    int threads = 32;
    while (threads < 1024 && threads * 4 < width) threads <<= 1;
    asb::launch(rmsnorm_kernel<T>, num_rows, threads, 0, stream, (T*)out, (const T*)x, gain, rows, width, eps);
  }
  return asb::check_launch("rmsnorm");
}

}  // namespace

extern "C" int asb_rmsnorm(void* out, const void* x, const float* gain, const int* rows,
                           int num_rows, int width, float eps, int dtype, cudaStream_t stream) {
  if (num_rows == 0) return 0;
  ASB_DISPATCH_DTYPE(dtype, T, return launch<T>(out, x, gain, rows, num_rows, width, eps, stream));
  return 0;
}

// sum_out = partial sums + residual (bfloat16 [tokens, width]); normed_out = RMSNorm(sum_out).
// The partial sums are those of asb_gemm_tcgen05 mode 3 on [tokens, K] x [width, K]; widths that
// are a multiple of 8 up to 8192, pointers 16-byte aligned.
extern "C" int asb_partial_add_rmsnorm(void* sum_out, void* normed_out, const float* ws, int max_slots,
                                       int bn, int kb_per_tile, int num_tiles, int blocks,
                                       const void* residual, const float* gain, int tokens, int width,
                                       float eps, cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (width % 8 || width / 8 > 1024) return asb::fail("partial_add_rmsnorm: width %d must be a multiple of 8 up to 8192", width);
  if (tokens > bn || num_tiles * asb::kPartialRows < width)
    return asb::fail("partial_add_rmsnorm: %d tokens x %d columns do not fit the partial sums (%d x %d)", tokens,
                     width, bn, num_tiles * asb::kPartialRows);
  if (((uintptr_t)sum_out | (uintptr_t)normed_out | (uintptr_t)residual | (uintptr_t)gain | (uintptr_t)ws) & 15)
    return asb::fail("partial_add_rmsnorm: pointers must be 16-byte aligned");
  const asb::PartialSums ps = {ws, max_slots, bn, kb_per_tile, num_tiles, blocks};
  const int threads = ((width / 8) + 31) / 32 * 32;
  asb::launch(partial_add_rmsnorm_kernel, tokens, threads, 0, stream, (__nv_bfloat16*)sum_out,
              (__nv_bfloat16*)normed_out, ps, (const __nv_bfloat16*)residual, gain, width, eps);
  return asb::check_launch("partial_add_rmsnorm");
}
