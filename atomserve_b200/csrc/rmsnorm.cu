// RMSNorm over the last dimension: y = gain * x / sqrt(mean(x^2) + eps), accumulated in
// float32 and rounded once (atomserve/model.py:125-139). Gains are float32 whatever the
// activation type. An optional row list gathers the rows to normalise, which is how the
// final norm runs only on the rows whose logits are wanted (atomserve/model.py:383-384).
//
// Rows whose width is a multiple of a 16-byte vector and fits one vector per thread are read
// once into registers (one 16-byte load per thread); other widths take the strided loop.
#include "common.cuh"

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
