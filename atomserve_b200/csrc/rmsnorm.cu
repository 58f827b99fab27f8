// RMSNorm over the last dimension: y = gain * x / sqrt(mean(x^2) + eps), accumulated in
// float32 and rounded once (atomserve/model.py:125-139). Gains are float32 whatever the
// activation type. An optional row list gathers the rows to normalise, which is how the
// final norm runs only on the rows whose logits are wanted (atomserve/model.py:383-384).
#include "common.cuh"

namespace {

template <typename T>
__global__ void rmsnorm_kernel(T* __restrict__ out, const T* __restrict__ x,
                               const float* __restrict__ gain, const int* __restrict__ rows,
                               int width, float eps) {
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

}  // namespace

extern "C" int asb_rmsnorm(void* out, const void* x, const float* gain, const int* rows,
                           int num_rows, int width, float eps, int dtype, cudaStream_t stream) {
  if (num_rows == 0) return 0;
  int threads = 32;
  while (threads < 1024 && threads * 4 < width) threads <<= 1;
  ASB_DISPATCH_DTYPE(dtype, T,
                     rmsnorm_kernel<T><<<num_rows, threads, 0, stream>>>(
                         (T*)out, (const T*)x, gain, rows, width, eps));
  return asb::check_launch("rmsnorm");
}
