// SwiGLU's elementwise half: out[t, i] = silu(gu[t, i]) * gu[t, I + i], silu(g) = g / (1 + exp(-g)),
// computed in float32 and rounded once (atomserve/kernels.py:437-449; gate is the first half
// of the stacked projection, atomserve/model.py:354-358).
#include "common.cuh"

namespace {

template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int inter) {
  const size_t t = blockIdx.y;
  const T* row = gate_up + t * 2 * (size_t)inter;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < inter; i += gridDim.x * blockDim.x) {
    const float g = asb::to_float(row[i]);
    const float u = asb::to_float(row[inter + i]);
    out[t * inter + i] = asb::from_float<T>(g / (1.f + expf(-g)) * u);
  }
}

}  // namespace

extern "C" int asb_silu_mul(void* out, const void* gate_up, int num_tokens, int inter, int dtype,
                            cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (num_tokens > 65535 * 16) return asb::fail("silu_mul: %d tokens exceed the grid", num_tokens);
  const int threads = 256;
  int bx = (inter + threads - 1) / threads;
  if (bx > 64) bx = 64;
  // grid.y is limited to 65535 rows per launch
  for (int t0 = 0; t0 < num_tokens; t0 += 65535) {
    const int rows = num_tokens - t0 < 65535 ? num_tokens - t0 : 65535;
    ASB_DISPATCH_DTYPE(
        dtype, T,
        silu_mul_kernel<T><<<dim3(bx, rows), threads, 0, stream>>>(
            (T*)out + (size_t)t0 * inter, (const T*)gate_up + (size_t)t0 * 2 * inter, inter));
  }
  return asb::check_launch("silu_mul");
}
