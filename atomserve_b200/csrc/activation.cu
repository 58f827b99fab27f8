// SwiGLU's elementwise half: out[t, i] = silu(gu[t, i]) * gu[t, I + i], silu(g) = g / (1 + exp(-g)),
// computed in float32 and rounded once (atomserve/kernels.py:437-449; gate is the first half
// of the stacked projection, atomserve/model.py:354-358). 16-byte vectors when the width allows.
#include "common.cuh"

namespace {

template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int inter,
                                long long total) {
  asb::pdl_wait();  // the stream's previous kernel has completed (programmatic dependent launch)
  asb::pdl_launch_dependents();
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / inter;
    const int i = (int)(idx - t * inter);
    const float g = asb::to_float(gate_up[t * 2 * inter + i]);
    const float u = asb::to_float(gate_up[t * 2 * inter + inter + i]);
    out[idx] = asb::from_float<T>(g / (1.f + expf(-g)) * u);
  }
}

template <typename T, int VEC>
__global__ void silu_mul_vec_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int inter,
                                    long long total_vecs) {
  asb::pdl_wait();  // the stream's previous kernel has completed (programmatic dependent launch)
  asb::pdl_launch_dependents();
  const int vecs_per_row = inter / VEC;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total_vecs;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / vecs_per_row;
    const int i = (int)(idx - t * vecs_per_row) * VEC;
    const uint4 graw = *reinterpret_cast<const uint4*>(gate_up + t * 2 * inter + i);
    const uint4 uraw = *reinterpret_cast<const uint4*>(gate_up + t * 2 * inter + inter + i);
    const T* g = reinterpret_cast<const T*>(&graw);
    const T* u = reinterpret_cast<const T*>(&uraw);
    uint4 packed;
    T* o = reinterpret_cast<T*>(&packed);
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      const float gv = asb::to_float(g[k]);
      o[k] = asb::from_float<T>(gv / (1.f + expf(-gv)) * asb::to_float(u[k]));
    }
    *reinterpret_cast<uint4*>(out + t * inter + i) = packed;
  }
}

template <typename T>
int launch(void* out, const void* gate_up, int num_tokens, int inter, cudaStream_t stream) {
  constexpr int VEC = 16 / sizeof(T);
  const bool aligned = ((uintptr_t)out % 16 == 0) && ((uintptr_t)gate_up % 16 == 0);
  const int threads = 256;
  if (inter % VEC == 0 && aligned) {
    const long long total = (long long)num_tokens * (inter / VEC);
    const long long blocks = (total + threads - 1) / threads;
    asb::launch(silu_mul_vec_kernel<T, VEC>, (unsigned)(blocks < 148 * 32 ? blocks : 148 * 32), threads, 0, stream, 
        (T*)out, (const T*)gate_up, inter, total);
  } else {
    const long long total = (long long)num_tokens * inter;
    const long long blocks = (total + threads - 1) / threads;
    asb::launch(silu_mul_kernel<T>, (unsigned)(blocks < 148 * 32 ? blocks : 148 * 32), threads, 0, stream, 
        (T*)out, (const T*)gate_up, inter, total);
  }
  return asb::check_launch("silu_mul");
}

}  // namespace

extern "C" int asb_silu_mul(void* out, const void* gate_up, int num_tokens, int inter, int dtype,
                            cudaStream_t stream) {
  if (num_tokens == 0 || inter == 0) return 0;
  ASB_DISPATCH_DTYPE(dtype, T, return launch<T>(out, gate_up, num_tokens, inter, stream));
  return 0;
}
