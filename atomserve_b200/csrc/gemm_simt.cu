// out[M, N] = x[M, K] . w[N, K]^T (+ residual[M, N]) on CUDA cores with float32 multiply-adds:
// the matrix product of the true 32-bit path (no tensor-core mode of reduced precision is
// involved), also instantiated for bfloat16 inputs as the fallback and the checker of the
// tensor-core kernels. Weights keep the checkpoint layout [out_features, in_features], so
// both operands are contiguous along K (atomserve/model.py:15-16; the residual form is the
// reference's addmm, atomserve/quant.py:89-91).
//
// Each output element is summed in a fixed order that depends on k alone: a chain of fused
// multiply-adds over each run of kChunk consecutive k, the runs' sums added up in ascending
// order, whatever M and N are and wherever the element lies in its tile. A row's result
// therefore does not depend on which other rows share the batch. The two levels keep the
// rounding error of a long sum (K = 12,288 in the served models) near that of a sum of
// sqrt(K) terms: one chain over all of K drifted 2.5e-5 of the largest logit from a float64
// oracle through two full-width layers, the blocked sum a fifth of that.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
constexpr int kChunk = 256;  // k per inner chain; a multiple of BK

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(TOut* __restrict__ out, const TIn* __restrict__ x, const TIn* __restrict__ w,
                 const TOut* __restrict__ residual, int M, int N, int K) {
  asb::pdl_wait();  // the stream's previous kernel has completed (programmatic dependent launch)
  asb::pdl_launch_dependents();
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = tid % 16, ty = tid / 16;  // 16 x 16 threads, each TM x TN outputs
  const int lrow = tid / 4, lk = (tid % 4) * 4;  // loader: row 0..63, k offset 0,4,8,12

  float acc[TM][TN], total[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = total[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = k0 + lk + u;
      const int xm = m0 + lrow, wn = n0 + lrow;
      xs[lk + u][lrow] = (xm < M && k < K) ? asb::to_float(x[(size_t)xm * K + k]) : 0.f;
      ws[lk + u][lrow] = (wn < N && k < K) ? asb::to_float(w[(size_t)wn * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = xs[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if ((k0 + BK) % kChunk == 0 || k0 + BK >= K) {  // the run is complete: bank its sum
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          total[i][j] += acc[i][j];
          acc[i][j] = 0.f;
        }
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= N) continue;
      float v = total[i][j];
      if (residual) v += asb::to_float(residual[(size_t)m * N + n]);
      out[(size_t)m * N + n] = asb::from_float<TOut>(v);
    }
  }
}

}  // namespace

// in_dtype: element type of x and w. out_dtype: element type of out and residual (float32 out
// from bfloat16 inputs gives logits straight from the accumulator).
extern "C" int asb_gemm_simt(void* out, const void* x, const void* w, const void* residual,
                             int M, int N, int K, int in_dtype, int out_dtype,
                             cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (K < 1) return asb::fail("gemm_simt: K = %d", K);
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return asb::fail("gemm_simt: M = %d exceeds the grid", M);
  if (in_dtype == asb::kFloat32 && out_dtype == asb::kFloat32) {
    asb::launch(gemm_simt_kernel<float, float>, grid, 256, 0, stream, 
        (float*)out, (const float*)x, (const float*)w, (const float*)residual, M, N, K);
  } else if (in_dtype == asb::kBFloat16 && out_dtype == asb::kBFloat16) {
    asb::launch(gemm_simt_kernel<__nv_bfloat16, __nv_bfloat16>, grid, 256, 0, stream, 
        (__nv_bfloat16*)out, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
        (const __nv_bfloat16*)residual, M, N, K);
  } else if (in_dtype == asb::kBFloat16 && out_dtype == asb::kFloat32) {
    asb::launch(gemm_simt_kernel<__nv_bfloat16, float>, grid, 256, 0, stream, 
        (float*)out, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const float*)residual, M,
        N, K);
  } else {
    return asb::fail("gemm_simt: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
  }
  return asb::check_launch("gemm_simt");
}
