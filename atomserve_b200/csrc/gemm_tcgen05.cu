// bfloat16 GEMM on the fifth-generation tensor cores: out[M, N] = x[M, K] . w[N, K]^T with
// float32 accumulation in tensor memory (TMEM), operands brought to shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle, no multicast), MMAs issued by one thread
// (tcgen05.mma.cta_group::1.kind::f16), results read back with tcgen05.ld for the epilogue.
// Epilogues: plain bfloat16, + residual (the reference's addmm, atomserve/quant.py:89-91),
// float32 result (logits from the accumulator, atomserve/model.py:388-412), and float32
// partial sums for split K. These are the products of atomserve/model.py:317,336,354,360,412.
//
// The kernel multiplies two K-major operands: P (rows become TMEM lanes, tile of 128) and Q
// (rows become TMEM columns, tile of BN = 16..256). With many tokens P = x and Q = w. With few
// tokens (decoding) the operands swap: P = w, so that the 128-row MMA shape is filled with
// weight rows and the handful of tokens is the narrow N; the kernel then streams weights at
// HBM speed with a deep TMA pipeline, and splits K over grid.z when there are too few weight
// tiles to occupy every SM (partials are summed by `splitk_reduce_kernel`).
//
// Warp roles (192 threads): warp 0 issues TMA loads, warp 1 allocates TMEM and issues MMAs,
// warps 2-5 run the epilogue (warp w reads TMEM lanes 32*(w%4)..+31). Stages are handed over
// with mbarriers: full[s] (TMA bytes landed) and empty[s] (tcgen05.commit after the MMAs that
// read stage s), and one barrier tells the epilogue that the accumulator is complete.
//
// Every wait on a barrier is bounded. A wait that runs out sets *status (non-zero) and the
// role stops waiting; all roles still meet at the final barrier, TMEM is freed and the block
// returns, so a fault in the pipeline shows as an error code, never as a hang.
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int kThreads = 192;
constexpr int BM = 128;   // P rows per tile = TMEM lanes
constexpr int BK = 64;    // K elements per stage: 128 bytes, one swizzle atom
constexpr int UMMA_K = 16;
constexpr uint32_t kMaxPolls = 1u << 24;

enum Epilogue : int { kStoreBf16 = 0, kStoreBf16Residual = 1, kStoreF32 = 2, kStorePartial = 3 };

struct GemmParams {
  void* out;             // bf16 or f32 [M, N]; for partials f32 [splits, M, N]
  const void* residual;  // bf16 [M, N] or null
  int* status;           // device word, set non-zero by a wait that ran out
  int p_rows, q_rows;    // rows of P and Q (M and N, or N and M when swapped)
  int ldo;               // row stride of out (N)
  int K, kb_per_split;   // K blocks of BK each split handles
  int swap;              // 1: P = w (lanes are output columns), Q = x
  int epilogue;
  long long split_stride;  // elements between split partials (M * N)
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity. False if it ran out of polls.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int code) {
  for (uint32_t i = 0; i < kMaxPolls; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  atomicExch(status, code);
  return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// Shared-memory matrix descriptor: K-major tile, rows of 128 bytes, 128-byte swizzle; groups of
// eight rows are 1024 bytes apart (SBO), LBO is 1 for swizzled K-major layouts, version 1.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor: D = f32, A = B = bf16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t instr_desc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

template <int BN>
struct Config {
  static constexpr int kTileP = BM * BK * 2;   // 16 KB
  static constexpr int kTileQ = BN * BK * 2;
  static constexpr int kStage = kTileP + kTileQ;
  static constexpr int kStages = BN >= 256 ? 4 : (BN >= 128 ? 6 : 8);
  static constexpr int kTmemCols = BN < 32 ? 32 : BN;
  static constexpr int kSmem = kStages * kStage + 1024 /* alignment slack */ + 256 /* barriers */;
};

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
                    const GemmParams p) {
  using C = Config<BN>;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;   // swizzle atoms need 1024-byte alignment
  unsigned char* aligned = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + C::kStages * C::kStage;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (C::kStages + s); };
  const uint32_t acc_bar = bars + 8u * (2 * C::kStages);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(aligned + C::kStages * C::kStage + 8 * (2 * C::kStages + 1));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int p0 = blockIdx.x * BM, q0 = blockIdx.y * BN;
  const int total_kb = (p.K + BK - 1) / BK;
  const int kb_begin = blockIdx.z * p.kb_per_split;
  const int num_kb = min(p.kb_per_split, total_kb - kb_begin);

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"((uint32_t)C::kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0 && num_kb > 0) {
      for (int i = 0; i < num_kb; ++i) {
        const int s = i % C::kStages;
        const uint32_t phase = (uint32_t)(i / C::kStages) & 1u;
        if (!mbar_wait(empty_bar(s), phase ^ 1u, p.status, 1)) break;
        mbar_expect_tx(full_bar(s), C::kStage);
        const int k0 = (kb_begin + i) * BK;
        tma_load_2d(base + s * C::kStage, &map_p, full_bar(s), k0, p0);
        tma_load_2d(base + s * C::kStage + C::kTileP, &map_q, full_bar(s), k0, q0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && num_kb > 0) {
      constexpr uint32_t idesc = instr_desc(BM, BN);
      bool ok = true;
      for (int i = 0; i < num_kb && ok; ++i) {
        const int s = i % C::kStages;
        const uint32_t phase = (uint32_t)(i / C::kStages) & 1u;
        ok = mbar_wait(full_bar(s), phase, p.status, 2);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t da = smem_desc(base + s * C::kStage);
        const uint64_t db = smem_desc(base + s * C::kStage + C::kTileP);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)  // 32 bytes further along K inside the swizzle atom
          umma(tmem_base, da + (uint64_t)(k * UMMA_K * 2 >> 4), db + (uint64_t)(k * UMMA_K * 2 >> 4), idesc,
               (uint32_t)((i | k) != 0));
        umma_commit(empty_bar(s));  // stage s may be refilled once these MMAs have read it
      }
      umma_commit(acc_bar);  // arrives when every MMA issued above has completed
    }
  } else {
    // Epilogue: this warp owns TMEM lanes 32*(warp%4)..+31, one lane (P row) per thread.
    const int quad = warp & 3;
    const int prow = p0 + quad * 32 + lane;
    int ok_i = num_kb > 0;
    if (ok_i && lane == 0) ok_i = mbar_wait(acc_bar, 0, p.status, 3) ? 1 : 0;  // one poller per warp
    const bool ok = __shfl_sync(0xffffffffu, ok_i, 0) != 0;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
      constexpr int kChunk = 16;
#pragma unroll 1
      for (int c = 0; c < BN; c += kChunk) {
        if (q0 + c >= p.q_rows) break;  // uniform: depends on the block and c only
        uint32_t raw[16];
        tmem_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c, raw);
        if (prow >= p.p_rows) continue;
        if (p.swap) {
          // lanes are output columns (weight rows), TMEM columns are tokens: out[token, prow]
#pragma unroll
          for (int j = 0; j < kChunk; ++j) {
            const int tok = q0 + c + j;
            if (tok >= p.q_rows) break;
            const size_t at = (size_t)tok * p.ldo + prow;
            float v = __uint_as_float(raw[j]);
            if (p.epilogue == kStorePartial) {
              ((float*)p.out)[(size_t)blockIdx.z * p.split_stride + at] = v;
            } else if (p.epilogue == kStoreF32) {
              ((float*)p.out)[at] = v;
            } else {
              if (p.epilogue == kStoreBf16Residual) v += __bfloat162float(((const __nv_bfloat16*)p.residual)[at]);
              ((__nv_bfloat16*)p.out)[at] = __float2bfloat16_rn(v);
            }
          }
        } else {
          // lanes are tokens, TMEM columns are output columns: out[prow, q0 + c + j], contiguous in j
          const size_t at = (size_t)prow * p.ldo + q0 + c;
          const int valid = min(kChunk, p.q_rows - (q0 + c));
          if (p.epilogue == kStorePartial || p.epilogue == kStoreF32) {
            float* o = (float*)p.out + (p.epilogue == kStorePartial ? (size_t)blockIdx.z * p.split_stride : 0) + at;
            if (valid == kChunk && (((uintptr_t)o) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < kChunk; j += 4)
                *reinterpret_cast<uint4*>(o + j) = make_uint4(raw[j], raw[j + 1], raw[j + 2], raw[j + 3]);
            } else {
              for (int j = 0; j < valid; ++j) o[j] = __uint_as_float(raw[j]);
            }
          } else {
            __nv_bfloat16* o = (__nv_bfloat16*)p.out + at;
            const __nv_bfloat16* res = p.epilogue == kStoreBf16Residual ? (const __nv_bfloat16*)p.residual + at : nullptr;
            if (valid == kChunk && (((uintptr_t)o) & 15) == 0 && (!res || (((uintptr_t)res) & 15) == 0)) {
              uint4 rv[2];
              if (res) {
                rv[0] = *reinterpret_cast<const uint4*>(res);
                rv[1] = *reinterpret_cast<const uint4*>(res + 8);
              }
              const __nv_bfloat16* rb = reinterpret_cast<const __nv_bfloat16*>(rv);
              uint4 ov[2];
              __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(ov);
#pragma unroll
              for (int j = 0; j < kChunk; j += 2) {
                float a = __uint_as_float(raw[j]), b = __uint_as_float(raw[j + 1]);
                if (res) { a += __bfloat162float(rb[j]); b += __bfloat162float(rb[j + 1]); }
                ob[j >> 1] = __floats2bfloat162_rn(a, b);
              }
              *reinterpret_cast<uint4*>(o) = ov[0];
              *reinterpret_cast<uint4*>(o + 8) = ov[1];
            } else {
              for (int j = 0; j < valid; ++j) {
                float v = __uint_as_float(raw[j]);
                if (res) v += __bfloat162float(res[j]);
                o[j] = __float2bfloat16_rn(v);
              }
            }
          }
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::kTmemCols) : "memory");
  }
}

// out[m, n] = sum over splits of partial[s, m, n] (+ residual), rounded once.
__global__ void splitk_reduce_kernel(void* __restrict__ out, const float* __restrict__ partial,
                                     const __nv_bfloat16* __restrict__ residual, long long total,
                                     int splits, int out_f32) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < splits; ++s) v += partial[(size_t)s * total + i];
    if (residual) v += __bfloat162float(residual[i]);
    if (out_f32) ((float*)out)[i] = v; else ((__nv_bfloat16*)out)[i] = __float2bfloat16_rn(v);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)ptr;
  }
  return fn;
}

// A [rows, K] row-major bfloat16 matrix as a 2-D tensor map with boxes of box_rows x 64.
int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return asb::fail("gemm_tcgen05: cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return asb::fail("gemm_tcgen05: cuTensorMapEncodeTiled failed with %d (rows %d, K %d)", (int)r, rows, K);
  return 0;
}

template <int BN>
int launch(const CUtensorMap& mp, const CUtensorMap& mq, const GemmParams& p, dim3 grid, cudaStream_t stream) {
  auto kern = gemm_tcgen05_kernel<BN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Config<BN>::kSmem);
  if (e != cudaSuccess) return asb::fail("gemm_tcgen05: shared memory %d: %s", Config<BN>::kSmem, cudaGetErrorString(e));
  kern<<<grid, kThreads, Config<BN>::kSmem, stream>>>(mp, mq, p);
  return asb::check_launch("gemm_tcgen05");
}

}  // namespace

static int sm_count() {
  static int count = 0;
  if (!count) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count < 1)
      count = 148;
  }
  return count;
}

// How the shape is run: operands swap at up to 64 tokens. One block runs per SM, so K is split
// where that shortens the slowest SM's share of the weight stream by more than the float32
// partial sums cost to write and read back; every split keeps at least four K blocks.
static void plan(int M, int N, int K, int* swap, int* bn, int* splits, int* kb_per_split) {
  *swap = M <= 64 ? 1 : 0;
  const int total_kb = (K + BK - 1) / BK;
  int best = 1;
  if (*swap) {
    *bn = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    const int tiles = (N + BM - 1) / BM, sms = sm_count();
    const double weight_bytes = 2.0 * N * K;
    double best_cost = 0;
    for (int s = 1; s <= 16 && total_kb / s >= 4; ++s) {
      const int waves = (tiles * s + sms - 1) / sms;
      // bytes the busiest SM streams, scaled to the whole device, plus the partials' round trip
      double cost = weight_bytes * waves * sms / ((double)tiles * s);
      if (s > 1) cost += 2.0 * s * M * N * 4.0;
      if (s == 1 || cost < best_cost * 0.97) {
        best_cost = cost;
        best = s;
      }
    }
  } else {
    *bn = N <= 128 ? 128 : 256;
  }
  const int per = (total_kb + best - 1) / best;
  *splits = (total_kb + per - 1) / per;  // no empty split
  *kb_per_split = per;
}

// Float32 workspace elements a call needs (0 when K is not split).
extern "C" long long asb_gemm_tcgen05_workspace(int M, int N, int K, int* splits_out) {
  int swap, bn, splits, per;
  plan(M, N, K, &swap, &bn, &splits, &per);
  if (splits_out) *splits_out = splits;
  return splits > 1 ? (long long)splits * M * N : 0;
}

// out = x . w^T (+ residual). x [M, K] and w [N, K] bfloat16, contiguous, K a multiple of 8 and
// both bases 16-byte aligned (TMA's rules). out bfloat16 [M, N], or float32 when out_f32.
// workspace: float32, asb_gemm_tcgen05_workspace(M, N, K) elements (null if that is 0).
// status: one int on the device; it stays 0 unless a pipeline wait ran out.
extern "C" int asb_gemm_tcgen05(void* out, const void* x, const void* w, const void* residual, int M,
                                int N, int K, int out_f32, float* workspace, int* status,
                                cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (K < 8 || K % 8) return asb::fail("gemm_tcgen05: K = %d must be a positive multiple of 8 (16-byte TMA rows)", K);
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return asb::fail("gemm_tcgen05: operands must be 16-byte aligned");
  if (out_f32 && residual) return asb::fail("gemm_tcgen05: the float32 result form takes no residual");
  if (!status) return asb::fail("gemm_tcgen05: a status word is required");
  int swap, bn, splits, per;
  plan(M, N, K, &swap, &bn, &splits, &per);
  if (splits > 1 && !workspace) return asb::fail("gemm_tcgen05: %d K splits need a workspace", splits);

  GemmParams p;
  p.status = status;
  p.K = K;
  p.kb_per_split = per;
  p.swap = swap;
  p.ldo = N;
  p.split_stride = (long long)M * N;
  p.p_rows = swap ? N : M;
  p.q_rows = swap ? M : N;
  p.residual = residual;
  if (splits > 1) {
    p.out = workspace;
    p.epilogue = kStorePartial;
  } else {
    p.out = out;
    p.epilogue = out_f32 ? kStoreF32 : (residual ? kStoreBf16Residual : kStoreBf16);
  }
  alignas(64) CUtensorMap mp, mq;
  if (int rc = make_map(&mp, swap ? w : x, p.p_rows, K, BM)) return rc;
  if (int rc = make_map(&mq, swap ? x : w, p.q_rows, K, bn)) return rc;
  dim3 grid((p.p_rows + BM - 1) / BM, (p.q_rows + bn - 1) / bn, splits);
  if (grid.y > 65535 || grid.z > 65535) return asb::fail("gemm_tcgen05: grid too large");
  int rc = 0;
  switch (bn) {
    case 16: rc = launch<16>(mp, mq, p, grid, stream); break;
    case 32: rc = launch<32>(mp, mq, p, grid, stream); break;
    case 64: rc = launch<64>(mp, mq, p, grid, stream); break;
    case 128: rc = launch<128>(mp, mq, p, grid, stream); break;
    default: rc = launch<256>(mp, mq, p, grid, stream); break;
  }
  if (rc) return rc;
  if (splits > 1) {
    const long long total = (long long)M * N;
    const int threads = 256;
    long long blocks = (total + threads - 1) / threads;
    if (blocks > 148 * 8) blocks = 148 * 8;
    splitk_reduce_kernel<<<(unsigned)blocks, threads, 0, stream>>>(out, workspace, (const __nv_bfloat16*)residual,
                                                                  total, splits, out_f32);
    return asb::check_launch("splitk_reduce");
  }
  return 0;
}
