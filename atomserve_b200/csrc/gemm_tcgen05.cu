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
// tokens (decoding, and up to 256 tokens on matrices of few rows) the operands swap: P = w, so
// that the 128-row MMA shape is filled with weight rows and the tokens are its N; the kernel
// then streams weights at HBM speed with a deep TMA pipeline (make_plan has the rule).
//
// The kernel is persistent: one block per SM walks a list of work segments (output tile, range
// of K blocks), the TMA pipeline running on across segment boundaries. Two schedules: whole
// tiles dealt round-robin (many tokens), or the flattened (tile, K block) sequence cut into one
// equal contiguous range per block (few tokens), so that every SM streams the same number of
// weight bytes whatever the number of tiles. A segment that covers all of K is stored
// directly; one that covers a part writes float32 partial sums to a workspace slot, and
// `segment_reduce_kernel` sums a tile's slots afterwards, unless the caller asked for the partial
// sums themselves (csrc/gemm_partials.cuh).
//
// Warp roles: warp 0 issues TMA loads, warp 1 allocates TMEM and issues MMAs, warps 2-5 run the
// epilogue (warp w reads TMEM lanes 32*(w%4)..+31). With narrow tiles (few tokens) a tcgen05.mma
// takes the tensor pipe far less time than its issue takes the issuing thread (60-80 cycles an
// instruction, whatever its shape: measured), so one thread cannot keep up with the weight stream:
// there, warps 6.. issue too. Issuer i takes every kIssuers-th K block of a segment into an
// accumulator of its own, and the epilogue adds the accumulators up. Stages are handed over
// with mbarriers: full[s] (TMA bytes landed) and empty[s] (tcgen05.commit after the MMAs that
// read stage s). The accumulator is double-buffered in TMEM: acc_full[b] tells the epilogue
// that buffer b is complete, acc_empty[b] tells the MMA warp that it has been read out, so the
// epilogue of one segment overlaps the MMAs of the next.
//
// Every wait on a barrier is bounded. A wait that runs out sets *status (non-zero) and the
// role stops waiting; all roles still meet at the final barrier, TMEM is freed and the block
// returns, so a fault in the pipeline shows as an error code, never as a hang.
#include <cuda.h>

#include "common.cuh"
#include "gemm_partials.cuh"
#include "tcgen05.cuh"

// How the pair kernel cuts its last round of tiles along K (gemm_tcgen05_pair.cu).
extern "C" long long asb_gemm_tcgen05_pair_cut(int M, int N, int K, int bn, int* out3);
extern "C" double asb_gemm_tcgen05_pair_us_per_kb(int bn);

namespace {

using asb::block_of;
using asb::range_begin;

constexpr int kMaxLoaders = 1;
constexpr int kMaxThreads = 192 + 32 + 32 * (kMaxLoaders - 1);
constexpr int BM = 128;   // P rows per tile = TMEM lanes
constexpr int BK = 64;    // K elements per stage: 128 bytes, one swizzle atom
constexpr int UMMA_K = 16;

enum Epilogue : int { kStoreBf16 = 0, kStoreBf16Residual = 1, kStoreF32 = 2, kStoreSwiGLU = 4, kPartialsOnly = 8 };

struct GemmParams {
  void* out;             // bf16 or f32 [M, N]
  const void* residual;  // bf16 [M, N] or null
  float* workspace;      // f32 [tiles][max_slots][128][BN] partial sums (stream schedule)
  int* status;           // device word, set non-zero by a wait that ran out
  int p_rows, q_rows;    // rows of P and Q (M and N, or N and M when swapped)
  int ldo;               // row stride of out (N)
  int swap;              // 1: P = w (lanes are output columns), Q = x
  int epilogue;          // kStoreBf16 / kStoreBf16Residual / kStoreF32 / kStoreSwiGLU (out is [M, N / 2]) /
                         // kPartialsOnly (every segment leaves its sums in a workspace slot; no out)
  int tiles_p, num_tiles;  // tile t -> (t % tiles_p, t / tiles_p)
  int kb_per_tile;       // K blocks of BK per tile
  int stream;            // 0: whole tiles round-robin; 1: equal contiguous ranges of K blocks
  int max_slots;         // workspace slots per tile
  int bn;                // Q rows per tile actually used (<= the kernel's BN; narrower tiles of unswapped weights)
  int stages;            // pipeline stages in use (a narrower tile leaves room for more of them)
  int stage_size;        // bytes from one stage's slot to the next: the P tile, then bn rows of Q, to a multiple of 1024
  // Optional timeline for profiling, null in normal use: %globaltimer stamps in rows of 8 words, 7
  // used per block (entry, set-up done, dependency wait over, first stage complete, last MMA
  // issued, last accumulator complete, epilogue done) and a row after the blocks for the reduction
  // kernel (entry, wait over, end).
  unsigned long long* stamps;
};

// Walks the segments of one block: the same sequence in every warp role.
struct SegmentWalk {
  int tile, kb0, kb1;       // current segment
  long long pos, end;       // stream schedule
  int step, stream, kb_per_tile, num_tiles;
  __device__ SegmentWalk(const GemmParams& p) {
    stream = p.stream; kb_per_tile = p.kb_per_tile; num_tiles = p.num_tiles; step = gridDim.x;
    if (stream) {
      const long long total = (long long)p.num_tiles * p.kb_per_tile;
      pos = range_begin(total, gridDim.x, blockIdx.x);
      end = range_begin(total, gridDim.x, blockIdx.x + 1);
    } else {
      pos = blockIdx.x; end = p.num_tiles;
    }
  }
  __device__ bool next() {
    if (pos >= end) return false;
    if (stream) {
      tile = (int)(pos / kb_per_tile);
      kb0 = (int)(pos - (long long)tile * kb_per_tile);
      const long long left = end - pos;
      kb1 = (int)((long long)kb_per_tile - kb0 < left ? kb_per_tile : kb0 + left);
      pos += kb1 - kb0;
    } else {
      tile = (int)pos; kb0 = 0; kb1 = kb_per_tile;
      pos += step;
    }
    return true;
  }
};

__device__ __forceinline__ unsigned long long global_timer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)::"memory");
  return t;
}
__device__ __forceinline__ void stamp(const GemmParams& p, int which) {
  if (p.stamps) p.stamps[(size_t)blockIdx.x * 8 + which] = global_timer();
}

// The PTX building blocks (mbarriers with bounded waits, TMA loads, descriptors, tcgen05.mma,
// commit and ld) are those of tcgen05.cuh, shared with the attention kernel.
using asb::t5::mbar_expect_tx;
using asb::t5::mbar_init;
using asb::t5::mbar_wait;
using asb::t5::smem_u32;
using asb::t5::tma_load_2d;
using asb::t5::umma_commit;

// K-major operand tiles, rows of 128 bytes in the 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) { return asb::t5::desc_k_major(addr, 1024); }
// D = f32, A = B = bf16, both K-major.
__host__ __device__ constexpr uint32_t instr_desc(int m, int n) { return asb::t5::instr_desc_bf16(m, n, false); }
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asb::t5::umma_bf16(tmem_d, a, b, idesc, accumulate);
}
// 32 lanes x N consecutive columns (N = 16 or 32): thread i of the warp gets lane (base lane + i).
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[32]) { asb::t5::tmem_ld32(taddr, r); }
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[16]) { asb::t5::tmem_ld16(taddr, r); }

template <int BN>
struct Config {
  static constexpr int kTileP = BM * BK * 2;   // 16 KB
  static constexpr int kTileQ = BN * BK * 2;
  static constexpr int kStage = kTileP + kTileQ;
  static constexpr int kStages = BN >= 256 ? 4 : (BN >= 128 ? 6 : 8);   // with tiles of the full BN rows of Q
  static constexpr int kIssuers = BN <= 128 ? 2 : 1;            // threads that issue MMAs, an accumulator each
  // Threads that request operands, a warp each (warp 0 and the warps after the issuing ones).
  // One thread's chain of wait, announcement and two TMA requests takes about 700 cycles per K
  // block whatever the boxes' sizes (714 with one thread, 353 with four, MMAs switched off), but
  // so does the chain of the thread that issues the MMAs, which is the one that bounds this
  // kernel: two or four loaders changed no shape's time here, so there is one.
  static constexpr int kLoaders = kMaxLoaders;
  static constexpr int kThreads = 192 + 32 * (kIssuers - 1) + 32 * (kLoaders - 1);
  static constexpr int kAccCols = kIssuers * BN;                // tensor-memory columns of one buffer
  static constexpr int kTmemCols = 2 * kAccCols < 32 ? 32 : 2 * kAccCols;   // two buffers
  // the 256-row kernel also runs narrower tiles, of which more stages fit: it takes all an SM has
  static constexpr int kStageRoom = BN >= 256 ? 227 * 1024 - 1024 - 256 : kStages * kStage;
  static constexpr int kSmem = kStageRoom + 1024 /* alignment slack */ + 256 /* barriers */;
  static constexpr int kMaxStages = 12;   // the barriers' 256 bytes hold 2 * 12 + 4 of them and the tensor-memory slot
};

// SwiGLU on a (gate, up) pair of float32 sums (atomserve/kernels.py:437-449).
__device__ __forceinline__ float swiglu(float gate, float up) { return gate / (1.f + __expf(-gate)) * up; }

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

template <int BN>
__global__ void __launch_bounds__(kMaxThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
                    const GemmParams p) {
  using C = Config<BN>;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;   // swizzle atoms need 1024-byte alignment
  unsigned char* aligned = smem_raw + (base - smem_u32(smem_raw));
  // the 256-column kernel takes both from the plan (narrower tiles leave room for more stages);
  // the others keep them as constants, which the one thread that issues their MMAs has no time to compute
  const int stages = BN >= 256 ? p.stages : C::kStages;
  const uint32_t stage_size = BN >= 256 ? (uint32_t)p.stage_size : (uint32_t)C::kStage;
  const uint32_t bars = base + stages * stage_size;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (stages + s); };
  auto acc_full = [&](int b) { return bars + 8u * (2 * stages + b); };
  auto acc_empty = [&](int b) { return bars + 8u * (2 * stages + 2 + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(aligned + stages * stage_size + 8 * (2 * stages + 4));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bn = p.bn;                                               // Q rows per tile: BN unless the plan narrowed it
  const uint32_t stage_bytes = (uint32_t)(C::kTileP + bn * BK * 2);  // what one K block's two boxes bring

  if (threadIdx.x == 0) {
    stamp(p, 0);
    for (int s = 0; s < stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full(b), C::kIssuers);  // one commit per issuing thread
      mbar_init(acc_empty(b), 4);  // one arrival per epilogue warp
    }
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
  if (threadIdx.x == 0) stamp(p, 1);
  // Everything above touched only this block's shared and tensor memory: with a programmatic
  // dependent launch it ran while the stream's previous kernel was finishing. Each role calls
  // pdl_wait() before it first reads that kernel's output; the TMA warp first fills the pipeline
  // with the weight operand, which no kernel writes.

  constexpr int kFirstExtraLoader = 6 + C::kIssuers - 1;  // warps 0 and kFirstExtraLoader.. load
  if (warp == 0 || warp >= kFirstExtraLoader) {
    if (lane == 0) {
      // Loader `me` of kLoaders brings every kLoaders-th K block of the block's sequence. The
      // weights are operand P when swapped, Q otherwise. Before waiting for the previous kernel,
      // the first `stages` stages are filled with the weight half; the activation half follows.
      const uint32_t me = warp == 0 ? 0u : (uint32_t)(warp - kFirstExtraLoader + 1);
      {
        SegmentWalk ahead(p);
        uint32_t it = 0;
        while (it < (uint32_t)stages && ahead.next()) {
          const int p0 = (ahead.tile % p.tiles_p) * BM, q0 = (ahead.tile / p.tiles_p) * bn;
          for (int kb = ahead.kb0; kb < ahead.kb1 && it < (uint32_t)stages; ++kb, ++it) {
            if (it % C::kLoaders != me) continue;
            mbar_expect_tx(full_bar(it), stage_bytes);
            if (p.swap) tma_load_2d(base + it * stage_size, &map_p, full_bar(it), kb * BK, p0);
            else tma_load_2d(base + it * stage_size + C::kTileP, &map_q, full_bar(it), kb * BK, q0);
          }
        }
      }
      asb::pdl_wait();
      if (me == 0) {
        stamp(p, 2);
        asb::pdl_launch_dependents();
      }
      SegmentWalk walk(p);
      uint32_t it = 0;  // K blocks of this block so far, across segments
      uint32_t turn = 0;    // it % kLoaders: whose K block this is
      int s = 0;            // the stage K block `it` goes to, and the phase of its barriers:
      uint32_t phase = 0;   // it % stages and (it / stages) & 1, kept by counting
      bool ok = true;
      while (ok && walk.next()) {
        const int p0 = (walk.tile % p.tiles_p) * BM, q0 = (walk.tile / p.tiles_p) * bn;
        for (int kb = walk.kb0; kb < walk.kb1; ++kb, ++it) {
          if (turn == me) {
            if (it < (uint32_t)stages) {  // the weight half is already on its way
              if (p.swap) tma_load_2d(base + s * stage_size + C::kTileP, &map_q, full_bar(s), kb * BK, q0);
              else tma_load_2d(base + s * stage_size, &map_p, full_bar(s), kb * BK, p0);
            } else {
              ok = mbar_wait(empty_bar(s), phase ^ 1u, p.status, 1);
              if (!ok) break;
              mbar_expect_tx(full_bar(s), stage_bytes);
              tma_load_2d(base + s * stage_size, &map_p, full_bar(s), kb * BK, p0);
              tma_load_2d(base + s * stage_size + C::kTileP, &map_q, full_bar(s), kb * BK, q0);
            }
          }
          if (++turn == (uint32_t)C::kLoaders) turn = 0;
          if (++s == stages) { s = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1 || (warp >= 6 && warp < kFirstExtraLoader)) {
    asb::pdl_wait();
    if (lane == 0) {
      const int me = warp == 1 ? 0 : warp - 5;  // which of the kIssuers issuing threads
      const uint32_t idesc = instr_desc(BM, bn);
      SegmentWalk walk(p);
      uint32_t it = 0, seg = 0;
      int s = -1;           // the stage of K block `it`, it % stages, and its barriers' phase,
      uint32_t phase = 0;   // (it / stages) & 1: advanced at the top of every K block
      bool ok = true;
      while (ok && walk.next()) {
        const uint32_t buf = seg & 1u;
        // the epilogue must have read this accumulator out (its use two segments ago)
        ok = mbar_wait(acc_empty(buf), ((seg >> 1) & 1u) ^ 1u, p.status, 4);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_acc = tmem_base + buf * C::kAccCols + me * BN;
        for (int kb = walk.kb0; kb < walk.kb1; ++kb, ++it) {
          if (++s == stages) { s = 0; phase ^= 1u; }
          if (C::kIssuers > 1 && (kb - walk.kb0) % C::kIssuers != me) continue;
          ok = mbar_wait(full_bar(s), phase, p.status, 2);
          if (!ok) break;
          if (it == 0) stamp(p, 3);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint64_t da = smem_desc(base + s * stage_size);
          const uint64_t db = smem_desc(base + s * stage_size + C::kTileP);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)  // 32 bytes further along K inside the swizzle atom
            umma(tmem_acc, da + (uint64_t)(k * UMMA_K * 2 >> 4), db + (uint64_t)(k * UMMA_K * 2 >> 4), idesc,
                 (uint32_t)((kb - walk.kb0 >= C::kIssuers) | (k != 0)));
          umma_commit(empty_bar(s));  // stage s may be refilled once these MMAs have read it
        }
        umma_commit(acc_full(buf));  // arrives when every MMA this thread issued for the segment has completed
        if (me == 0) stamp(p, 4);
        ++seg;
      }
    }
  } else {
    // Epilogue: this warp owns TMEM lanes 32*(warp%4)..+31, one lane (P row) per thread.
    asb::pdl_wait();  // it reads the residual and writes where earlier kernels may still be reading
    const int quad = warp & 3;
    SegmentWalk walk(p);
    uint32_t seg = 0;
    bool ok = true;
    while (ok && walk.next()) {
      const uint32_t buf = seg & 1u;
      int ok_i = 1;
      if (lane == 0) ok_i = mbar_wait(acc_full(buf), (seg >> 1) & 1u, p.status, 3) ? 1 : 0;  // one poller per warp
      ok = __shfl_sync(0xffffffffu, ok_i, 0) != 0;
      if (!ok) break;
      if (warp == 2 && lane == 0) stamp(p, 5);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int p0 = (walk.tile % p.tiles_p) * BM, q0 = (walk.tile / p.tiles_p) * bn;
      const int prow = p0 + quad * 32 + lane;
      const bool whole = walk.kb0 == 0 && walk.kb1 == p.kb_per_tile && p.epilogue != kPartialsOnly;
      float* slot = nullptr;
      if (!whole) {
        const long long total = (long long)p.num_tiles * p.kb_per_tile;
        const int first = block_of(total, gridDim.x, (long long)walk.tile * p.kb_per_tile);
        // a slot is laid out [column][lane] (csrc/gemm_partials.cuh)
        slot = p.workspace + ((size_t)walk.tile * p.max_slots + (blockIdx.x - first)) * BM * BN;
      }
      constexpr int kChunk = BN >= 32 ? 32 : 16;  // columns read from tensor memory at a time
#pragma unroll 1
      for (int c = 0; c < bn; c += kChunk) {
        if (q0 + c >= p.q_rows) break;  // uniform: depends on the segment and c only
        uint32_t raw[kChunk];
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * C::kAccCols + (uint32_t)c;
        tmem_ld(taddr, raw);
        // the other issuing threads' accumulators, as far as the segment gave them K blocks
#pragma unroll
        for (int i = 1; i < C::kIssuers; ++i) {
          if (walk.kb1 - walk.kb0 <= i) break;
          uint32_t more[kChunk];
          tmem_ld(taddr + i * BN, more);
#pragma unroll
          for (int j = 0; j < kChunk; ++j) raw[j] = __float_as_uint(__uint_as_float(raw[j]) + __uint_as_float(more[j]));
        }
        if (!whole) {  // partial sums; rows beyond the matrix hold zeros
          const int row = quad * 32 + lane;
          // K is cut only with swapped operands: lanes are output columns, and a warp's 32 lanes
          // store 128 contiguous bytes of the slot's [column][lane] layout per instruction
#pragma unroll
          for (int j = 0; j < kChunk; ++j)
            if (q0 + c + j < p.q_rows) slot[(size_t)(c + j) * BM + row] = __uint_as_float(raw[j]);  // tokens that exist
          continue;
        }
        if (p.epilogue == kStoreSwiGLU) {
          // weight rows alternate gate, up: output column n / 2 = silu(sum[n]) * sum[n + 1]
          if (p.swap) {
            // lanes are weight rows: the up sum sits in the next lane
#pragma unroll
            for (int j = 0; j < kChunk; ++j) {
              const float up = __shfl_down_sync(0xffffffffu, __uint_as_float(raw[j]), 1);
              const int tok = q0 + c + j;
              if ((lane & 1) == 0 && prow < p.p_rows && tok < p.q_rows)
                ((__nv_bfloat16*)p.out)[(size_t)tok * (p.ldo / 2) + prow / 2] = __float2bfloat16_rn(swiglu(__uint_as_float(raw[j]), up));
            }
          } else if (prow < p.p_rows) {
            // columns are weight rows: this thread holds kChunk / 2 (gate, up) pairs of its token
            __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)prow * (p.ldo / 2) + (q0 + c) / 2;
            const int valid = min(kChunk, p.q_rows - (q0 + c)) / 2;
            uint4 packed[kChunk / 16];
            __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(packed);
#pragma unroll
            for (int j = 0; j < kChunk / 2; ++j)
              ob[j] = __float2bfloat16_rn(swiglu(__uint_as_float(raw[2 * j]), __uint_as_float(raw[2 * j + 1])));
            if (valid == kChunk / 2 && (((uintptr_t)o) & 15) == 0) {
#pragma unroll
              for (int v = 0; v < kChunk / 16; ++v) *reinterpret_cast<uint4*>(o + 8 * v) = packed[v];
            } else {
#pragma unroll
              for (int j = 0; j < kChunk / 2; ++j)
                if (j < valid) o[j] = ob[j];
            }
          }
          continue;
        }
        if (prow >= p.p_rows) continue;
        if (p.swap) {
          // lanes are output columns (weight rows), TMEM columns are tokens: out[token, prow]
#pragma unroll
          for (int j = 0; j < kChunk; ++j) {
            const int tok = q0 + c + j;
            if (tok < p.q_rows) {
              const size_t at = (size_t)tok * p.ldo + prow;
              float v = __uint_as_float(raw[j]);
              if (p.epilogue == kStoreF32) {
                ((float*)p.out)[at] = v;
              } else {
                if (p.epilogue == kStoreBf16Residual) v += __bfloat162float(((const __nv_bfloat16*)p.residual)[at]);
                ((__nv_bfloat16*)p.out)[at] = __float2bfloat16_rn(v);
              }
            }
          }
        } else {
          // lanes are tokens, TMEM columns are output columns: out[prow, q0 + c + j], contiguous in j
          const size_t at = (size_t)prow * p.ldo + q0 + c;
          const int valid = min(kChunk, p.q_rows - (q0 + c));
          if (p.epilogue == kStoreF32) {
            float* o = (float*)p.out + at;
            if (valid == kChunk && (((uintptr_t)o) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < kChunk; j += 4)
                *reinterpret_cast<uint4*>(o + j) = make_uint4(raw[j], raw[j + 1], raw[j + 2], raw[j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < kChunk; ++j)
                if (j < valid) o[j] = __uint_as_float(raw[j]);
            }
          } else {
            __nv_bfloat16* o = (__nv_bfloat16*)p.out + at;
            const __nv_bfloat16* res = p.epilogue == kStoreBf16Residual ? (const __nv_bfloat16*)p.residual + at : nullptr;
            if (valid == kChunk && (((uintptr_t)o) & 15) == 0 && (!res || (((uintptr_t)res) & 15) == 0)) {
              uint4 rv[kChunk / 8];
              if (res) {
#pragma unroll
                for (int v = 0; v < kChunk / 8; ++v) rv[v] = *reinterpret_cast<const uint4*>(res + 8 * v);
              }
              const __nv_bfloat16* rb = reinterpret_cast<const __nv_bfloat16*>(rv);
              uint4 ov[kChunk / 8];
              __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(ov);
#pragma unroll
              for (int j = 0; j < kChunk; j += 2) {
                float a = __uint_as_float(raw[j]), b = __uint_as_float(raw[j + 1]);
                if (res) { a += __bfloat162float(rb[j]); b += __bfloat162float(rb[j + 1]); }
                ob[j >> 1] = __floats2bfloat162_rn(a, b);
              }
#pragma unroll
              for (int v = 0; v < kChunk / 8; ++v) *reinterpret_cast<uint4*>(o + 8 * v) = ov[v];
            } else {
#pragma unroll
              for (int j = 0; j < kChunk; ++j)
                if (j < valid) {
                  float v = __uint_as_float(raw[j]);
                  if (res) v += __bfloat162float(res[j]);
                  o[j] = __float2bfloat16_rn(v);
                }
            }
          }
        }
      }
      // this warp has read its lanes of the accumulator: hand the buffer back to the MMA warp
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty(buf));
      ++seg;
    }
    if (warp == 2 && lane == 0) stamp(p, 6);
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::kTmemCols) : "memory");
  }
}

// Sums the workspace slots of every tile that was computed in parts, adds the residual and
// stores in the output's orientation. grid = (tiles, pieces of the tile); each thread owns four
// consecutive elements along the output's contiguous dimension. Tiles stored whole are skipped.
template <int BN>
__global__ void segment_reduce_kernel(const GemmParams p, int parts) {
  // the index arithmetic needs nothing from the GEMM: it runs while the GEMM drains
  const int tile = blockIdx.x;
  const long long total = (long long)p.num_tiles * p.kb_per_tile;
  const long long begin = (long long)tile * p.kb_per_tile;
  const int first = block_of(total, parts, begin), last = block_of(total, parts, begin + p.kb_per_tile - 1);
  const int slots = last - first + 1;
  const int p0 = (tile % p.tiles_p) * BM, q0 = (tile / p.tiles_p) * BN;
  const float* ws = p.workspace + (size_t)tile * p.max_slots * BM * BN;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  unsigned long long* stamps = p.stamps ? p.stamps + (size_t)parts * 8 : nullptr;
  const bool first_thread = blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0;
  if (stamps && first_thread) stamps[0] = global_timer();
  asb::pdl_wait();  // the GEMM has completed (programmatic dependent launch)
  if (stamps && first_thread) stamps[1] = global_timer();
  struct AtExit {
    unsigned long long* stamps;
    __device__ ~AtExit() { if (stamps && threadIdx.x == 0) atomicMax(stamps + 2, global_timer()); }
  } at_exit{stamps};
  asb::pdl_launch_dependents();
  if (slots == 1) return;  // one block covered all of K and stored the tile itself
  if (i >= BM * BN) return;
  if (q0 + i / BM >= p.q_rows) return;  // a column (token) beyond the matrix: its slots were not written
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s0 = 0; s0 < slots; s0 += 4) {  // four loads in flight; the sum still runs in slot order
    float4 a[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (s0 + u < slots) a[u] = *reinterpret_cast<const float4*>(ws + (size_t)(s0 + u) * BM * BN + i);
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (s0 + u < slots) { v.x += a[u].x; v.y += a[u].y; v.z += a[u].z; v.w += a[u].w; }
  }
  const float e[4] = {v.x, v.y, v.z, v.w};
  if (p.epilogue == kStoreSwiGLU) {
    // the four sums are two (gate, up) pairs along the weight-row dimension, the slot's contiguous one
#pragma unroll
    for (int k = 0; k < 4; k += 2) {
      const int row = (i + k) % BM, col = (i + k) / BM;
      const int prow = p0 + row, qrow = q0 + col;
      if (prow >= p.p_rows || qrow >= p.q_rows) continue;
      const size_t at = (size_t)qrow * (p.ldo / 2) + prow / 2;
      ((__nv_bfloat16*)p.out)[at] = __float2bfloat16_rn(swiglu(e[k], e[k + 1]));
    }
    return;
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    // slot layout [column][lane]: lanes are output columns (weight rows), columns are tokens
    const int row = (i + k) % BM, col = (i + k) / BM;
    const int prow = p0 + row, qrow = q0 + col;
    if (prow >= p.p_rows || qrow >= p.q_rows) continue;
    const size_t at = (size_t)qrow * p.ldo + prow;
    float o = e[k];
    if (p.epilogue == kStoreF32) {
      ((float*)p.out)[at] = o;
    } else {
      if (p.epilogue == kStoreBf16Residual) o += __bfloat162float(((const __nv_bfloat16*)p.residual)[at]);
      ((__nv_bfloat16*)p.out)[at] = __float2bfloat16_rn(o);
    }
  }
}

// A [rows, K] row-major bfloat16 matrix as a 2-D tensor map with boxes of box_rows x 64.
int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  return asb::t5::make_bf16_map(map, ptr, 2, dims, strides, box);
}

int sm_count() {
  static int count = 0;
  if (!count) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count < 1)
      count = 148;
  }
  return count;
}

unsigned long long* g_stamps = nullptr;  // asb_gemm_tcgen05_timeline

struct Plan {
  int swap, bn, bn_kernel, tiles_p, tiles_q, kb_per_tile, stream, blocks, max_slots;
  int stages, stage_size;
  int pair;             // 0, or the weight rows (128 to 256 in steps of 32) of the tiles that pairs of SMs compute (gemm_tcgen05_pair.cu)
  long long workspace;  // float32 elements
};

// Tuning aid (asb_gemm_tcgen05_tune): orientation and tile width forced for the calls that follow.
int g_force_swap = -1, g_force_bn = 0;

int stage_room(int bn_kernel) {
  switch (bn_kernel) {
    case 16: return Config<16>::kStageRoom;
    case 32: return Config<32>::kStageRoom;
    case 64: return Config<64>::kStageRoom;
    case 128: return Config<128>::kStageRoom;
    default: return Config<256>::kStageRoom;
  }
}

// How a shape is run. One block runs per SM (or one pair of blocks per pair of SMs).
//
// Up to 128 tokens the operands swap (weights fill the 128-row MMA, tokens are its N = 16..256)
// always for up to 32 tokens, and beyond where the unswapped tiles of 128 x 256 would leave over
// half of the SMs idle (few weight rows: qkv, o, down); where they fill the machine (gate/up, the
// head) whole unswapped tiles win from 33 tokens on (measured on the 8B and 14B shapes).
//
// With more than 128 tokens the forms are compared by an estimate of their time in microseconds,
// a fixed part plus rounds of tiles times K blocks times the form's time per K block, with
// constants fitted to the twelve projection shapes of Qwen3-8B, -14B and -32B at 200 to 2,048
// tokens (over those 84 cases the estimate's choice is within 0.1 % of the best form's time
// summed, and never more than 2 % behind it on one):
//   unswapped tiles of 128 tokens by bn weight rows, bn a multiple of 32 from 64 to 256 (the
//     epilogue reads 32 columns at a time): up to 128 rows in the 128-column kernel (six stages),
//     wider ones in the 256-column kernel with as many stages as fit; an SM's time per K block
//     goes with the bytes it takes in, so narrower tiles that occupy more SMs win where wide
//     ones leave SMs idle, as long as they need no further round;
//   tiles of 256 tokens by 128 to 256 weight rows (in steps of 32) on pairs of SMs (gemm_tcgen05_pair.cu), whose
//     last round can be cut along K: twice the arithmetic per byte taken in, so with enough
//     tiles to fill the device the 256-row tile wins (gate/up at 2,048 tokens: 339 -> 268 us, the
//     vendor library 284), and the 128-row tile where there are few weight rows and a few
//     hundred tokens (o at 512 tokens on the 14B shape: 34.5 -> 27.6 us);
//   swapped operands with the flattened K-block sequence cut into equal ranges, up to 512 tokens:
//     the partial sums cost about 14 us, which only long K over few tokens repays (down at 200).
// With swapped operands, whole tiles are dealt round-robin unless cutting the flattened K-block
// sequence into equal ranges shortens the busiest SM's share of the operand stream by more than
// the partial sums cost to write and read back; unswapped single-SM tiles are never cut.
Plan make_plan(int M, int N, int K) {
  Plan pl;
  const int sms_now = sm_count();
  const int unswapped_tiles = ((M + BM - 1) / BM) * ((N + 255) / 256);
  const int kb_per_tile = (K + BK - 1) / BK;
  pl.pair = 0;
  pl.swap = M <= 32 || (M <= BM && 2 * unswapped_tiles < sms_now) ? 1 : 0;
  pl.bn = pl.swap ? (M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128))) : (N <= 128 ? 128 : 256);
  pl.bn_kernel = pl.bn;
  if (M <= BM && !pl.swap && N > 128) {
    // one row of unswapped tiles: the narrowest tiles that need no further round (time per K
    // block goes with the bytes taken in, the tokens' box and bn weight rows)
    double best = 1e30;
    for (int bn = 256; bn >= 64; bn -= 32) {
      const int tiles = (N + bn - 1) / bn;
      const double cost = (double)((tiles + sms_now - 1) / sms_now) * (128 + bn);
      if (cost < best) { best = cost; pl.bn = bn; pl.bn_kernel = bn <= 128 ? 128 : 256; }
    }
  }
  if (M > BM && g_force_swap < 0) {
    const double kb = kb_per_tile;
    const int token_tiles = (M + BM - 1) / BM, pairs = sms_now / 2;
    double best = 1e30;
    if (N > 128) {
      for (int bn = 256; bn >= 64; bn -= 32) {
        const int tiles = token_tiles * ((N + bn - 1) / bn);
        const double per_kb = bn <= 128 ? 0.1724 + 0.0595 * bn / 128.0 : 0.26 + 0.1337 * bn / 256.0;
        const double cost = 4.0 + (double)((tiles + sms_now - 1) / sms_now) * kb * per_kb;
        if (cost < best) { best = cost; pl.swap = 0; pl.pair = 0; pl.bn = bn; pl.bn_kernel = bn <= 128 ? 128 : 256; }
      }
    } else {
      best = 4.0 + (double)((token_tiles + sms_now - 1) / sms_now) * kb * 0.2319;
      pl.swap = 0; pl.bn = pl.bn_kernel = 128;
    }
    for (int bn = 256; bn >= 128; bn -= 32) {
      const int tiles = ((M + 255) / 256) * ((N + bn - 1) / bn);
      const double per_kb = asb_gemm_tcgen05_pair_us_per_kb(bn);
      double cost = (double)((tiles + pairs - 1) / pairs) * kb * per_kb;
      int cut[3];
      const long long floats = asb_gemm_tcgen05_pair_cut(M, N, K, bn, cut);
      if (floats > 0)  // the last round cut along K: its pieces, and their sums written and read back
        cost = (double)(cut[0] / pairs) * kb * per_kb + 2.0 * cut[2] * per_kb + 3.0 + 8.0 * floats / 3.0e6;
      cost += 5.98;
      if (cost < best) { best = cost; pl.swap = 0; pl.pair = bn; }
    }
    if (M <= 512) {
      const double share = (double)((N + BM - 1) / BM) * ((M + 255) / 256) * kb / sms_now;  // K blocks per SM
      const double cost = 14.0 + (share < 4 ? 4 : share) * 0.457;
      if (cost < best) { best = cost; pl.swap = 1; pl.pair = 0; pl.bn = pl.bn_kernel = 256; }
    }
  }
  if (g_force_swap >= 0) {  // the tuning aid's choice
    pl.swap = g_force_swap == 1 ? 1 : 0;
    pl.pair = g_force_swap == 2 && M > BM ? (g_force_bn >= 128 && g_force_bn <= 256 && g_force_bn % 32 == 0 ? g_force_bn : 256) : 0;
    if (pl.swap) pl.bn = pl.bn_kernel = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256)));
    else if (N <= 128) pl.bn = pl.bn_kernel = 128;
    else {
      pl.bn = g_force_bn && g_force_swap != 2 ? g_force_bn : 256;
      pl.bn_kernel = pl.bn <= 128 ? 128 : 256;
    }
  }
  pl.stage_size = BM * BK * 2 + ((pl.bn * BK * 2 + 1023) / 1024) * 1024;
  pl.stages = stage_room(pl.bn_kernel) / pl.stage_size;
  if (pl.stages > Config<256>::kMaxStages) pl.stages = Config<256>::kMaxStages;
  const int p_rows = pl.swap ? N : M, q_rows = pl.swap ? M : N;
  pl.tiles_p = (p_rows + BM - 1) / BM;
  pl.tiles_q = (q_rows + pl.bn - 1) / pl.bn;
  pl.kb_per_tile = (K + BK - 1) / BK;
  const int tiles = pl.tiles_p * pl.tiles_q, sms = sm_count();
  const long long total = (long long)tiles * pl.kb_per_tile;
  // whole tiles: the busiest block runs ceil(tiles / blocks) tiles
  const int whole_blocks = tiles < sms ? tiles : sms;
  const double whole_cost = (double)((tiles + whole_blocks - 1) / whole_blocks) * pl.kb_per_tile;
  // equal ranges: every block runs total / blocks K blocks (at least four), plus the partials
  int stream_blocks = (int)(total / 4 < sms ? total / 4 : sms);
  if (stream_blocks < 1) stream_blocks = 1;
  const double per_block = (double)total / stream_blocks;
  const double kb_bytes = (double)(BM + pl.bn) * BK * 2;             // operand bytes one K block brings
  const double cut_tiles = stream_blocks < tiles ? stream_blocks : tiles;  // tiles a range boundary falls into
  const double partial_bytes = 2.0 * 2.0 * cut_tiles * BM * pl.bn * 4;     // two slots each, written and read
  const double stream_cost = per_block + partial_bytes / kb_bytes / stream_blocks;
  // (measured: one SM draws about 60 GB/s however deep its pipeline, so few tiles never fill the
  // device without cutting K; many tiles in nearly whole waves are best left whole)
  pl.stream = pl.swap && stream_cost < whole_cost * 0.97 ? 1 : 0;
  pl.blocks = pl.stream ? stream_blocks : whole_blocks;
  if (pl.pair) pl.stream = 0;
  pl.max_slots = 0;
  pl.workspace = 0;
  if (pl.pair) {
    int cut[3];
    pl.workspace = asb_gemm_tcgen05_pair_cut(M, N, K, pl.pair, cut);
  }
  if (pl.stream) {
    const long long shortest = total / pl.blocks;  // the shortest range
    pl.max_slots = (int)((pl.kb_per_tile + shortest - 1) / shortest) + 1;
    pl.workspace = (long long)tiles * pl.max_slots * BM * pl.bn;
  }
  return pl;
}

template <int BN>
int launch(const CUtensorMap& mp, const CUtensorMap& mq, const GemmParams& p, const Plan& pl, cudaStream_t stream) {
  auto kern = gemm_tcgen05_kernel<BN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Config<BN>::kSmem);
  if (e != cudaSuccess) return asb::fail("gemm_tcgen05: shared memory %d: %s", Config<BN>::kSmem, cudaGetErrorString(e));
  asb::launch(kern, pl.blocks, Config<BN>::kThreads, Config<BN>::kSmem, stream, mp, mq, p);
  if (int rc = asb::check_launch("gemm_tcgen05")) return rc;
  if (pl.stream && p.epilogue != kPartialsOnly) {
    asb::launch(segment_reduce_kernel<BN>, dim3(p.num_tiles, (BM * BN / 4 + 255) / 256), 256, 0, stream, p, pl.blocks);
    return asb::check_launch("gemm_tcgen05 segment_reduce");
  }
  return 0;
}

}  // namespace

// The form for many tokens on pairs of SMs (gemm_tcgen05_pair.cu).
extern "C" int asb_gemm_tcgen05_pair(void* out, const void* x, const void* w, const void* residual, int M, int N,
                                     int K, int mode, int bn, float* workspace, int* status, cudaStream_t stream);

// Float32 workspace elements a call needs (0 when every tile is computed whole).
extern "C" long long asb_gemm_tcgen05_workspace(int M, int N, int K, int* stream_out) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const Plan pl = make_plan(M, N, K);
  if (stream_out) *stream_out = pl.stream;
  return pl.workspace;
}

// Profiling aid: later calls write their timeline (see GemmParams::stamps) into `buffer`, device
// memory of (blocks + 1) * 8 64-bit words that the caller zeroes; null switches it off again.
extern "C" void asb_gemm_tcgen05_timeline(void* buffer) { g_stamps = (unsigned long long*)buffer; }

// Tuning aid: force the orientation (swap 0: unswapped on single SMs, 1: swapped, 2: pairs of
// SMs; -1 automatic) and, for unswapped tiles, the weight rows per tile (single SMs: a multiple of
// 32 from 64 to 256; pairs: 128 to 256 in steps of 32; 0 automatic) of the calls that follow.
extern "C" void asb_gemm_tcgen05_tune(int swap, int bn) { g_force_swap = swap; g_force_bn = bn; }

// How a shape is run: out8 = {cuts K (1) or whole tiles (0), swapped operands, workspace slots per
// tile, token columns (swapped) or weight rows (unswapped) per tile, K blocks per tile, tiles,
// thread blocks, weight rows of the tiles of pairs of SMs (0: single SMs)}. With pairs, a tile is
// 256 tokens by that many weight rows and two thread blocks share it; how the last round of
// tiles is cut along K, asb_gemm_tcgen05_pair_cut tells. A shape that cuts K with
// swapped operands can leave its product as partial sums (mode 3 of asb_gemm_tcgen05), which
// csrc/gemm_partials.cuh describes.
extern "C" int asb_gemm_tcgen05_plan(int M, int N, int K, int* out8) {
  if (M <= 0 || N <= 0 || K <= 0) return asb::fail("gemm_tcgen05_plan: empty shape");
  const Plan pl = make_plan(M, N, K);
  out8[0] = pl.stream; out8[1] = pl.swap; out8[2] = pl.max_slots; out8[3] = pl.bn;
  out8[4] = pl.kb_per_tile; out8[5] = pl.tiles_p * pl.tiles_q; out8[6] = pl.blocks;
  out8[7] = pl.pair;
  if (pl.pair) {
    const int tiles = ((M + 255) / 256) * ((N + pl.pair - 1) / pl.pair), pairs = sm_count() / 2;
    int cut[3];
    asb_gemm_tcgen05_pair_cut(M, N, K, pl.pair, cut);  // with few tiles, cut[1] pairs share each
    out8[3] = pl.pair; out8[5] = tiles; out8[6] = 2 * (tiles < pairs ? tiles * cut[1] : pairs);
  }
  return 0;
}

// out = x . w^T (+ residual). x [M, K] and w [N, K] bfloat16, contiguous, K a multiple of 8 and
// both bases 16-byte aligned (TMA's rules). out bfloat16 [M, N], float32, or [M, N / 2] by mode.
// workspace: float32, asb_gemm_tcgen05_workspace(M, N, K) elements (null if that is 0); calls that
// may overlap on the GPU need separate workspaces.
// status: one int on the device; it stays 0 unless a pipeline wait ran out.
// mode 0: out bfloat16 (+ residual); 1: out float32; 2: SwiGLU: the rows of w alternate gate and
// up (row 2i gate_i, row 2i + 1 up_i) and out is bfloat16 [M, N / 2] = silu(gate) * up; 3: no out:
// the product stays in the workspace as float32 partial sums for a consumer kernel to add up
// (only for shapes whose plan cuts K with swapped operands, and then tiles_q is 1).
extern "C" int asb_gemm_tcgen05(void* out, const void* x, const void* w, const void* residual, int M,
                                int N, int K, int mode, float* workspace, int* status,
                                cudaStream_t stream) {
  const int out_f32 = mode == 1;
  if (mode < 0 || mode > 3) return asb::fail("gemm_tcgen05: unknown mode %d", mode);
  if (mode == 3 && residual) return asb::fail("gemm_tcgen05: the partial-sum form takes no residual");
  if (mode == 2 && (residual || N % 2)) return asb::fail("gemm_tcgen05: the SwiGLU form takes no residual and an even N");
  if (M == 0 || N == 0) return 0;
  if (K < 8 || K % 8) return asb::fail("gemm_tcgen05: K = %d must be a positive multiple of 8 (16-byte TMA rows)", K);
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return asb::fail("gemm_tcgen05: operands must be 16-byte aligned");
  if (out_f32 && residual) return asb::fail("gemm_tcgen05: the float32 result form takes no residual");
  if (!status) return asb::fail("gemm_tcgen05: a status word is required");
  const Plan pl = make_plan(M, N, K);
  if (mode == 3 && !(pl.stream && pl.swap && pl.tiles_q == 1))
    return asb::fail("gemm_tcgen05: [%d, %d] x [%d, %d] does not run with partial sums", M, K, N, K);
  if (pl.pair && mode != 3)
    return asb_gemm_tcgen05_pair(out, x, w, residual, M, N, K, mode, pl.pair, workspace, status, stream);
  if (pl.workspace > 0 && !workspace) return asb::fail("gemm_tcgen05: this shape needs a workspace of %lld floats", pl.workspace);

  GemmParams p;
  p.out = out;
  p.residual = residual;
  p.workspace = workspace;
  p.status = status;
  p.swap = pl.swap;
  p.ldo = N;
  p.p_rows = pl.swap ? N : M;
  p.q_rows = pl.swap ? M : N;
  p.epilogue = mode == 3 ? kPartialsOnly : mode == 2 ? kStoreSwiGLU : (out_f32 ? kStoreF32 : (residual ? kStoreBf16Residual : kStoreBf16));
  p.tiles_p = pl.tiles_p;
  p.num_tiles = pl.tiles_p * pl.tiles_q;
  p.kb_per_tile = pl.kb_per_tile;
  p.stream = pl.stream;
  p.max_slots = pl.max_slots;
  p.bn = pl.bn;
  p.stages = pl.stages;
  p.stage_size = pl.stage_size;
  p.stamps = g_stamps;
  alignas(64) CUtensorMap mp, mq;
  if (int rc = make_map(&mp, pl.swap ? w : x, p.p_rows, K, BM)) return rc;
  if (int rc = make_map(&mq, pl.swap ? x : w, p.q_rows, K, pl.bn)) return rc;
  switch (pl.bn_kernel) {
    case 16: return launch<16>(mp, mq, p, pl, stream);
    case 32: return launch<32>(mp, mq, p, pl, stream);
    case 64: return launch<64>(mp, mq, p, pl, stream);
    case 128: return launch<128>(mp, mq, p, pl, stream);
    default: return launch<256>(mp, mq, p, pl, stream);
  }
}
