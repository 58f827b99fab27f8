// bfloat16 GEMM for many tokens on pairs of SMs: out[M, N] = x[M, K] . w[N, K]^T with
// tcgen05.mma.cta_group::2. Two CTAs on the two SMs of a pair (a cluster of two) compute one tile
// of 256 tokens by up to BN weight rows (the kernel built for 256 also runs tiles of 160, 192 and
// 224 rows: narrower tiles let one round occupy more pairs). Each CTA loads its own 128 token rows and half of the tile's
// weight rows, the pair's MMA reads both halves of the weights from the two shared memories, and
// each CTA's tensor memory receives its 128 token rows of the result. Per unit of arithmetic an
// SM so takes in two thirds (BN = 256) of the bytes a single CTA's 128 x 256 tile asks for, and
// its shared memory holds that much more work in flight, which is what the single-CTA kernel
// lacks with many tokens: the round trip of one of its four stages (MMAs done, commit, producer
// wakes, TMA request, L2 latency, barrier, MMA thread wakes) is longer than the MMAs of the other
// three (csrc/gemm_tcgen05.cu has that kernel and the swapped, few-token forms).
//
// Roles per CTA: warps 0 and 6-8 load (TMA, no multicast), warp 1 of the even CTA issues the pair's MMAs,
// warps 2-5 run the epilogue for the CTA's 128 token rows. Barriers: full[s] lives in the even
// CTA and counts both CTAs' arrivals and bytes (the odd CTA's TMA completes there through the
// cluster address); empty[s] and acc_full[b] exist in both CTAs and are signalled in both by one
// tcgen05.commit with a multicast of the arrival (not of any load); acc_empty[b] lives in the
// even CTA and takes one arrival per epilogue warp of either CTA. Before a CTA leaves, its first
// loader waits for the last use of every stage to be handed back, so that no commit is still on
// its way into a CTA that has gone. Every wait is bounded
// (tcgen05.cuh); a wait that runs out sets the status word, the roles wind down, both CTAs meet at
// a cluster barrier, tensor memory is freed and the kernel returns.
#include <cuda.h>

#include "common.cuh"
#include "tcgen05.cuh"

namespace {

using namespace asb::t5;

constexpr int BM = 128;  // token rows per CTA
constexpr int BK = 64;   // K elements per stage: 128 bytes, one swizzle atom
constexpr int UMMA_K = 16;
constexpr int kMaxLoaders = 4;   // threads that request operands, a warp each: warps 0, 6, 7, 8
constexpr int kThreads = 192 + 32 * (kMaxLoaders - 1);

enum Epilogue : int { kStoreBf16 = 0, kStoreBf16Residual = 1, kStoreF32 = 2, kStoreSwiGLU = 4 };

struct PairParams {
  void* out;             // bf16 [M, N], f32 [M, N], or bf16 [M, N / 2] (SwiGLU)
  const void* residual;  // bf16 [M, N] or null
  int* status;
  int M, N, ldo;
  int epilogue;
  int bn;                  // weight rows per tile: a multiple of 32, at most the kernel's BN
  int tiles_m, num_tiles;  // tile t -> tokens (t % tiles_m) * 256, weight rows (t / tiles_m) * bn
  int kb_per_tile;
  // The last, partial round of tiles can be cut along K so that every pair has a share of it:
  // tiles [0, whole_tiles) are dealt whole, round-robin; each later tile is computed by `split`
  // pairs, piece j taking the stages [j * piece_stages, (j + 1) * piece_stages) of the tile's K
  // and leaving its float32 sums in workspace slot (tile - whole_tiles) * split + j, a slot being
  // [256 tokens][BN]; tail_reduce_kernel adds the slots up and stores the result. With
  // whole_tiles = num_tiles nothing is cut.
  float* workspace;
  int whole_tiles, split, piece_stages;
};

template <int BN>
struct PairConfig {
  static constexpr int kA = BM * BK * 2;           // 16 KB: this CTA's token rows of one K block
  static constexpr int kB = (BN / 2) * BK * 2;     // its half of the weight rows of one K block
  // A stage holds kSub K blocks (each operand's K blocks side by side): the thread that issues
  // the MMAs pays its wait for the operands, the fence and the commit once per stage, and with
  // four MMAs a stage those cost it as much as the MMAs themselves (about 700 cycles a K block
  // against the 512 the tensor pipe needs); with eight it keeps ahead of the pipe.
  static constexpr int kSub = 2;
  static constexpr int kStage = kSub * (kA + kB);
  static constexpr int kRoom = 227 * 1024 - 1024 - 384;
  static constexpr int kStages = kRoom / kStage > 10 ? 10 : kRoom / kStage;
  static constexpr int kSmem = kStages * kStage + 1024 + 384;
  static constexpr int kTmemCols = 2 * BN;          // two accumulators of BN columns
  // Loader j takes the stages j, j + kLoaders, ...: never more loaders than slots, or two of them
  // would wait for the same slot's same phase (and a step of more than kStages slots would leave
  // the ring: an earlier build did, and faulted).
  static constexpr int kLoaders = kStages < kMaxLoaders ? kStages : kMaxLoaders;
  static_assert(kLoaders >= 1 && kLoaders <= kStages, "a loader's step must stay inside the ring of stages");
};

__device__ __forceinline__ float swiglu(float gate, float up) { return gate / (1.f + __expf(-gate)) * up; }

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The address, in the cluster's shared window, of this CTA's shared address `addr` in CTA `rank`.
__device__ __forceinline__ uint32_t cluster_address(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t cluster_bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// A TMA tile load (no multicast) whose bytes are counted on a barrier of the CTA pair.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives, when the pair's MMAs so far have completed, on the barrier at this shared address in
// both CTAs.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(both) : "memory");
}

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                         const PairParams p) {
  using C = PairConfig<BN>;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* aligned = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + C::kStages * C::kStage;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (C::kStages + s); };
  auto acc_full = [&](int b) { return bars + 8u * (2 * C::kStages + b); };
  auto acc_empty = [&](int b) { return bars + 8u * (2 * C::kStages + 2 + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(aligned + C::kStages * C::kStage + 8 * (2 * C::kStages + 4));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0: the CTA that issues the MMAs and owns full and acc_empty
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(full_bar(s), 2);   // one arrival (with its byte count) per CTA
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full(b), 1);
      mbar_init(acc_empty(b), 8);  // one arrival per epilogue warp of either CTA
    }
    mbar_init_fence();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"((uint32_t)C::kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  fence_before_sync();
  __syncthreads();
  cluster_sync();  // both CTAs' barriers exist before either signals into the other
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // This pair's work: its whole tiles (pair, pair + pairs, ... below whole_tiles), then at most
  // one piece of a tile of the cut round.
  const int stages_per_tile = (p.kb_per_tile + C::kSub - 1) / C::kSub;  // a K block beyond K is filled with zeros
  const int n_whole = p.whole_tiles > pair ? (p.whole_tiles - pair + pairs - 1) / pairs : 0;
  const int cut_tiles = p.num_tiles - p.whole_tiles;
  const bool has_piece = pair < cut_tiles * p.split;
  const int piece_tile = p.whole_tiles + (has_piece ? pair / p.split : 0);
  const int piece_begin = has_piece ? (pair % p.split) * p.piece_stages : 0;
  const int piece_len = has_piece ? min(p.piece_stages, stages_per_tile - piece_begin) : 0;
  const int n_items = n_whole + (piece_len > 0 ? 1 : 0);
  const uint32_t total = (uint32_t)n_whole * (uint32_t)stages_per_tile + (uint32_t)piece_len;  // stages this pair runs
  auto item_tile = [&](int i) { return i < n_whole ? pair + i * pairs : piece_tile; };
  auto item_len = [&](int i) { return i < n_whole ? stages_per_tile : (i < n_items ? piece_len : 0x3fffffff); };

  if (warp == 0 || warp >= 6) {
    if (lane == 0 && (warp == 0 ? 0 : warp - 5) < C::kLoaders) {  // a spare loader warp has nothing to do
      // Loader `me` of kLoaders (warps 0, 6, 7, ...) brings every kLoaders-th stage: this CTA's 128
      // token rows and its half of the weight rows; the bytes are counted in the even CTA. One
      // thread's chain of wait, announcement and requests takes about 700 cycles per stage,
      // whatever the boxes' sizes, so several threads share the stages (the loads alone, MMAs
      // switched off: 714 cycles per K block with one loader, 353 with four). The tile and its
      // rows are carried along instead of being divided out of the stage count each time.
      const int me = warp == 0 ? 0 : warp - 5;
      // bytes a stage brings into this CTA: its token rows and its half of the tile's weight rows
      const uint32_t stage_bytes = (uint32_t)(C::kSub * (C::kA + (p.bn / 2) * BK * 2));
      int item = 0, ks = 0, s = 0;   // work item, stage within it, slot
      int len = item_len(0);
      uint32_t phase = 0;
      int x0 = 0, w0 = 0, k0 = 0;    // the item's token rows, weight rows and first stage of K
      auto place = [&]() {
        const int t = item_tile(item);
        x0 = (t % p.tiles_m) * 256 + (int)rank * BM;
        w0 = (t / p.tiles_m) * p.bn + (int)rank * (p.bn / 2);
        k0 = item < n_whole ? 0 : piece_begin;
      };
      auto advance = [&](int by) {
        ks += by;
        bool moved = false;
        while (ks >= len) { ks -= len; len = item_len(++item); moved = true; }
        if (moved) place();
        s += by;  // by <= kLoaders <= kStages: at most one turn of the ring
        if (s >= C::kStages) { s -= C::kStages; phase ^= 1u; }
      };
      place();
      advance(me);
      // the weights, which no kernel writes, fill the pipeline before the wait for the previous kernel
      const uint32_t ahead = total < (uint32_t)C::kStages ? total : (uint32_t)C::kStages;
      {
        const int item1 = item, ks1 = ks, s1 = s, len1 = len;
        const uint32_t phase1 = phase;
        for (uint32_t it = me; it < ahead; it += C::kLoaders) {
          const uint32_t bar = cluster_address(full_bar(s), 0);
          mbar_expect_tx_cluster(bar, stage_bytes);
#pragma unroll
          for (int j = 0; j < C::kSub; ++j)
            tma_load_2d_pair(base + s * C::kStage + C::kSub * C::kA + j * C::kB, &map_w, bar, ((k0 + ks) * C::kSub + j) * BK, w0);
          advance(C::kLoaders);
        }
        item = item1; ks = ks1; s = s1; len = len1; phase = phase1;
        place();
      }
      asb::pdl_wait();
      if (me == 0) asb::pdl_launch_dependents();
      for (uint32_t it = me; it < total; it += C::kLoaders) {
        const uint32_t bar = cluster_address(full_bar(s), 0);
        const uint32_t dst = base + s * C::kStage;
        if (it >= (uint32_t)C::kStages) {
          if (!mbar_wait(empty_bar(s), phase ^ 1u, p.status, 31)) break;
          mbar_expect_tx_cluster(bar, stage_bytes);
#pragma unroll
          for (int j = 0; j < C::kSub; ++j)
            tma_load_2d_pair(dst + C::kSub * C::kA + j * C::kB, &map_w, bar, ((k0 + ks) * C::kSub + j) * BK, w0);
        }
#pragma unroll
        for (int j = 0; j < C::kSub; ++j) tma_load_2d_pair(dst + j * C::kA, &map_x, bar, ((k0 + ks) * C::kSub + j) * BK, x0);
        advance(C::kLoaders);
      }
      if (me == 0) {
        // Nobody has waited for the last use of each slot to be handed back, and the commits that
        // hand them back arrive in both CTAs on their own, after the MMAs, not as part of any
        // thread's work: a CTA that left before the last of them had landed could have its shared
        // memory, by then perhaps another kernel's, written by the pair's other half. So one
        // thread of each CTA sees every slot's last use complete before the CTA goes on to leave.
        for (int slot = 0; slot < C::kStages && (uint32_t)slot < total; ++slot) {
          const uint32_t last = (uint32_t)slot + (uint32_t)C::kStages * ((total - 1u - (uint32_t)slot) / (uint32_t)C::kStages);
          if (!mbar_wait(empty_bar(slot), (last / (uint32_t)C::kStages) & 1u, p.status, 38)) break;
        }
      }
    }
  } else if (warp == 1) {
    asb::pdl_wait();
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = instr_desc_bf16(256, p.bn, false);
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (uint32_t seg = 0; ok && seg < (uint32_t)n_items; ++seg) {
        const int stages_here = item_len((int)seg);
        const uint32_t buf = seg & 1u;
        ok = mbar_wait(acc_empty(buf), ((seg >> 1) & 1u) ^ 1u, p.status, 34);
        if (!ok) break;
        fence_after_sync();
        const uint32_t tmem_acc = tmem_base + buf * BN;
        for (int ks = 0; ks < stages_here; ++ks) {
          ok = mbar_wait(full_bar(s), phase, p.status, 32);
          if (!ok) break;
          fence_after_sync();
#pragma unroll
          for (int j = 0; j < C::kSub; ++j) {
            const uint64_t da = desc_k_major(base + s * C::kStage + j * C::kA, 1024);
            const uint64_t db = desc_k_major(base + s * C::kStage + C::kSub * C::kA + j * C::kB, 1024);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              umma_pair(tmem_acc, da + (uint64_t)(k * UMMA_K * 2 >> 4), db + (uint64_t)(k * UMMA_K * 2 >> 4), idesc,
                        (uint32_t)((ks > 0) | (j != 0) | (k != 0)));
          }
          umma_commit_pair(empty_bar(s));  // both CTAs may refill the stage once these MMAs have read it
          if (++s == C::kStages) { s = 0; phase ^= 1u; }
        }
        umma_commit_pair(acc_full(buf));  // both CTAs' epilogues
      }
    }
  } else {
    // Epilogue: this warp owns lanes 32 * (warp % 4) .. + 31 of this CTA's 128 token rows.
    asb::pdl_wait();
    const int quad = warp & 3;
    bool ok = true;
    for (uint32_t seg = 0; ok && seg < (uint32_t)n_items; ++seg) {
      const int t = item_tile((int)seg);
      const uint32_t buf = seg & 1u;
      int ok_i = 1;
      if (lane == 0) ok_i = mbar_wait(acc_full(buf), (seg >> 1) & 1u, p.status, 33) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok_i, 0) != 0;
      if (!ok) break;
      fence_after_sync();
      const int row = (t % p.tiles_m) * 256 + (int)rank * BM + quad * 32 + lane;  // this thread's token
      const int n0 = (t / p.tiles_m) * p.bn;
      if ((int)seg >= n_whole) {
        // a piece of a cut tile: the sums go to this pair's workspace slot as they are
        float* slot_row = p.workspace + ((size_t)pair * 256 + (size_t)((int)rank * BM + quad * 32 + lane)) * BN;
#pragma unroll 1
        for (int c = 0; c < p.bn; c += 32) {
          if (n0 + c >= p.N) break;  // uniform
          uint32_t raw[32];
          tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + buf * BN + (uint32_t)c, raw);
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<uint4*>(slot_row + c + j) = make_uint4(raw[j], raw[j + 1], raw[j + 2], raw[j + 3]);
        }
        fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(cluster_address(acc_empty(buf), 0));
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < p.bn; c += 32) {
        if (n0 + c >= p.N) break;  // uniform
        uint32_t raw[32];
        tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + buf * BN + (uint32_t)c, raw);
        if (row >= p.M) continue;
        const int valid = min(32, p.N - (n0 + c));
        if (p.epilogue == kStoreSwiGLU) {
          // weight rows alternate gate, up: this thread holds 16 (gate, up) pairs of its token
          __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)row * (p.ldo / 2) + (n0 + c) / 2;
          uint4 packed[2];
          __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(packed);
#pragma unroll
          for (int j = 0; j < 16; ++j) ob[j] = __float2bfloat16_rn(swiglu(__uint_as_float(raw[2 * j]), __uint_as_float(raw[2 * j + 1])));
          if (valid == 32 && (((uintptr_t)o) & 15) == 0) {
            *reinterpret_cast<uint4*>(o) = packed[0];
            *reinterpret_cast<uint4*>(o + 8) = packed[1];
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (j < valid / 2) o[j] = ob[j];
          }
          continue;
        }
        const size_t at = (size_t)row * p.ldo + n0 + c;
        if (p.epilogue == kStoreF32) {
          float* o = (float*)p.out + at;
          if (valid == 32 && (((uintptr_t)o) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) *reinterpret_cast<uint4*>(o + j) = make_uint4(raw[j], raw[j + 1], raw[j + 2], raw[j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < valid) o[j] = __uint_as_float(raw[j]);
          }
          continue;
        }
        __nv_bfloat16* o = (__nv_bfloat16*)p.out + at;
        const __nv_bfloat16* res = p.epilogue == kStoreBf16Residual ? (const __nv_bfloat16*)p.residual + at : nullptr;
        if (valid == 32 && (((uintptr_t)o) & 15) == 0 && (!res || (((uintptr_t)res) & 15) == 0)) {
          uint4 rv[4];
          if (res) {
#pragma unroll
            for (int v = 0; v < 4; ++v) rv[v] = *reinterpret_cast<const uint4*>(res + 8 * v);
          }
          const __nv_bfloat16* rb = reinterpret_cast<const __nv_bfloat16*>(rv);
          uint4 ov[4];
          __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(ov);
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            float a = __uint_as_float(raw[j]), b = __uint_as_float(raw[j + 1]);
            if (res) { a += __bfloat162float(rb[j]); b += __bfloat162float(rb[j + 1]); }
            ob[j >> 1] = __floats2bfloat162_rn(a, b);
          }
#pragma unroll
          for (int v = 0; v < 4; ++v) *reinterpret_cast<uint4*>(o + 8 * v) = ov[v];
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < valid) {
              float v = __uint_as_float(raw[j]);
              if (res) v += __bfloat162float(res[j]);
              o[j] = __float2bfloat16_rn(v);
            }
        }
      }
      // this warp has read its lanes of the accumulator: hand the buffer back to the MMA thread
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(cluster_address(acc_empty(buf), 0));
    }
  }

  fence_before_sync();
  __syncthreads();
  cluster_sync();  // neither CTA leaves while the other may still signal into its barriers
  if (warp == 1) {
    fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::kTmemCols) : "memory");
  }
}

// Adds up the pieces of the tiles that the GEMM cut along K and stores them as the GEMM stores
// whole tiles. grid = (cut tiles, pieces of a tile's 256 x BN elements); a thread owns four
// consecutive weight rows of one token.
template <int BN>
__global__ void tail_reduce_kernel(const PairParams p) {
  const int cut = blockIdx.x, tile = p.whole_tiles + cut;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  const int r = i / BN, c = i % BN;
  const int row = (tile % p.tiles_m) * 256 + r, n = (tile / p.tiles_m) * p.bn + c;
  asb::pdl_wait();  // the GEMM has completed
  asb::pdl_launch_dependents();
  if (i >= 256 * BN || c >= p.bn || row >= p.M || n >= p.N) return;
  const float* ws = p.workspace + ((size_t)cut * p.split * 256 + r) * BN + c;
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int j0 = 0; j0 < p.split; j0 += 4) {  // four loads in flight; the sum still runs in piece order
    float4 a[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (j0 + u < p.split) a[u] = *reinterpret_cast<const float4*>(ws + (size_t)(j0 + u) * 256 * BN);
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (j0 + u < p.split) { v.x += a[u].x; v.y += a[u].y; v.z += a[u].z; v.w += a[u].w; }
  }
  const float e[4] = {v.x, v.y, v.z, v.w};
  if (p.epilogue == kStoreSwiGLU) {
    __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)row * (p.ldo / 2) + n / 2;
#pragma unroll
    for (int k = 0; k < 4; k += 2)
      if (n + k + 1 < p.N) o[k / 2] = __float2bfloat16_rn(swiglu(e[k], e[k + 1]));
    return;
  }
  const size_t at = (size_t)row * p.ldo + n;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    if (n + k >= p.N) break;
    float o = e[k];
    if (p.epilogue == kStoreF32) {
      ((float*)p.out)[at + k] = o;
    } else {
      if (p.epilogue == kStoreBf16Residual) o += __bfloat162float(((const __nv_bfloat16*)p.residual)[at + k]);
      ((__nv_bfloat16*)p.out)[at + k] = __float2bfloat16_rn(o);
    }
  }
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

template <int BN>
int launch_pairs(const CUtensorMap& mx, const CUtensorMap& mw, const PairParams& p, cudaStream_t stream) {
  using C = PairConfig<BN>;
  auto kern = gemm_tcgen05_pair_kernel<BN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem);
  if (e != cudaSuccess) return asb::fail("gemm_tcgen05_pair: shared memory %d: %s", C::kSmem, cudaGetErrorString(e));
  int pairs = sm_count() / 2;
  if (p.num_tiles < pairs) pairs = p.num_tiles * p.split;  // (the planner keeps tiles * split within the pairs)
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(2 * pairs);
  config.blockDim = dim3(kThreads);
  config.dynamicSmemBytes = C::kSmem;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = 2;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = asb::pdl_enabled() ? 2 : 1;
  asb::prefer_shared_carveout((const void*)kern);
  asb::count_launch();
  cudaLaunchKernelEx(&config, kern, mx, mw, p);
  if (int rc = asb::check_launch("gemm_tcgen05_pair")) return rc;
  if (p.whole_tiles < p.num_tiles) {
    asb::launch(tail_reduce_kernel<BN>, dim3(p.num_tiles - p.whole_tiles, 256 * BN / 4 / 256), 256, 0, stream, p);
    return asb::check_launch("gemm_tcgen05_pair tail_reduce");
  }
  return 0;
}

}  // namespace

// Whether, and how, the pair kernel cuts the last round of tiles along K. With fewer tiles left
// over than half the pairs, `split` pairs share each of them, a piece being at least four stages
// (eight K blocks), as long as the K blocks that the last round so saves outweigh what the pieces'
// float32 sums cost to write and read back (a launch and about 3 TB/s). out3 = {tiles dealt
// whole, pairs per cut tile, stages per piece}; returns the workspace's float32 elements.
static int g_cut_enabled = 1;
// Microseconds a pair takes per K block of 64 on a tile of 256 tokens by bn weight rows (fitted to
// sweeps over the projection shapes of Qwen3-8B, -14B and -32B): at 256 rows the tensor pipe's 512
// cycles at the clock a long GEMM runs at; at 128 the issuing thread's time for eight MMAs.
extern "C" double asb_gemm_tcgen05_pair_us_per_kb(int bn) {
  return bn <= 128 ? 0.2 : 0.2 + (0.3116 - 0.2) * (bn - 128) / 128.0;
}
static int kernel_rows(int bn) { return bn <= 128 ? 128 : 256; }  // the instantiation that runs tiles of bn weight rows
// Tuning aid: 0 keeps every tile whole in the calls that follow, 1 (the default) lets the last round be cut.
extern "C" void asb_gemm_tcgen05_pair_tune(int cut) { g_cut_enabled = cut; }

extern "C" long long asb_gemm_tcgen05_pair_cut(int M, int N, int K, int bn, int* out3) {
  const int tiles = ((M + 255) / 256) * ((N + bn - 1) / bn), pairs = sm_count() / 2;
  const int stages = ((K + BK - 1) / BK + 1) / 2;
  out3[0] = tiles; out3[1] = 1; out3[2] = stages;
  const int left = tiles % pairs;
  if (!g_cut_enabled || left == 0 || 2 * left > pairs || stages < 8) return 0;
  int split = pairs / left;
  if (split > stages / 4) split = stages / 4;
  if (split < 2) return 0;
  const int piece = (stages + split - 1) / split;
  split = (stages + piece - 1) / piece;  // no empty piece
  const double us_per_stage = 2 * asb_gemm_tcgen05_pair_us_per_kb(bn);
  const double bytes = (double)left * split * 256 * bn * 4 * 2;
  if ((stages - piece) * us_per_stage <= 3.0 + bytes / 3.0e6) return 0;
  out3[0] = tiles - left; out3[1] = split; out3[2] = piece;
  return (long long)left * split * 256 * kernel_rows(bn);  // a slot is as wide as the kernel's widest tile
}

// out = x . w^T (+ residual) on pairs of SMs, for more than 128 tokens. x [M, K] and w [N, K]
// bfloat16, contiguous, K a multiple of 8, both bases 16-byte aligned. mode 0: out bfloat16
// (+ residual); 1: out float32; 2: SwiGLU (rows of w alternate gate and up; out [M, N / 2]).
// bn: weight rows per pair tile: 128, or a multiple of 32 from 160 to 256 (one kernel, built for 256
// rows, runs those: narrower tiles let one round of them occupy more pairs of SMs).
// workspace: float32, asb_gemm_tcgen05_pair_cut(M, N, K, bn) elements (null if that is 0).
extern "C" int asb_gemm_tcgen05_pair(void* out, const void* x, const void* w, const void* residual, int M, int N,
                                     int K, int mode, int bn, float* workspace, int* status, cudaStream_t stream) {
  if (mode < 0 || mode > 2) return asb::fail("gemm_tcgen05_pair: unknown mode %d", mode);
  if (mode == 2 && (residual || N % 2)) return asb::fail("gemm_tcgen05_pair: the SwiGLU form takes no residual and an even N");
  if (mode == 1 && residual) return asb::fail("gemm_tcgen05_pair: the float32 result form takes no residual");
  if (M == 0 || N == 0) return 0;
  if (K < 8 || K % 8) return asb::fail("gemm_tcgen05_pair: K = %d must be a positive multiple of 8 (16-byte TMA rows)", K);
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return asb::fail("gemm_tcgen05_pair: operands must be 16-byte aligned");
  if (!status) return asb::fail("gemm_tcgen05_pair: a status word is required");
  if (bn != 128 && !(bn >= 160 && bn <= 256 && bn % 32 == 0))
    return asb::fail("gemm_tcgen05_pair: %d weight rows per tile (128, or a multiple of 32 from 160 to 256)", bn);
  PairParams p;
  p.out = out;
  p.residual = residual;
  p.status = status;
  p.M = M;
  p.N = N;
  p.ldo = N;
  p.epilogue = mode == 2 ? kStoreSwiGLU : (mode == 1 ? kStoreF32 : (residual ? kStoreBf16Residual : kStoreBf16));
  p.bn = bn;
  p.tiles_m = (M + 255) / 256;
  p.num_tiles = p.tiles_m * ((N + bn - 1) / bn);
  p.kb_per_tile = (K + BK - 1) / BK;
  int cut[3];
  const long long need = asb_gemm_tcgen05_pair_cut(M, N, K, bn, cut);
  if (need > 0 && !workspace) return asb::fail("gemm_tcgen05_pair: this shape needs a workspace of %lld floats", need);
  p.workspace = workspace;
  p.whole_tiles = cut[0];
  p.split = cut[1];
  p.piece_stages = cut[2];
  alignas(64) CUtensorMap mx, mw;
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint64_t dims_x[2] = {(cuuint64_t)K, (cuuint64_t)M}, dims_w[2] = {(cuuint64_t)K, (cuuint64_t)N};
  const cuuint32_t box_x[2] = {(cuuint32_t)BK, (cuuint32_t)BM}, box_w[2] = {(cuuint32_t)BK, (cuuint32_t)(bn / 2)};
  if (int rc = make_bf16_map(&mx, x, 2, dims_x, strides, box_x)) return rc;
  if (int rc = make_bf16_map(&mw, w, 2, dims_w, strides, box_w)) return rc;
  return bn == 128 ? launch_pairs<128>(mx, mw, p, stream) : launch_pairs<256>(mx, mw, p, stream);
}
