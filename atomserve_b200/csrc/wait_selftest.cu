// A self-test of the way every tcgen05 kernel here ends when one of its waits runs out.
//
// The GEMM and the prefill attention wait on mbarriers only through asb::t5::mbar_wait, which
// gives up after a bounded number of polls, writes a code into the device's status word and
// returns false; the block then goes on to its final barrier, frees its tensor memory and
// returns. In a healthy run that path never executes. This kernel executes it on purpose and
// safely: it takes tensor memory as those kernels do, waits with a small poll limit on a barrier
// that nothing will ever arrive at, reports through the status word, frees the tensor memory and
// ends. Nothing faults and nothing hangs; the host then reads the code, and the kernels that run
// after it show that the context and the tensor memory are intact.
#include "tcgen05.cuh"

namespace {

constexpr int kSelfTestCode = 90;
constexpr uint32_t kColumns = 64;

__global__ void __launch_bounds__(128) bounded_wait_selftest_kernel(int* status, uint32_t polls, int* freed) {
  using namespace asb::t5;
  __shared__ __align__(8) unsigned long long never_arrives;
  __shared__ uint32_t tmem_slot;
  __shared__ int gave_up;
  asb::pdl_wait();
  asb::pdl_launch_dependents();
  const uint32_t bar = smem_u32(&never_arrives);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    mbar_init_fence();
    gave_up = 0;
  }
  if (threadIdx.x < 32) {
    __syncwarp();  // the allocation is a warp-wide instruction: lane 0 has rejoined
    tmem_alloc(smem_u32(&tmem_slot), kColumns);
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  if (threadIdx.x == 0 && !mbar_wait(bar, 0, status, kSelfTestCode, polls)) gave_up = 1;  // the role that waits
  // what every role does after a wait that ran out: on to the final barrier, then free and return
  fence_before_sync();
  __syncthreads();
  if (threadIdx.x < 32) {
    fence_after_sync();
    tmem_dealloc(tmem_base, kColumns);
    if (threadIdx.x == 0) *freed = gave_up ? 1 : 2;
  }
}

}  // namespace

// status: the device's status word; freed: one int on the device, set to 1 once the block has
// given up its wait and freed its tensor memory (2 if, against all expectation, the wait ended).
extern "C" int asb_bounded_wait_selftest(int* status, int polls, int* freed, cudaStream_t stream) {
  if (!status || !freed) return asb::fail("bounded_wait_selftest: status and freed words are required");
  if (polls < 1 || polls > (1 << 20)) return asb::fail("bounded_wait_selftest: %d polls (1..2^20)", polls);
  asb::launch(bounded_wait_selftest_kernel, dim3(1), dim3(128), 0, stream, status, (uint32_t)polls, freed);
  return asb::check_launch("bounded_wait_selftest");
}
