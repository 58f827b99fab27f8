// asb_paged_attention_static_scratch: see attention_noalloc.h for what it is for, its limits
// and its rules. The partial results of the split-key attention live in the file-scope device
// array below; the kernels are the ones asb_paged_attention launches, handed that array.
#include "attention_noalloc.h"

#include <mutex>

#include "common.cuh"

extern "C" int asb_paged_attention(void* out, const void* q, const void* k_cache,
                                   const void* v_cache, const int* block_tables,
                                   const int* req_q_start, const int* req_pos_start,
                                   float* part_m, float* part_l, float* part_acc, int num_tokens,
                                   int R, int H, int KV, int hd, int bs, int table_width,
                                   int window, int PS, int NP, float scale, int dtype,
                                   cudaStream_t stream);

namespace {

// One copy per GPU that loads this library, resident until the process exits.
static __device__ __align__(256) float static_scratch[ASB_STATIC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* scratch_of_device[kMaxDevices];  // device addresses, filled on a device's first call
std::mutex setup_mutex;

// In host code `static_scratch` is only a handle for the runtime, not an address the GPU can
// use; the address comes from cudaGetSymbolAddress with the owning device current.
int scratch_address(float** ptr) {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return asb::fail("static scratch: cudaGetDevice: %s", cudaGetErrorString(e));
  if (device < 0 || device >= kMaxDevices) return asb::fail("static scratch: device %d is beyond the %d this library tracks", device, kMaxDevices);
  std::lock_guard<std::mutex> lock(setup_mutex);
  if (scratch_of_device[device] == nullptr) {
    float* address = nullptr;
    e = cudaGetSymbolAddress((void**)&address, static_scratch);
    if (e != cudaSuccess || address == nullptr)
      return asb::fail("static scratch: cudaGetSymbolAddress on device %d: %s", device, cudaGetErrorString(e));
    scratch_of_device[device] = address;
  }
  *ptr = scratch_of_device[device];
  return 0;
}

}  // namespace

extern "C" unsigned int asb_static_scratch_floats(void) { return ASB_STATIC_SCRATCH_FLOATS; }

extern "C" int asb_paged_attention_static_scratch(void* out, const void* q, const void* k_cache,
                                                  const void* v_cache, const int* block_tables,
                                                  const int* req_q_start, const int* req_pos_start,
                                                  int num_tokens, int R, int H, int KV, int hd,
                                                  int bs, int table_width, int window, int PS,
                                                  int NP, float scale, int dtype,
                                                  cudaStream_t stream) {
  if (num_tokens <= 0 || R <= 0) return 0;
  // the same ranges asb_paged_attention accepts, checked here first so that the product below
  // is formed from numbers that cannot wrap it
  if (H < 1 || H > 65535 || hd < 1 || hd > 256 || NP < 1 || NP > 65535)
    return asb::fail("static scratch attention: heads %d (1..65535), head size %d (1..256) or partitions %d (1..65535) out of range", H, hd, NP);
  if (NP == 1)
    // unpartitioned: the kernel writes `out` itself and no partial result exists, so the array
    // is neither needed nor looked up, whatever the number of tokens
    return asb_paged_attention(out, q, k_cache, v_cache, block_tables, req_q_start, req_pos_start,
                               nullptr, nullptr, nullptr, num_tokens, R, H, KV, hd, bs, table_width,
                               window, PS, NP, scale, dtype, stream);
  // part_m and part_l take rows * NP floats each, part_acc rows * NP * hd, rows = tokens * heads;
  // each factor is checked against the capacity before the next is multiplied in
  const unsigned long long capacity = ASB_STATIC_SCRATCH_FLOATS;
  unsigned long long slots = (unsigned long long)num_tokens * (unsigned long long)H;  // < 2^47
  unsigned long long need = capacity + 1;
  if (slots <= capacity) {
    slots *= (unsigned long long)NP;  // < 2^38
    if (slots <= capacity) need = slots * (unsigned long long)(hd + 2);
  }
  if (need > capacity)
    return asb::fail(
        "static scratch attention: %d tokens x %d heads x %d partitions x (%d + 2) floats exceed the "
        "built-in scratch of %u floats; use fewer partitions or tokens per call, or asb_paged_attention with "
        "caller-provided scratch",
        num_tokens, H, NP, hd, (unsigned)ASB_STATIC_SCRATCH_FLOATS);
  float* base = nullptr;
  if (int rc = scratch_address(&base)) return rc;
  float* part_m = base;
  float* part_l = base + slots;
  float* part_acc = base + 2 * slots;
  return asb_paged_attention(out, q, k_cache, v_cache, block_tables, req_q_start, req_pos_start,
                             part_m, part_l, part_acc, num_tokens, R, H, KV, hd, bs, table_width,
                             window, PS, NP, scale, dtype, stream);
}
