// Token embedding: out[t, :] = table[ids[t], :]  (atomserve/model.py:373; no scaling).
#include "common.cuh"

namespace {

template <typename T>
__global__ void embedding_kernel(T* __restrict__ out, const T* __restrict__ table,
                                 const int* __restrict__ ids, int width, int vocab,
                                 int* __restrict__ status) {
  asb::pdl_wait();  // the stream's previous kernel has completed (programmatic dependent launch)
  asb::pdl_launch_dependents();
  const int t = blockIdx.x;
  const int id = ids[t];
  if (id < 0 || id >= vocab) {  // refuse rather than read outside the table
    if (threadIdx.x == 0) atomicExch(status, 1);
    for (int i = threadIdx.x; i < width; i += blockDim.x) out[(size_t)t * width + i] = asb::from_float<T>(0.f);
    return;
  }
  const T* src = table + (size_t)id * width;
  T* dst = out + (size_t)t * width;
  const int vec = 16 / sizeof(T);
  if (width % vec == 0) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    for (int i = threadIdx.x; i < width / vec; i += blockDim.x) d4[i] = s4[i];
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
  }
}

}  // namespace

// status: one int on the device, set to 1 if any id was outside [0, vocab).
extern "C" int asb_embedding(void* out, const void* table, const int* ids, int num_tokens,
                             int width, int vocab, int dtype, int* status, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  const int threads = width >= 2048 ? 256 : 128;
  ASB_DISPATCH_DTYPE(dtype, T,
                     asb::launch(embedding_kernel<T>, num_tokens, threads, 0, stream, 
                         (T*)out, (const T*)table, ids, width, vocab, status));
  return asb::check_launch("embedding");
}
