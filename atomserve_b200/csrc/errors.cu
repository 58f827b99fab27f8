// Error text of the last refused call on this thread, and the library's identity.
#include <atomic>
#include <mutex>

#include "common.cuh"

namespace asb {

char* error_buffer() {
  static thread_local char buffer[512];
  return buffer;
}

int fail(const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(error_buffer(), 512, fmt, args);
  va_end(args);
  return 1;
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail("%s: %s", what, cudaGetErrorString(e));
  return 0;
}

void prefer_shared_carveout(const void* kernel) {
  static std::mutex lock;
  static const void* done[128];
  static int count = 0;
  std::lock_guard<std::mutex> guard(lock);
  for (int i = 0; i < count; ++i)
    if (done[i] == kernel) return;
  if (count < 128) done[count++] = kernel;
  cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

static std::atomic<long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
long long launch_count() { return g_launches.load(std::memory_order_relaxed); }

static bool g_pdl = false;
bool pdl_enabled() { return g_pdl; }
void set_pdl(bool on) { g_pdl = on; }

}  // namespace asb

namespace asb {
void set_pdl(bool on);
long long launch_count();
}  // namespace asb

// Kernels launched by this library's entry points in this process (a launch recorded into a CUDA
// graph counts once, at capture).
extern "C" long long asb_launch_count() { return asb::launch_count(); }

// Switch programmatic dependent launch on or off for every later launch of this library.
extern "C" void asb_set_pdl(int on) { asb::set_pdl(on != 0); }

extern "C" const char* asb_last_error() { return asb::error_buffer(); }

// Architecture the kernels were compiled for; the loader checks it against the device.
extern "C" int asb_compiled_arch() { return 100; }
