// The library's device status word and its host-visible mirror.
//
// Every wait inside the tensor-core and decode kernels is bounded (ptx::mbar_wait).  A wait that
// gives up stores its code in ONE word of device memory shared by all kernels of the library; the
// word is sticky: every later CTA reads it when it starts and bails out at its first wait, so a
// protocol failure cannot be followed by silently wrong results.  So that the host learns of it
// without synchronising, the give-up path also stores the code in a word of mapped, pinned host
// memory; the C ABI entry points read that word before they launch anything and return an error
// until fa_device_status() has read and cleared the state.
#include <atomic>

#include "../fa_common.cuh"
#include "ptx.cuh"

namespace fa {

using namespace ptx;

namespace {

__device__ int g_status_word = 0;  // 0 = ok; otherwise code of the first wait that gave up

constexpr int kMaxDevices = 64;
int* g_dev_ptr[kMaxDevices] = {nullptr};            // device address of g_status_word, per device
std::atomic<int*> g_host_mirror{nullptr};           // kMaxDevices ints of mapped pinned host memory
int* g_host_dev_view[kMaxDevices] = {nullptr};      // the mirror slot of a device, as that device addresses it

int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    return -1;
  }
  return dev;
}

// A kernel that does nothing but wait, with a short limit, for a barrier phase that no one
// completes: exercises the give-up path (status word, mirror, wind-down) without any fault.
__global__ void wait_timeout_selftest_kernel(StatusRef status, long long limit_cycles, int code) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ __align__(8) int abort_block[kAbortBlockBytes / 4];
  volatile int* abort_flag = abort_block + 1;
  const uint32_t bar_addr = smem_addr(&bar);
  if (threadIdx.x == 0) {
    abort_init(abort_flag, status);
    mbar_init(bar_addr, 1);
    fence_barrier_init();
  }
  __syncthreads();
  mbar_wait(bar_addr, 0, code, abort_flag, 0, limit_cycles);  // nobody arrives
  __syncthreads();
}

}  // namespace

// Status pointers of the current device for a kernel launch.  `may_allocate` = false never
// allocates: the host mirror is then used only if an earlier call created it.
StatusRef status_ref(bool may_allocate) {
  StatusRef r{nullptr, nullptr};
  const int dev = current_device();
  if (dev < 0) return r;
  if (!g_dev_ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) {
      cudaGetLastError();
      return r;
    }
    g_dev_ptr[dev] = static_cast<int*>(p);
  }
  r.dev = g_dev_ptr[dev];
  int* mirror = g_host_mirror.load(std::memory_order_acquire);
  if (!mirror && may_allocate) {
    void* p = nullptr;
    if (cudaHostAlloc(&p, kMaxDevices * sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess) {
      for (int i = 0; i < kMaxDevices; ++i) static_cast<int*>(p)[i] = 0;
      int* expected = nullptr;
      if (g_host_mirror.compare_exchange_strong(expected, static_cast<int*>(p), std::memory_order_acq_rel)) {
        mirror = static_cast<int*>(p);
      } else {
        cudaFreeHost(p);
        mirror = expected;
      }
    } else {
      cudaGetLastError();
    }
  }
  if (mirror) {
    if (!g_host_dev_view[dev]) {
      void* dp = nullptr;
      if (cudaHostGetDevicePointer(&dp, mirror + dev, 0) == cudaSuccess)
        g_host_dev_view[dev] = static_cast<int*>(dp);
      else
        cudaGetLastError();
    }
    r.host = g_host_dev_view[dev];
  }
  return r;
}

// The mirror word of the current device, read without any synchronisation (0 when there is no mirror).
int status_peek() {
  const int dev = current_device();
  int* mirror = g_host_mirror.load(std::memory_order_acquire);
  if (dev < 0 || !mirror) return 0;
  return *reinterpret_cast<volatile int*>(mirror + dev);
}

// Synchronises the device, returns the status word and (optionally) clears word and mirror.
int status_read(bool clear) {
  const int dev = current_device();
  int v = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(&v, g_status_word, sizeof(int)) != cudaSuccess) return -1;
  if (clear && v) {
    const int z = 0;
    cudaMemcpyToSymbol(g_status_word, &z, sizeof(int));
    int* mirror = g_host_mirror.load(std::memory_order_acquire);
    if (mirror && dev >= 0) *reinterpret_cast<volatile int*>(mirror + dev) = 0;
  }
  return v;
}

int selftest_wait_timeout(long long limit_cycles, int code, cudaStream_t st) {
  StatusRef s = status_ref(true);
  if (!s.dev) {
    fa_host::set_error("status word of the current device is not available");
    return 2;
  }
  wait_timeout_selftest_kernel<<<1, 32, 0, st>>>(s, limit_cycles, code);
  return fa_host::check_launch("wait_timeout_selftest_kernel");
}

}  // namespace fa
