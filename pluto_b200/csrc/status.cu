// The kernel status word: one device-resident uint32 per GPU that kernels set when a bounded wait
// runs out.  Its device address is resolved once per device (the symbol's host-side name is not
// a device address) and cached; reading it back is an explicit, synchronising diagnostic call.
#include <mutex>

#include "../../include/pluto_b200.h"
#include "common.cuh"
#include "engine.h"

namespace pluto {
namespace {
__device__ uint32_t g_kernel_status = 0;
constexpr int kMaxDevices = 64;
std::once_flag g_once[kMaxDevices];
uint32_t* g_address[kMaxDevices] = {};
}  // namespace

uint32_t* kernel_status_word() {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return nullptr;
  std::call_once(g_once[device], [device] {
    void* address = nullptr;
    if (cudaGetSymbolAddress(&address, g_kernel_status) == cudaSuccess)
      g_address[device] = static_cast<uint32_t*>(address);
  });
  return g_address[device];
}

bool stream_on_current_device(cudaStream_t stream) {
  int current = -1, owner = -1;
  if (cudaGetDevice(&current) != cudaSuccess) return false;
  if (cudaStreamGetDevice(stream, &owner) != cudaSuccess) {
    cudaGetLastError();   // an invalid handle is the caller's error, not a sticky one
    return false;
  }
  return owner == current;
}

cudaError_t read_kernel_status(uint32_t* host_value, bool clear) {
  uint32_t* word = kernel_status_word();
  if (word == nullptr) return cudaErrorInvalidDevice;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return e;
  e = cudaMemcpy(host_value, word, sizeof(uint32_t), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess || !clear) return e;
  return cudaMemset(word, 0, sizeof(uint32_t));
}

namespace {
// One CTA, one thread, one mbarrier that nobody ever arrives at: the bounded wait must give up
// after `limit_ns`, record (site << 8) | kWaitTimeout and let the kernel return normally.
__global__ void bounded_wait_selftest_kernel(uint32_t* status, uint32_t site, uint64_t limit_ns,
                                             uint32_t* gave_up) {
  __shared__ uint64_t bar;
  mbar_init(&bar, 1);
  mbar_fence_init();
  const bool arrived = mbar_wait(&bar, 0, status, site, limit_ns);
  *gave_up = arrived ? 0u : 1u;
}
}  // namespace

}  // namespace pluto

extern "C" int pluto_selftest_bounded_wait(pluto_stream_t stream, unsigned long long limit_ns,
                                           uint32_t* gave_up) {
  if (gave_up == nullptr) return pluto::report(PLUTO_E_INVALID, "self-test requires a device flag");
  if (limit_ns == 0 || limit_ns > 100000000ull)
    return pluto::report(PLUTO_E_INVALID, "self-test wait limit must be in (0, 100 ms]");
  uint32_t* status = pluto::kernel_status_word();
  if (!status) return pluto::report(PLUTO_E_INTERNAL, "kernel status word unavailable");
  pluto::bounded_wait_selftest_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(
      status, PLUTO_SELFTEST_WAIT_SITE, limit_ns, gave_up);
  return pluto::report_cuda(cudaGetLastError(), "bounded-wait self-test launch");
}
