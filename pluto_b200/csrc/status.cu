// The kernel status word: one device-resident uint32 per GPU that kernels set when a bounded wait
// runs out.  Its device address is resolved once per device (the symbol's host-side name is not
// a device address) and cached; reading it back is an explicit, synchronising diagnostic call.
#include <mutex>

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

cudaError_t read_kernel_status(uint32_t* host_value, bool clear) {
  uint32_t* word = kernel_status_word();
  if (word == nullptr) return cudaErrorInvalidDevice;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return e;
  e = cudaMemcpy(host_value, word, sizeof(uint32_t), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess || !clear) return e;
  return cudaMemset(word, 0, sizeof(uint32_t));
}

}  // namespace pluto
