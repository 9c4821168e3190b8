// Local interleave after an all-gather of head-sharded activations: NCCL delivers rank-major
// [ranks][rows][local_bytes]; the next layer wants row-major [rows][ranks * local_bytes].
// Remote data has already landed in this GPU's own receive buffer, so the kernel only touches
// local memory.  The reference has no multi-GPU path (its thread pool pins one device,
// src/cuda/thread_pool.h:19-22); this is the one piece of data movement head sharding adds.
#include <dlfcn.h>

#include <mutex>

#include "../../include/pluto_b200.h"
#include "engine.h"

namespace pluto {
namespace {

template <typename V>
__global__ void interleave_kernel(const V* __restrict__ gathered, V* __restrict__ out, int ranks,
                                  long long rows, int local_vecs) {
  const long long total = static_cast<long long>(ranks) * rows * local_vecs;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(i % local_vecs);
    const long long row = (i / local_vecs) % rows;
    const int rank = static_cast<int>(i / (static_cast<long long>(local_vecs) * rows));
    out[(row * ranks + rank) * local_vecs + v] = gathered[i];
  }
}

}  // namespace

cudaError_t interleave_heads(cudaStream_t stream, const void* gathered, void* out, int ranks,
                             long long rows, size_t local_bytes) {
  const bool vec = local_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(gathered) & 15u) == 0 &&
                   (reinterpret_cast<uintptr_t>(out) & 15u) == 0;
  const long long units = static_cast<long long>(ranks) * rows * (vec ? local_bytes / 16 : local_bytes);
  const int blocks = static_cast<int>(units / 256 + 1 > 148 * 16 ? 148 * 16 : units / 256 + 1);
  if (vec)
    interleave_kernel<uint4><<<blocks, 256, 0, stream>>>(static_cast<const uint4*>(gathered),
                                                         static_cast<uint4*>(out), ranks, rows,
                                                         static_cast<int>(local_bytes / 16));
  else
    interleave_kernel<uint8_t><<<blocks, 256, 0, stream>>>(static_cast<const uint8_t*>(gathered),
                                                           static_cast<uint8_t*>(out), ranks, rows,
                                                           static_cast<int>(local_bytes));
  return cudaGetLastError();
}

}  // namespace pluto

// ---------------------------------------------------------------------------------------------
// All-gather + interleave behind one C entry point.  NCCL is bound at run time to the library
// the caller's communicator came from (symbols already in the process), so this shared object
// carries no NCCL dependency of its own and cannot end up talking to a second copy of NCCL.
// ---------------------------------------------------------------------------------------------
namespace {

using AllGatherFn = int (*)(const void*, void*, size_t, int /*ncclDataType_t*/, void* /*comm*/,
                            cudaStream_t);
using ErrorStringFn = const char* (*)(int);
AllGatherFn g_all_gather = nullptr;
ErrorStringFn g_error_string = nullptr;
std::once_flag g_nccl_once;

void bind_nccl() {
  void* sym = dlsym(RTLD_DEFAULT, "ncclAllGather");
  void* handle = nullptr;
  if (sym == nullptr) {
    handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (handle != nullptr) sym = dlsym(handle, "ncclAllGather");
  }
  g_all_gather = reinterpret_cast<AllGatherFn>(sym);
  void* text = dlsym(handle ? handle : RTLD_DEFAULT, "ncclGetErrorString");
  g_error_string = reinterpret_cast<ErrorStringFn>(text);
}

}  // namespace

extern "C" int pluto_allgather_heads(pluto_stream_t stream, void* nccl_comm, const void* local,
                                     void* gathered, void* out, int ranks, long long rows,
                                     size_t local_bytes) {
  if (ranks <= 0 || rows <= 0 || local_bytes == 0 || local_bytes > 0x7fffffffu)
    return pluto::report(PLUTO_E_INVALID, "invalid head-gather dimensions");
  if (!nccl_comm || !local || !gathered || !out)
    return pluto::report(PLUTO_E_INVALID, "head gather requires a communicator and non-null device pointers");
  std::call_once(g_nccl_once, bind_nccl);
  if (g_all_gather == nullptr)
    return pluto::report(PLUTO_E_UNIMPLEMENTED, "no NCCL library is loaded in this process (ncclAllGather not found)");
  const int rc = g_all_gather(local, gathered, static_cast<size_t>(rows) * local_bytes, /*ncclInt8*/ 0,
                              nccl_comm, static_cast<cudaStream_t>(stream));
  if (rc != 0) {
    pluto::report(PLUTO_E_INTERNAL, g_error_string ? g_error_string(rc) : "ncclAllGather failed");
    return 10000 + rc;
  }
  return pluto::report_cuda(pluto::interleave_heads(static_cast<cudaStream_t>(stream), gathered, out, ranks,
                                                    rows, local_bytes),
                            "head interleave launch");
}
