// Local interleave after an all-gather of head-sharded activations: NCCL delivers rank-major
// [ranks][rows][local_bytes]; the next layer wants row-major [rows][ranks * local_bytes].
// Remote data has already landed in this GPU's own receive buffer, so the kernel only touches
// local memory.  The reference has no multi-GPU path (its thread pool pins one device,
// src/cuda/thread_pool.h:19-22); this is the one piece of data movement head sharding adds.
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
