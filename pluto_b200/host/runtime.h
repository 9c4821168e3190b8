// Executor and Buffer of the C++ host adapter: the device-runtime types the reference's layers
// are written against (src/cuda/executor.h:16-58, src/cuda/buffer.h:19-40).  One Executor owns a
// non-blocking compute stream; a Buffer is a shared handle to a stream-ordered allocation
// (cudaMallocAsync / cudaFreeAsync on that stream) and gives its bytes no type.
#pragma once

#include <cuda_runtime_api.h>

#include <cstddef>
#include <memory>

#include "status.h"

namespace pluto::cuda {

Status CudaStatus(cudaError_t error, const char* operation);

class Executor final {
 public:
  static StatusOr<std::unique_ptr<Executor>> Create();
  Executor(const Executor&) = delete;
  Executor& operator=(const Executor&) = delete;
  ~Executor();
  Status Synchronize() const;
  cudaStream_t stream() const { return stream_; }

 private:
  Executor() = default;
  cudaStream_t stream_ = nullptr;
};

class Buffer final {
 public:
  static StatusOr<Buffer> Allocate(Executor& executor, size_t size_bytes);
  void* data() const;
  size_t size_bytes() const;
  Executor& executor() const;

 private:
  struct Allocation;
  explicit Buffer(std::shared_ptr<Allocation> allocation) : allocation_(std::move(allocation)) {}
  std::shared_ptr<Allocation> allocation_;
};

}  // namespace pluto::cuda
