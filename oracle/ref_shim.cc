// TEST INFRASTRUCTURE -- not part of the shipped engine.
//
// C entry points over the reference project's own scalar CPU attention layer
// (AttentionLayerReference, src/llm/layers/attention_reference.cc:20-230 with the buffer type of
// src/host/buffer.cc).  The reference sources are compiled where they lie by oracle/Makefile; this
// file only adapts them to plain pointers so tests and the CPU-baseline timer can call them
// through ctypes.  Sequences are independent in the layer (attention resets at every
// context_length boundary), so `threads` > 1 splits whole sequences across std::threads, each with
// its own layer instance; every output byte is the same as a single-threaded run.
#include <algorithm>
#include <cstring>
#include <thread>
#include <vector>

#include "src/llm/layers/attention.h"

namespace {
using pluto::llm::AttentionLayerReference;
using pluto::llm::DataType;
using pluto::llm::HostBuffer;
using pluto::llm::HostBufferVec;

// Runs forward (and backward when d_out != nullptr) on rows [row_begin, row_end).
int RunRange(const unsigned char* qkv, const float* d_out, int row_begin, int row_end, int context,
             int heads, int embed, bool bf16, unsigned char* out, float* d_qkv) {
  const DataType type = bf16 ? DataType::BF16 : DataType::FP16;  // FP16 policy stores fp32
  const size_t element = bf16 ? 2 : 4;
  auto layer = AttentionLayerReference::Create(context, heads, embed, type);
  if (!layer.ok()) return static_cast<int>(layer.status().code());
  const size_t rows = static_cast<size_t>(row_end - row_begin);
  auto input = HostBuffer::Allocate(rows * 3 * embed * element);
  if (!input.ok()) return 100;
  std::memcpy(input->data(), qkv + static_cast<size_t>(row_begin) * 3 * embed * element,
              input->size_bytes());
  HostBufferVec inputs = {*input};
  auto forward = (*layer)->fwd(inputs);
  if (!forward.ok()) return static_cast<int>(forward.status().code());
  if (out != nullptr)
    std::memcpy(out + static_cast<size_t>(row_begin) * embed * element,
                forward->outputs[0].data(), forward->outputs[0].size_bytes());
  if (d_out == nullptr) return 0;
  auto gradient = HostBuffer::Allocate(rows * embed * sizeof(float));
  if (!gradient.ok()) return 100;
  std::memcpy(gradient->data(), d_out + static_cast<size_t>(row_begin) * embed,
              gradient->size_bytes());
  HostBufferVec gradients = {*gradient};
  auto backward = (*layer)->bwd(gradients, std::move(forward->state));
  if (!backward.ok()) return static_cast<int>(backward.status().code());
  std::memcpy(d_qkv + static_cast<size_t>(row_begin) * 3 * embed, backward->front().data(),
              backward->front().size_bytes());
  return 0;
}
}  // namespace

extern "C" {

// qkv: packed [rows, 3*embed] (fp32, or bf16 bit patterns when is_bf16); out: [rows, embed] same
// storage type (may be null); d_out: fp32 [rows, embed] or null to skip backward; d_qkv: fp32
// [rows, 3*embed].  Returns 0 or the absl::StatusCode of the reference's error.
int pluto_ref_attention(const void* qkv, const float* d_out, int rows, int context, int heads,
                        int embed, int is_bf16, int threads, void* out, float* d_qkv) {
  if (context <= 0 || rows <= 0 || rows % context != 0 || threads <= 1)
    return RunRange(static_cast<const unsigned char*>(qkv), d_out, 0, rows, context, heads, embed,
                    is_bf16 != 0, static_cast<unsigned char*>(out), d_qkv);
  const int sequences = rows / context;
  threads = std::min(threads, sequences);
  std::vector<int> codes(threads, 0);
  std::vector<std::thread> workers;
  for (int t = 0; t < threads; ++t) {
    const int begin = static_cast<int>(static_cast<long long>(sequences) * t / threads);
    const int end = static_cast<int>(static_cast<long long>(sequences) * (t + 1) / threads);
    workers.emplace_back([=, &codes] {
      codes[t] = RunRange(static_cast<const unsigned char*>(qkv), d_out, begin * context,
                          end * context, context, heads, embed, is_bf16 != 0,
                          static_cast<unsigned char*>(out), d_qkv);
    });
  }
  for (auto& worker : workers) worker.join();
  for (int code : codes)
    if (code != 0) return code;
  return 0;
}

}  // extern "C"
