// C++ host adapter: the reference's layer interface for the attention hot path, implemented over
// the C ABI of include/pluto_b200.h.  Class and function names, argument meaning, saved-state
// layout and error behaviour follow the reference so that its call sites keep compiling:
//   Layer, FwdResult, BackwardState, LayerHooks     src/llm/layer.h:96-185, layer_hooks.h:104-108
//   AttentionLayer                                  src/llm/layers/attention.h:25-77
//   KeyValueCache                                   src/llm/key_value_cache.h:25-57
//   FullAttentionParameters, ValidateCachedAttention, CachedAttentionStep,
//   DeltaNetParameters, DeltaNetState               src/llm/layers/util/cached_attention_ops.h:13-89
// Allocation happens here (stream-ordered Buffers), never inside the C ABI.
#pragma once

#include <cstdint>
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "runtime.h"
#include "status.h"

namespace pluto::llm {

using Buffer = cuda::Buffer;
using BufferVec = std::vector<Buffer>;

enum class DataType { FP16, BF16, FP8, FP32, INT32 };
inline DataType ActivationDataType(DataType compute) {
  return compute == DataType::FP16 ? DataType::FP32 : compute;
}

struct ActivationType {
  static constexpr int64_t kBatchDimension = -2;
  DataType data_type;
  std::vector<int64_t> dimensions;
  bool operator==(const ActivationType& o) const {
    return data_type == o.data_type && dimensions == o.dimensions;
  }
};

class Layer;
struct BackwardState {
  const Layer* layer = nullptr;
  BufferVec intermediates;
  std::vector<BackwardState> children;
};
struct FwdResult {
  BufferVec outputs;
  BackwardState state;
};
struct LayerHooks {
  std::function<Status(cuda::Executor&, const std::string&, const ActivationType&, const Buffer&)>
      attention_probabilities_hook;
};

class Layer {
 public:
  virtual ~Layer() = default;
  virtual const char* name() const = 0;
  virtual std::vector<ActivationType> input_types() const = 0;
  virtual std::vector<ActivationType> output_types() const = 0;
  virtual DataType output_type() const = 0;
  StatusOr<FwdResult> fwd(cuda::Executor& executor, const BufferVec& inputs,
                          LayerHooks* hooks = nullptr) const;
  StatusOr<BufferVec> bwd(cuda::Executor& executor, const BufferVec& output_gradients,
                          BackwardState state, LayerHooks* hooks = nullptr);

 private:
  virtual StatusOr<FwdResult> fwd_impl(cuda::Executor& executor, const BufferVec& inputs,
                                       LayerHooks* hooks) const = 0;
  virtual StatusOr<BufferVec> bwd_impl(cuda::Executor& executor, const BufferVec& output_gradients,
                                       BackwardState state, LayerHooks* hooks) = 0;
};

class AttentionLayer final : public Layer {
 public:
  static StatusOr<std::unique_ptr<AttentionLayer>> Create(cuda::Executor& executor,
                                                         int context_length, int num_heads,
                                                         int embedding_dim, DataType data_type);
  const char* name() const override { return "AttentionLayer"; }
  DataType output_type() const override { return output_type_; }
  std::vector<ActivationType> input_types() const override;
  std::vector<ActivationType> output_types() const override;

 private:
  AttentionLayer(cuda::Executor& executor, int context_length, int num_heads, int embedding_dim,
                 DataType data_type)
      : executor_(executor), context_length_(context_length), num_heads_(num_heads),
        embedding_dim_(embedding_dim), output_type_(data_type) {}
  StatusOr<FwdResult> fwd_impl(cuda::Executor& executor, const BufferVec& inputs,
                               LayerHooks* hooks) const override;
  StatusOr<BufferVec> bwd_impl(cuda::Executor& executor, const BufferVec& output_gradients,
                               BackwardState state, LayerHooks* hooks) override;
  cuda::Executor& executor_;
  int context_length_, num_heads_, embedding_dim_;
  DataType output_type_;
};

// Per-sequence K/V storage [capacity, kv_heads, head_dim] plus the position counter.  `bfloat16`
// selects 2-byte storage (the same values the reference keeps in fp32 when rounding is on).
class KeyValueCache final {
 public:
  static StatusOr<std::unique_ptr<KeyValueCache>> Create(cuda::Executor& executor, int capacity,
                                                         int key_value_heads, int head_dim,
                                                         bool bfloat16 = false);
  int capacity() const { return capacity_; }
  int key_value_heads() const { return key_value_heads_; }
  int head_dim() const { return head_dim_; }
  int position() const { return position_; }
  bool bfloat16() const { return bfloat16_; }
  const Buffer& keys() const { return keys_; }
  const Buffer& values() const { return values_; }
  cuda::Executor& executor() const { return keys_.executor(); }
  Status Advance();
  void Reset() { position_ = 0; }

 private:
  KeyValueCache(int capacity, int heads, int dim, bool bf16, Buffer keys, Buffer values)
      : capacity_(capacity), key_value_heads_(heads), head_dim_(dim), bfloat16_(bf16),
        keys_(std::move(keys)), values_(std::move(values)) {}
  int capacity_, key_value_heads_, head_dim_;
  bool bfloat16_;
  int position_ = 0;
  Buffer keys_, values_;
};

namespace cached_attention_ops {

struct FullAttentionParameters {
  int query_heads = 24;
  int key_value_heads = 4;
  int head_dim = 256;
  int rotary_dim = 64;
  int capacity = 4096;
  float rms_norm_epsilon = 1e-6f;
  float rope_theta = 10000000.0f;
  bool round_to_bfloat16 = true;
};

Status ValidateCachedAttention(cuda::Executor& executor, const FullAttentionParameters& parameters,
                               const KeyValueCache& cache);

// One token of batch-one causal attention; device fp32 pointers as in the reference.  Validates
// everything before queuing work and advances the cache only after every launch succeeded.
Status CachedAttentionStep(cuda::Executor& executor, const FullAttentionParameters& parameters,
                           KeyValueCache& cache, const float* q_gate, const float* k,
                           const float* v, const float* q_norm, const float* k_norm, float* output,
                           float* probabilities = nullptr);

// The same step for activations that are not fp32: q_gate, k, v are read as `input_dtype`
// (PLUTO_FP32 / PLUTO_BF16 of include/pluto_b200.h) and the output is written as `output_dtype`,
// so a layer whose activations are bf16 needs no cast launches either side (the reference's
// QwenAttentionLayer::CachedForward converts with ToFloat / ToBFloat16,
// src/llm/layers/qwen_attention.cc:370-412).  Norm weights and probabilities stay fp32.
Status CachedAttentionStepTyped(cuda::Executor& executor, const FullAttentionParameters& parameters,
                                KeyValueCache& cache, const void* q_gate, const void* k,
                                const void* v, int input_dtype, const float* q_norm,
                                const float* k_norm, void* output, int output_dtype,
                                float* probabilities = nullptr);

struct DeltaNetParameters {
  int key_heads = 16;
  int value_heads = 48;
  int key_head_dim = 128;
  int value_head_dim = 128;
  int conv_kernel_dim = 4;
  float rms_norm_epsilon = 1e-6f;
  bool round_to_bfloat16 = true;
};

class DeltaNetState final {
 public:
  static StatusOr<std::unique_ptr<DeltaNetState>> Create(cuda::Executor& executor,
                                                        DeltaNetParameters parameters);
  Status Step(const float* qkv, const float* z, const float* a, const float* b,
              const float* conv_weight, const float* a_log, const float* dt_bias,
              const float* norm_weight, float* output);
  // Step for activations stored as `input_dtype` with the output written as `output_dtype`
  // (see CachedAttentionStepTyped); weights stay fp32.
  Status StepTyped(const void* qkv, const void* z, const void* a, const void* b, int input_dtype,
                   const float* conv_weight, const float* a_log, const float* dt_bias,
                   const float* norm_weight, void* output, int output_dtype);
  Status Reset();

 private:
  DeltaNetState(cuda::Executor& executor, DeltaNetParameters p, Buffer conv, Buffer recurrent,
                Buffer convolved, Buffer core, Buffer gates)
      : executor_(executor), parameters_(p), convolution_state_(std::move(conv)),
        recurrent_state_(std::move(recurrent)), convolved_qkv_(std::move(convolved)),
        core_output_(std::move(core)), gates_(std::move(gates)) {}
  cuda::Executor& executor_;
  DeltaNetParameters parameters_;
  Buffer convolution_state_, recurrent_state_, convolved_qkv_, core_output_, gates_;
};

}  // namespace cached_attention_ops
}  // namespace pluto::llm
