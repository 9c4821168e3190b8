// C++ host adapter, second part: the three layer classes of the Qwen decoder and the block
// parameter they share, with the reference's names, Create signatures, validation order, error
// codes and saved-state order, implemented over the C ABI of include/pluto_b200.h:
//   BlockParameter          src/llm/block_parameter.h:15-47 (FP32 storage; see Activate)
//   QwenAttentionLayer      src/llm/layers/qwen_attention.h:29-99, .cc:291-499
//   DeltaNetLayer           src/llm/layers/delta_net.h:20-60, .cc:38-110
//   SequenceDeltaNetLayer   src/llm/layers/sequence_delta_net.h:20-67, .cc:396-561
// What differs from the reference, on purpose:
//   * activations stay bf16 end to end (no ToFloat / ToBFloat16 round trips, util.cc:14-72);
//   * the sequence layers keep no [Hq, T, T] probabilities and no per-token states, so their
//     T <= 128 limit is gone; the saved state keeps the reference's slots in the reference's order
//     (unused ones are empty buffers) and appends what replaces them.
#pragma once

#include <memory>
#include <optional>

#include "layers.h"

namespace pluto::llm {

using FullAttentionParameters = cached_attention_ops::FullAttentionParameters;
using DeltaNetParameters = cached_attention_ops::DeltaNetParameters;

// A resident parameter the block optimizer may activate: active parameters own an FP32 master
// copy and an FP32 gradient that layers ACCUMULATE into.  Only FP32 storage is built here (the
// norm, convolution and gate parameters of these layers are FP32); BF16 storage is accepted by
// Create, as in the reference, but cannot be activated.
class BlockParameter final {
 public:
  static StatusOr<std::shared_ptr<BlockParameter>> Create(cuda::Executor& executor, Buffer value,
                                                         DataType storage);
  Status Activate();
  Status Publish();
  Status Deactivate();
  bool active() const { return master_.has_value(); }
  const Buffer& value() const { return value_; }
  const Buffer& master() const { return *master_; }
  const Buffer& gradient() const { return *gradient_; }
  size_t elements() const { return elements_; }
  DataType storage() const { return storage_; }

 private:
  BlockParameter(Buffer value, DataType storage, size_t elements)
      : value_(std::move(value)), storage_(storage), elements_(elements) {}
  Buffer value_;
  DataType storage_;
  size_t elements_;
  std::optional<Buffer> master_, gradient_;
};

class QwenAttentionLayer final : public Layer {
 public:
  static constexpr int kMaximumDimension = 1048576;
  static StatusOr<std::unique_ptr<QwenAttentionLayer>> Create(
      cuda::Executor& executor, FullAttentionParameters parameters,
      std::shared_ptr<BlockParameter> q_norm, std::shared_ptr<BlockParameter> k_norm,
      int sequence_length, KeyValueCache* cache = nullptr);
  static StatusOr<std::unique_ptr<QwenAttentionLayer>> Create(
      cuda::Executor& executor, FullAttentionParameters parameters, Buffer q_norm, Buffer k_norm,
      int sequence_length, KeyValueCache* cache = nullptr);
  const char* name() const override { return "QwenAttentionLayer"; }
  DataType output_type() const override { return DataType::BF16; }
  std::vector<ActivationType> input_types() const override;
  std::vector<ActivationType> output_types() const override;
  const Buffer* weights() const { return weights_; }   // query norm, key norm

  // Saved state of the sequence forward: the reference's seven buffers {Q/gate input, K input,
  // V input, prepared q, prepared k, probabilities (empty unless a hook asked), unrounded core}
  // followed by {row maxima, row normalizers, rounded v}.
  static constexpr size_t kSavedBuffers = 10;

 private:
  QwenAttentionLayer(cuda::Executor& executor, FullAttentionParameters parameters,
                     std::shared_ptr<BlockParameter> q_norm, std::shared_ptr<BlockParameter> k_norm,
                     int sequence_length, KeyValueCache* cache);
  StatusOr<FwdResult> fwd_impl(cuda::Executor& executor, const BufferVec& inputs,
                               LayerHooks* hooks) const override;
  StatusOr<BufferVec> bwd_impl(cuda::Executor& executor, const BufferVec& gradients,
                               BackwardState state, LayerHooks* hooks) override;
  StatusOr<FwdResult> CachedForward(cuda::Executor& executor, const BufferVec& inputs,
                                    LayerHooks* hooks) const;
  StatusOr<FwdResult> SequenceForward(cuda::Executor& executor, const BufferVec& inputs,
                                      LayerHooks* hooks) const;
  StatusOr<BufferVec> SequenceBackward(cuda::Executor& executor, const BufferVec& gradients,
                                       BackwardState state);
  cuda::Executor& executor_;
  FullAttentionParameters parameters_;
  std::shared_ptr<BlockParameter> q_norm_, k_norm_;
  int sequence_length_;
  Buffer weights_[2];
  KeyValueCache* cache_;   // borrowed; null = stateless sequence layer
};

class DeltaNetLayer final : public Layer {
 public:
  static constexpr int kMaximumDimension = 1048576;
  static StatusOr<std::unique_ptr<DeltaNetLayer>> Create(cuda::Executor& executor,
                                                        DeltaNetParameters parameters,
                                                        Buffer convolution, Buffer a_log,
                                                        Buffer dt_bias, Buffer norm);
  const char* name() const override { return "DeltaNetLayer"; }
  DataType output_type() const override { return DataType::BF16; }
  std::vector<ActivationType> input_types() const override;
  std::vector<ActivationType> output_types() const override;
  const Buffer* weights() const { return weights_; }
  Status Reset();

 private:
  DeltaNetLayer(cuda::Executor& executor, DeltaNetParameters parameters, Buffer convolution,
                Buffer a_log, Buffer dt_bias, Buffer norm,
                std::unique_ptr<cached_attention_ops::DeltaNetState> cache);
  StatusOr<FwdResult> fwd_impl(cuda::Executor& executor, const BufferVec& inputs,
                               LayerHooks* hooks) const override;
  StatusOr<BufferVec> bwd_impl(cuda::Executor& executor, const BufferVec& gradients,
                               BackwardState state, LayerHooks* hooks) override;
  cuda::Executor& executor_;
  DeltaNetParameters parameters_;
  Buffer weights_[4];
  std::unique_ptr<cached_attention_ops::DeltaNetState> cache_;
};

class SequenceDeltaNetLayer final : public Layer {
 public:
  static StatusOr<std::unique_ptr<SequenceDeltaNetLayer>> Create(
      cuda::Executor& executor, DeltaNetParameters parameters,
      std::shared_ptr<BlockParameter> convolution, std::shared_ptr<BlockParameter> a_log,
      std::shared_ptr<BlockParameter> dt_bias, std::shared_ptr<BlockParameter> norm,
      int sequence_length);
  const char* name() const override { return "SequenceDeltaNetLayer"; }
  DataType output_type() const override { return DataType::BF16; }
  std::vector<ActivationType> input_types() const override;
  std::vector<ActivationType> output_types() const override;
  const Buffer* weights() const { return weights_; }

  // Saved state: the reference's eight slots {QKV, Z, A, B inputs, convolution pre-activation
  // (empty: recomputed in backward), convolved + SiLU'd activations, rounded recurrence output,
  // recurrent states (the final state only)}.
  static constexpr size_t kSavedBuffers = 8;

 private:
  SequenceDeltaNetLayer(cuda::Executor& executor, DeltaNetParameters parameters,
                        std::shared_ptr<BlockParameter> convolution,
                        std::shared_ptr<BlockParameter> a_log,
                        std::shared_ptr<BlockParameter> dt_bias,
                        std::shared_ptr<BlockParameter> norm, int sequence_length);
  StatusOr<FwdResult> fwd_impl(cuda::Executor& executor, const BufferVec& inputs,
                               LayerHooks* hooks) const override;
  StatusOr<BufferVec> bwd_impl(cuda::Executor& executor, const BufferVec& gradients,
                               BackwardState state, LayerHooks* hooks) override;
  cuda::Executor& executor_;
  DeltaNetParameters parameters_;
  int sequence_length_;
  std::shared_ptr<BlockParameter> parameters_owned_[4];
  Buffer weights_[4];
};

}  // namespace pluto::llm
