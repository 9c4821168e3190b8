// Implementation of the Qwen decoder layer classes (qwen_layers.h) over the C ABI.
#include "qwen_layers.h"

#include <cmath>
#include <cstdint>
#include <limits>
#include <string>

#include "../../include/pluto_b200.h"

namespace pluto::llm {
namespace {

// internal::ValidateBFloat16Inputs (src/llm/layers/util.cc:60-72): count, executor, byte sizes.
Status ValidateBFloat16Inputs(cuda::Executor& executor, const BufferVec& inputs, const int64_t* counts,
                              size_t expected_inputs, const char* layer) {
  if (inputs.size() != expected_inputs)
    return InvalidArgumentError(std::string(layer) + " expects " + std::to_string(expected_inputs) + " inputs");
  for (size_t i = 0; i < inputs.size(); ++i) {
    if (&inputs[i].executor() != &executor)
      return InvalidArgumentError(std::string(layer) + " input belongs to a different Executor");
    if (inputs[i].size_bytes() != static_cast<size_t>(counts[i]) * 2)
      return InvalidArgumentError(std::string(layer) + " input has " + std::to_string(inputs[i].size_bytes()) +
                                  " bytes; expected " + std::to_string(counts[i] * 2));
  }
  return OkStatus();
}

StatusOr<Buffer> AllocateAligned(cuda::Executor& executor, size_t bytes) {
  // stream-ordered allocations are 256-byte aligned or better, which every workspace here needs
  return Buffer::Allocate(executor, bytes);
}

float* F(const Buffer& b) { return static_cast<float*>(b.data()); }
char* Bytes(const Buffer& b) { return static_cast<char*>(b.data()); }

pluto_kv_cache SequenceView(const Buffer& k, const Buffer& v, int tokens, int kv_heads, int head_dim) {
  pluto_kv_cache view{};
  view.k_base = k.data();
  view.v_base = v.data();
  view.page_size = tokens;
  view.token_stride = static_cast<size_t>(kv_heads) * head_dim;
  view.page_stride = view.token_stride * tokens;
  view.dtype = PLUTO_BF16;
  view.num_pages = 1;
  return view;
}

}  // namespace

// ---- BlockParameter (src/llm/block_parameter.cc:25-95) ------------------------------------------
StatusOr<std::shared_ptr<BlockParameter>> BlockParameter::Create(cuda::Executor& executor, Buffer value,
                                                                DataType storage) {
  if (storage != DataType::BF16 && storage != DataType::FP32)
    return InvalidArgumentError("block parameter must use BF16 or FP32");
  const size_t size = storage == DataType::BF16 ? 2 : 4;
  if (&value.executor() != &executor || value.size_bytes() == 0 || value.size_bytes() % size != 0 ||
      value.size_bytes() / size > static_cast<size_t>(std::numeric_limits<int>::max()))
    return InvalidArgumentError("invalid block parameter buffer");
  const size_t elements = value.size_bytes() / size;
  return std::shared_ptr<BlockParameter>(new BlockParameter(std::move(value), storage, elements));
}

Status BlockParameter::Activate() {
  if (active()) return OkStatus();
  if (storage_ != DataType::FP32)
    return UnimplementedError("activating a BF16 block parameter is outside the attention path");
  cuda::Executor& executor = value_.executor();
  PLUTO_ASSIGN_OR_RETURN(Buffer master, Buffer::Allocate(executor, elements_ * 4));
  PLUTO_ASSIGN_OR_RETURN(Buffer gradient, Buffer::Allocate(executor, elements_ * 4));
  PLUTO_RETURN_IF_ERROR(cuda::CudaStatus(
      cudaMemcpyAsync(master.data(), value_.data(), value_.size_bytes(), cudaMemcpyDeviceToDevice,
                      executor.stream()),
      "activate FP32 block weight"));
  PLUTO_RETURN_IF_ERROR(cuda::CudaStatus(
      cudaMemsetAsync(gradient.data(), 0, gradient.size_bytes(), executor.stream()), "zero block gradient"));
  master_ = std::move(master);
  gradient_ = std::move(gradient);
  return OkStatus();
}

Status BlockParameter::Publish() {
  if (!active()) return OkStatus();
  return cuda::CudaStatus(cudaMemcpyAsync(value_.data(), master_->data(), value_.size_bytes(),
                                          cudaMemcpyDeviceToDevice, value_.executor().stream()),
                          "publish FP32 block weight");
}

Status BlockParameter::Deactivate() {
  master_.reset();
  gradient_.reset();
  return OkStatus();
}

// ---- QwenAttentionLayer (src/llm/layers/qwen_attention.cc:291-499) ------------------------------
QwenAttentionLayer::QwenAttentionLayer(cuda::Executor& executor, FullAttentionParameters parameters,
                                       std::shared_ptr<BlockParameter> q_norm,
                                       std::shared_ptr<BlockParameter> k_norm, int sequence_length,
                                       KeyValueCache* cache)
    : executor_(executor), parameters_(parameters), q_norm_(std::move(q_norm)), k_norm_(std::move(k_norm)),
      sequence_length_(sequence_length), weights_{q_norm_->value(), k_norm_->value()}, cache_(cache) {}

StatusOr<std::unique_ptr<QwenAttentionLayer>> QwenAttentionLayer::Create(
    cuda::Executor& executor, FullAttentionParameters p, std::shared_ptr<BlockParameter> q_norm,
    std::shared_ptr<BlockParameter> k_norm, int sequence_length, KeyValueCache* cache) {
  if (cache != nullptr) {
    if (sequence_length != 1)
      return InvalidArgumentError("cached Qwen attention requires sequence_length == 1");
    if (p.query_heads <= 0 || p.key_value_heads <= 0 || p.head_dim <= 0)
      return InvalidArgumentError("QwenAttentionLayer dimensions must be positive");
    const int64_t query_width = 1LL * p.query_heads * p.head_dim;
    const int64_t key_width = 1LL * p.key_value_heads * p.head_dim;
    if (query_width > kMaximumDimension / 2 || key_width > kMaximumDimension)
      return InvalidArgumentError("QwenAttentionLayer activation exceeds the layer dimension limit");
    PLUTO_RETURN_IF_ERROR(cached_attention_ops::ValidateCachedAttention(executor, p, *cache));
  } else {
    // The reference also bounds 1 <= T <= 128 here because it stores [Hq, T, T] probabilities.
    if (p.query_heads <= 0 || p.query_heads > 256 || p.key_value_heads <= 0 ||
        p.query_heads % p.key_value_heads != 0 || p.head_dim <= 0 || p.head_dim > 256 ||
        p.rotary_dim <= 0 || p.rotary_dim > p.head_dim || p.rotary_dim % 2 != 0 || sequence_length <= 0 ||
        !(p.rms_norm_epsilon > 0) || !std::isfinite(p.rms_norm_epsilon) || !(p.rope_theta > 0) ||
        !std::isfinite(p.rope_theta))
      return InvalidArgumentError("sequence Qwen attention requires valid GQA dimensions and D<=256");
    if (!p.round_to_bfloat16)
      return UnimplementedError("sequence Qwen attention without bf16 rounding is not built");
  }
  for (const auto& norm : {q_norm, k_norm})
    if (!norm || norm->storage() != DataType::FP32 || norm->elements() != static_cast<size_t>(p.head_dim) ||
        &norm->value().executor() != &executor)
      return InvalidArgumentError("Qwen attention norms must be FP32 head-width parameters on its Executor");
  return std::unique_ptr<QwenAttentionLayer>(
      new QwenAttentionLayer(executor, p, std::move(q_norm), std::move(k_norm), sequence_length, cache));
}

StatusOr<std::unique_ptr<QwenAttentionLayer>> QwenAttentionLayer::Create(
    cuda::Executor& executor, FullAttentionParameters parameters, Buffer q_norm, Buffer k_norm,
    int sequence_length, KeyValueCache* cache) {
  PLUTO_ASSIGN_OR_RETURN(auto query_parameter, BlockParameter::Create(executor, std::move(q_norm), DataType::FP32));
  PLUTO_ASSIGN_OR_RETURN(auto key_parameter, BlockParameter::Create(executor, std::move(k_norm), DataType::FP32));
  return Create(executor, parameters, std::move(query_parameter), std::move(key_parameter), sequence_length,
                cache);
}

std::vector<ActivationType> QwenAttentionLayer::input_types() const {
  const auto& p = parameters_;
  const int64_t t = sequence_length_;
  return {{DataType::BF16, {ActivationType::kBatchDimension, t, 2LL * p.query_heads * p.head_dim}},
          {DataType::BF16, {ActivationType::kBatchDimension, t, 1LL * p.key_value_heads * p.head_dim}},
          {DataType::BF16, {ActivationType::kBatchDimension, t, 1LL * p.key_value_heads * p.head_dim}}};
}
std::vector<ActivationType> QwenAttentionLayer::output_types() const {
  return {{DataType::BF16,
           {ActivationType::kBatchDimension, sequence_length_, 1LL * parameters_.query_heads * parameters_.head_dim}}};
}

StatusOr<FwdResult> QwenAttentionLayer::fwd_impl(cuda::Executor& executor, const BufferVec& inputs,
                                                 LayerHooks* hooks) const {
  if (&executor != &executor_)
    return InvalidArgumentError("QwenAttentionLayer used with a different Executor");
  return cache_ != nullptr ? CachedForward(executor, inputs, hooks) : SequenceForward(executor, inputs, hooks);
}

StatusOr<BufferVec> QwenAttentionLayer::bwd_impl(cuda::Executor& executor, const BufferVec& gradients,
                                                 BackwardState state, LayerHooks*) {
  if (cache_ != nullptr)
    return UnimplementedError("QwenAttentionLayer with a KV cache supports inference only");
  return SequenceBackward(executor, gradients, std::move(state));
}

StatusOr<FwdResult> QwenAttentionLayer::CachedForward(cuda::Executor& executor, const BufferVec& inputs,
                                                      LayerHooks* hooks) const {
  const auto& p = parameters_;
  const int64_t width = 1LL * p.query_heads * p.head_dim, kv = 1LL * p.key_value_heads * p.head_dim;
  const int64_t counts[] = {2 * width, kv, kv};
  PLUTO_RETURN_IF_ERROR(ValidateBFloat16Inputs(executor, inputs, counts, 3, "QwenAttentionLayer"));
  if (cache_->position() >= cache_->capacity())
    return ResourceExhaustedError("full-attention cache capacity reached");
  const int length = cache_->position() + 1;
  const bool inspect = hooks != nullptr && static_cast<bool>(hooks->attention_probabilities_hook);
  PLUTO_ASSIGN_OR_RETURN(Buffer output, Buffer::Allocate(executor, static_cast<size_t>(width) * 2));
  PLUTO_ASSIGN_OR_RETURN(Buffer probabilities,
                         Buffer::Allocate(executor, inspect ? static_cast<size_t>(p.query_heads) * length * 4 : 0));
  PLUTO_RETURN_IF_ERROR(cached_attention_ops::CachedAttentionStepTyped(
      executor, p, *cache_, inputs[0].data(), inputs[1].data(), inputs[2].data(), PLUTO_BF16, F(weights_[0]),
      F(weights_[1]), output.data(), PLUTO_BF16, inspect ? F(probabilities) : nullptr));
  if (inspect)
    PLUTO_RETURN_IF_ERROR(hooks->attention_probabilities_hook(
        executor, name(), ActivationType{DataType::FP32, {1, p.query_heads, 1, length}}, probabilities));
  FwdResult result;
  result.outputs = {output};
  return result;
}

StatusOr<FwdResult> QwenAttentionLayer::SequenceForward(cuda::Executor& executor, const BufferVec& inputs,
                                                        LayerHooks* hooks) const {
  const auto& p = parameters_;
  const int t = sequence_length_, hq = p.query_heads, hkv = p.key_value_heads, d = p.head_dim;
  const int64_t counts[] = {2LL * t * hq * d, 1LL * t * hkv * d, 1LL * t * hkv * d};
  PLUTO_RETURN_IF_ERROR(ValidateBFloat16Inputs(executor, inputs, counts, 3, "QwenAttentionLayer"));
  const size_t q_elements = static_cast<size_t>(t) * hq * d, kv_elements = static_cast<size_t>(t) * hkv * d;
  const bool inspect = hooks != nullptr && static_cast<bool>(hooks->attention_probabilities_hook);
  PLUTO_ASSIGN_OR_RETURN(Buffer q, Buffer::Allocate(executor, q_elements * 2));
  PLUTO_ASSIGN_OR_RETURN(Buffer k, Buffer::Allocate(executor, kv_elements * 2));
  PLUTO_ASSIGN_OR_RETURN(Buffer v, Buffer::Allocate(executor, kv_elements * 2));
  PLUTO_ASSIGN_OR_RETURN(Buffer output, Buffer::Allocate(executor, q_elements * 2));
  PLUTO_ASSIGN_OR_RETURN(Buffer core, Buffer::Allocate(executor, q_elements * 4));
  PLUTO_ASSIGN_OR_RETURN(Buffer maxima, Buffer::Allocate(executor, static_cast<size_t>(hq) * t * 4));
  PLUTO_ASSIGN_OR_RETURN(Buffer normalizers, Buffer::Allocate(executor, static_cast<size_t>(hq) * t * 4));
  PLUTO_ASSIGN_OR_RETURN(Buffer probabilities,
                         Buffer::Allocate(executor, inspect ? static_cast<size_t>(hq) * t * t * 4 : 0));
  // the key/value split only pays when the query tiles of all heads cannot fill the GPU
  const bool few_tiles = t >= 1024 && static_cast<long long>(hq) * ((t + 127) / 128) <= 148;
  const size_t fwd_ws = few_tiles ? pluto_gqa_prefill_fwd_workspace_bytes(1, t, hq, d) : 0;
  PLUTO_ASSIGN_OR_RETURN(Buffer workspace, AllocateAligned(executor, fwd_ws));
  // PrepareKernel (:30-63): RMSNorm(1+w), bf16 rounding, partial RoPE; rows of the prepared k and
  // the rounded v land in the two sequence buffers through the cache-append path (position = row)
  const pluto_kv_cache view = SequenceView(k, v, t, hkv, d);
  PLUTO_RETURN_IF_ERROR(FromEngine(
      pluto_qk_prepare(executor.stream(), inputs[0].data(), inputs[1].data(), inputs[2].data(), PLUTO_BF16,
                       2 * static_cast<size_t>(hq) * d, 2 * static_cast<size_t>(d), F(weights_[0]), F(weights_[1]),
                       nullptr, q.data(), PLUTO_BF16, &view, 1, t, hq, hkv, d, p.rotary_dim, p.rms_norm_epsilon,
                       p.rope_theta, 1),
      "prepare sequence full attention"));
  // ForwardKernel (:68-119): causal attention core + sigmoid gate, saving the unrounded core
  PLUTO_RETURN_IF_ERROR(FromEngine(
      pluto_gqa_prefill_fwd(executor.stream(), q.data(), Bytes(inputs[0]) + static_cast<size_t>(d) * 2, k.data(),
                            v.data(), output.data(), F(core), F(maxima), F(normalizers), 1, t, hq, hkv, d,
                            static_cast<size_t>(hq) * d, d, 2 * static_cast<size_t>(hq) * d,
                            2 * static_cast<size_t>(d), 1, fwd_ws ? workspace.data() : nullptr, fwd_ws),
      "sequence full attention forward"));
  if (inspect) {
    // [Hq, T, T] with zeros above the diagonal: row r of the sequence is a cached step of length r+1
    PLUTO_RETURN_IF_ERROR(cuda::CudaStatus(
        cudaMemsetAsync(probabilities.data(), 0, probabilities.size_bytes(), executor.stream()),
        "clear attention probabilities"));
    std::vector<int32_t> host(static_cast<size_t>(2) * t, 0);
    for (int r = 0; r < t; ++r) host[r] = r + 1;   // lengths, then a block table of zeros
    PLUTO_ASSIGN_OR_RETURN(Buffer rows, Buffer::Allocate(executor, host.size() * sizeof(int32_t)));
    PLUTO_RETURN_IF_ERROR(cuda::CudaStatus(
        cudaMemcpyAsync(rows.data(), host.data(), host.size() * sizeof(int32_t), cudaMemcpyHostToDevice,
                        executor.stream()),
        "upload probability row lengths"));
    // (a copy from pageable host memory is staged before the call returns: `host` may go away)
    pluto_kv_cache paged = view;
    paged.block_table = static_cast<const int32_t*>(rows.data()) + t;
    paged.max_blocks = 1;
    PLUTO_RETURN_IF_ERROR(FromEngine(
        pluto_gqa_decode_probs(executor.stream(), q.data(), PLUTO_BF16, &paged,
                               static_cast<const int32_t*>(rows.data()), F(probabilities), t,
                               static_cast<size_t>(t) * t, t, hq, hkv, d),
        "sequence attention probabilities"));
    PLUTO_RETURN_IF_ERROR(hooks->attention_probabilities_hook(
        executor, name(), ActivationType{DataType::FP32, {1, hq, t, t}}, probabilities));
  }
  FwdResult result;
  result.outputs = {output};
  result.state.intermediates = {inputs[0], inputs[1], inputs[2], q, k, probabilities, core,
                                maxima,    normalizers, v};
  return result;
}

StatusOr<BufferVec> QwenAttentionLayer::SequenceBackward(cuda::Executor& executor, const BufferVec& gradients,
                                                         BackwardState state) {
  const auto& p = parameters_;
  const int t = sequence_length_, hq = p.query_heads, hkv = p.key_value_heads, d = p.head_dim;
  if (&executor != &executor_ || state.intermediates.size() != kSavedBuffers)
    return InvalidArgumentError("sequence attention backward Executor/state mismatch");
  if (gradients.size() != 1)
    return InvalidArgumentError("sequence attention received an unexpected number of buffers");
  const size_t q_elements = static_cast<size_t>(t) * hq * d, kv_elements = static_cast<size_t>(t) * hkv * d;
  if (&gradients[0].executor() != &executor || gradients[0].size_bytes() != q_elements * 4)
    return InvalidArgumentError("sequence attention buffer has an invalid size or Executor");
  const auto& s = state.intermediates;
  const size_t expected[] = {2 * q_elements * 2, kv_elements * 2, kv_elements * 2, q_elements * 2,
                             kv_elements * 2,    s[5].size_bytes(), q_elements * 4,
                             static_cast<size_t>(hq) * t * 4, static_cast<size_t>(hq) * t * 4, kv_elements * 2};
  for (size_t i = 0; i < kSavedBuffers; ++i)
    if (&s[i].executor() != &executor || s[i].size_bytes() != expected[i])
      return InvalidArgumentError("sequence attention buffer has an invalid size or Executor");
  PLUTO_ASSIGN_OR_RETURN(Buffer dqg, Buffer::Allocate(executor, 2 * q_elements * 4));
  PLUTO_ASSIGN_OR_RETURN(Buffer dk, Buffer::Allocate(executor, kv_elements * 4));
  PLUTO_ASSIGN_OR_RETURN(Buffer dv, Buffer::Allocate(executor, kv_elements * 4));
  PLUTO_ASSIGN_OR_RETURN(Buffer dq_rope, Buffer::Allocate(executor, q_elements * 4));
  PLUTO_ASSIGN_OR_RETURN(Buffer dk_rope, Buffer::Allocate(executor, kv_elements * 4));
  PLUTO_ASSIGN_OR_RETURN(Buffer dc, Buffer::Allocate(executor, q_elements * 4));
  PLUTO_ASSIGN_OR_RETURN(Buffer deltas, Buffer::Allocate(executor, static_cast<size_t>(hq) * t * 4));
  const size_t token = 2 * static_cast<size_t>(hq) * d, head = 2 * static_cast<size_t>(d);
  // GateBackwardKernel (:123-138) + the row term of the softmax backward
  PLUTO_RETURN_IF_ERROR(FromEngine(
      pluto_gqa_gate_bwd(executor.stream(), Bytes(s[0]) + static_cast<size_t>(d) * 2, token, head, F(s[6]),
                         F(gradients[0]), F(dc), F(dqg) + d, token, head, F(deltas), 1, t, hq, d,
                         p.round_to_bfloat16),
      "sequence full attention backward (gate)"));
  // QueryBackwardKernel + KeyValueBackwardKernel (:140-190)
  const size_t core_ws = pluto_gqa_prefill_bwd_workspace_bytes(1, t, hq, d, PLUTO_BF16);
  PLUTO_ASSIGN_OR_RETURN(Buffer workspace, AllocateAligned(executor, core_ws));
  PLUTO_RETURN_IF_ERROR(FromEngine(
      pluto_gqa_prefill_bwd(executor.stream(), s[3].data(), s[4].data(), s[9].data(), PLUTO_BF16,
                            static_cast<size_t>(hq) * d, d, F(dc), F(s[7]), F(s[8]), F(deltas), F(dq_rope),
                            F(dk_rope), F(dv), core_ws ? workspace.data() : nullptr, core_ws, 1, t, hq, hkv, d),
      "sequence full attention backward"));
  // NormBackwardKernel + ReduceNormKernel (:192-239) for the queries, then the keys
  struct Side { const Buffer* x; size_t x_token, x_head; BlockParameter* norm; Buffer* grad; float* dx; int heads; };
  const Side sides[2] = {{&s[0], token, head, q_norm_.get(), &dq_rope, F(dqg), hq},
                         {&s[1], static_cast<size_t>(hkv) * d, static_cast<size_t>(d), k_norm_.get(), &dk_rope,
                          F(dk), hkv}};
  for (const Side& side : sides) {
    const bool active = side.norm->active();
    const size_t norm_ws = active ? pluto_qk_prepare_bwd_workspace_bytes(1, t, side.heads, d) : 0;
    PLUTO_ASSIGN_OR_RETURN(Buffer scratch, Buffer::Allocate(executor, norm_ws));
    PLUTO_RETURN_IF_ERROR(FromEngine(
        pluto_qk_prepare_bwd(executor.stream(), side.x->data(), side.x_token, side.x_head, F(side.norm->value()),
                             F(*side.grad), nullptr, side.dx, side.x_token, side.x_head,
                             active ? F(side.norm->gradient()) : nullptr, active ? scratch.data() : nullptr,
                             norm_ws, 1, t, side.heads, d, p.rotary_dim, p.rms_norm_epsilon, p.rope_theta,
                             p.round_to_bfloat16),
        "sequence full attention backward (norm)"));
  }
  return BufferVec{dqg, dk, dv};
}

// ---- DeltaNetLayer (src/llm/layers/delta_net.cc:38-110) -----------------------------------------
DeltaNetLayer::DeltaNetLayer(cuda::Executor& executor, DeltaNetParameters parameters, Buffer convolution,
                             Buffer a_log, Buffer dt_bias, Buffer norm,
                             std::unique_ptr<cached_attention_ops::DeltaNetState> cache)
    : executor_(executor), parameters_(parameters),
      weights_{std::move(convolution), std::move(a_log), std::move(dt_bias), std::move(norm)},
      cache_(std::move(cache)) {}

StatusOr<std::unique_ptr<DeltaNetLayer>> DeltaNetLayer::Create(cuda::Executor& executor, DeltaNetParameters p,
                                                              Buffer convolution, Buffer a_log,
                                                              Buffer dt_bias, Buffer norm) {
  if (p.key_heads <= 0 || p.value_heads <= 0 || p.key_head_dim <= 0 || p.value_head_dim <= 0 ||
      p.conv_kernel_dim <= 0)
    return InvalidArgumentError("DeltaNetLayer dimensions must be positive");
  const int64_t key_width = 1LL * p.key_heads * p.key_head_dim;
  const int64_t value_width = 1LL * p.value_heads * p.value_head_dim;
  if (key_width > kMaximumDimension / 2 || value_width > kMaximumDimension ||
      2 * key_width + value_width > kMaximumDimension)
    return InvalidArgumentError("DeltaNetLayer activation exceeds the layer dimension limit");
  const int64_t channels = 2 * key_width + value_width;
  const Buffer* weights[] = {&convolution, &a_log, &dt_bias, &norm};
  const int64_t counts[] = {channels * p.conv_kernel_dim, p.value_heads, p.value_heads, p.value_head_dim};
  for (int i = 0; i < 4; ++i)
    if (&weights[i]->executor() != &executor ||
        weights[i]->size_bytes() != static_cast<size_t>(counts[i]) * sizeof(float))
      return InvalidArgumentError("DeltaNetLayer weight has incorrect FP32 size or Executor");
  PLUTO_ASSIGN_OR_RETURN(auto cache, cached_attention_ops::DeltaNetState::Create(executor, p));
  return std::unique_ptr<DeltaNetLayer>(new DeltaNetLayer(executor, p, std::move(convolution), std::move(a_log),
                                                          std::move(dt_bias), std::move(norm), std::move(cache)));
}

std::vector<ActivationType> DeltaNetLayer::input_types() const {
  const auto& p = parameters_;
  const int64_t width = 1LL * p.value_heads * p.value_head_dim;
  const int64_t channels = 2LL * p.key_heads * p.key_head_dim + width;
  return {{DataType::BF16, {ActivationType::kBatchDimension, 1, channels}},
          {DataType::BF16, {ActivationType::kBatchDimension, 1, width}},
          {DataType::BF16, {ActivationType::kBatchDimension, 1, p.value_heads}},
          {DataType::BF16, {ActivationType::kBatchDimension, 1, p.value_heads}}};
}
std::vector<ActivationType> DeltaNetLayer::output_types() const {
  return {{DataType::BF16,
           {ActivationType::kBatchDimension, 1, 1LL * parameters_.value_heads * parameters_.value_head_dim}}};
}

StatusOr<FwdResult> DeltaNetLayer::fwd_impl(cuda::Executor& executor, const BufferVec& inputs,
                                            LayerHooks*) const {
  if (&executor != &executor_) return InvalidArgumentError("DeltaNetLayer used with a different Executor");
  const auto& p = parameters_;
  const int64_t width = 1LL * p.value_heads * p.value_head_dim;
  const int64_t counts[] = {2LL * p.key_heads * p.key_head_dim + width, width, p.value_heads, p.value_heads};
  PLUTO_RETURN_IF_ERROR(ValidateBFloat16Inputs(executor, inputs, counts, 4, "DeltaNetLayer"));
  PLUTO_ASSIGN_OR_RETURN(Buffer output, Buffer::Allocate(executor, static_cast<size_t>(width) * 2));
  PLUTO_RETURN_IF_ERROR(cache_->StepTyped(inputs[0].data(), inputs[1].data(), inputs[2].data(), inputs[3].data(),
                                          PLUTO_BF16, F(weights_[0]), F(weights_[1]), F(weights_[2]),
                                          F(weights_[3]), output.data(), PLUTO_BF16));
  FwdResult result;
  result.outputs = {output};
  return result;
}

StatusOr<BufferVec> DeltaNetLayer::bwd_impl(cuda::Executor&, const BufferVec&, BackwardState, LayerHooks*) {
  return UnimplementedError("DeltaNetLayer supports cached inference only");
}

Status DeltaNetLayer::Reset() { return cache_->Reset(); }

// ---- SequenceDeltaNetLayer (src/llm/layers/sequence_delta_net.cc:396-561) -----------------------
SequenceDeltaNetLayer::SequenceDeltaNetLayer(cuda::Executor& executor, DeltaNetParameters parameters,
                                             std::shared_ptr<BlockParameter> convolution,
                                             std::shared_ptr<BlockParameter> a_log,
                                             std::shared_ptr<BlockParameter> dt_bias,
                                             std::shared_ptr<BlockParameter> norm, int sequence_length)
    : executor_(executor), parameters_(parameters), sequence_length_(sequence_length),
      parameters_owned_{std::move(convolution), std::move(a_log), std::move(dt_bias), std::move(norm)},
      weights_{parameters_owned_[0]->value(), parameters_owned_[1]->value(), parameters_owned_[2]->value(),
               parameters_owned_[3]->value()} {}

StatusOr<std::unique_ptr<SequenceDeltaNetLayer>> SequenceDeltaNetLayer::Create(
    cuda::Executor& executor, DeltaNetParameters p, std::shared_ptr<BlockParameter> convolution,
    std::shared_ptr<BlockParameter> a_log, std::shared_ptr<BlockParameter> dt_bias,
    std::shared_ptr<BlockParameter> norm, int sequence_length) {
  // (the reference also bounds T <= 128 here because it stores every intermediate state)
  if (sequence_length < 1 || p.key_heads < 1 || p.value_heads < 1 || p.value_heads % p.key_heads != 0 ||
      p.key_head_dim < 1 || p.key_head_dim > 128 || p.value_head_dim < 1 || p.value_head_dim > 256 ||
      p.conv_kernel_dim < 1 || p.conv_kernel_dim > 32 || !std::isfinite(p.rms_norm_epsilon) ||
      p.rms_norm_epsilon <= 0)
    return InvalidArgumentError("unsupported SequenceDeltaNetLayer shape");
  if (!p.round_to_bfloat16)
    return UnimplementedError("sequence delta-net without bf16 rounding is not built");
  const int64_t channels = 2LL * p.key_heads * p.key_head_dim + 1LL * p.value_heads * p.value_head_dim;
  if (channels * sequence_length > std::numeric_limits<int>::max())
    return InvalidArgumentError("unsupported SequenceDeltaNetLayer shape");
  const std::shared_ptr<BlockParameter>* parameters[] = {&convolution, &a_log, &dt_bias, &norm};
  const int64_t counts[] = {channels * p.conv_kernel_dim, p.value_heads, p.value_heads, p.value_head_dim};
  for (int i = 0; i < 4; ++i) {
    const auto& parameter = *parameters[i];
    if (!parameter || parameter->storage() != DataType::FP32)
      return InvalidArgumentError("DeltaNet parameters must be FP32");
    if (&parameter->value().executor() != &executor ||
        parameter->elements() != static_cast<size_t>(counts[i]))
      return InvalidArgumentError("DeltaNet parameter has " + std::to_string(parameter->elements() * 4) +
                                  " bytes; expected " + std::to_string(counts[i] * 4));
  }
  return std::unique_ptr<SequenceDeltaNetLayer>(new SequenceDeltaNetLayer(
      executor, p, std::move(convolution), std::move(a_log), std::move(dt_bias), std::move(norm),
      sequence_length));
}

std::vector<ActivationType> SequenceDeltaNetLayer::input_types() const {
  const auto& p = parameters_;
  const int64_t t = sequence_length_, width = 1LL * p.value_heads * p.value_head_dim;
  const int64_t channels = 2LL * p.key_heads * p.key_head_dim + width;
  return {{DataType::BF16, {1, t, channels}},
          {DataType::BF16, {1, t, width}},
          {DataType::BF16, {1, t, p.value_heads}},
          {DataType::BF16, {1, t, p.value_heads}}};
}
std::vector<ActivationType> SequenceDeltaNetLayer::output_types() const {
  return {{DataType::BF16, {1, sequence_length_, 1LL * parameters_.value_heads * parameters_.value_head_dim}}};
}

StatusOr<FwdResult> SequenceDeltaNetLayer::fwd_impl(cuda::Executor& executor, const BufferVec& inputs,
                                                    LayerHooks*) const {
  const auto& p = parameters_;
  const int t = sequence_length_;
  const int width = p.value_heads * p.value_head_dim, kq = p.key_heads * p.key_head_dim;
  const int channels = 2 * kq + width;
  if (&executor != &executor_ || inputs.size() != 4)
    return InvalidArgumentError("DeltaNet expects four inputs on its Executor");
  const int64_t counts[] = {1LL * t * channels, 1LL * t * width, 1LL * t * p.value_heads, 1LL * t * p.value_heads};
  PLUTO_RETURN_IF_ERROR(ValidateBFloat16Inputs(executor, inputs, counts, 4, "SequenceDeltaNetLayer"));
  cudaStream_t stream = executor.stream();
  PLUTO_ASSIGN_OR_RETURN(Buffer pre, Buffer::Allocate(executor, 0));
  PLUTO_ASSIGN_OR_RETURN(Buffer post, Buffer::Allocate(executor, static_cast<size_t>(t) * channels * 2));
  PLUTO_ASSIGN_OR_RETURN(Buffer conv_state,
                         Buffer::Allocate(executor, static_cast<size_t>(channels) * p.conv_kernel_dim * 4));
  PLUTO_ASSIGN_OR_RETURN(Buffer gates, Buffer::Allocate(executor, 2 * static_cast<size_t>(t) * p.value_heads * 4));
  PLUTO_ASSIGN_OR_RETURN(Buffer states, Buffer::Allocate(executor, static_cast<size_t>(p.value_heads) *
                                                                       p.key_head_dim * p.value_head_dim * 4));
  PLUTO_ASSIGN_OR_RETURN(Buffer core, Buffer::Allocate(executor, static_cast<size_t>(t) * width * 2));
  PLUTO_ASSIGN_OR_RETURN(Buffer output, Buffer::Allocate(executor, static_cast<size_t>(t) * width * 2));
  PLUTO_RETURN_IF_ERROR(cuda::CudaStatus(cudaMemsetAsync(conv_state.data(), 0, conv_state.size_bytes(), stream),
                                         "clear convolution history"));
  PLUTO_RETURN_IF_ERROR(cuda::CudaStatus(cudaMemsetAsync(states.data(), 0, states.size_bytes(), stream),
                                         "clear recurrent state"));
  // ConvForward (:31-51)
  PLUTO_RETURN_IF_ERROR(FromEngine(
      pluto_gdn_conv_silu(stream, inputs[0].data(), F(weights_[0]), PLUTO_BF16, 1, t, channels, p.conv_kernel_dim,
                          1, F(conv_state), post.data(), PLUTO_BF16),
      "sequence DeltaNet forward (convolution)"));
  float* g = F(gates);
  float* beta = g + static_cast<size_t>(t) * p.value_heads;
  PLUTO_RETURN_IF_ERROR(FromEngine(
      pluto_gdn_gates(stream, inputs[2].data(), inputs[3].data(), F(weights_[1]), F(weights_[2]), PLUTO_BF16, t,
                      p.value_heads, 1, g, beta),
      "sequence DeltaNet forward (gates)"));
  // RecurrenceForward (:55-102): the chunked tensor-core form when the shape has one
  size_t chunk_ws = pluto_gdn_prefill_workspace_bytes(1, t, p.key_heads, p.value_heads, p.key_head_dim,
                                                      p.value_head_dim, PLUTO_BF16);
  if (channels % 8 != 0 || kq % 8 != 0) chunk_ws = 0;   // the chunked path reads 16-byte pieces of a token row
  PLUTO_ASSIGN_OR_RETURN(Buffer workspace, AllocateAligned(executor, chunk_ws));
  const char* packed = Bytes(post);
  PLUTO_RETURN_IF_ERROR(FromEngine(
      pluto_gdn_prefill(stream, packed, packed + static_cast<size_t>(kq) * 2, packed + 2 * static_cast<size_t>(kq) * 2,
                        PLUTO_BF16, g, beta, F(states), core.data(), PLUTO_BF16, 1, t, p.key_heads, p.value_heads,
                        p.key_head_dim, p.value_head_dim, channels, channels, 1, 1.0f, 1,
                        chunk_ws ? workspace.data() : nullptr, chunk_ws),
      "sequence DeltaNet forward (recurrence)"));
  // OutputForward (:104-121): the last product is stored without an extra rounding
  PLUTO_RETURN_IF_ERROR(FromEngine(
      pluto_gdn_out_norm_gate(stream, core.data(), PLUTO_BF16, inputs[1].data(), PLUTO_BF16, F(weights_[3]),
                              1LL * t * p.value_heads, p.value_head_dim, p.rms_norm_epsilon, 1, 0, output.data(),
                              PLUTO_BF16),
      "sequence DeltaNet forward"));
  FwdResult result;
  result.outputs = {output};
  result.state.intermediates = {inputs[0], inputs[1], inputs[2], inputs[3], pre, post, core, states};
  return result;
}

StatusOr<BufferVec> SequenceDeltaNetLayer::bwd_impl(cuda::Executor& executor, const BufferVec& gradients,
                                                    BackwardState state, LayerHooks*) {
  if (&executor != &executor_ || gradients.size() != 1 || state.intermediates.size() != kSavedBuffers)
    return InvalidArgumentError("invalid DeltaNet backward state or gradient");
  const auto& p = parameters_;
  const int t = sequence_length_;
  const int width = p.value_heads * p.value_head_dim, kq = p.key_heads * p.key_head_dim;
  const int channels = 2 * kq + width;
  const auto& s = state.intermediates;
  if (&gradients[0].executor() != &executor || gradients[0].size_bytes() != static_cast<size_t>(t) * width * 4)
    return InvalidArgumentError("SequenceDeltaNetLayer requires batch-one buffers of the declared shape");
  const size_t expected[] = {static_cast<size_t>(t) * channels * 2, static_cast<size_t>(t) * width * 2,
                             static_cast<size_t>(t) * p.value_heads * 2, static_cast<size_t>(t) * p.value_heads * 2,
                             0, static_cast<size_t>(t) * channels * 2, static_cast<size_t>(t) * width * 2,
                             static_cast<size_t>(p.value_heads) * p.key_head_dim * p.value_head_dim * 4};
  for (size_t i = 0; i < kSavedBuffers; ++i)
    if (&s[i].executor() != &executor || s[i].size_bytes() != expected[i])
      return InvalidArgumentError("SequenceDeltaNetLayer requires batch-one buffers of the declared shape");
  cudaStream_t stream = executor.stream();
  BlockParameter* conv_p = parameters_owned_[0].get();
  BlockParameter* a_log_p = parameters_owned_[1].get();
  BlockParameter* dt_bias_p = parameters_owned_[2].get();
  BlockParameter* norm_p = parameters_owned_[3].get();
  auto gradient_of = [](BlockParameter* parameter) { return parameter->active() ? F(parameter->gradient()) : nullptr; };
  PLUTO_ASSIGN_OR_RETURN(Buffer dqkv, Buffer::Allocate(executor, static_cast<size_t>(t) * channels * 4));
  PLUTO_ASSIGN_OR_RETURN(Buffer dz, Buffer::Allocate(executor, static_cast<size_t>(t) * width * 4));
  PLUTO_ASSIGN_OR_RETURN(Buffer da, Buffer::Allocate(executor, static_cast<size_t>(t) * p.value_heads * 4));
  PLUTO_ASSIGN_OR_RETURN(Buffer db, Buffer::Allocate(executor, static_cast<size_t>(t) * p.value_heads * 4));
  PLUTO_ASSIGN_OR_RETURN(Buffer dcore, Buffer::Allocate(executor, static_cast<size_t>(t) * width * 4));
  PLUTO_ASSIGN_OR_RETURN(Buffer dpost, Buffer::Allocate(executor, static_cast<size_t>(t) * channels * 4));
  // OutputBackward + SumNormGradient (:126-171)
  const long long rows = 1LL * t * p.value_heads;
  const size_t out_ws = norm_p->active() ? pluto_gdn_out_norm_gate_bwd_workspace_bytes(rows, p.value_head_dim) : 0;
  PLUTO_ASSIGN_OR_RETURN(Buffer out_scratch, Buffer::Allocate(executor, out_ws));
  PLUTO_RETURN_IF_ERROR(FromEngine(
      pluto_gdn_out_norm_gate_bwd(stream, s[6].data(), PLUTO_BF16, s[1].data(), PLUTO_BF16, F(norm_p->value()),
                                  F(gradients[0]), F(dcore), F(dz), gradient_of(norm_p),
                                  out_ws ? out_scratch.data() : nullptr, out_ws, rows, p.value_head_dim,
                                  p.rms_norm_epsilon, 1),
      "sequence DeltaNet backward (output)"));
  // RecurrenceBackward + GatherQkGradient + GatherScalarGradient (:176-309)
  const size_t rec_ws = pluto_gdn_recurrence_bwd_workspace_bytes(1, t, p.key_heads, p.value_heads, p.key_head_dim,
                                                                 p.value_head_dim);
  PLUTO_ASSIGN_OR_RETURN(Buffer rec_scratch, Buffer::Allocate(executor, rec_ws));
  const char* packed = Bytes(s[5]);
  float* dpacked = F(dpost);
  PLUTO_RETURN_IF_ERROR(FromEngine(
      pluto_gdn_recurrence_bwd(stream, packed, packed + static_cast<size_t>(kq) * 2,
                               packed + 2 * static_cast<size_t>(kq) * 2, PLUTO_BF16, channels, channels,
                               s[2].data(), s[3].data(), PLUTO_BF16, F(a_log_p->value()), F(dt_bias_p->value()),
                               F(dcore), dpacked, dpacked + kq, channels, dpacked + 2 * kq, channels, F(da), F(db),
                               gradient_of(a_log_p), gradient_of(dt_bias_p), rec_scratch.data(), rec_ws, 1, t,
                               p.key_heads, p.value_heads, p.key_head_dim, p.value_head_dim, 1),
      "sequence DeltaNet backward (recurrence)"));
  // ConvSiluBackward + ConvInputBackward + ConvWeightBackward (:311-362)
  PLUTO_RETURN_IF_ERROR(FromEngine(
      pluto_gdn_conv_silu_bwd(stream, s[0].data(), PLUTO_BF16, F(conv_p->value()), F(dpost), F(dqkv),
                              gradient_of(conv_p), 1, t, channels, p.conv_kernel_dim, 1),
      "sequence DeltaNet backward (convolution)"));
  return BufferVec{dqkv, dz, da, db};
}

}  // namespace pluto::llm
