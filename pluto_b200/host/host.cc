// Implementation of the C++ host adapter (runtime.h, layers.h) over the C ABI.
#include <cmath>
#include <limits>
#include <string>

#include "../../include/pluto_b200.h"
#include "layers.h"

namespace pluto {

Status FromEngine(int code, const char* operation) {
  if (code == PLUTO_OK) return OkStatus();
  const std::string text = pluto_last_error();
  switch (code) {
    case PLUTO_E_INVALID: return InvalidArgumentError(text);
    case PLUTO_E_UNIMPLEMENTED: return UnimplementedError(text);
    case PLUTO_E_EXHAUSTED: return ResourceExhaustedError(text);
    case PLUTO_E_INTERNAL: return InternalError(text);
    default: return InternalError(std::string(operation) + ": " + text);  // a cudaError_t
  }
}

namespace cuda {

Status CudaStatus(cudaError_t error, const char* operation) {
  if (error == cudaSuccess) return OkStatus();
  const std::string text = std::string(operation) + ": " + cudaGetErrorString(error);
  return error == cudaErrorMemoryAllocation ? ResourceExhaustedError(text) : InternalError(text);
}

StatusOr<std::unique_ptr<Executor>> Executor::Create() {
  std::unique_ptr<Executor> executor(new Executor());
  PLUTO_RETURN_IF_ERROR(CudaStatus(
      cudaStreamCreateWithFlags(&executor->stream_, cudaStreamNonBlocking), "create compute stream"));
  return executor;
}
Executor::~Executor() {
  if (stream_ != nullptr) {
    cudaStreamSynchronize(stream_);
    cudaStreamDestroy(stream_);
  }
}
Status Executor::Synchronize() const {
  return CudaStatus(cudaStreamSynchronize(stream_), "synchronize compute stream");
}

struct Buffer::Allocation {
  Executor* executor;
  void* data;
  size_t size_bytes;
  ~Allocation() {
    if (data != nullptr) cudaFreeAsync(data, executor->stream());  // stream-ordered, like the reference
  }
};

StatusOr<Buffer> Buffer::Allocate(Executor& executor, size_t size_bytes) {
  void* data = nullptr;
  if (size_bytes > 0)
    PLUTO_RETURN_IF_ERROR(
        CudaStatus(cudaMallocAsync(&data, size_bytes, executor.stream()), "allocate device buffer"));
  return Buffer(std::shared_ptr<Allocation>(new Allocation{&executor, data, size_bytes}));
}
void* Buffer::data() const { return allocation_->data; }
size_t Buffer::size_bytes() const { return allocation_->size_bytes; }
Executor& Buffer::executor() const { return *allocation_->executor; }

}  // namespace cuda

namespace llm {
namespace {

size_t ElementBytes(DataType type) { return type == DataType::BF16 ? 2 : 4; }

Status ValidateExecutor(const cuda::Executor& owner, const cuda::Executor& caller, const char* layer) {
  if (&owner != &caller)
    return InvalidArgumentError(std::string(layer) + " was created for a different Executor");
  return OkStatus();
}

StatusOr<int> MatrixRows(cuda::Executor& executor, const Buffer& buffer, size_t element_bytes,
                         int columns, const char* name) {
  if (&buffer.executor() != &executor)
    return InvalidArgumentError(std::string(name) + " belongs to a different Executor");
  if (buffer.size_bytes() == 0 || buffer.size_bytes() % element_bytes != 0)
    return InvalidArgumentError(std::string(name) + " has an invalid byte size");
  const size_t elements = buffer.size_bytes() / element_bytes;
  if (elements > static_cast<size_t>(std::numeric_limits<int>::max()))
    return InvalidArgumentError(std::string(name) + " has too many elements");
  if (elements % static_cast<size_t>(columns) != 0)
    return InvalidArgumentError(std::string(name) + " is not an activation matrix");
  return static_cast<int>(elements / columns);
}

Status ValidateBuffer(cuda::Executor& executor, const Buffer& buffer, size_t expected, const char* name) {
  if (&buffer.executor() != &executor)
    return InvalidArgumentError(std::string(name) + " belongs to a different Executor");
  if (buffer.size_bytes() != expected)
    return InvalidArgumentError(std::string(name) + " has " + std::to_string(buffer.size_bytes()) +
                                " bytes; expected " + std::to_string(expected));
  return OkStatus();
}

}  // namespace

// ---- Layer: public wrappers with the state-identity check (src/llm/layer.cc:35-84) -------------
StatusOr<FwdResult> Layer::fwd(cuda::Executor& executor, const BufferVec& inputs,
                               LayerHooks* hooks) const {
  auto result = fwd_impl(executor, inputs, hooks);
  if (result.ok()) result->state.layer = this;
  return result;
}
StatusOr<BufferVec> Layer::bwd(cuda::Executor& executor, const BufferVec& output_gradients,
                               BackwardState state, LayerHooks* hooks) {
  if (state.layer != this)
    return InvalidArgumentError("bwd requires a state from this layer's successful fwd");
  return bwd_impl(executor, output_gradients, std::move(state), hooks);
}

// ---- AttentionLayer (src/llm/layers/attention.cc:400-596) ---------------------------------------
StatusOr<std::unique_ptr<AttentionLayer>> AttentionLayer::Create(cuda::Executor& executor,
                                                                int context_length, int num_heads,
                                                                int embedding_dim,
                                                                DataType data_type) {
  if (data_type != DataType::FP16 && data_type != DataType::BF16)
    return UnimplementedError("backend supports only FP16 and BF16 compute policies");
  if (context_length <= 0 || num_heads <= 0 || embedding_dim <= 0)
    return InvalidArgumentError("attention dimensions must all be positive");
  if (embedding_dim % num_heads != 0)
    return InvalidArgumentError("embedding_dim must be divisible by num_heads");
  return std::unique_ptr<AttentionLayer>(
      new AttentionLayer(executor, context_length, num_heads, embedding_dim, data_type));
}

std::vector<ActivationType> AttentionLayer::input_types() const {
  return {{ActivationDataType(output_type_),
           {ActivationType::kBatchDimension, context_length_, 3LL * embedding_dim_}}};
}
std::vector<ActivationType> AttentionLayer::output_types() const {
  return {{ActivationDataType(output_type_),
           {ActivationType::kBatchDimension, context_length_, embedding_dim_}}};
}

StatusOr<FwdResult> AttentionLayer::fwd_impl(cuda::Executor& executor, const BufferVec& inputs,
                                             LayerHooks* hooks) const {
  PLUTO_RETURN_IF_ERROR(ValidateExecutor(executor_, executor, "AttentionLayer"));
  if (inputs.size() != 1) return InvalidArgumentError("AttentionLayer fwd expects packed Q/K/V");
  const size_t element = ElementBytes(output_type_);
  PLUTO_ASSIGN_OR_RETURN(int rows, MatrixRows(executor, inputs[0], element, 3 * embedding_dim_,
                                              "attention packed Q/K/V input"));
  if (rows % context_length_ != 0)
    return InvalidArgumentError("attention rows must be divisible by context_length");
  const bool inspect = hooks != nullptr && static_cast<bool>(hooks->attention_probabilities_hook);
  const int batch = rows / context_length_, head_dim = embedding_dim_ / num_heads_;
  const int dtype = output_type_ == DataType::BF16 ? PLUTO_BF16 : PLUTO_FP32;
  size_t probability_bytes = 0;
  if (inspect) {
    probability_bytes = static_cast<size_t>(rows);
    for (size_t factor : {static_cast<size_t>(num_heads_), static_cast<size_t>(context_length_), sizeof(float)}) {
      if (probability_bytes > std::numeric_limits<size_t>::max() / factor)
        return ResourceExhaustedError("attention probabilities tensor byte size overflows size_t");
      probability_bytes *= factor;
    }
  }
  PLUTO_ASSIGN_OR_RETURN(Buffer output, Buffer::Allocate(executor, static_cast<size_t>(rows) * embedding_dim_ * element));
  const size_t stats_bytes = static_cast<size_t>(rows) * num_heads_ * sizeof(float);
  PLUTO_ASSIGN_OR_RETURN(Buffer maxima, Buffer::Allocate(executor, stats_bytes));
  PLUTO_ASSIGN_OR_RETURN(Buffer normalizers, Buffer::Allocate(executor, stats_bytes));
  PLUTO_RETURN_IF_ERROR(FromEngine(
      pluto_attn_fwd(executor.stream(), inputs[0].data(), output.data(),
                     static_cast<float*>(maxima.data()), static_cast<float*>(normalizers.data()),
                     batch, context_length_, num_heads_, head_dim, dtype),
      "attention forward launch"));
  if (inspect) {
    PLUTO_ASSIGN_OR_RETURN(Buffer probabilities, Buffer::Allocate(executor, probability_bytes));
    PLUTO_RETURN_IF_ERROR(FromEngine(
        pluto_attn_probs(executor.stream(), inputs[0].data(),
                         static_cast<const float*>(maxima.data()),
                         static_cast<const float*>(normalizers.data()),
                         static_cast<float*>(probabilities.data()), batch, context_length_,
                         num_heads_, head_dim, dtype),
        "attention probabilities launch"));
    const ActivationType type{DataType::FP32, {batch, num_heads_, context_length_, context_length_}};
    PLUTO_RETURN_IF_ERROR(hooks->attention_probabilities_hook(executor, name(), type, probabilities));
  }
  FwdResult result;
  result.state.intermediates = {inputs[0], output, maxima, normalizers};
  result.outputs = {output};
  return result;
}

StatusOr<BufferVec> AttentionLayer::bwd_impl(cuda::Executor& executor,
                                             const BufferVec& output_gradients, BackwardState state,
                                             LayerHooks*) {
  PLUTO_RETURN_IF_ERROR(ValidateExecutor(executor_, executor, "AttentionLayer"));
  if (output_gradients.size() != 1 || state.intermediates.size() != 4)
    return InvalidArgumentError("AttentionLayer bwd received an incompatible gradient or state");
  PLUTO_ASSIGN_OR_RETURN(int rows, MatrixRows(executor, output_gradients[0], sizeof(float),
                                              embedding_dim_, "attention output gradient"));
  if (rows % context_length_ != 0)
    return InvalidArgumentError("attention gradient rows must be divisible by context_length");
  const size_t element = ElementBytes(output_type_);
  const size_t stats_bytes = static_cast<size_t>(rows) * num_heads_ * sizeof(float);
  PLUTO_RETURN_IF_ERROR(ValidateBuffer(executor, state.intermediates[0],
                                       static_cast<size_t>(rows) * 3 * embedding_dim_ * element,
                                       "attention saved Q/K/V"));
  PLUTO_RETURN_IF_ERROR(ValidateBuffer(executor, state.intermediates[1],
                                       static_cast<size_t>(rows) * embedding_dim_ * element,
                                       "attention saved output"));
  PLUTO_RETURN_IF_ERROR(ValidateBuffer(executor, state.intermediates[2], stats_bytes, "attention saved maxima"));
  PLUTO_RETURN_IF_ERROR(ValidateBuffer(executor, state.intermediates[3], stats_bytes, "attention saved normalizers"));
  PLUTO_ASSIGN_OR_RETURN(Buffer gradient, Buffer::Allocate(executor, static_cast<size_t>(rows) * 3 * embedding_dim_ * sizeof(float)));
  PLUTO_ASSIGN_OR_RETURN(Buffer deltas, Buffer::Allocate(executor, stats_bytes));
  const int dtype = output_type_ == DataType::BF16 ? PLUTO_BF16 : PLUTO_FP32;
  const size_t workspace_bytes = pluto_attn_bwd_workspace_bytes(
      rows / context_length_, context_length_, num_heads_, embedding_dim_ / num_heads_, dtype);
  PLUTO_ASSIGN_OR_RETURN(Buffer workspace, Buffer::Allocate(executor, workspace_bytes));
  PLUTO_RETURN_IF_ERROR(FromEngine(
      pluto_attn_bwd(executor.stream(), state.intermediates[0].data(), state.intermediates[1].data(),
                     static_cast<const float*>(output_gradients[0].data()),
                     static_cast<const float*>(state.intermediates[2].data()),
                     static_cast<const float*>(state.intermediates[3].data()),
                     static_cast<float*>(gradient.data()), static_cast<float*>(deltas.data()),
                     rows / context_length_, context_length_, num_heads_,
                     embedding_dim_ / num_heads_, dtype, workspace.data(), workspace_bytes),
      "attention backward launch"));
  return BufferVec{gradient};
}

// ---- KeyValueCache (src/llm/key_value_cache.cc:20-45) -------------------------------------------
StatusOr<std::unique_ptr<KeyValueCache>> KeyValueCache::Create(cuda::Executor& executor, int capacity,
                                                              int key_value_heads, int head_dim,
                                                              bool bfloat16) {
  if (capacity <= 0 || key_value_heads <= 0 || head_dim <= 0)
    return InvalidArgumentError("key-value cache dimensions must be positive");
  const size_t bytes = static_cast<size_t>(capacity) * key_value_heads * head_dim * (bfloat16 ? 2 : 4);
  PLUTO_ASSIGN_OR_RETURN(Buffer keys, Buffer::Allocate(executor, bytes));
  PLUTO_ASSIGN_OR_RETURN(Buffer values, Buffer::Allocate(executor, bytes));
  return std::unique_ptr<KeyValueCache>(
      new KeyValueCache(capacity, key_value_heads, head_dim, bfloat16, keys, values));
}
Status KeyValueCache::Advance() {
  if (position_ >= capacity_) return ResourceExhaustedError("key-value cache capacity reached");
  ++position_;
  return OkStatus();
}

namespace cached_attention_ops {
namespace {

pluto_kv_cache View(const KeyValueCache& cache) {
  pluto_kv_cache view{};
  view.k_base = cache.keys().data();
  view.v_base = cache.values().data();
  view.block_table = nullptr;  // one contiguous region, page 0
  view.max_blocks = 0;
  view.page_size = cache.capacity();
  view.token_stride = static_cast<size_t>(cache.key_value_heads()) * cache.head_dim();
  view.page_stride = view.token_stride * cache.capacity();
  view.dtype = cache.bfloat16() ? PLUTO_BF16 : PLUTO_FP32;
  view.num_pages = 1;
  return view;
}

}  // namespace

Status ValidateCachedAttention(cuda::Executor& executor, const FullAttentionParameters& p,
                               const KeyValueCache& cache) {
  constexpr int kIntMax = std::numeric_limits<int>::max();
  if (p.query_heads <= 0 || p.key_value_heads <= 0 || p.query_heads % p.key_value_heads != 0 ||
      p.head_dim <= 0 || p.head_dim > 256 || p.rotary_dim <= 0 || p.rotary_dim > p.head_dim ||
      p.rotary_dim % 2 != 0 || p.capacity <= 0 || p.capacity > kIntMax - 32 ||
      !std::isfinite(p.rope_theta) || p.rope_theta <= 0.0f || !std::isfinite(p.rms_norm_epsilon) ||
      p.rms_norm_epsilon <= 0.0f || p.query_heads > kIntMax / (2 * p.head_dim) ||
      p.query_heads > kIntMax - p.key_value_heads)
    return InvalidArgumentError("invalid full-attention dimensions or parameters");
  if (&cache.executor() != &executor)
    return InvalidArgumentError("attention cache belongs to a different Executor");
  if (cache.capacity() != p.capacity || cache.key_value_heads() != p.key_value_heads ||
      cache.head_dim() != p.head_dim)
    return InvalidArgumentError("attention cache shape or capacity does not match parameters");
  return OkStatus();
}

Status CachedAttentionStep(cuda::Executor& executor, const FullAttentionParameters& p,
                           KeyValueCache& cache, const float* q_gate, const float* k, const float* v,
                           const float* q_norm, const float* k_norm, float* output,
                           float* probabilities) {
  return CachedAttentionStepTyped(executor, p, cache, q_gate, k, v, PLUTO_FP32, q_norm, k_norm, output,
                                  PLUTO_FP32, probabilities);
}

Status CachedAttentionStepTyped(cuda::Executor& executor, const FullAttentionParameters& p,
                                KeyValueCache& cache, const void* q_gate, const void* k, const void* v,
                                int input_dtype, const float* q_norm, const float* k_norm, void* output,
                                int output_dtype, float* probabilities) {
  PLUTO_RETURN_IF_ERROR(ValidateCachedAttention(executor, p, cache));
  if ((input_dtype != PLUTO_FP32 && input_dtype != PLUTO_BF16) ||
      (output_dtype != PLUTO_FP32 && output_dtype != PLUTO_BF16))
    return InvalidArgumentError("attention activations must be FP32 or BF16");
  if (!q_gate || !k || !v || !q_norm || !k_norm || !output)
    return InvalidArgumentError("attention requires non-null device pointers");
  if (cache.position() >= cache.capacity())
    return ResourceExhaustedError("full-attention cache capacity reached");
  const int position = cache.position();
  const size_t ws_bytes = pluto_gqa_decode_workspace_bytes(1, p.query_heads, p.key_value_heads,
                                                           p.head_dim, position + 1);
  PLUTO_ASSIGN_OR_RETURN(Buffer queries, Buffer::Allocate(executor, static_cast<size_t>(p.query_heads) * p.head_dim * sizeof(float)));
  PLUTO_ASSIGN_OR_RETURN(Buffer counters, Buffer::Allocate(executor, 2 * sizeof(int32_t)));
  PLUTO_ASSIGN_OR_RETURN(Buffer workspace, Buffer::Allocate(executor, ws_bytes));
  // position and length travel as two device words written in stream order (no host wait)
  const int32_t host_counters[2] = {position, position + 1};
  PLUTO_RETURN_IF_ERROR(cuda::CudaStatus(
      cudaMemcpyAsync(counters.data(), host_counters, sizeof(host_counters), cudaMemcpyHostToDevice,
                      executor.stream()),
      "upload cache position"));
  const auto* device_counters = static_cast<const int32_t*>(counters.data());
  const pluto_kv_cache view = View(cache);
  const size_t token = 2 * static_cast<size_t>(p.query_heads) * p.head_dim, head = 2 * static_cast<size_t>(p.head_dim);
  PLUTO_RETURN_IF_ERROR(FromEngine(
      pluto_qk_prepare(executor.stream(), q_gate, k, v, input_dtype, token, head, q_norm, k_norm,
                       device_counters, queries.data(), PLUTO_FP32, &view, 1, 1, p.query_heads,
                       p.key_value_heads, p.head_dim, p.rotary_dim, p.rms_norm_epsilon,
                       p.rope_theta, p.round_to_bfloat16),
      "prepare Qwen attention"));
  PLUTO_RETURN_IF_ERROR(FromEngine(
      pluto_gqa_decode(executor.stream(), queries.data(), PLUTO_FP32,
                       static_cast<const char*>(q_gate) +
                           static_cast<size_t>(p.head_dim) * (input_dtype == PLUTO_BF16 ? 2 : 4),
                       input_dtype, token, head, &view, device_counters + 1, position + 1, output,
                       output_dtype,
                       nullptr, workspace.data(), ws_bytes, 1, p.query_heads, p.key_value_heads,
                       p.head_dim, p.round_to_bfloat16),
      "Qwen full attention"));
  if (probabilities)
    PLUTO_RETURN_IF_ERROR(FromEngine(
        pluto_gqa_decode_probs(executor.stream(), queries.data(), PLUTO_FP32, &view,
                               device_counters + 1, probabilities, 0, position + 1, 1,
                               p.query_heads, p.key_value_heads, p.head_dim),
        "inspect cached attention probabilities"));
  return cache.Advance();
}

StatusOr<std::unique_ptr<DeltaNetState>> DeltaNetState::Create(cuda::Executor& executor,
                                                              DeltaNetParameters p) {
  if (p.key_heads <= 0 || p.value_heads <= 0 || p.value_heads % p.key_heads != 0 ||
      p.key_head_dim <= 0 || p.key_head_dim > 128 || p.value_head_dim <= 0 ||
      p.value_head_dim > 256 || p.conv_kernel_dim <= 0 || p.conv_kernel_dim > 32 ||
      !std::isfinite(p.rms_norm_epsilon) || p.rms_norm_epsilon <= 0.0f)
    return InvalidArgumentError("invalid DeltaNet dimensions or parameters");
  const size_t channels = 2 * static_cast<size_t>(p.key_heads) * p.key_head_dim +
                          static_cast<size_t>(p.value_heads) * p.value_head_dim;
  if (channels > static_cast<size_t>(std::numeric_limits<int>::max()) / p.conv_kernel_dim)
    return ResourceExhaustedError("DeltaNet dimensions exceed indexing limit");
  PLUTO_ASSIGN_OR_RETURN(Buffer conv, Buffer::Allocate(executor, channels * p.conv_kernel_dim * sizeof(float)));
  PLUTO_ASSIGN_OR_RETURN(Buffer recurrent, Buffer::Allocate(executor, static_cast<size_t>(p.value_heads) * p.key_head_dim * p.value_head_dim * sizeof(float)));
  PLUTO_ASSIGN_OR_RETURN(Buffer convolved, Buffer::Allocate(executor, channels * sizeof(float)));
  PLUTO_ASSIGN_OR_RETURN(Buffer core, Buffer::Allocate(executor, static_cast<size_t>(p.value_heads) * p.value_head_dim * sizeof(float)));
  PLUTO_ASSIGN_OR_RETURN(Buffer gates, Buffer::Allocate(executor, 2 * static_cast<size_t>(p.value_heads) * sizeof(float)));
  std::unique_ptr<DeltaNetState> state(
      new DeltaNetState(executor, p, conv, recurrent, convolved, core, gates));
  PLUTO_RETURN_IF_ERROR(state->Reset());
  return state;
}

Status DeltaNetState::Step(const float* qkv, const float* z, const float* a, const float* b,
                           const float* conv_weight, const float* a_log, const float* dt_bias,
                           const float* norm_weight, float* output) {
  return StepTyped(qkv, z, a, b, PLUTO_FP32, conv_weight, a_log, dt_bias, norm_weight, output, PLUTO_FP32);
}

Status DeltaNetState::StepTyped(const void* qkv, const void* z, const void* a, const void* b,
                                int input_dtype, const float* conv_weight, const float* a_log,
                                const float* dt_bias, const float* norm_weight, void* output,
                                int output_dtype) {
  if ((input_dtype != PLUTO_FP32 && input_dtype != PLUTO_BF16) ||
      (output_dtype != PLUTO_FP32 && output_dtype != PLUTO_BF16))
    return InvalidArgumentError("DeltaNet activations must be FP32 or BF16");
  if (!qkv || !z || !a || !b || !conv_weight || !a_log || !dt_bias || !norm_weight || !output)
    return InvalidArgumentError("DeltaNet requires non-null device pointers");
  const auto& p = parameters_;
  const int channels = 2 * p.key_heads * p.key_head_dim + p.value_heads * p.value_head_dim;
  const int kq = p.key_heads * p.key_head_dim;
  auto* convolved = static_cast<float*>(convolved_qkv_.data());
  auto* g = static_cast<float*>(gates_.data());
  float* beta = g + p.value_heads;
  cudaStream_t stream = executor_.stream();
  PLUTO_RETURN_IF_ERROR(FromEngine(
      pluto_gdn_conv_silu(stream, qkv, conv_weight, input_dtype, 1, 1, channels, p.conv_kernel_dim,
                          p.round_to_bfloat16, static_cast<float*>(convolution_state_.data()),
                          convolved, PLUTO_FP32),
      "Qwen causal convolution"));
  PLUTO_RETURN_IF_ERROR(FromEngine(
      pluto_gdn_gates(stream, a, b, a_log, dt_bias, input_dtype, 1, p.value_heads,
                      p.round_to_bfloat16, g, beta),
      "Qwen gated delta gates"));
  PLUTO_RETURN_IF_ERROR(FromEngine(
      pluto_gdn_step(stream, convolved, convolved + kq, convolved + 2 * kq, PLUTO_FP32, g, beta,
                     static_cast<float*>(recurrent_state_.data()), core_output_.data(), PLUTO_FP32,
                     1, p.key_heads, p.value_heads, p.key_head_dim, p.value_head_dim, 1, 1.0f,
                     p.round_to_bfloat16),
      "Qwen gated delta recurrence"));
  return FromEngine(
      pluto_gdn_out_norm_gate(stream, core_output_.data(), PLUTO_FP32, z, input_dtype, norm_weight,
                              p.value_heads, p.value_head_dim, p.rms_norm_epsilon,
                              p.round_to_bfloat16, 1, output, output_dtype),
      "Qwen gated delta output norm");
}

Status DeltaNetState::Reset() {
  PLUTO_RETURN_IF_ERROR(cuda::CudaStatus(
      cudaMemsetAsync(convolution_state_.data(), 0, convolution_state_.size_bytes(), executor_.stream()),
      "reset Qwen convolution state"));
  return cuda::CudaStatus(
      cudaMemsetAsync(recurrent_state_.data(), 0, recurrent_state_.size_bytes(), executor_.stream()),
      "reset Qwen recurrent state");
}

}  // namespace cached_attention_ops
}  // namespace llm
}  // namespace pluto
