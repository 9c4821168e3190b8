// extern "C" entry points declared in include/pluto_b200.h: argument validation (the same checks,
// in the same order, as the reference layers make before queuing GPU work) and dispatch to the
// kernel files.  No allocation, no synchronisation, no mutable global state beyond the per-thread
// error text and the per-device status-word address cache.
#include <math.h>
#include <stdio.h>

#include <limits>
#include <mutex>

#include "../../include/pluto_b200.h"
#include "engine.h"

namespace {

thread_local char g_error[256] = "";

int fail(int code, const char* message) {
  snprintf(g_error, sizeof(g_error), "%s", message);
  return code;
}
int from_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return PLUTO_OK;
  snprintf(g_error, sizeof(g_error), "%s: %s", what, cudaGetErrorString(e));
  return static_cast<int>(e);
}
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
}  // namespace

// the same two helpers for entry points defined in other files
namespace pluto {
int report(int code, const char* message) { return fail(code, message); }
int report_cuda(cudaError_t e, const char* what) { return from_cuda(e, what); }
}  // namespace pluto

namespace {

// AttentionLayer::Create's checks (src/llm/layers/attention.cc:400-416) plus the extents the
// kernels index with.
int check_mha(int batch, int seq, int heads, int head_dim, int dtype) {
  if (dtype != PLUTO_FP32 && dtype != PLUTO_BF16)
    return fail(PLUTO_E_UNIMPLEMENTED, "attention supports only the FP16 (fp32 storage) and BF16 policies");
  if (batch <= 0 || seq <= 0 || heads <= 0 || head_dim <= 0)
    return fail(PLUTO_E_INVALID, "attention dimensions must all be positive");
  if (head_dim > 256) return fail(PLUTO_E_UNIMPLEMENTED, "attention head width above 256");
  if (batch > 65535 || heads > 65535)
    return fail(PLUTO_E_EXHAUSTED, "attention batch or head count exceeds CUDA's grid limits");
  const long long rows = static_cast<long long>(batch) * seq;
  if (rows * 3 * heads * head_dim > static_cast<long long>(std::numeric_limits<int>::max()) * 8LL)
    return fail(PLUTO_E_EXHAUSTED, "attention activation exceeds the indexing limit");
  return PLUTO_OK;
}

bool tensor_core_shape(int head_dim, int dtype) {
  return dtype == PLUTO_BF16 && (head_dim == 64 || head_dim == 128);
}

}  // namespace

extern "C" {

const char* pluto_last_error(void) { return g_error; }
const char* pluto_build_info(void) { return "pluto_b200 0.1 (sm_100a)"; }

int pluto_kernel_status(uint32_t* value, int clear) {
  if (!value) return fail(PLUTO_E_INVALID, "pluto_kernel_status requires a host pointer");
  return from_cuda(pluto::read_kernel_status(value, clear != 0), "read kernel status");
}

int pluto_attn_fwd(pluto_stream_t stream, const void* qkv, void* out, float* maxima,
                   float* normalizers, int batch, int seq, int heads, int head_dim, int dtype) {
  if (int c = check_mha(batch, seq, heads, head_dim, dtype)) return c;
  if (!qkv || !out || !maxima || !normalizers)
    return fail(PLUTO_E_INVALID, "attention forward requires non-null device pointers");
  const size_t E = static_cast<size_t>(heads) * head_dim;
  if (tensor_core_shape(head_dim, dtype) && aligned16(qkv) && aligned16(out)) {
    pluto::AttnFwdArgs a{};
    a.q = a.k = a.v = qkv;
    a.q_cols = a.kv_cols = static_cast<int>(3 * E);
    a.q_token = a.kv_token = 3 * E;
    a.q_col0 = 0;
    a.k_col0 = static_cast<int>(E);
    a.v_col0 = static_cast<int>(2 * E);
    a.q_head_cols = head_dim;
    a.batch = batch; a.seq = seq; a.heads = heads; a.group = 1; a.head_dim = head_dim;
    a.out = out; a.out_token = E; a.out_head = head_dim;
    a.maxima = maxima; a.normalizers = normalizers;
    a.status = pluto::kernel_status_word();
    if (!a.status) return fail(PLUTO_E_INTERNAL, "kernel status word unavailable");
    return from_cuda(pluto::attn_fwd_tc(stream, a), "attention forward (tcgen05) launch");
  }
  const char* base = static_cast<const char*>(qkv);
  const size_t es = dtype == PLUTO_BF16 ? 2 : 4;
  return from_cuda(
      pluto::attn_generic_fwd(stream, base, base + E * es, base + 2 * E * es, out, maxima,
                              normalizers, batch, seq, heads, head_dim, 3 * E, head_dim, 3 * E,
                              head_dim, E, head_dim, 1, nullptr, 0, 0, nullptr, 0,
                              dtype == PLUTO_BF16),
      "attention forward launch");
}

int pluto_attn_bwd(pluto_stream_t stream, const void* qkv, const void* out, const float* d_out,
                   const float* maxima, const float* normalizers, float* d_qkv, float* deltas,
                   int batch, int seq, int heads, int head_dim, int dtype, void* workspace,
                   size_t workspace_bytes) {
  if (int c = check_mha(batch, seq, heads, head_dim, dtype)) return c;
  if (!qkv) return fail(PLUTO_E_INVALID, "attention backward requires the saved Q/K/V");
  if (!out) return fail(PLUTO_E_INVALID, "attention backward requires the saved output");
  if (!maxima) return fail(PLUTO_E_INVALID, "attention backward requires the saved maxima");
  if (!normalizers) return fail(PLUTO_E_INVALID, "attention backward requires the saved normalizers");
  if (!d_out || !d_qkv || !deltas)
    return fail(PLUTO_E_INVALID, "attention backward requires non-null gradient pointers");
  if (workspace != nullptr) {
    const size_t need = pluto_attn_bwd_workspace_bytes(batch, seq, heads, head_dim, dtype);
    if (need == 0)
      return fail(PLUTO_E_INVALID, "attention backward has no tensor-core path for this shape; pass a null workspace");
    if (workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0 ||
        !aligned16(qkv) || !aligned16(d_qkv) || !aligned16(out) || !aligned16(d_out))
      return fail(PLUTO_E_INVALID, "attention backward workspace is too small or a tensor is misaligned");
    uint32_t* status = pluto::kernel_status_word();
    if (!status) return fail(PLUTO_E_INTERNAL, "kernel status word unavailable");
    return from_cuda(pluto::attn_bwd_tc(stream, qkv, out, d_out, maxima, normalizers, d_qkv, deltas,
                                        workspace, batch, seq, heads, head_dim, status),
                     "attention backward (tcgen05) launch");
  }
  return from_cuda(pluto::attn_generic_bwd(stream, qkv, out, d_out, maxima, normalizers, d_qkv,
                                           deltas, batch, seq, heads, head_dim,
                                           dtype == PLUTO_BF16),
                   "attention backward launch");
}

size_t pluto_attn_bwd_workspace_bytes(int batch, int seq, int heads, int head_dim, int dtype) {
  if (batch <= 0 || seq <= 0 || heads <= 0 || !tensor_core_shape(head_dim, dtype)) return 0;
  return pluto::attn_bwd_tc_workspace_bytes(batch, seq, heads, head_dim);
}

int pluto_attn_probs(pluto_stream_t stream, const void* qkv, const float* maxima,
                     const float* normalizers, float* probs, int batch, int seq, int heads,
                     int head_dim, int dtype) {
  if (int c = check_mha(batch, seq, heads, head_dim, dtype)) return c;
  if (!qkv || !maxima || !normalizers || !probs)
    return fail(PLUTO_E_INVALID, "attention probabilities require non-null device pointers");
  // src/llm/layers/attention.cc:39-50: the quadratic tensor's byte size must be representable.
  size_t bytes = static_cast<size_t>(batch) * seq;
  for (size_t factor : {static_cast<size_t>(heads), static_cast<size_t>(seq), sizeof(float)}) {
    if (bytes > std::numeric_limits<size_t>::max() / factor)
      return fail(PLUTO_E_EXHAUSTED, "attention probabilities tensor byte size overflows size_t");
    bytes *= factor;
  }
  return from_cuda(pluto::attn_generic_probs(stream, qkv, maxima, normalizers, probs, batch, seq,
                                             heads, head_dim, dtype == PLUTO_BF16),
                   "attention probabilities launch");
}

int pluto_gqa_prefill_fwd(pluto_stream_t stream, const void* q, const void* gate, const void* k,
                          const void* v, void* out, float* core, float* maxima,
                          float* normalizers, int batch, int seq, int q_heads, int kv_heads,
                          int head_dim, size_t q_token_stride, size_t q_head_stride,
                          size_t gate_token_stride, size_t gate_head_stride, int round_to_bf16,
                          void* workspace, size_t workspace_bytes) {
  if (batch <= 0 || seq <= 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 ||
      q_heads % kv_heads != 0 || head_dim > 256 || batch > 65535 || q_heads > 65535)
    return fail(PLUTO_E_INVALID, "invalid full-attention dimensions or parameters");
  if (!q || !k || !v || !out)
    return fail(PLUTO_E_INVALID, "attention requires non-null device pointers");
  if ((maxima == nullptr) != (normalizers == nullptr))
    return fail(PLUTO_E_INVALID, "attention statistics must be requested together");
  if (q_head_stride < static_cast<size_t>(head_dim) ||
      q_token_stride < (static_cast<size_t>(q_heads) - 1) * q_head_stride + head_dim)
    return fail(PLUTO_E_INVALID, "attention query strides overlap");
  const int group = q_heads / kv_heads;
  const size_t kv_token = static_cast<size_t>(kv_heads) * head_dim;
  const size_t out_token = static_cast<size_t>(q_heads) * head_dim;
  const bool tma_ok = aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out) &&
                      q_token_stride % 8 == 0 && q_head_stride % 8 == 0 &&
                      q_token_stride <= 0x7fffffffu;
  if ((head_dim == 64 || head_dim == 128) && tma_ok) {
    pluto::AttnFwdArgs a{};
    a.q = q; a.k = k; a.v = v;
    a.q_cols = static_cast<int>((static_cast<size_t>(q_heads) - 1) * q_head_stride + head_dim);
    a.kv_cols = static_cast<int>(kv_token);
    a.q_token = q_token_stride; a.kv_token = kv_token;
    a.q_col0 = a.k_col0 = a.v_col0 = 0;
    a.q_head_cols = static_cast<int>(q_head_stride);
    a.batch = batch; a.seq = seq; a.heads = q_heads; a.group = group; a.head_dim = head_dim;
    a.out = out; a.out_token = out_token; a.out_head = head_dim;
    a.maxima = maxima; a.normalizers = normalizers; a.core = core;
    a.gate = gate; a.gate_token = gate_token_stride; a.gate_head = gate_head_stride;
    a.round_gate = round_to_bf16;
    // the optional workspace enables the key/value split for shapes with few (sequence, head) units
    if (workspace != nullptr && aligned16(workspace) &&
        workspace_bytes >= pluto::attn_fwd_tc_workspace_bytes(batch, seq, q_heads, head_dim))
      a.workspace = workspace;
    a.status = pluto::kernel_status_word();
    if (!a.status) return fail(PLUTO_E_INTERNAL, "kernel status word unavailable");
    return from_cuda(pluto::attn_fwd_tc(stream, a), "GQA prefill (tcgen05) launch");
  }
  return from_cuda(
      pluto::attn_generic_fwd(stream, q, k, v, out, maxima, normalizers, batch, seq, q_heads,
                              head_dim, q_token_stride, q_head_stride, kv_token, head_dim,
                              out_token, head_dim, group, gate, gate_token_stride, gate_head_stride,
                              core, round_to_bf16, true),
      "GQA prefill launch");
}

int pluto_gqa_gate_bwd(pluto_stream_t stream, const void* gate, size_t gate_token_stride,
                       size_t gate_head_stride, const float* core, const float* dy, float* dc,
                       float* d_gate, size_t d_gate_token_stride, size_t d_gate_head_stride,
                       float* deltas, int batch, int seq, int q_heads, int head_dim,
                       int round_to_bf16) {
  if (batch <= 0 || seq <= 0 || q_heads <= 0 || head_dim <= 0 || head_dim > 256 ||
      static_cast<long long>(batch) * seq * q_heads > 0x7fffffffLL)
    return fail(PLUTO_E_INVALID, "invalid full-attention dimensions or parameters");
  if (!gate || !core || !dy || !dc || !d_gate || !deltas)
    return fail(PLUTO_E_INVALID, "attention requires non-null device pointers");
  pluto::GateBwdArgs a{};
  a.gate = static_cast<const __nv_bfloat16*>(gate);
  a.gate_token = gate_token_stride; a.gate_head = gate_head_stride;
  a.core = core; a.dy = dy; a.dc = dc; a.d_gate = d_gate;
  a.dgate_token = d_gate_token_stride; a.dgate_head = d_gate_head_stride;
  a.deltas = deltas;
  a.batch = batch; a.seq = seq; a.q_heads = q_heads; a.head_dim = head_dim;
  a.round = round_to_bf16;
  return from_cuda(pluto::gqa_gate_bwd(stream, a), "sequence full attention backward (gate)");
}

int pluto_gqa_prefill_bwd(pluto_stream_t stream, const void* q, const void* k, const void* v,
                          int dtype, size_t q_token_stride, size_t q_head_stride, const float* dc,
                          const float* maxima, const float* normalizers, const float* deltas,
                          float* dq, float* dk, float* dv, void* workspace, size_t workspace_bytes,
                          int batch, int seq, int q_heads, int kv_heads, int head_dim) {
  if (batch <= 0 || seq <= 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 ||
      q_heads % kv_heads != 0 || head_dim > 256 || batch > 65535 || q_heads > 65535)
    return fail(PLUTO_E_INVALID, "invalid full-attention dimensions or parameters");
  if (dtype != PLUTO_FP32 && dtype != PLUTO_BF16)
    return fail(PLUTO_E_INVALID, "attention tensors have an unknown dtype");
  if (!q || !k || !v || !dc || !dq || !dk || !dv)
    return fail(PLUTO_E_INVALID, "attention requires non-null device pointers");
  if (!maxima) return fail(PLUTO_E_INVALID, "attention backward requires saved maxima");
  if (!normalizers) return fail(PLUTO_E_INVALID, "attention backward requires saved normalizers");
  if (!deltas) return fail(PLUTO_E_INVALID, "attention backward requires the gate pass deltas");
  if (q_head_stride < static_cast<size_t>(head_dim) ||
      q_token_stride < (static_cast<size_t>(q_heads) - 1) * q_head_stride + head_dim)
    return fail(PLUTO_E_INVALID, "attention query strides overlap");
  const size_t D = head_dim, qd = static_cast<size_t>(q_heads) * D, kd = static_cast<size_t>(kv_heads) * D;
  // bf16 tensors of head width 64/128 with a dense query run on tcgen05 when a workspace is given
  if (workspace != nullptr && tensor_core_shape(head_dim, dtype) && q_head_stride == D &&
      q_token_stride % 8 == 0 && q_token_stride <= 0x7fffffffu && aligned16(q) && aligned16(k) &&
      aligned16(v) && aligned16(dc) && aligned16(workspace)) {
    if (workspace_bytes < pluto::attn_bwd_tc_workspace_bytes(batch, seq, q_heads, head_dim))
      return fail(PLUTO_E_INVALID, "attention backward workspace is too small");
    pluto::GqaBwdTcArgs t{};
    t.q = q; t.k = k; t.v = v; t.out = nullptr;
    t.q_cols = static_cast<int>(qd); t.kv_cols = static_cast<int>(kd);
    t.q_col0 = t.k_col0 = t.v_col0 = 0;
    t.q_token = q_token_stride; t.kv_token = kd;
    t.d_out = dc; t.maxima = maxima; t.normalizers = normalizers;
    t.deltas = const_cast<float*>(deltas);   // only read when out is null
    t.dq = dq; t.dk = dk; t.dv = dv; t.dq_token = qd; t.dkv_token = kd;
    t.workspace = workspace;
    t.batch = batch; t.seq = seq; t.q_heads = q_heads; t.kv_heads = kv_heads; t.head_dim = head_dim;
    t.status = pluto::kernel_status_word();
    if (!t.status) return fail(PLUTO_E_INTERNAL, "kernel status word unavailable");
    return from_cuda(pluto::gqa_bwd_tc(stream, t), "sequence full attention backward (tcgen05)");
  }
  pluto::GqaBwdArgs a{};
  a.q = q; a.k = k; a.v = v; a.out = nullptr;
  a.d_out = dc; a.maxima = maxima; a.normalizers = normalizers;
  a.deltas = const_cast<float*>(deltas);   // only read when out is null
  a.dq = dq; a.dk = dk; a.dv = dv;
  a.batch = batch; a.seq = seq; a.q_heads = q_heads; a.kv_heads = kv_heads; a.head_dim = head_dim;
  a.q_token = q_token_stride; a.q_head = q_head_stride;
  a.kv_token = kd; a.kv_head = D;
  a.o_token = qd; a.o_head = D; a.g_token = qd; a.g_head = D;
  a.dq_token = qd; a.dq_head = D; a.dkv_token = kd; a.dkv_head = D;
  a.bf16 = dtype == PLUTO_BF16;
  return from_cuda(pluto::gqa_generic_bwd(stream, a), "sequence full attention backward");
}

size_t pluto_gqa_prefill_fwd_workspace_bytes(int batch, int seq, int q_heads, int head_dim) {
  if (batch <= 0 || seq <= 0 || q_heads <= 0 || (head_dim != 64 && head_dim != 128)) return 0;
  return pluto::attn_fwd_tc_split_workspace_bytes(batch, seq, q_heads, head_dim);
}

size_t pluto_gqa_prefill_bwd_workspace_bytes(int batch, int seq, int q_heads, int head_dim, int dtype) {
  if (batch <= 0 || seq <= 0 || q_heads <= 0 || !tensor_core_shape(head_dim, dtype)) return 0;
  return pluto::attn_bwd_tc_workspace_bytes(batch, seq, q_heads, head_dim);
}

size_t pluto_qk_prepare_bwd_workspace_bytes(int batch, int tokens, int heads, int head_dim) {
  if (batch <= 0 || tokens <= 0 || heads <= 0 || head_dim <= 0) return 0;
  return pluto::qk_prepare_bwd_workspace_bytes(static_cast<long long>(batch) * tokens * heads, head_dim);
}

int pluto_qk_prepare_bwd(pluto_stream_t stream, const void* x, size_t x_token_stride,
                         size_t x_head_stride, const float* weight, const float* grad,
                         const int32_t* positions, float* dx, size_t dx_token_stride,
                         size_t dx_head_stride, float* d_weight, void* workspace,
                         size_t workspace_bytes, int batch, int tokens, int heads, int head_dim,
                         int rotary_dim, float rms_norm_epsilon, float rope_theta,
                         int round_to_bf16) {
  if (batch <= 0 || tokens <= 0 || heads <= 0 || head_dim <= 0 || head_dim > 256 ||
      rotary_dim <= 0 || rotary_dim > head_dim || rotary_dim % 2 != 0 ||
      !(rms_norm_epsilon > 0.0f) || !std::isfinite(rms_norm_epsilon) || !(rope_theta > 0.0f) ||
      !std::isfinite(rope_theta) ||
      static_cast<long long>(batch) * tokens * heads > 0x7fffffffLL)
    return fail(PLUTO_E_INVALID, "invalid full-attention dimensions or parameters");
  if (!x || !weight || !grad || !dx)
    return fail(PLUTO_E_INVALID, "attention requires non-null device pointers");
  if (d_weight != nullptr &&
      (workspace == nullptr ||
       workspace_bytes < pluto_qk_prepare_bwd_workspace_bytes(batch, tokens, heads, head_dim)))
    return fail(PLUTO_E_INVALID, "norm-weight gradient requires its workspace");
  pluto::NormBwdArgs a{};
  a.x = static_cast<const __nv_bfloat16*>(x);
  a.x_token = x_token_stride; a.x_head = x_head_stride;
  a.weight = weight; a.grad = grad; a.positions = positions;
  a.dx = dx; a.dx_token = dx_token_stride; a.dx_head = dx_head_stride;
  a.batch = batch; a.tokens = tokens; a.heads = heads; a.head_dim = head_dim; a.rotary = rotary_dim;
  a.epsilon = rms_norm_epsilon; a.log_theta = logf(rope_theta);
  a.round = round_to_bf16;
  return from_cuda(pluto::qk_prepare_bwd(stream, a, d_weight, workspace),
                   "sequence full attention backward (norm)");
}

}  // extern "C"

namespace {

bool dtype_ok(int d) { return d == PLUTO_FP32 || d == PLUTO_BF16; }

int check_cache(const pluto_kv_cache* cache, int kv_heads, int head_dim) {
  const bool separate = cache && (cache->k_bases || cache->v_bases);
  if (!cache || (separate ? (!cache->k_bases || !cache->v_bases || cache->block_table)
                          : (!cache->k_base || !cache->v_base)))
    return fail(PLUTO_E_INVALID, "attention requires non-null device pointers");
  if (!dtype_ok(cache->dtype)) return fail(PLUTO_E_INVALID, "attention cache has an unknown dtype");
  if (cache->page_size <= 0 || (cache->block_table && cache->max_blocks <= 0) ||
      cache->token_stride < static_cast<size_t>(kv_heads) * head_dim ||
      (!separate && cache->page_stride < cache->token_stride))
    return fail(PLUTO_E_INVALID, "attention cache shape or capacity does not match parameters");
  return PLUTO_OK;
}

// Chunk length of the split-KV decode: the largest of {2048,...,256} tokens that still yields
// at least 8 work items per SM, so ragged lengths balance across the 148 SMs.  (16 per SM halved
// the chunks of a one-KV-head shard at batch 64 for nothing: 140 against 132 us.)
int decode_split_tokens(int batch, int kv_heads, int max_seq_len) {
  for (int s : {2048, 1024, 512}) {
    const long long items = static_cast<long long>(batch) * kv_heads * ((max_seq_len + s - 1) / s);
    if (items >= 148 * 8) return s;
  }
  return 256;
}

int fill_decode(pluto::DecodeArgs* a, const void* q, int q_dtype, const pluto_kv_cache* cache,
                const int32_t* seq_lens, int max_seq_len, int batch, int q_heads, int kv_heads,
                int head_dim) {
  if (batch <= 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0 || head_dim <= 0 ||
      head_dim > 256 || max_seq_len <= 0 || batch > 65535 || q_heads > 65535 || !dtype_ok(q_dtype))
    return fail(PLUTO_E_INVALID, "invalid full-attention dimensions or parameters");
  if (int c = check_cache(cache, kv_heads, head_dim)) return c;
  if (!q || !seq_lens) return fail(PLUTO_E_INVALID, "attention requires non-null device pointers");
  *a = pluto::DecodeArgs{};
  a->q = q;
  a->q_is_bf16 = q_dtype == PLUTO_BF16;
  a->k_base = cache->k_base;
  a->v_base = cache->v_base;
  a->k_bases = cache->k_bases;
  a->v_bases = cache->v_bases;
  a->kv_is_bf16 = cache->dtype == PLUTO_BF16;
  a->block_table = cache->block_table;
  a->max_blocks = cache->max_blocks;
  a->page_size = cache->page_size;
  a->page_stride = cache->page_stride;
  a->token_stride = cache->token_stride;
  a->num_pages = cache->num_pages;
  a->seq_lens = seq_lens;
  a->batch = batch; a->q_heads = q_heads; a->kv_heads = kv_heads; a->head_dim = head_dim;
  a->split_tokens = decode_split_tokens(batch, kv_heads, max_seq_len);
  a->splits = pluto::decode_chunk_count(max_seq_len, a->split_tokens);
  if (a->splits > 65535) return fail(PLUTO_E_INVALID, "max_seq_len exceeds what one decode launch can split");
  a->scale = 1.0f / sqrtf(static_cast<float>(head_dim));
  a->status = pluto::kernel_status_word();
  if (!a->status) return fail(PLUTO_E_INTERNAL, "kernel status word unavailable");
  return PLUTO_OK;
}

int check_gdn(int batch, int tokens, int key_heads, int value_heads, int key_dim, int value_dim) {
  // DeltaNetState::Create, src/llm/layers/util/cached_attention_ops.cc:370-376
  if (batch <= 0 || tokens <= 0 || key_heads <= 0 || value_heads <= 0 ||
      value_heads % key_heads != 0 || key_dim <= 0 || key_dim > 128 || value_dim <= 0 ||
      value_dim > 256 || batch > 65535 || value_heads > 65535)
    return fail(PLUTO_E_INVALID, "invalid DeltaNet dimensions or parameters");
  return PLUTO_OK;
}

}  // namespace

extern "C" {

int pluto_qk_prepare(pluto_stream_t stream, const void* q_in, const void* k_in, const void* v_in,
                     int in_dtype, size_t q_token_stride, size_t q_head_stride,
                     const float* q_norm, const float* k_norm, const int32_t* positions,
                     void* q_out, int q_out_dtype, const pluto_kv_cache* cache, int batch,
                     int tokens, int q_heads, int kv_heads, int head_dim, int rotary_dim,
                     float rms_norm_epsilon, float rope_theta, int round_to_bf16) {
  // ValidateCachedAttention, src/llm/layers/util/cached_attention_ops.cc:283-306
  if (batch <= 0 || tokens <= 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0 ||
      head_dim <= 0 || head_dim > 256 || rotary_dim <= 0 || rotary_dim > head_dim ||
      rotary_dim % 2 != 0 || !isfinite(rope_theta) || rope_theta <= 0.0f ||
      !isfinite(rms_norm_epsilon) || rms_norm_epsilon <= 0.0f || !dtype_ok(in_dtype) ||
      !dtype_ok(q_out_dtype) ||
      static_cast<long long>(batch) * tokens * (q_heads + kv_heads) > 0x7fffffffLL)
    return fail(PLUTO_E_INVALID, "invalid full-attention dimensions or parameters");
  if (int c = check_cache(cache, kv_heads, head_dim)) return c;
  if (!q_in || !k_in || !v_in || !q_norm || !k_norm || !q_out)
    return fail(PLUTO_E_INVALID, "attention requires non-null device pointers");
  pluto::PrepareArgs a{};
  a.q_in = q_in; a.k_in = k_in; a.v_in = v_in; a.in_is_bf16 = in_dtype == PLUTO_BF16;
  a.q_token = q_token_stride; a.q_head = q_head_stride;
  a.q_norm = q_norm; a.k_norm = k_norm; a.positions = positions;
  a.q_out = q_out; a.q_out_is_bf16 = q_out_dtype == PLUTO_BF16;
  a.k_cache = cache->k_base; a.v_cache = cache->v_base; a.kv_is_bf16 = cache->dtype == PLUTO_BF16;
  a.k_bases = cache->k_bases; a.v_bases = cache->v_bases;
  a.block_table = cache->block_table; a.max_blocks = cache->max_blocks;
  a.page_size = cache->page_size; a.page_stride = cache->page_stride;
  a.token_stride = cache->token_stride;
  a.batch = batch; a.tokens = tokens; a.q_heads = q_heads; a.kv_heads = kv_heads;
  a.head_dim = head_dim; a.rotary = rotary_dim;
  a.epsilon = rms_norm_epsilon; a.log_theta = logf(rope_theta); a.round = round_to_bf16;
  return from_cuda(pluto::qk_prepare(stream, a), "prepare Qwen attention");
}

size_t pluto_gqa_decode_workspace_bytes(int batch, int q_heads, int kv_heads, int head_dim,
                                        int max_seq_len) {
  if (batch <= 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 || max_seq_len <= 0) return 0;
  const int s = decode_split_tokens(batch, kv_heads, max_seq_len);
  const size_t splits = static_cast<size_t>(pluto::decode_chunk_count(max_seq_len, s));
  return static_cast<size_t>(batch) * q_heads * splits * (head_dim + 2) * sizeof(float);
}

int pluto_gqa_decode(pluto_stream_t stream, const void* q, int q_dtype, const void* gate,
                     int gate_dtype, size_t gate_token_stride, size_t gate_head_stride,
                     const pluto_kv_cache* cache, const int32_t* seq_lens, int max_seq_len,
                     void* out, int out_dtype, float* lse, void* workspace, size_t workspace_bytes,
                     int batch, int q_heads, int kv_heads, int head_dim, int round_to_bf16) {
  pluto::DecodeArgs a;
  if (int c = fill_decode(&a, q, q_dtype, cache, seq_lens, max_seq_len, batch, q_heads, kv_heads,
                          head_dim))
    return c;
  if (!out || !workspace || !dtype_ok(out_dtype) || (gate && !dtype_ok(gate_dtype)))
    return fail(PLUTO_E_INVALID, "attention requires non-null device pointers");
  if (workspace_bytes <
          pluto_gqa_decode_workspace_bytes(batch, q_heads, kv_heads, head_dim, max_seq_len) ||
      !aligned16(workspace))
    return fail(PLUTO_E_INVALID, "attention decode workspace is too small or misaligned");
  a.gate = gate; a.gate_is_bf16 = gate_dtype == PLUTO_BF16;
  a.gate_token = gate_token_stride; a.gate_head = gate_head_stride;
  a.out = out; a.out_is_bf16 = out_dtype == PLUTO_BF16; a.lse = lse;
  a.round = round_to_bf16;
  // (max, sum) pairs first: the merge reads them as 8-byte pairs, and the workspace start is the
  // only address here whose alignment does not depend on head_dim (odd widths are legal).
  a.partial_ml = static_cast<float*>(workspace);
  a.partial_acc = a.partial_ml + pluto::decode_ml_floats(batch, q_heads, a.splits);
  return from_cuda(pluto::gqa_decode(stream, a), "Qwen full attention");
}

int pluto_gqa_decode_probs(pluto_stream_t stream, const void* q, int q_dtype,
                           const pluto_kv_cache* cache, const int32_t* seq_lens, float* probs,
                           size_t probs_batch_stride, size_t probs_head_stride, int batch,
                           int q_heads, int kv_heads, int head_dim) {
  pluto::DecodeArgs a;
  if (int c = fill_decode(&a, q, q_dtype, cache, seq_lens, 1, batch, q_heads, kv_heads, head_dim))
    return c;
  if (!probs) return fail(PLUTO_E_INVALID, "attention requires non-null device pointers");
  return from_cuda(pluto::gqa_decode_probabilities(stream, a, probs, probs_batch_stride,
                                                   probs_head_stride),
                   "inspect cached attention probabilities");
}

int pluto_gdn_gates(pluto_stream_t stream, const void* a, const void* b, const float* a_log,
                    const float* dt_bias, int in_dtype, long long tokens, int heads,
                    int round_to_bf16, float* g, float* beta) {
  if (tokens <= 0 || heads <= 0 || !dtype_ok(in_dtype) || tokens * heads > 0x7fffffff00LL)
    return fail(PLUTO_E_INVALID, "invalid DeltaNet dimensions or parameters");
  if (!a || !b || !a_log || !dt_bias || !g || !beta)
    return fail(PLUTO_E_INVALID, "DeltaNet requires non-null device pointers");
  return from_cuda(pluto::gdn_gates(stream, a, b, a_log, dt_bias, in_dtype == PLUTO_BF16, tokens,
                                    heads, round_to_bf16, g, beta),
                   "Qwen gated delta gates");
}

int pluto_gdn_conv_silu(pluto_stream_t stream, const void* input, const float* weight,
                        int in_dtype, int batch, int tokens, int channels, int width,
                        int round_to_bf16, float* state, void* output, int out_dtype) {
  if (batch <= 0 || tokens <= 0 || channels <= 0 || width <= 0 || width > 32 ||
      !dtype_ok(in_dtype) || !dtype_ok(out_dtype))
    return fail(PLUTO_E_INVALID, "invalid DeltaNet dimensions or parameters");
  if (!input || !weight || !state || !output)
    return fail(PLUTO_E_INVALID, "DeltaNet requires non-null device pointers");
  return from_cuda(pluto::gdn_conv(stream, input, weight, in_dtype == PLUTO_BF16, batch, tokens,
                                   channels, width, round_to_bf16, state, output,
                                   out_dtype == PLUTO_BF16),
                   "Qwen causal convolution");
}

int pluto_gdn_prefill(pluto_stream_t stream, const void* q, const void* k, const void* v,
                      int in_dtype, const float* g, const float* beta, float* state, void* out,
                      int out_dtype, int batch, int tokens, int key_heads, int value_heads,
                      int key_dim, int value_dim, size_t qk_token_stride, size_t v_token_stride,
                      int normalize_qk, float q_scale, int round_to_bf16, void* workspace,
                      size_t workspace_bytes) {
  if (int c = check_gdn(batch, tokens, key_heads, value_heads, key_dim, value_dim)) return c;
  const size_t qk_dense = static_cast<size_t>(key_heads) * key_dim;
  const size_t v_dense = static_cast<size_t>(value_heads) * value_dim;
  if (qk_token_stride == 0) qk_token_stride = qk_dense;
  if (v_token_stride == 0) v_token_stride = v_dense;
  if (qk_token_stride < qk_dense || v_token_stride < v_dense)
    return fail(PLUTO_E_INVALID, "DeltaNet token strides overlap");
  if (!dtype_ok(in_dtype) || !dtype_ok(out_dtype))
    return fail(PLUTO_E_INVALID, "invalid DeltaNet dimensions or parameters");
  if (!q || !k || !v || !g || !beta || !state || !out)
    return fail(PLUTO_E_INVALID, "DeltaNet requires non-null device pointers");
  pluto::GdnArgs a{};
  a.q = q; a.k = k; a.v = v; a.in_is_bf16 = in_dtype == PLUTO_BF16;
  a.qk_token = qk_token_stride; a.v_token = v_token_stride;
  a.g = g; a.beta = beta; a.state = state; a.out = out; a.out_is_bf16 = out_dtype == PLUTO_BF16;
  a.batch = batch; a.tokens = tokens; a.key_heads = key_heads; a.value_heads = value_heads;
  a.key_dim = key_dim; a.value_dim = value_dim;
  a.normalize_qk = normalize_qk; a.q_scale = q_scale; a.round = round_to_bf16;
  if (workspace != nullptr) {
    if (!pluto::gdn_chunked_supported(a))
      return fail(PLUTO_E_INVALID, "DeltaNet shape has no chunked prefill path; pass a null workspace");
    if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0 ||
        workspace_bytes < pluto::gdn_chunked_workspace_bytes(batch, tokens, value_heads, value_dim))
      return fail(PLUTO_E_INVALID, "DeltaNet prefill workspace is too small or misaligned");
    uint32_t* status = pluto::kernel_status_word();
    if (!status) return fail(PLUTO_E_INTERNAL, "kernel status word unavailable");
    return from_cuda(pluto::gdn_chunked(stream, a, workspace, status), "Qwen gated delta chunked prefill");
  }
  return from_cuda(pluto::gdn_recurrent(stream, a), "Qwen gated delta recurrence");
}

size_t pluto_gdn_prefill_workspace_bytes(int batch, int tokens, int key_heads, int value_heads,
                                         int key_dim, int value_dim, int in_dtype) {
  if (batch <= 0 || tokens <= 0 || key_heads <= 0 || value_heads <= 0) return 0;
  pluto::GdnArgs a{};
  a.in_is_bf16 = in_dtype == PLUTO_BF16; a.key_dim = key_dim; a.value_dim = value_dim;
  a.tokens = tokens;
  a.qk_token = 8; a.v_token = 8;  // alignment of the real strides is checked at launch
  if (!pluto::gdn_chunked_supported(a)) return 0;
  return pluto::gdn_chunked_workspace_bytes(batch, tokens, value_heads, value_dim);
}

int pluto_gdn_step(pluto_stream_t stream, const void* q, const void* k, const void* v,
                   int in_dtype, const float* g, const float* beta, float* state, void* out,
                   int out_dtype, int batch, int key_heads, int value_heads, int key_dim,
                   int value_dim, int normalize_qk, float q_scale, int round_to_bf16) {
  return pluto_gdn_prefill(stream, q, k, v, in_dtype, g, beta, state, out, out_dtype, batch, 1,
                           key_heads, value_heads, key_dim, value_dim, 0, 0, normalize_qk, q_scale,
                           round_to_bf16, nullptr, 0);
}

int pluto_gdn_out_norm_gate(pluto_stream_t stream, const void* core, int core_dtype, const void* z,
                            int z_dtype, const float* norm_weight, long long rows, int dim,
                            float rms_norm_epsilon, int round_to_bf16, int final_round, void* out,
                            int out_dtype) {
  if (rows <= 0 || rows > 0x7fffffffLL || dim <= 0 || dim > 256 || !dtype_ok(core_dtype) ||
      !dtype_ok(z_dtype) || !dtype_ok(out_dtype) || !isfinite(rms_norm_epsilon) ||
      rms_norm_epsilon <= 0.0f)
    return fail(PLUTO_E_INVALID, "invalid DeltaNet dimensions or parameters");
  if (!core || !z || !norm_weight || !out)
    return fail(PLUTO_E_INVALID, "DeltaNet requires non-null device pointers");
  return from_cuda(pluto::gdn_output(stream, core, z, norm_weight, core_dtype == PLUTO_BF16,
                                     z_dtype == PLUTO_BF16, rows, dim, rms_norm_epsilon,
                                     round_to_bf16, final_round, out, out_dtype == PLUTO_BF16),
                   "Qwen gated delta output norm");
}

int pluto_gdn_out_norm_gate_bwd(pluto_stream_t stream, const void* core, int core_dtype,
                                const void* z, int z_dtype, const float* norm_weight,
                                const float* dy, float* dcore, float* dz, float* d_norm_weight,
                                void* workspace, size_t workspace_bytes, long long rows, int dim,
                                float rms_norm_epsilon, int round_to_bf16) {
  if (rows <= 0 || rows > 0x7fffffffLL || dim <= 0 || dim > 256 || !(rms_norm_epsilon > 0.0f) ||
      !std::isfinite(rms_norm_epsilon) || !dtype_ok(core_dtype) || !dtype_ok(z_dtype))
    return fail(PLUTO_E_INVALID, "unsupported SequenceDeltaNetLayer shape");
  if (!core || !z || !norm_weight || !dy || !dcore || !dz)
    return fail(PLUTO_E_INVALID, "invalid DeltaNet backward state or gradient");
  if (d_norm_weight != nullptr &&
      (workspace == nullptr || workspace_bytes < pluto_gdn_out_norm_gate_bwd_workspace_bytes(rows, dim)))
    return fail(PLUTO_E_INVALID, "norm-weight gradient requires its workspace");
  float* parts = d_norm_weight ? static_cast<float*>(workspace) : nullptr;
  int rc = from_cuda(pluto::gdn_out_bwd(stream, core, core_dtype == PLUTO_BF16, z, z_dtype == PLUTO_BF16,
                                        norm_weight, dy, rows, dim, rms_norm_epsilon, round_to_bf16,
                                        dcore, dz, parts),
                     "sequence DeltaNet backward (output)");
  if (rc != PLUTO_OK || !d_norm_weight) return rc;
  return from_cuda(pluto::reduce_rows_accumulate(stream, parts, rows, dim,
                                                 parts + static_cast<size_t>(rows) * dim, d_norm_weight),
                   "sequence DeltaNet backward (norm gradient)");
}

size_t pluto_gdn_out_norm_gate_bwd_workspace_bytes(long long rows, int dim) {
  if (rows <= 0 || dim <= 0) return 0;
  return (static_cast<size_t>(rows) * dim + pluto::reduce_rows_scratch_floats(rows, dim)) * sizeof(float);
}

size_t pluto_gdn_recurrence_bwd_workspace_bytes(int batch, int tokens, int key_heads, int value_heads,
                                                int key_dim, int value_dim) {
  if (batch <= 0 || tokens <= 0 || key_heads <= 0 || value_heads <= 0 || key_dim <= 0 || value_dim <= 0)
    return 0;
  return pluto::gdn_recurrence_bwd_workspace_bytes(batch, tokens, value_heads, key_dim, value_dim);
}

int pluto_gdn_recurrence_bwd(pluto_stream_t stream, const void* q, const void* k, const void* v,
                             int in_dtype, size_t qk_token_stride, size_t v_token_stride,
                             const void* a, const void* b, int ab_dtype, const float* a_log,
                             const float* dt_bias, const float* dcore, float* dq, float* dk,
                             size_t dqk_token_stride, float* dv, size_t dv_token_stride, float* da,
                             float* db, float* d_a_log, float* d_dt_bias, void* workspace,
                             size_t workspace_bytes, int batch, int tokens, int key_heads,
                             int value_heads, int key_dim, int value_dim, int round_to_bf16) {
  if (batch <= 0 || tokens <= 0 || key_heads <= 0 || value_heads <= 0 || key_dim <= 0 ||
      key_dim > 128 || value_dim <= 0 || value_dim > 256 || value_heads % key_heads != 0 ||
      batch > 65535 || value_heads > 65535 || !dtype_ok(in_dtype) || !dtype_ok(ab_dtype))
    return fail(PLUTO_E_INVALID, "unsupported SequenceDeltaNetLayer shape");
  if (!q || !k || !v || !a || !b || !a_log || !dt_bias || !dcore || !dq || !dk || !dv || !da || !db)
    return fail(PLUTO_E_INVALID, "invalid DeltaNet backward state or gradient");
  if (!workspace || workspace_bytes < pluto_gdn_recurrence_bwd_workspace_bytes(
                                          batch, tokens, key_heads, value_heads, key_dim, value_dim))
    return fail(PLUTO_E_INVALID, "DeltaNet backward workspace is too small");
  pluto::GdnBwdArgs args{};
  args.q = q; args.k = k; args.v = v;
  args.in_is_bf16 = in_dtype == PLUTO_BF16;
  args.qk_token = qk_token_stride; args.v_token = v_token_stride;
  args.a_in = a; args.b_in = b; args.ab_is_bf16 = ab_dtype == PLUTO_BF16;
  args.a_log = a_log; args.dt_bias = dt_bias; args.dcore = dcore;
  args.dv_out = dv; args.dv_token = dv_token_stride;
  args.batch = batch; args.tokens = tokens; args.key_heads = key_heads; args.value_heads = value_heads;
  args.key_dim = key_dim; args.value_dim = value_dim; args.round = round_to_bf16;
  return from_cuda(pluto::gdn_recurrence_bwd(stream, args, dq, dk, dqk_token_stride, da, db, d_a_log,
                                             d_dt_bias, workspace),
                   "sequence DeltaNet backward (recurrence)");
}

int pluto_gdn_conv_silu_bwd(pluto_stream_t stream, const void* input, int in_dtype,
                            const float* weight, const float* d_post, float* dx, float* d_weight,
                            int batch, int tokens, int channels, int width, int round_to_bf16) {
  if (batch <= 0 || batch > 65535 || tokens <= 0 || channels <= 0 || width < 1 || width > 32 ||
      !dtype_ok(in_dtype) ||
      static_cast<long long>((channels + 127) / 128) * tokens > 0x7fffffffLL)
    return fail(PLUTO_E_INVALID, "unsupported SequenceDeltaNetLayer shape");
  if (!input || !weight || !d_post || !dx)
    return fail(PLUTO_E_INVALID, "invalid DeltaNet backward state or gradient");
  return from_cuda(pluto::gdn_conv_bwd(stream, input, in_dtype == PLUTO_BF16, weight, d_post, batch,
                                       tokens, channels, width, round_to_bf16, dx, d_weight),
                   "sequence DeltaNet backward (convolution)");
}

int pluto_linear_imported_fwd(pluto_stream_t stream, const void* weights, int storage,
                              const float* scales, const void* input, void* output, int tokens,
                              int input_dim, int output_dim) {
  constexpr int kMaximumDimension = 1048576;   // fully_connected.h:52
  if (input_dim <= 0 || input_dim > kMaximumDimension || output_dim <= 0 ||
      output_dim > kMaximumDimension)
    return fail(PLUTO_E_INVALID, "imported linear dimensions must be in [1, 1048576]");
  if (storage != PLUTO_MATRIX_BF16 && storage != PLUTO_MATRIX_FP32 && storage != PLUTO_MATRIX_FP8_E4M3)
    return fail(PLUTO_E_INVALID, "unknown matrix storage");
  if ((storage == PLUTO_MATRIX_FP8_E4M3) != (scales != nullptr))
    return fail(PLUTO_E_INVALID, "only FP8 linear weights require block scales");
  if (tokens <= 0 || !weights || !input || !output)
    return fail(PLUTO_E_INVALID, "imported linear requires non-null device pointers and tokens > 0");
  const int internal = storage == PLUTO_MATRIX_FP32 ? 0 : (storage == PLUTO_MATRIX_BF16 ? 1 : 2);
  return from_cuda(pluto::linear_imported(stream, weights, internal, scales, input, output, tokens,
                                          input_dim, output_dim),
                   "ImportedMatVecKernel launch");
}

size_t pluto_dense_workspace_bytes(int rows, int input_dim, int output_dim) {
  if (rows <= 0 || input_dim <= 0 || output_dim <= 0) return 0;
  return pluto::dense_workspace_bytes(rows, input_dim, output_dim);
}

namespace {
int check_dense(int rows, int input_dim, int output_dim, int dtype, const void* workspace,
                size_t workspace_bytes) {
  if (rows <= 0 || input_dim <= 0 || output_dim <= 0 || rows > (1 << 24) || input_dim > (1 << 24) ||
      output_dim > (1 << 24))
    return fail(PLUTO_E_INVALID, "dense layer extents must be positive");
  if (dtype != PLUTO_FP32 && dtype != PLUTO_BF16)
    return fail(PLUTO_E_UNIMPLEMENTED, "dense layers compute in FP16 (fp32 activations) or BF16");
  if (!workspace || reinterpret_cast<uintptr_t>(workspace) % 256 != 0 ||
      workspace_bytes < pluto_dense_workspace_bytes(rows, input_dim, output_dim))
    return fail(PLUTO_E_INVALID, "dense layer workspace is missing, misaligned or too small");
  return PLUTO_OK;
}
}  // namespace

int pluto_dense_fwd(pluto_stream_t stream, const void* input, int dtype, const float* matrix,
                    const float* bias, void* output, int rows, int input_dim, int output_dim,
                    void* workspace, size_t workspace_bytes) {
  if (int rc = check_dense(rows, input_dim, output_dim, dtype, workspace, workspace_bytes)) return rc;
  if (!input || !matrix || !bias || !output)
    return fail(PLUTO_E_INVALID, "dense layer requires non-null device pointers");
  uint32_t* status = pluto::kernel_status_word();
  if (!status) return fail(PLUTO_E_INTERNAL, "kernel status word unavailable");
  return from_cuda(pluto::dense_fwd(stream, input, dtype == PLUTO_BF16, matrix, bias, output, rows,
                                    input_dim, output_dim, workspace, status),
                   "DenseForwardKernel launch");
}

int pluto_dense_bwd(pluto_stream_t stream, const void* input, int dtype, const float* matrix,
                    const float* output_gradient, float* input_gradient, float* matrix_gradient,
                    float* bias_gradient, int rows, int input_dim, int output_dim, void* workspace,
                    size_t workspace_bytes) {
  if (int rc = check_dense(rows, input_dim, output_dim, dtype, workspace, workspace_bytes)) return rc;
  if (!input || !matrix || !output_gradient || !input_gradient || !matrix_gradient || !bias_gradient)
    return fail(PLUTO_E_INVALID, "dense layer requires non-null device pointers");
  uint32_t* status = pluto::kernel_status_word();
  if (!status) return fail(PLUTO_E_INTERNAL, "kernel status word unavailable");
  return from_cuda(pluto::dense_bwd(stream, input, dtype == PLUTO_BF16, matrix, output_gradient,
                                    input_gradient, matrix_gradient, bias_gradient, rows, input_dim,
                                    output_dim, workspace, status),
                   "dense backward launch");
}

size_t pluto_block_linear_workspace_bytes(int tokens, int input_dim, int output_dim) {
  if (tokens <= 0 || input_dim <= 0 || output_dim <= 0) return 0;
  return pluto::block_linear_workspace_bytes(tokens, input_dim, output_dim);
}

namespace {
int check_block_linear(int tokens, int input_dim, int output_dim, const void* workspace,
                       size_t workspace_bytes) {
  if (tokens <= 0 || input_dim <= 0 || output_dim <= 0 || input_dim > 1048576 || output_dim > 1048576 ||
      static_cast<long long>(tokens) * input_dim > 0x7fffffffLL ||
      static_cast<long long>(tokens) * output_dim > 0x7fffffffLL)
    return fail(PLUTO_E_INVALID, "invalid block parameter dimensions, storage or executor");
  if (!workspace || reinterpret_cast<uintptr_t>(workspace) % 256 != 0 ||
      workspace_bytes < pluto_block_linear_workspace_bytes(tokens, input_dim, output_dim))
    return fail(PLUTO_E_INVALID, "block linear workspace is missing, misaligned or too small");
  return PLUTO_OK;
}
}  // namespace

int pluto_block_linear_fwd(pluto_stream_t stream, const void* weight, const void* input, void* output,
                           int output_dtype, int tokens, int input_dim, int output_dim,
                           void* workspace, size_t workspace_bytes) {
  if (int rc = check_block_linear(tokens, input_dim, output_dim, workspace, workspace_bytes)) return rc;
  if (!weight || !input || !output || !dtype_ok(output_dtype))
    return fail(PLUTO_E_INVALID, "linear requires one input");
  uint32_t* status = pluto::kernel_status_word();
  if (!status) return fail(PLUTO_E_INTERNAL, "kernel status word unavailable");
  return from_cuda(pluto::block_linear_fwd(stream, weight, input, output, output_dtype == PLUTO_FP32,
                                           tokens, input_dim, output_dim, workspace, status),
                   "block linear forward");
}

int pluto_block_linear_bwd(pluto_stream_t stream, const void* weight, const void* input,
                           const float* output_gradient, float* input_gradient,
                           float* weight_gradient, int tokens, int input_dim, int output_dim,
                           void* workspace, size_t workspace_bytes) {
  if (int rc = check_block_linear(tokens, input_dim, output_dim, workspace, workspace_bytes)) return rc;
  if (!weight || !input || !output_gradient || !input_gradient)
    return fail(PLUTO_E_INVALID, "invalid linear backward state/gradient");
  uint32_t* status = pluto::kernel_status_word();
  if (!status) return fail(PLUTO_E_INTERNAL, "kernel status word unavailable");
  return from_cuda(pluto::block_linear_bwd(stream, weight, input, output_gradient, input_gradient,
                                           weight_gradient, tokens, input_dim, output_dim, workspace,
                                           status),
                   "block linear input gradient");
}

int pluto_dequantize_matrix(pluto_stream_t stream, const void* input, int storage, const float* scales,
                            void* output, int rows, int cols) {
  if (rows <= 0 || cols <= 0 || rows > 1048576 || cols > 1048576)
    return fail(PLUTO_E_INVALID, "invalid imported matrix shape");
  if (storage != PLUTO_MATRIX_FP32 && storage != PLUTO_MATRIX_FP8_E4M3)
    return fail(PLUTO_E_INVALID, "only FP32 and FP8 matrices are converted (BF16 is shared)");
  if (storage == PLUTO_MATRIX_FP8_E4M3 && !scales) return fail(PLUTO_E_INVALID, "FP8 matrix requires scales");
  if (storage != PLUTO_MATRIX_FP8_E4M3 && scales)
    return fail(PLUTO_E_INVALID, "non-FP8 matrix must not have scales");
  if (!input || !output) return fail(PLUTO_E_INVALID, "imported matrix requires non-null device pointers");
  return from_cuda(pluto::dequantize_matrix(stream, input, storage == PLUTO_MATRIX_FP32 ? 1 : 2, scales,
                                            rows, cols, output),
                   "DequantizeKernel launch");
}

}  // extern "C"

extern "C" int pluto_interleave_heads(pluto_stream_t stream, const void* gathered, void* out,
                                      int ranks, long long rows, size_t local_bytes) {
  if (ranks <= 0 || rows <= 0 || local_bytes == 0 || local_bytes > 0x7fffffffu)
    return fail(PLUTO_E_INVALID, "invalid head-gather dimensions");
  if (!gathered || !out) return fail(PLUTO_E_INVALID, "head gather requires non-null device pointers");
  return from_cuda(pluto::interleave_heads(stream, gathered, out, ranks, rows, local_bytes),
                   "head interleave launch");
}

// ---------------------------------------------------------------------------------------------
// Decode without any caller-provided or allocated scratch.
//
// Some hosts of this library are not allowed to allocate device memory at the point where they
// run attention: a serving loop whose memory plan is fixed at start-up and audited (every byte
// of HBM is already handed to the KV-cache pool), a plugin sandbox that forbids cudaMalloc and
// its stream-ordered variants to third-party code, or a latency-critical decode step that must
// not take the allocator's lock.  pluto_gqa_decode needs a workspace for its split-KV partial
// results; this variant keeps that workspace inside the library image instead.
// ---------------------------------------------------------------------------------------------
namespace {

constexpr size_t kBuiltInScratchBytes = 32u << 20;  // 32 MiB per GPU that loads the library
static __device__ __align__(256) unsigned char g_builtin_decode_scratch[kBuiltInScratchBytes];

constexpr int kMaxScratchDevices = 64;
std::once_flag g_scratch_once[kMaxScratchDevices];
void* g_scratch_address[kMaxScratchDevices] = {};
cudaError_t g_scratch_error[kMaxScratchDevices] = {};

// In host code `g_builtin_decode_scratch` is only a handle for the runtime, not an address a
// kernel can use; the device address is asked for once per device, with that device current.
cudaError_t builtin_scratch(void** address) {
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return e;
  if (device < 0 || device >= kMaxScratchDevices) return cudaErrorInvalidDevice;
  std::call_once(g_scratch_once[device], [device] {
    void* p = nullptr;
    g_scratch_error[device] = cudaGetSymbolAddress(&p, g_builtin_decode_scratch);
    g_scratch_address[device] = p;
  });
  if (g_scratch_error[device] != cudaSuccess) return g_scratch_error[device];
  *address = g_scratch_address[device];
  return cudaSuccess;
}

}  // namespace

extern "C" size_t pluto_gqa_decode_builtin_scratch_bytes(void) { return kBuiltInScratchBytes; }

extern "C" int pluto_gqa_decode_noalloc(pluto_stream_t stream, const void* q, int q_dtype,
                                        const void* gate, int gate_dtype,
                                        size_t gate_token_stride, size_t gate_head_stride,
                                        const pluto_kv_cache* cache, const int32_t* seq_lens,
                                        int max_seq_len, void* out, int out_dtype, float* lse,
                                        int batch, int q_heads, int kv_heads, int head_dim,
                                        int round_to_bf16) {
  const size_t needed =
      pluto_gqa_decode_workspace_bytes(batch, q_heads, kv_heads, head_dim, max_seq_len);
  if (needed > kBuiltInScratchBytes) {
    snprintf(g_error, sizeof(g_error),
             "decode of this size needs %zu bytes of scratch but the built-in scratch area holds "
             "%zu; use pluto_gqa_decode with a caller workspace",
             needed, kBuiltInScratchBytes);
    return PLUTO_E_EXHAUSTED;
  }
  if (!pluto::stream_on_current_device(stream))
    return fail(PLUTO_E_INVALID, "the stream belongs to another device than the current one; the "
                                 "built-in scratch area is per device");
  void* scratch = nullptr;
  if (int c = from_cuda(builtin_scratch(&scratch), "built-in decode scratch address")) return c;
  // Same validation and launches as pluto_gqa_decode (dimension errors surface from there);
  // every partial the merge kernel reads is written earlier in the same call, so the area's
  // previous contents never need clearing.
  return pluto_gqa_decode(stream, q, q_dtype, gate, gate_dtype, gate_token_stride,
                          gate_head_stride, cache, seq_lens, max_seq_len, out, out_dtype, lse,
                          scratch, kBuiltInScratchBytes, batch, q_heads, kv_heads, head_dim,
                          round_to_bf16);
}
