// extern "C" entry points declared in include/pluto_b200.h: argument validation (the same checks,
// in the same order, as the reference layers make before queuing GPU work) and dispatch to the
// kernel files.  No allocation, no synchronisation, no mutable global state beyond the per-thread
// error text and the per-device status-word address cache.
#include <math.h>
#include <stdio.h>

#include <limits>

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
                              head_dim, E, head_dim, 1, nullptr, nullptr, 0, dtype == PLUTO_BF16),
      "attention forward launch");
}

int pluto_attn_bwd(pluto_stream_t stream, const void* qkv, const void* out, const float* d_out,
                   const float* maxima, const float* normalizers, float* d_qkv, float* deltas,
                   int batch, int seq, int heads, int head_dim, int dtype) {
  if (int c = check_mha(batch, seq, heads, head_dim, dtype)) return c;
  if (!qkv) return fail(PLUTO_E_INVALID, "attention backward requires the saved Q/K/V");
  if (!out) return fail(PLUTO_E_INVALID, "attention backward requires the saved output");
  if (!maxima) return fail(PLUTO_E_INVALID, "attention backward requires the saved maxima");
  if (!normalizers) return fail(PLUTO_E_INVALID, "attention backward requires the saved normalizers");
  if (!d_out || !d_qkv || !deltas)
    return fail(PLUTO_E_INVALID, "attention backward requires non-null gradient pointers");
  return from_cuda(pluto::attn_generic_bwd(stream, qkv, out, d_out, maxima, normalizers, d_qkv,
                                           deltas, batch, seq, heads, head_dim,
                                           dtype == PLUTO_BF16),
                   "attention backward launch");
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
                          int round_to_bf16) {
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
                      q_token_stride <= 0x7fffffffu && (!gate || aligned16(gate));
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
    a.gate = gate; a.gate_token = q_token_stride; a.gate_head = q_head_stride;
    a.round_gate = round_to_bf16;
    a.status = pluto::kernel_status_word();
    if (!a.status) return fail(PLUTO_E_INTERNAL, "kernel status word unavailable");
    return from_cuda(pluto::attn_fwd_tc(stream, a), "GQA prefill (tcgen05) launch");
  }
  return from_cuda(
      pluto::attn_generic_fwd(stream, q, k, v, out, maxima, normalizers, batch, seq, q_heads,
                              head_dim, q_token_stride, q_head_stride, kv_token, head_dim,
                              out_token, head_dim, group, gate, core, round_to_bf16, true),
      "GQA prefill launch");
}

}  // extern "C"
