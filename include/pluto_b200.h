/*
 * pluto_b200 -- C ABI of the B200 attention engine.
 *
 * These are the entry points a binding inside the Pluto tree (C++20, no exceptions, absl::Status)
 * calls from its Layer::fwd_impl / bwd_impl bodies and from cached_attention_ops.  Each comment
 * names the reference interface the function stands in for (paths relative to the reference
 * tree).  Conventions shared by every function:
 *
 *   - every pointer is a DEVICE pointer owned by the caller (a pluto::cuda::Buffer::data()),
 *     unless the comment says "host";
 *   - work is queued on `stream` (the caller's Executor::stream()); nothing synchronises, nothing
 *     touches the default stream, nothing allocates or frees -- scratch comes in through
 *     explicit workspace arguments whose size the *_workspace_bytes functions report;
 *   - all validation happens before any GPU work is queued;
 *   - return value: 0 = queued; > 0 = a cudaError_t from the launch; < 0 = one of PLUTO_E_*.
 *     PLUTO_E_INVALID maps to absl::InvalidArgumentError, PLUTO_E_UNIMPLEMENTED to
 *     UnimplementedError, PLUTO_E_EXHAUSTED to ResourceExhaustedError, PLUTO_E_INTERNAL to
 *     InternalError (src/util/status_macros.h:11-38, src/cuda/executor.cc:15-21);
 *   - bf16 tensors are raw uint16 bit patterns (round-to-nearest-even), fp32 tensors IEEE floats.
 */
#ifndef PLUTO_B200_H_
#define PLUTO_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* pluto_stream_t; /* == cudaStream_t */

enum {
  PLUTO_OK = 0,
  PLUTO_E_INVALID = -1,
  PLUTO_E_UNIMPLEMENTED = -2,
  PLUTO_E_EXHAUSTED = -3,
  PLUTO_E_INTERNAL = -4
};

/* Activation storage of a layer.  PLUTO_FP32 is the reference's DataType::FP16 compute policy,
 * whose activations are stored as fp32 (src/llm/layer.h:83-88); PLUTO_BF16 is DataType::BF16. */
enum { PLUTO_FP32 = 0, PLUTO_BF16 = 1 };

/* Human-readable text for the last PLUTO_E_* returned on this host thread (host pointer, valid
 * until the next call on the thread).  The strings carry the phrases the reference's tests look
 * for ("divisible by context_length", "saved maxima", ...). */
const char* pluto_last_error(void);

/* Library version and the SM architecture it was compiled for ("sm_100a"). */
const char* pluto_build_info(void);

/* Diagnostic: reads (and optionally clears) the device status word that kernels set when one of
 * their bounded waits ran out.  SYNCHRONISES the device.  *value == 0 means healthy. */
int pluto_kernel_status(uint32_t* value /* host */, int clear);

/* --------------------------------------------------------------------------------------------
 * Causal multi-head attention over a packed activation (GPT-2 recipe).
 * Stands in for AttentionLayer::fwd_impl + FlashAttentionForwardKernel
 * (src/llm/layers/attention.cc:418-507, :98-170).
 *   qkv          [batch*seq, 3*heads*head_dim], row-major; columns = all Q, then all K, then all V;
 *                head h at h*head_dim inside each third.  fp32 or bf16 per `dtype`.
 *   out          [batch*seq, heads*head_dim], same dtype.
 *   maxima, normalizers   fp32 [batch*heads*seq] at (b*heads+h)*seq + s: the row maximum of the
 *                scaled scores and sum exp(score - max), the state backward reuses.
 * Attention restarts at every multiple of seq (the layer's context_length); scale = 1/sqrt(head_dim).
 * head_dim <= 256.  bf16 with head_dim 64 or 128 runs on the tcgen05 tensor-core kernel, every
 * other shape on the exact fp32 kernel. */
int pluto_attn_fwd(pluto_stream_t stream, const void* qkv, void* out, float* maxima,
                   float* normalizers, int batch, int seq, int heads, int head_dim, int dtype);

/* Stands in for AttentionLayer::bwd_impl + FlashAttentionQueryBackwardKernel +
 * FlashAttentionKeyValueBackwardKernel (src/llm/layers/attention.cc:509-596, :235-314, :319-396).
 *   d_out        fp32 [batch*seq, heads*head_dim] (upstream gradient is always fp32)
 *   d_qkv        fp32 [batch*seq, 3*heads*head_dim]: dQ third, dK third, dV third (fully written)
 *   deltas       fp32 scratch [batch*heads*seq] (sum dO*O per row; written then read)
 * Deterministic: single-writer tiles, fixed-order reductions, no floating-point atomics. */
int pluto_attn_bwd(pluto_stream_t stream, const void* qkv, const void* out, const float* d_out,
                   const float* maxima, const float* normalizers, float* d_qkv, float* deltas,
                   int batch, int seq, int heads, int head_dim, int dtype);

/* Stands in for AttentionProbabilitiesKernel behind LayerHooks::attention_probabilities_hook
 * (src/llm/layers/attention.cc:176-230, :475-502).  probs: fp32 [batch, heads, seq, seq], zeros
 * above the diagonal. */
int pluto_attn_probs(pluto_stream_t stream, const void* qkv, const float* maxima,
                     const float* normalizers, float* probs, int batch, int seq, int heads,
                     int head_dim, int dtype);

/* --------------------------------------------------------------------------------------------
 * Grouped-query causal attention over a whole sequence (prefill / stateless sequence forward).
 * Stands in for the attention core of QwenAttentionLayer::SequenceForward + ForwardKernel
 * (src/llm/layers/qwen_attention.cc:414-448, :68-119); q and k are expected already normalised
 * and rotated (pluto_qk_prepare).
 *   q            bf16, token t / head h at q + (b*seq + t)*q_token_stride + h*q_head_stride
 *                (element strides; [T,Hq,D] is (Hq*D, D); the query half of [T,Hq,2,D] is
 *                (2*Hq*D, 2*D))
 *   gate         optional bf16, indexed with the same two strides (pass q + D for [T,Hq,2,D]);
 *                when non-null out = R(R(core) * R(sigmoid(gate))), R = bf16 rounding when
 *                round_to_bf16, as the reference does
 *   k, v         bf16 [batch, seq, kv_heads, head_dim] contiguous
 *   out          bf16 [batch, seq, q_heads, head_dim] contiguous
 *   core         optional fp32 [batch, seq, q_heads, head_dim]: the ungated, unrounded result the
 *                reference saves for backward
 *   maxima, normalizers   optional fp32 [batch*q_heads*seq] as in pluto_attn_fwd (both or neither)
 * q_heads % kv_heads == 0, head_dim <= 256; head_dim 64/128 runs on tcgen05. */
int pluto_gqa_prefill_fwd(pluto_stream_t stream, const void* q, const void* gate, const void* k,
                          const void* v, void* out, float* core, float* maxima,
                          float* normalizers, int batch, int seq, int q_heads, int kv_heads,
                          int head_dim, size_t q_token_stride, size_t q_head_stride,
                          int round_to_bf16);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* PLUTO_B200_H_ */
