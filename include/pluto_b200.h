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
 *   - the device that owns `stream` must be the calling thread's current device: per-device state
 *     (the kernel status word, the built-in decode scratch, the host-prefill copy streams) is
 *     looked up by the current device;
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
 * their bounded waits ran out.  SYNCHRONISES the device.  *value == 0 means healthy; otherwise
 * (site << 8) | kind with kind 1 = a bounded wait ran out, 2 = a device-side sequence length lay
 * outside the declared bound, 3 = a block-table entry lay outside the page pool, 4 = a kernel found
 * its dynamic shared memory off the boundary it needs (it returns without computing). */
int pluto_kernel_status(uint32_t* value /* host */, int clear);

/* Diagnostic with no counterpart in the reference: proves on the running GPU that a bounded wait
 * gives up instead of hanging.  Queues a one-thread kernel that waits on a barrier nobody arrives
 * at; after limit_ns (at most 100 ms) the wait gives up, the kernel stores 1 to *gave_up (device
 * uint32) and returns, and the status word reads (PLUTO_SELFTEST_WAIT_SITE << 8) | 1 until it is
 * cleared.  Clear it (pluto_kernel_status with clear = 1) before queuing other work: while the
 * word is non-zero every other bounded wait that has to spin gives up early too. */
#define PLUTO_SELFTEST_WAIT_SITE 63u
int pluto_selftest_bounded_wait(pluto_stream_t stream, unsigned long long limit_ns,
                                uint32_t* gave_up);

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

/* Bytes of scratch the tensor-core backward needs (host-only query; 0 when the shape has no
 * tensor-core path: it needs bf16 activations and head_dim 64 or 128). */
size_t pluto_attn_bwd_workspace_bytes(int batch, int seq, int heads, int head_dim, int dtype);

/* Stands in for AttentionLayer::bwd_impl + FlashAttentionQueryBackwardKernel +
 * FlashAttentionKeyValueBackwardKernel (src/llm/layers/attention.cc:509-596, :235-314, :319-396).
 *   d_out        fp32 [batch*seq, heads*head_dim] (upstream gradient is always fp32)
 *   d_qkv        fp32 [batch*seq, 3*heads*head_dim]: dQ third, dK third, dV third (fully written)
 *   deltas       fp32 scratch [batch*heads*seq] (sum dO*O per row; written then read)
 *   workspace    NULL: exact fp32 kernels (every shape).  >= pluto_attn_bwd_workspace_bytes(...)
 *                bytes, 256-byte aligned: tcgen05 kernels (holds the gradient rounded to bf16 and
 *                a padded per-row statistics record).
 * Deterministic either way: single-writer tiles, fixed-order reductions, no floating-point
 * atomics. */
int pluto_attn_bwd(pluto_stream_t stream, const void* qkv, const void* out, const float* d_out,
                   const float* maxima, const float* normalizers, float* d_qkv, float* deltas,
                   int batch, int seq, int heads, int head_dim, int dtype, void* workspace,
                   size_t workspace_bytes);

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
 *   gate         optional bf16; token t / head h at gate + (b*seq + t)*gate_token_stride +
 *                h*gate_head_stride (for [T,Hq,2,D] pass base + D and strides (2*Hq*D, 2*D));
 *                when non-null out = R(R(core) * R(sigmoid(gate))), R = bf16 rounding when
 *                round_to_bf16, as the reference does
 *   k, v         bf16 [batch, seq, kv_heads, head_dim] contiguous
 *   out          bf16 [batch, seq, q_heads, head_dim] contiguous
 *   core         optional fp32 [batch, seq, q_heads, head_dim]: the ungated, unrounded result the
 *                reference saves for backward
 *   maxima, normalizers   optional fp32 [batch*q_heads*seq] as in pluto_attn_fwd (both or neither)
 *   workspace    optional (may be null): with pluto_gqa_prefill_fwd_workspace_bytes of 16-byte
 *                aligned device memory, shapes whose whole query tiles cannot load the SMs evenly
 *                (a few heads of a long causal prompt, e.g. one GPU's share of a head-sharded
 *                layer) have their longest query-tile pairs cut along the keys into 2 to 4 CTAs,
 *                combined by a second kernel; the query returns 0 for shapes that are not cut
 * q_heads % kv_heads == 0, head_dim <= 256; head_dim 64/128 runs on tcgen05. */
int pluto_gqa_prefill_fwd(pluto_stream_t stream, const void* q, const void* gate, const void* k,
                          const void* v, void* out, float* core, float* maxima,
                          float* normalizers, int batch, int seq, int q_heads, int kv_heads,
                          int head_dim, size_t q_token_stride, size_t q_head_stride,
                          size_t gate_token_stride, size_t gate_head_stride, int round_to_bf16,
                          void* workspace, size_t workspace_bytes);
size_t pluto_gqa_prefill_fwd_workspace_bytes(int batch, int seq, int q_heads, int head_dim);

/* --------------------------------------------------------------------------------------------
 * pluto_gqa_prefill_fwd (the attention core of src/llm/layers/qwen_attention.cc:414-448) for
 * activations that live in pinned HOST memory; the one entry point that takes host pointers
 * (the reference stages such buffers with one cudaMemcpyAsync per tensor, as its tests do,
 * src/llm/layers/qwen_attention_test.cc:118-131): q_host / out_host bf16 [batch, seq, q_heads, head_dim], k_host /
 * v_host bf16 [batch, seq, kv_heads, head_dim], all dense.  The key/value heads are processed in
 * groups of kv_heads_per_group (with their query heads); each group's host->device copy, kernel
 * and device->host copy run on separate streams, two groups in flight, so the PCIe transfers of
 * both directions overlap each other and the kernels.  kv_heads_per_group = 0 (head width 64 or
 * 128) cuts the prompt by query tokens instead: chunks of 1024 tokens or more (at least 4 MB of input) are copied as contiguous
 * pieces (queries, keys and values alike), a chunk's queries run against all keys copied so far
 * (causal attention needs no later ones), and its output rows leave as one contiguous piece; the
 * workspace then holds the whole Q, K, V and output.  No gate, statistics or core output.
 * workspace: device memory of pluto_gqa_prefill_host_workspace_bytes, 256-byte aligned.  Ordered
 * behind `stream`; `stream` waits for the last output copy, so synchronising it (or ordering
 * later work on it) is enough.  Uses two internal copy streams and a few events per device,
 * created on first use; calls for one device must not run concurrently from several threads. */
size_t pluto_gqa_prefill_host_workspace_bytes(int batch, int seq, int q_heads, int kv_heads,
                                              int head_dim, int kv_heads_per_group);
int pluto_gqa_prefill_fwd_host(pluto_stream_t stream, const void* q_host, const void* k_host,
                               const void* v_host, void* out_host, void* workspace,
                               size_t workspace_bytes, int batch, int seq, int q_heads, int kv_heads,
                               int head_dim, int kv_heads_per_group);

/* --------------------------------------------------------------------------------------------
 * Backward of the Qwen sequence attention, QwenAttentionLayer::SequenceBackward
 * (src/llm/layers/qwen_attention.cc:450-499), in the reference's three stages.  None of them
 * materialises the [Hq,T,T] probabilities or score gradients the reference saves: the core pass
 * recomputes P from the saved maxima / normalizers, so the T <= 128 limit does not apply.
 *
 * 1. pluto_gqa_gate_bwd: GateBackwardKernel (:123-138) plus the row term of the softmax
 *    backward (QueryBackwardKernel :153-155):
 *      dc = dy * R(sigmoid(gate)),  d_gate = dy * R(core) * s * (1 - s),  deltas = sum_c dc * core
 *    gate bf16 and d_gate fp32 are addressed by (token, head) element strides (the gate half of
 *    [T,Hq,2,D] is base + D with strides (2*Hq*D, 2*D)); core, dy, dc fp32 dense
 *    [batch, seq, q_heads, head_dim]; deltas fp32 [batch*q_heads*seq] indexed like maxima.
 * 2. pluto_gqa_prefill_bwd: QueryBackwardKernel + KeyValueBackwardKernel (:140-190):
 *      dS = P * (dc . v - delta),  dq = scale * dS k,  dk = scale * sum dS^T q,  dv = sum P^T dc
 *    with dk / dv summed over the query heads of the group and the later rows in a fixed order
 *    (single writer, no atomics: repeated runs are bitwise equal).  q (strided like the forward),
 *    k, v are the prepared tensors of the forward, bf16 or fp32 (dtype); dq fp32
 *    [batch, seq, q_heads, head_dim], dk / dv fp32 [batch, seq, kv_heads, head_dim]: gradients
 *    of the normalised, rotated vectors.  With a workspace of
 *    pluto_gqa_prefill_bwd_workspace_bytes (non-zero for bf16 tensors of head width 64/128) and
 *    a dense query (q_head_stride == head_dim) the two passes run on tcgen05 with bf16 operands;
 *    with workspace null, or for any other shape, in exact fp32 arithmetic.
 * 3. pluto_qk_prepare_bwd: NormBackwardKernel + ReduceNormKernel (:192-239): inverse partial
 *    RoPE with the forward's (rounded) cos/sin, RMSNorm backward through the layer input x
 *    (bf16, strided), dx fp32 strided (the query half of dQG [T,Hq,2,D], or dK [T,Hkv,D]).
 *    d_weight (optional fp32 [head_dim]) is ACCUMULATED into, as the reference accumulates into
 *    BlockParameter::gradient(); it needs a workspace of pluto_qk_prepare_bwd_workspace_bytes
 *    (per-row parts reduced in a fixed order).  positions as in pluto_qk_prepare (null: token t of
 *    every sequence sits at position t). */
int pluto_gqa_gate_bwd(pluto_stream_t stream, const void* gate, size_t gate_token_stride,
                       size_t gate_head_stride, const float* core, const float* dy, float* dc,
                       float* d_gate, size_t d_gate_token_stride, size_t d_gate_head_stride,
                       float* deltas, int batch, int seq, int q_heads, int head_dim,
                       int round_to_bf16);
int pluto_gqa_prefill_bwd(pluto_stream_t stream, const void* q, const void* k, const void* v,
                          int dtype, size_t q_token_stride, size_t q_head_stride, const float* dc,
                          const float* maxima, const float* normalizers, const float* deltas,
                          float* dq, float* dk, float* dv, void* workspace, size_t workspace_bytes,
                          int batch, int seq, int q_heads, int kv_heads, int head_dim);
size_t pluto_gqa_prefill_bwd_workspace_bytes(int batch, int seq, int q_heads, int head_dim, int dtype);
size_t pluto_qk_prepare_bwd_workspace_bytes(int batch, int tokens, int heads, int head_dim);
int pluto_qk_prepare_bwd(pluto_stream_t stream, const void* x, size_t x_token_stride,
                         size_t x_head_stride, const float* weight, const float* grad,
                         const int32_t* positions, float* dx, size_t dx_token_stride,
                         size_t dx_head_stride, float* d_weight, void* workspace,
                         size_t workspace_bytes, int batch, int tokens, int heads, int head_dim,
                         int rotary_dim, float rms_norm_epsilon, float rope_theta,
                         int round_to_bf16);

/* --------------------------------------------------------------------------------------------
 * KV cache addressing shared by prepare and decode.  The reference keeps one KeyValueCache per
 * sequence: two fp32 buffers [capacity, kv_heads, head_dim] plus a position counter
 * (src/llm/key_value_cache.h:25-57).  Every value it stores is already rounded to bf16 when
 * round_to_bfloat16 is set (cached_attention_ops.cc:48,64-67,76), so a bf16 cache holds the same
 * numbers in half the bytes; both storage types are accepted.
 * Token t of sequence b, kv head h starts at element
 *     page(b, t) * page_stride + (t % page_size) * token_stride + h * head_dim
 * with page(b, t) = block_table ? block_table[b * max_blocks + t / page_size] : b.
 * One contiguous [capacity, kv_heads, head_dim] region per sequence is block_table = NULL,
 * page_size = capacity, page_stride = capacity * kv_heads * head_dim,
 * token_stride = kv_heads * head_dim.  The position counter stays with the caller.
 * A shard of KV heads [h0, h0 + n) of a wider cache is addressed in place: k_base / v_base advanced
 * by h0 * head_dim elements, kv_heads = n in the call, token_stride left at the full row.
 * Separately allocated per-sequence caches (the reference's one KeyValueCache object per
 * sequence) are passed as two device arrays of base pointers, k_bases / v_bases [batch]: token t of
 * sequence b, kv head h then starts at element t * token_stride + h * head_dim of k_bases[b]; no
 * block table, page_size = the sequences' capacity, k_base / v_base / page_stride unused.  Decode
 * over pointer arrays runs on the plain-load kernel (one pool or a block table is what the
 * tensor-map path addresses). */
typedef struct pluto_kv_cache {
  void* k_base;
  void* v_base;
  const int32_t* block_table; /* device int32 [batch, max_blocks] or NULL */
  int max_blocks;
  int page_size;
  size_t page_stride;  /* elements */
  size_t token_stride; /* elements */
  int dtype;           /* PLUTO_BF16 or PLUTO_FP32 */
  int num_pages;       /* pages in the pool when block_table is used (0 = unknown: decode then
                          takes its plain-load path); ignored without a block table */
  const void* const* k_bases; /* device arrays [batch] of per-sequence base pointers, or both NULL */
  const void* const* v_bases;
} pluto_kv_cache;

/* Per-head RMSNorm(1+w) -> bf16 rounding -> split-half partial RoPE of queries and keys, and the
 * append of the new K/V rows to the cache.  Stands in for PrepareAttentionKernel
 * (src/llm/layers/util/cached_attention_ops.cc:30-79) and PrepareKernel
 * (src/llm/layers/qwen_attention.cc:30-63).
 *   q_in         token (b,t), head h at q_in + (b*tokens+t)*q_token_stride + h*q_head_stride;
 *                [.., Hq, 2, D] query halves are (2*Hq*D, 2*D).  k_in, v_in [batch*tokens, Hkv, D].
 *                in_dtype says whether these three are fp32 or bf16.
 *   q_norm, k_norm   fp32 [head_dim], zero-centred (multiplier 1 + w)
 *   positions    device int32 [batch] position of token 0 of each sequence (NULL = 0): the cache
 *                row written and the RoPE angle use positions[b] + t
 *   q_out        [batch*tokens, Hq, D] in q_out_dtype
 *   rotary_dim even, <= head_dim; head_dim <= 256. */
int pluto_qk_prepare(pluto_stream_t stream, const void* q_in, const void* k_in, const void* v_in,
                     int in_dtype, size_t q_token_stride, size_t q_head_stride,
                     const float* q_norm, const float* k_norm, const int32_t* positions,
                     void* q_out, int q_out_dtype, const pluto_kv_cache* cache /* host */,
                     int batch, int tokens, int q_heads, int kv_heads, int head_dim,
                     int rotary_dim, float rms_norm_epsilon, float rope_theta, int round_to_bf16);

/* Bytes of scratch pluto_gqa_decode needs for split-KV partial results (host-only query). */
size_t pluto_gqa_decode_workspace_bytes(int batch, int q_heads, int kv_heads, int head_dim,
                                        int max_seq_len);

/* One new query token per sequence against the cache.  Stands in for FullAttentionKernel and the
 * launch sequence of CachedAttentionStep (src/llm/layers/util/cached_attention_ops.cc:83-126,
 * :308-353) with a batch dimension added (the reference is batch one).
 *   q            [batch, Hq, D] prepared queries (q_dtype)
 *   gate         optional; element (b,h,d) at gate + b*gate_token_stride + h*gate_head_stride + d
 *                ([B,Hq,2,D]: pass base + D, strides (2*Hq*D, 2*D)); out = R(R(core)*R(sigmoid))
 *   seq_lens     device int32 [batch]: tokens to attend to (position + 1, each >= 1)
 *   max_seq_len  host upper bound of seq_lens (sizes the grid; no device read-back)
 *   out          [batch, Hq, D] (out_dtype);  lse optional fp32 [batch, Hq]
 *   workspace    >= pluto_gqa_decode_workspace_bytes(...) bytes, 16-byte aligned
 * bf16 cache with head_dim 64/128 takes the bandwidth-bound path (bulk copies + mma); anything
 * else the exact fp32 path.  The result does not depend on which SM ran which chunk. */
int pluto_gqa_decode(pluto_stream_t stream, const void* q, int q_dtype, const void* gate,
                     int gate_dtype, size_t gate_token_stride, size_t gate_head_stride,
                     const pluto_kv_cache* cache /* host */, const int32_t* seq_lens,
                     int max_seq_len, void* out, int out_dtype, float* lse, void* workspace,
                     size_t workspace_bytes, int batch, int q_heads, int kv_heads, int head_dim,
                     int round_to_bf16);

/* pluto_gqa_decode for callers that may not allocate device memory and have no workspace to lend:
 * hosts whose HBM plan is fixed and fully committed at start-up, plugin sandboxes that forbid
 * cudaMalloc (and the stream-ordered allocators) to loaded libraries, decode loops that must not
 * contend for an allocator lock.  It has no counterpart in the reference, whose CachedAttentionStep
 * allocates its scratch with a stream-ordered Buffer on every token.  The split-KV partials live
 * in a 32 MiB area inside the library image (pluto_gqa_decode_builtin_scratch_bytes()).  Arguments,
 * results and kernels are those of pluto_gqa_decode minus the workspace pair.
 *   - A call whose pluto_gqa_decode_workspace_bytes(...) exceeds the area returns
 *     PLUTO_E_EXHAUSTED with the two sizes in pluto_last_error(); nothing is launched.
 *   - The entry point itself calls no cudaMalloc/cudaFree or allocating library routine.  The
 *     area is a static device array: the CUDA runtime gives it memory when it loads this
 *     library's device code on a GPU, which with lazy module loading (the default) happens at the
 *     first call on that GPU, not when the process loads the .so; the GPU then holds the 32 MiB
 *     until the process exits.  So make ONE warm-up call per device at start-up -- before the HBM
 *     plan is committed and before any stream capture: that call loads the device code, looks up
 *     the area's device address (cudaGetSymbolAddress, with that device current) and the status
 *     word's, and sets the kernels' shared-memory attribute.  Later calls touch no allocator.
 *   - `stream` must belong to the current device (PLUTO_E_INVALID otherwise): the area and the
 *     status word are per device and are looked up by the current device.
 *   - All calls share the one area.  Nothing in it has to start at zero (each call overwrites
 *     every partial it later reads), but two calls whose kernels overlap on the GPU -- different
 *     streams, or different host threads -- race on it: order them on one stream. */
int pluto_gqa_decode_noalloc(pluto_stream_t stream, const void* q, int q_dtype, const void* gate,
                             int gate_dtype, size_t gate_token_stride, size_t gate_head_stride,
                             const pluto_kv_cache* cache /* host */, const int32_t* seq_lens,
                             int max_seq_len, void* out, int out_dtype, float* lse, int batch,
                             int q_heads, int kv_heads, int head_dim, int round_to_bf16);

/* Size in bytes of the built-in area pluto_gqa_decode_noalloc uses (host-only query; no
 * counterpart in the reference). */
size_t pluto_gqa_decode_builtin_scratch_bytes(void);

/* Softmax row of the current query for the inspection hook.  Stands in for the cached
 * AttentionProbabilitiesKernel (cached_attention_ops.cc:131-178).  probs: fp32, row (b,h) at
 * probs + b*probs_batch_stride + h*probs_head_stride, seq_lens[b] entries written.  The
 * reference's [Hq, length] is (anything, length); the [Hq, T, T] tensor of the sequence layer's
 * hook is rows b = 0..T-1 with strides (T, T*T), seq_lens[b] = b + 1 and a block table that maps
 * every row to the same page. */
int pluto_gqa_decode_probs(pluto_stream_t stream, const void* q, int q_dtype,
                           const pluto_kv_cache* cache /* host */, const int32_t* seq_lens,
                           float* probs, size_t probs_batch_stride, size_t probs_head_stride,
                           int batch, int q_heads, int kv_heads, int head_dim);

/* --------------------------------------------------------------------------------------------
 * Gated delta-net.
 * pluto_gdn_gates: g = exp(-exp(A_log) * softplus(a + dt_bias)), beta = R(sigmoid(b)); the decay
 * and write-strength arithmetic of DeltaRecurrenceKernel (cached_attention_ops.cc:231-238).
 * a, b: [tokens, heads] (in_dtype); A_log, dt_bias fp32 [heads]; g, beta fp32 [tokens, heads]. */
int pluto_gdn_gates(pluto_stream_t stream, const void* a, const void* b, const float* a_log,
                    const float* dt_bias, int in_dtype, long long tokens, int heads,
                    int round_to_bf16, float* g, float* beta);

/* Causal depthwise convolution + SiLU.  Stands in for ConvolutionKernel
 * (cached_attention_ops.cc:180-203; tokens = 1) and ConvForward (sequence_delta_net.cc:31-51).
 * input/output [batch, tokens, channels]; weight fp32 [channels, width] oldest to newest;
 * state fp32 [batch, channels, width]: the last `width` rounded inputs, updated in place (zero it
 * for a fresh sequence).  width <= 32. */
int pluto_gdn_conv_silu(pluto_stream_t stream, const void* input, const float* weight,
                        int in_dtype, int batch, int tokens, int channels, int width,
                        int round_to_bf16, float* state, void* output, int out_dtype);

/* Bytes of scratch the chunked prefill path of pluto_gdn_prefill needs (host-only query; 0 when
 * the shape has no chunked path: it needs bf16 q/k/v, key_dim 128, value_dim a multiple of 32,
 * tokens >= 64). */
size_t pluto_gdn_prefill_workspace_bytes(int batch, int tokens, int key_heads, int value_heads,
                                         int key_dim, int value_dim, int in_dtype);

/* The recurrence over `tokens` tokens from the given state.  Stands in for RecurrenceForward
 * (src/llm/layers/sequence_delta_net.cc:55-102) without its per-token state history; with
 * tokens = 1 it is DeltaRecurrenceKernel (cached_attention_ops.cc:205-251).
 *   q, k         [batch, tokens, key_heads, key_dim];  v, out [batch, tokens, value_heads, value_dim]
 *   qk_token_stride, v_token_stride   elements between consecutive tokens of q/k and of v
 *                (0 = dense).  The reference's packed [T, all Q | all K | all V] activation is
 *                q = base, k = base + Hk*dk, v = base + 2*Hk*dk with both strides = channels.
 *   g, beta      fp32 [batch, tokens, value_heads]
 *   state        fp32 [batch, value_heads, key_dim, value_dim], read and updated in place
 *   normalize_qk 1: q^ = q*rsqrt(sum q^2 + 1e-6)/sqrt(key_dim), k^ = k*rsqrt(sum k^2 + 1e-6) as
 *                the reference; 0: use k as given and q * q_scale
 *   workspace    NULL: token-sequential kernel (the reference's arithmetic, state on chip).
 *                >= pluto_gdn_prefill_workspace_bytes(...) bytes, 256-byte aligned: chunked form
 *                (64-token chunks, in-chunk products on the tensor cores, fp32 state carried
 *                across chunks); same result within bf16 operand rounding.
 * key_dim <= 128, value_dim <= 256, value_heads % key_heads == 0. */
int pluto_gdn_prefill(pluto_stream_t stream, const void* q, const void* k, const void* v,
                      int in_dtype, const float* g, const float* beta, float* state, void* out,
                      int out_dtype, int batch, int tokens, int key_heads, int value_heads,
                      int key_dim, int value_dim, size_t qk_token_stride, size_t v_token_stride,
                      int normalize_qk, float q_scale, int round_to_bf16, void* workspace,
                      size_t workspace_bytes);

/* Single-token form of pluto_gdn_prefill (tokens = 1): DeltaRecurrenceKernel as launched by
 * DeltaNetState::Step (src/llm/layers/util/cached_attention_ops.cc:205-251, :401-431). */
int pluto_gdn_step(pluto_stream_t stream, const void* q, const void* k, const void* v,
                   int in_dtype, const float* g, const float* beta, float* state, void* out,
                   int out_dtype, int batch, int key_heads, int value_heads, int key_dim,
                   int value_dim, int normalize_qk, float q_scale, int round_to_bf16);

/* Per (token, head) RMSNorm * weight * SiLU(z).  Stands in for DeltaOutputKernel
 * (cached_attention_ops.cc:253-272; final_round = 1) and OutputForward
 * (sequence_delta_net.cc:104-121; final_round = 0: last product stored without the extra
 * rounding).  core, z, out: [rows, dim]; norm_weight fp32 [dim] (plain multiplier). */
int pluto_gdn_out_norm_gate(pluto_stream_t stream, const void* core, int core_dtype, const void* z,
                            int z_dtype, const float* norm_weight, long long rows, int dim,
                            float rms_norm_epsilon, int round_to_bf16, int final_round, void* out,
                            int out_dtype);

/* --------------------------------------------------------------------------------------------
 * Backward of the sequence gated delta-net, SequenceDeltaNetLayer::bwd_impl
 * (src/llm/layers/sequence_delta_net.cc:482-561), in the reference's three stages.  The
 * reference stores every intermediate state S_t and is limited to 128 tokens; the recurrence
 * pass here keeps one state per 64 tokens and recomputes inside a chunk, so any length runs.
 * Parameter gradients (d_norm_weight, d_a_log, d_dt_bias, d_weight; all optional) are
 * ACCUMULATED into, as the reference accumulates into BlockParameter::gradient().
 *
 * 1. pluto_gdn_out_norm_gate_bwd: OutputBackward + SumNormGradient (:126-171).  core (the rounded
 *    recurrence output saved by the forward, bf16 or fp32) and z are [rows, dim]; dy, dcore, dz
 *    fp32 [rows, dim]; rows = batch * tokens * value_heads.  The workspace is needed only with
 *    d_norm_weight.
 * 2. pluto_gdn_recurrence_bwd: RecurrenceBackward + GatherQkGradient + GatherScalarGradient
 *    (:176-309).  q, k, v are the convolved, SiLU'd activations (raw: the L2 normalisation of q
 *    and k and the 1/sqrt(key_dim) query scale are part of this stage and are differentiated
 *    here), addressed as in pluto_gdn_prefill; a, b the raw gate inputs [batch, tokens,
 *    value_heads]; dcore from stage 1.  dq, dk (token stride dqk_token_stride) and dv (token
 *    stride dv_token_stride) are fp32 and normally point into one [batch, tokens, channels]
 *    gradient of the convolved activations; da, db fp32 [batch, tokens, value_heads].
 *    key_dim <= 128, value_dim <= 256.  bf16 activations with key_dim = value_dim = 128 and 256
 *    tokens or more run chunk-parallel (the chunked forward again with the state kept at every
 *    64-token boundary, a reverse scan for the state gradients, then all chunks at once); everything
 *    else walks the sequence token by token.  The workspace query covers both.
 * 3. pluto_gdn_conv_silu_bwd: ConvSiluBackward + ConvInputBackward + ConvWeightBackward
 *    (:311-362) for sequences that start from an empty history.  input is the layer's QKV input
 *    [batch, tokens, channels]; d_post the gradient of the convolved activations; dx fp32. */
int pluto_gdn_out_norm_gate_bwd(pluto_stream_t stream, const void* core, int core_dtype,
                                const void* z, int z_dtype, const float* norm_weight,
                                const float* dy, float* dcore, float* dz, float* d_norm_weight,
                                void* workspace, size_t workspace_bytes, long long rows, int dim,
                                float rms_norm_epsilon, int round_to_bf16);
size_t pluto_gdn_out_norm_gate_bwd_workspace_bytes(long long rows, int dim);
size_t pluto_gdn_recurrence_bwd_workspace_bytes(int batch, int tokens, int key_heads, int value_heads,
                                                int key_dim, int value_dim);
int pluto_gdn_recurrence_bwd(pluto_stream_t stream, const void* q, const void* k, const void* v,
                             int in_dtype, size_t qk_token_stride, size_t v_token_stride,
                             const void* a, const void* b, int ab_dtype, const float* a_log,
                             const float* dt_bias, const float* dcore, float* dq, float* dk,
                             size_t dqk_token_stride, float* dv, size_t dv_token_stride, float* da,
                             float* db, float* d_a_log, float* d_dt_bias, void* workspace,
                             size_t workspace_bytes, int batch, int tokens, int key_heads,
                             int value_heads, int key_dim, int value_dim, int round_to_bf16);
int pluto_gdn_conv_silu_bwd(pluto_stream_t stream, const void* input, int in_dtype,
                            const float* weight, const float* d_post, float* dx, float* d_weight,
                            int batch, int tokens, int channels, int width, int round_to_bf16);

/* --------------------------------------------------------------------------------------------
 * Imported (frozen checkpoint) projection for a few tokens, FullyConnectedLayer::ImportedForward
 * (src/llm/layers/fully_connected.cc:295-341; kernels :40-95): output[t][r] = bf16(sum_c
 * W[r][c] * x[t][c]) in fp32 arithmetic.  weights [output_dim, input_dim] output-major in the
 * storage of MatrixStorage (src/llm/layers/matrix_common.h:11, same numbering): bf16, fp32, or
 * FP8 E4M3 bytes with fp32 block scales [ceil(output_dim/128), ceil(input_dim/128)]; for FP8 the
 * activation is first quantised to E4M3 in groups of 128 with a dynamic scale max|x|/448, as the
 * reference does.  input bf16 [tokens, input_dim], output bf16 [tokens, output_dim] (the reference
 * layer is single-token; several tokens share one pass over the weights here).  scales must be
 * null unless the storage is FP8. */
enum { PLUTO_MATRIX_BF16 = 0, PLUTO_MATRIX_FP32 = 1, PLUTO_MATRIX_FP8_E4M3 = 2 };
int pluto_linear_imported_fwd(pluto_stream_t stream, const void* weights, int storage,
                              const float* scales, const void* input, void* output, int tokens,
                              int input_dim, int output_dim);

/* --------------------------------------------------------------------------------------------
 * Trainable dense projection, FullyConnectedLayer::fwd_impl / bwd_impl
 * (src/llm/layers/fully_connected.cc:415-520; kernels :97-232), as tcgen05 GEMMs:
 *   forward   output = cast(input) * cast(matrix) + bias     [rows, output_dim], dtype of input
 *   backward  input_gradient  = cast(dY) * cast(matrix)^T    fp32 [rows, input_dim]
 *             matrix_gradient = cast(input)^T * cast(dY)     fp32 [input_dim, output_dim]
 *             bias_gradient   = column sums of dY            fp32 [output_dim]
 * matrix is the fp32 master copy [input_dim, output_dim] (input-major), bias fp32; input is bf16
 * (dtype PLUTO_BF16) or fp32 (PLUTO_FP32: the reference's FP16 compute policy); cast = bf16 or
 * fp16 respectively, accumulation fp32, as in the reference's tile MMAs.  The gradients are
 * overwritten, not accumulated, like the reference's.  workspace: device memory of
 * pluto_dense_workspace_bytes (the 2-byte operand copies), 256-byte aligned.  Any positive
 * extents (tiles are padded inside the workspace). */
size_t pluto_dense_workspace_bytes(int rows, int input_dim, int output_dim);
int pluto_dense_fwd(pluto_stream_t stream, const void* input, int dtype, const float* matrix,
                    const float* bias, void* output, int rows, int input_dim, int output_dim,
                    void* workspace, size_t workspace_bytes);
int pluto_dense_bwd(pluto_stream_t stream, const void* input, int dtype, const float* matrix,
                    const float* output_gradient, float* input_gradient, float* matrix_gradient,
                    float* bias_gradient, int rows, int input_dim, int output_dim, void* workspace,
                    size_t workspace_bytes);

/* --------------------------------------------------------------------------------------------
 * BlockLinearLayer and DequantizeMatrix (src/llm/layers/block_training.h:11-83,
 * block_training.cc:19-98, 281-399): resident bf16 weight [output_dim, input_dim] (output-major,
 * no bias), bf16 input [tokens, input_dim].
 *   forward   output[t][r] = sum_c x[t][c] W[r][c], fp32 accumulation, bf16 or fp32 output
 *   backward  input_gradient fp32 [tokens, input_dim] = dY W;  weight_gradient fp32
 *             [output_dim, input_dim] += dY^T x (ACCUMULATED; null for a frozen weight)
 * All three are tcgen05 GEMMs on the bf16 values; the fp32 dY enters as hi + lo bf16 halves so its
 * products keep 16 mantissa bits.  workspace: pluto_block_linear_workspace_bytes, 256-byte aligned.
 * pluto_dequantize_matrix converts an fp32 or FP8-E4M3 (fp32 block scales [ceil(rows/128),
 * ceil(cols/128)]) matrix to the resident bf16 form; bf16 matrices are shared, not converted. */
size_t pluto_block_linear_workspace_bytes(int tokens, int input_dim, int output_dim);
int pluto_block_linear_fwd(pluto_stream_t stream, const void* weight, const void* input, void* output,
                           int output_dtype, int tokens, int input_dim, int output_dim,
                           void* workspace, size_t workspace_bytes);
int pluto_block_linear_bwd(pluto_stream_t stream, const void* weight, const void* input,
                           const float* output_gradient, float* input_gradient,
                           float* weight_gradient, int tokens, int input_dim, int output_dim,
                           void* workspace, size_t workspace_bytes);
int pluto_dequantize_matrix(pluto_stream_t stream, const void* input, int storage, const float* scales,
                            void* output, int rows, int cols);

/* --------------------------------------------------------------------------------------------
 * Head-sharded multi-GPU support.  The reference is single-GPU (its only cudaSetDevice pins a
 * thread pool to one device, src/cuda/thread_pool.h:19-22, src/cuda/thread_pool.cc:109), so this
 * has no kernel to mirror: it is the local half of "all-gather the head-sharded output" for a
 * caller that wants the concatenated [rows, E] activation the next reference layer expects
 * (AttentionLayer output layout, src/llm/layers/attention.h:64-70).  The collective itself is the
 * caller's ncclAllGather into `gathered` = [ranks][rows][local_bytes]; this kernel rewrites it to
 * out = [rows][ranks * local_bytes].  Only local memory is touched. */
int pluto_interleave_heads(pluto_stream_t stream, const void* gathered, void* out, int ranks,
                           long long rows, size_t local_bytes);

/* The whole gather in one call, for a caller that owns an NCCL communicator over the head-sharded
 * ranks (same single-GPU reference as above, src/cuda/thread_pool.h:19-22: nothing to mirror; the
 * output is the [rows, E] layout of src/llm/layers/attention.h:64-70): ncclAllGather of `local`
 * ([rows][local_bytes], this rank's heads) into `gathered` ([ranks][rows][local_bytes], scratch
 * owned by the caller) on `stream`, then pluto_interleave_heads into out
 * ([rows][ranks * local_bytes]).  nccl_comm is the caller's ncclComm_t, passed as an opaque
 * pointer so this header needs no nccl.h; `ranks` must be its size.  The library does not link
 * NCCL: it binds ncclAllGather and ncclGetErrorString at first use to the NCCL already loaded in
 * the process (the communicator's own library), falling back to loading libnccl.so.2, and returns
 * PLUTO_E_UNIMPLEMENTED when neither is there.  NCCL moves the data over NVLink / NVSwitch into
 * this GPU's own memory; no kernel of this library reads peer memory.  Returns > 0 with the
 * ncclResult_t offset by 10000 when NCCL reports an error. */
int pluto_allgather_heads(pluto_stream_t stream, void* nccl_comm, const void* local,
                          void* gathered, void* out, int ranks, long long rows,
                          size_t local_bytes);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* PLUTO_B200_H_ */
