// Internal C++ interface between the C-ABI entry points (c_api.cu) and the kernel files.
// Everything here takes raw device pointers and a stream, allocates nothing and never
// synchronises; argument validation happens in c_api.cu before any of these run.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace pluto {

// Device word that kernels set when one of their bounded waits runs out (0 = healthy).
uint32_t* kernel_status_word();           // device address, per current device
cudaError_t read_kernel_status(uint32_t* host_value, bool clear);  // synchronising diagnostic
// Per-device state (status word, built-in scratch, copy lanes) is looked up by the CURRENT device;
// entry points that depend on it beyond the status word refuse a stream that belongs to another.
bool stream_on_current_device(cudaStream_t stream);

// ---- attn_generic.cu: exact fp32-math attention for every shape --------------------------------
cudaError_t attn_generic_fwd(cudaStream_t stream, const void* q, const void* k, const void* v,
                             void* out, float* maxima, float* normalizers, int batch, int seq,
                             int heads, int head_dim, size_t q_token, size_t q_head,
                             size_t kv_token, size_t kv_head, size_t out_token, size_t out_head,
                             int group, const void* gate, size_t gate_token, size_t gate_head,
                             float* core, int round_gate, bool bf16);
cudaError_t attn_generic_probs(cudaStream_t stream, const void* qkv, const float* maxima,
                               const float* normalizers, float* probs, int batch, int seq,
                               int heads, int head_dim, bool bf16);
cudaError_t attn_generic_bwd(cudaStream_t stream, const void* qkv, const void* out,
                             const float* d_out, const float* maxima, const float* normalizers,
                             float* d_qkv, float* deltas, int batch, int seq, int heads,
                             int head_dim, bool bf16);

// Backward of the causal attention core over separate tensors (element strides), `q_heads /
// kv_heads` query heads per key/value head.  q, k, v: bf16 or fp32 (`bf16`); d_out, dq, dk, dv,
// maxima, normalizers, deltas fp32; statistics indexed (b*q_heads + h)*seq + s.  With `out` set
// the deltas (row sums of d_out * out) are computed and stored; with `out` null they are read.
struct GqaBwdArgs {
  const void *q, *k, *v, *out;
  const float *d_out, *maxima, *normalizers;
  float *deltas, *dq, *dk, *dv;
  int batch, seq, q_heads, kv_heads, head_dim;
  size_t q_token, q_head, kv_token, kv_head, o_token, o_head, g_token, g_head;
  size_t dq_token, dq_head, dkv_token, dkv_head;
  bool bf16;
};
cudaError_t gqa_generic_bwd(cudaStream_t stream, const GqaBwdArgs& args);

// ---- qwen_bwd.cu: gate, RoPE^-1 + RMSNorm backward, norm-weight reduction -----------------------
struct GateBwdArgs {
  const __nv_bfloat16* gate;   // element strides gate_token / gate_head
  size_t gate_token, gate_head;
  const float* core;           // dense [B, S, Hq, D]
  const float* dy;             // dense
  float* dc;                   // dense
  float* d_gate;               // element strides dgate_token / dgate_head
  size_t dgate_token, dgate_head;
  float* deltas;               // [(b*Hq + h)*S + s]
  int batch, seq, q_heads, head_dim, round;
};
cudaError_t gqa_gate_bwd(cudaStream_t stream, const GateBwdArgs& args);
struct NormBwdArgs {
  const __nv_bfloat16* x;      // layer input, element strides x_token / x_head
  size_t x_token, x_head;
  const float* weight;         // zero-centred [D]
  const float* grad;           // dense [B, T, heads, D]: gradient of the rotated, normalised vector
  const int* positions;        // optional [B]: RoPE position of token 0 (null = 0)
  float* dx;                   // element strides dx_token / dx_head
  size_t dx_token, dx_head;
  float* parts;                // set by qk_prepare_bwd
  int batch, tokens, heads, head_dim, rotary;
  float epsilon, log_theta;
  int round;
};
size_t qk_prepare_bwd_workspace_bytes(long long rows, int head_dim);
cudaError_t qk_prepare_bwd(cudaStream_t stream, NormBwdArgs args, float* d_weight, void* workspace);

// ---- attn_bwd_sm100.cu: tcgen05 backward, bf16, head_dim 64 or 128 -----------------------------
size_t attn_bwd_tc_workspace_bytes(int batch, int seq, int heads, int head_dim);
cudaError_t attn_bwd_tc(cudaStream_t stream, const void* qkv, const void* out, const float* d_out,
                        const float* maxima, const float* normalizers, float* d_qkv, float* deltas,
                        void* workspace, int batch, int seq, int heads, int head_dim,
                        uint32_t* status);
// The same two passes over separate bf16 tensors with grouped query heads.  q has q_cols valid
// columns per token (token stride q_token elements), head h at column q_col0 + h*head_dim; k, v
// likewise with kv_cols / kv_token / k_col0, v_col0 and key/value head h/group.  d_out fp32 dense
// [batch, seq, q_heads*head_dim].  With `out` (bf16, dense) set, deltas are computed and stored;
// with `out` null they are read.  dq / dk / dv fp32, token strides dq_token / dkv_token, head
// stride head_dim.  workspace: attn_bwd_tc_workspace_bytes(batch, seq, q_heads, head_dim).
struct GqaBwdTcArgs {
  const void *q, *k, *v, *out;
  int q_cols, kv_cols, q_col0, k_col0, v_col0;
  size_t q_token, kv_token;
  const float *d_out, *maxima, *normalizers;
  float *deltas, *dq, *dk, *dv;
  size_t dq_token, dkv_token;
  void* workspace;
  int batch, seq, q_heads, kv_heads, head_dim;
  uint32_t* status;
};
cudaError_t gqa_bwd_tc(cudaStream_t stream, const GqaBwdTcArgs& args);

// ---- attn_fwd_sm100.cu: tcgen05 forward, bf16, head_dim 64 or 128 ------------------------------
struct AttnFwdArgs {
  const void* q;      // bf16; token stride q_token elements; q_cols valid columns per token
  const void* k;      // bf16; token stride kv_token; kv_cols valid columns per token
  const void* v;
  int q_cols, kv_cols;
  size_t q_token, kv_token;
  int q_col0, k_col0, v_col0;  // column of head 0 inside a token row
  int q_head_cols;             // column step between query heads (head_dim, or 2*head_dim when a
                               // gate is interleaved after every query head)
  int batch, seq, heads, group, head_dim;
  void* out;                   // bf16 [batch*seq tokens]: element stride out_token / out_head
  size_t out_token, out_head;
  float* maxima;               // optional fp32 [(b*heads+h)*seq + s]
  float* normalizers;
  float* core;                 // optional fp32, indexed like out
  const void* gate;            // optional bf16, gate_token / gate_head element strides
  size_t gate_token, gate_head;
  int round_gate;
  void* workspace;             // optional, attn_fwd_tc_workspace_bytes: enables the key/value split
  uint32_t* status;
  int tile_begin, tile_count;  // query tiles (128 rows) to compute; tile_count 0 = all of them
};
cudaError_t attn_fwd_tc(cudaStream_t stream, const AttnFwdArgs& args);
size_t attn_fwd_tc_workspace_bytes(int batch, int seq, int heads, int head_dim);
// ... or 0 when the launch plan for this shape cuts no tile pair (the scratch would not be used)
size_t attn_fwd_tc_split_workspace_bytes(int batch, int seq, int heads, int head_dim);
bool make_token_map(CUtensorMap* map, const void* base, int cols, int seq, int batch,
                    size_t token_stride, int box_rows);


// ---- gqa_decode.cu ------------------------------------------------------------------------------
// Cache addressing: token t of sequence b, kv head h starts at element
//   page(b, t) * page_stride + (t % page_size) * token_stride + h * head_dim,
// page(b, t) = block_table ? block_table[b * max_blocks + t / page_size] : b.
struct DecodeArgs {
  const void* q;            // [batch, q_heads, head_dim], already normalised/rotated
  int q_is_bf16;
  const void* gate;         // optional; element (b, h, d) at b*gate_token + h*gate_head + d
  int gate_is_bf16;
  size_t gate_token, gate_head;
  const void* k_base;
  const void* v_base;
  const void* const* k_bases;   // optional device arrays [batch] of per-sequence bases: sequence b's token
  const void* const* v_bases;   // t then starts at t * token_stride of k_bases[b] (no pages)
  int kv_is_bf16;
  const int32_t* block_table;
  int max_blocks, page_size;
  size_t page_stride, token_stride;
  int num_pages;            // pages in the pool (needed for the TMA map when a block table is used)
  int box_rows;             // filled by gqa_decode: tokens per TMA box
  const int32_t* seq_lens;  // [batch], number of cached tokens to attend to (>= 1)
  void* out;                // [batch, q_heads, head_dim]
  int out_is_bf16;
  float* lse;               // optional [batch, q_heads]
  float* partial_ml;        // workspace [batch, q_heads, splits, 2], 8-byte aligned (first section)
  float* partial_acc;       // workspace [batch, q_heads, splits, head_dim] (second section)
  int batch, q_heads, kv_heads, head_dim;
  int splits, split_tokens;
  float scale;
  int round;
  uint32_t* status;
};
// Chunks of the split-KV decode.  A sequence is cut into chunks of `split_tokens` tokens, except
// that its first split_tokens tokens form four chunks of a quarter each; the kernels run the
// chunks in decreasing index order, so that these short ones fill the end of the launch, where
// whole-length chunks would leave most SMs waiting for the last few.  (One KV head of 64 sequences:
// 4.1 waves of equal chunks cost 5.)  split_tokens is a multiple of 256.
__host__ __device__ inline int decode_chunk_begin(int s, int split_tokens) {
  return s < 4 ? s * (split_tokens / 4) : (s - 3) * split_tokens;
}
__host__ __device__ inline int decode_chunk_tokens(int s, int split_tokens) {
  return s < 4 ? split_tokens / 4 : split_tokens;
}
__host__ __device__ inline int decode_chunk_count(int length, int split_tokens) {   // chunks with a token
  if (length <= 0) return 0;
  return length <= split_tokens ? (length + split_tokens / 4 - 1) / (split_tokens / 4)
                                : 3 + (length + split_tokens - 1) / split_tokens;
}
__host__ __device__ inline long long decode_chunk_capacity(int splits, int split_tokens) {   // tokens `splits` chunks hold
  return splits < 4 ? static_cast<long long>(splits) * (split_tokens / 4)
                    : static_cast<long long>(splits - 3) * split_tokens;
}
bool gqa_decode_uses_tensor_cores(const DecodeArgs& args);
// Floats of the (max, sum) section at the start of the decode workspace; the accumulators
// [batch, q_heads, splits, head_dim] follow it.  Always an even count, so a workspace aligned to
// 8 bytes or more keeps the pairs 8-byte aligned whatever head_dim is.
inline size_t decode_ml_floats(int batch, int q_heads, int splits) {
  return static_cast<size_t>(batch) * q_heads * splits * 2;
}
cudaError_t gqa_decode(cudaStream_t stream, const DecodeArgs& args);
cudaError_t gqa_decode_probabilities(cudaStream_t stream, const DecodeArgs& args, float* probs,
                                     size_t batch_stride, size_t head_stride);

// ---- qk_prepare.cu ------------------------------------------------------------------------------
struct PrepareArgs {
  const void* q_in;         // token/head element strides q_token, q_head
  const void* k_in;         // [batch*tokens, kv_heads, head_dim]
  const void* v_in;
  int in_is_bf16;
  size_t q_token, q_head;
  const float* q_norm;      // [head_dim], zero-centred
  const float* k_norm;
  const int32_t* positions; // optional [batch]: position of token 0 of each sequence
  void* q_out;              // [batch*tokens, q_heads, head_dim]
  int q_out_is_bf16;
  void* k_cache;            // cache addressing as in DecodeArgs
  void* v_cache;
  const void* const* k_bases;   // optional per-sequence base pointers (then k_cache / v_cache are unused)
  const void* const* v_bases;
  int kv_is_bf16;
  const int32_t* block_table;
  int max_blocks, page_size;
  size_t page_stride, token_stride;
  int batch, tokens, q_heads, kv_heads, head_dim, rotary;
  float epsilon, log_theta;
  int round;
};
cudaError_t qk_prepare(cudaStream_t stream, const PrepareArgs& args);

// ---- gdn.cu -------------------------------------------------------------------------------------
struct GdnArgs {
  const void* q;            // [batch, tokens, key_heads, key_dim]
  const void* k;
  const void* v;            // [batch, tokens, value_heads, value_dim]
  int in_is_bf16;
  size_t qk_token;          // elements between tokens of q / k (key_heads*key_dim when dense)
  size_t v_token;           // elements between tokens of v (value_heads*value_dim when dense)
  const float* g;           // [batch, tokens, value_heads] decay in (0, 1]
  const float* beta;        // [batch, tokens, value_heads]
  float* state;             // [batch, value_heads, key_dim, value_dim], updated in place
  void* out;                // [batch, tokens, value_heads, value_dim]
  int out_is_bf16;
  int batch, tokens, key_heads, value_heads, key_dim, value_dim;
  int normalize_qk;
  float q_scale;
  int round;
};
cudaError_t gdn_recurrent(cudaStream_t stream, const GdnArgs& args);
// gdn_chunked.cu: chunked (64-token) form for bf16 inputs with key_dim 128
bool gdn_chunked_supported(const GdnArgs& args);
size_t gdn_chunked_workspace_bytes(int batch, int tokens, int value_heads, int value_dim);
cudaError_t gdn_chunked(cudaStream_t stream, const GdnArgs& args, void* workspace, uint32_t* status);
// ---- c_api.cu: per-thread error text for entry points defined outside it -----------------------------
int report(int code, const char* message);
int report_cuda(cudaError_t e, const char* what);

// ---- linear_gemv.cu: imported output-major projection; storage 0 fp32, 1 bf16, 2 FP8 E4M3 ---------
cudaError_t linear_imported(cudaStream_t stream, const void* weights, int storage, const float* scales,
                            const void* x, void* y, int tokens, int cols, int rows);

// ---- gemm_sm100.cu: trainable dense projection (tcgen05 GEMMs over 2-byte casts of the operands) --
size_t dense_workspace_bytes(int rows, int in, int out);
cudaError_t dense_fwd(cudaStream_t stream, const void* x, bool x_is_bf16, const float* w,
                      const float* bias, void* y, int rows, int in, int out, void* workspace,
                      uint32_t* status);
cudaError_t dense_bwd(cudaStream_t stream, const void* x, bool x_is_bf16, const float* w,
                      const float* dy, float* dx, float* dw, float* db, int rows, int in, int out,
                      void* workspace, uint32_t* status);

// BlockLinearLayer: resident bf16 weight [out, in], bf16 x [tokens, in]; see gemm_sm100.cu
size_t block_linear_workspace_bytes(int tokens, int in, int out);
cudaError_t block_linear_fwd(cudaStream_t stream, const void* weight, const void* x, void* y,
                             bool y_is_fp32, int tokens, int in, int out, void* workspace,
                             uint32_t* status);
cudaError_t block_linear_bwd(cudaStream_t stream, const void* weight, const void* x, const float* dy,
                             float* dx, float* d_weight, int tokens, int in, int out, void* workspace,
                             uint32_t* status);
// storage 1 = fp32, 2 = FP8 E4M3 with block scales -> bf16 [rows, cols]
cudaError_t dequantize_matrix(cudaStream_t stream, const void* input, int storage, const float* scales,
                              long long rows, int cols, void* output);

// gdn_bwd.cu: backward of the sequence layer
struct GdnBwdArgs {
  const void* q;            // convolved + SiLU'd activations, as GdnArgs (raw, not normalised)
  const void* k;
  const void* v;
  int in_is_bf16;
  size_t qk_token, v_token;
  const void* a_in;         // raw a, b inputs [batch, tokens, value_heads]
  const void* b_in;
  int ab_is_bf16;
  const float* a_log;       // [value_heads]
  const float* dt_bias;
  const float* dcore;       // [batch, tokens, value_heads, value_dim] fp32
  float* dv_out;            // gradient of v, element stride dv_token between tokens
  size_t dv_token;
  float *checkpoints, *scratch, *qk_partials, *scalar_partials;   // set by gdn_recurrence_bwd
  int batch, tokens, key_heads, value_heads, key_dim, value_dim, round;
};
cudaError_t gdn_out_bwd(cudaStream_t stream, const void* core, int core_is_bf16, const void* z,
                        int z_is_bf16, const float* norm, const float* dy, long long rows, int dim,
                        float epsilon, int round, float* dcore, float* dz, float* parts);
size_t gdn_recurrence_bwd_workspace_bytes(int batch, int tokens, int value_heads, int key_dim,
                                          int value_dim);
cudaError_t gdn_recurrence_bwd(cudaStream_t stream, GdnBwdArgs args, float* dq_out, float* dk_out,
                               size_t dqk_token, float* da, float* db, float* d_a_log,
                               float* d_dt_bias, void* workspace);
// gdn_bwd_chunked.cu: chunk-parallel form (two tensor-core scans + one CTA per chunk) for bf16
// activations with key width = value width = 128; fills scalar_partials (one tile per head), dv_out
// and the q / k gradients (directly when *qk_direct comes back true, else as qk_partials)
bool gdn_bwd_chunked_supported(const GdnBwdArgs& args);
size_t gdn_bwd_chunked_workspace_bytes(int batch, int tokens, int value_heads);
cudaError_t gdn_bwd_chunked(cudaStream_t stream, GdnBwdArgs& args, float* dq_out, float* dk_out, size_t dqk_token,
                            void* workspace, uint32_t* status, bool* qk_direct);
cudaError_t gdn_conv_bwd(cudaStream_t stream, const void* input, int in_is_bf16, const float* weight,
                         const float* dpost, int batch, int tokens, int channels, int width, int round,
                         float* dx, float* d_weight);
// qwen_bwd.cu: dst[c] += sum over rows of parts[row, c] in a fixed order; chunk_scratch holds
// ceil(rows / 1024) * dim floats
cudaError_t reduce_rows_accumulate(cudaStream_t stream, const float* parts, long long rows, int dim,
                                   float* chunk_scratch, float* dst);
size_t reduce_rows_scratch_floats(long long rows, int dim);
cudaError_t gdn_gates(cudaStream_t stream, const void* a_in, const void* b_in, const float* a_log,
                      const float* dt_bias, int in_is_bf16, long long tokens, int heads, int round,
                      float* g, float* beta);
cudaError_t gdn_conv(cudaStream_t stream, const void* input, const float* weight, int in_is_bf16,
                     int batch, int tokens, int channels, int width, int round, float* state,
                     void* output, int out_is_bf16);
cudaError_t gdn_output(cudaStream_t stream, const void* core, const void* z,
                       const float* norm_weight, int core_is_bf16, int z_is_bf16, long long rows,
                       int dim, float epsilon, int round, int final_round, void* output,
                       int out_is_bf16);


// ---- interleave.cu ------------------------------------------------------------------------------
cudaError_t interleave_heads(cudaStream_t stream, const void* gathered, void* out, int ranks,
                             long long rows, size_t local_bytes);

}  // namespace pluto
