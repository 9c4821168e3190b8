// Internal C++ interface between the C-ABI entry points (c_api.cu) and the kernel files.
// Everything here takes raw device pointers and a stream, allocates nothing and never
// synchronises; argument validation happens in c_api.cu before any of these run.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace pluto {

// Device word that kernels set when one of their bounded waits runs out (0 = healthy).
uint32_t* kernel_status_word();           // device address, per current device
cudaError_t read_kernel_status(uint32_t* host_value, bool clear);  // synchronising diagnostic

// ---- attn_generic.cu: exact fp32-math attention for every shape --------------------------------
cudaError_t attn_generic_fwd(cudaStream_t stream, const void* q, const void* k, const void* v,
                             void* out, float* maxima, float* normalizers, int batch, int seq,
                             int heads, int head_dim, size_t q_token, size_t q_head,
                             size_t kv_token, size_t kv_head, size_t out_token, size_t out_head,
                             int group, const void* gate, float* core, int round_gate,
                             bool bf16);
cudaError_t attn_generic_probs(cudaStream_t stream, const void* qkv, const float* maxima,
                               const float* normalizers, float* probs, int batch, int seq,
                               int heads, int head_dim, bool bf16);
cudaError_t attn_generic_bwd(cudaStream_t stream, const void* qkv, const void* out,
                             const float* d_out, const float* maxima, const float* normalizers,
                             float* d_qkv, float* deltas, int batch, int seq, int heads,
                             int head_dim, bool bf16);

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
  uint32_t* status;
};
cudaError_t attn_fwd_tc(cudaStream_t stream, const AttnFwdArgs& args);
bool make_token_map(CUtensorMap* map, const void* base, int cols, int seq, int batch,
                    size_t token_stride, int box_rows);

}  // namespace pluto
