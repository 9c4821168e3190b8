// Elementwise pieces of the Qwen sequence-attention backward
// (src/llm/layers/qwen_attention.cc:120-239): the sigmoid output gate, the inverse partial RoPE
// followed by the per-head RMSNorm backward, and the deterministic reduction of the shared
// norm-weight gradient.  The attention core between them runs in attn_generic.cu
// (gqa_generic_bwd).  One CTA of 256 threads per (token, head); head width <= 256.
#include "common.cuh"
#include "engine.h"

namespace pluto {
namespace {

__device__ __forceinline__ float rnd(float v, int round) { return round ? bf16_round(v) : v; }

// Sum over the 256 threads of a CTA in a fixed order (warp shuffles, then warp 0..7 in sequence).
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();   // red may still be read from a previous call
  if (threadIdx.x % 32 == 0) red[threadIdx.x / 32] = v;
  __syncthreads();
  float total = 0.0f;
#pragma unroll
  for (int w = 0; w < 8; ++w) total += red[w];
  return total;
}

// GateBackwardKernel (:123-138): dc = dy * R(sigmoid(gate)); d_gate = dy * R(core) * s * (1 - s),
// s in fp32.  Also the row term of the softmax backward, delta = dc . core with the unrounded
// core (QueryBackwardKernel :153-155), so the core pass only reads it.
// One warp per (token, head), eight per CTA; a lane covers kPer consecutive channels per step of
// 32 * kPer (kPer = 4 with 16-byte accesses when the width and strides allow it).
template <int kPer>
__global__ void __launch_bounds__(256) gate_bwd_kernel(GateBwdArgs a, long long rows) {
  const long long row = static_cast<long long>(blockIdx.x) * 8 + threadIdx.x / 32;
  if (row >= rows) return;
  const int lane = threadIdx.x % 32, D = a.head_dim;
  const long long token = row / a.q_heads;
  const int h = static_cast<int>(row % a.q_heads);
  const int b = static_cast<int>(token / a.seq), s = static_cast<int>(token % a.seq);
  const size_t dense = static_cast<size_t>(row) * D;
  const __nv_bfloat16* gate = a.gate + static_cast<size_t>(token) * a.gate_token + static_cast<size_t>(h) * a.gate_head;
  float* d_gate = a.d_gate + static_cast<size_t>(token) * a.dgate_token + static_cast<size_t>(h) * a.dgate_head;
  float part = 0.0f;
  for (int c0 = lane * kPer; c0 < D; c0 += 32 * kPer) {
    float g[kPer], grad[kPer], core[kPer], dc[kPer], dg[kPer];
    if (kPer == 4) {
      const uint2 raw = *reinterpret_cast<const uint2*>(gate + c0);
      g[0] = bf16_lo(raw.x); g[1] = bf16_hi(raw.x); g[2] = bf16_lo(raw.y); g[3] = bf16_hi(raw.y);
      const float4 y = *reinterpret_cast<const float4*>(a.dy + dense + c0);
      const float4 c = *reinterpret_cast<const float4*>(a.core + dense + c0);
      grad[0] = y.x; grad[1] = y.y; grad[2] = y.z; grad[3] = y.w;
      core[0] = c.x; core[1] = c.y; core[2] = c.z; core[3] = c.w;
    } else {
      g[0] = __bfloat162float(gate[c0]);
      grad[0] = a.dy[dense + c0];
      core[0] = a.core[dense + c0];
    }
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      const float sigmoid = 1.0f / (1.0f + expf(-g[i]));
      dc[i] = grad[i] * rnd(sigmoid, a.round);
      dg[i] = grad[i] * rnd(core[i], a.round) * sigmoid * (1.0f - sigmoid);
      part = fmaf(dc[i], core[i], part);
    }
    if (kPer == 4) {
      *reinterpret_cast<float4*>(a.dc + dense + c0) = make_float4(dc[0], dc[1], dc[2], dc[3]);
      *reinterpret_cast<float4*>(d_gate + c0) = make_float4(dg[0], dg[1], dg[2], dg[3]);
    } else {
      a.dc[dense + c0] = dc[0];
      d_gate[c0] = dg[0];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  if (lane == 0) a.deltas[(static_cast<size_t>(b) * a.q_heads + h) * a.seq + s] = part;
}

// NormBackwardKernel (:196-226): rotate the gradient back with the rounded cos/sin of the forward,
// then the RMSNorm backward; `parts` (optional) receives normalized_grad * x * inv per row.
__global__ void __launch_bounds__(256) norm_bwd_kernel(NormBwdArgs a) {
  __shared__ float red[8];
  const int token = blockIdx.x / a.heads, h = blockIdx.x % a.heads;
  const int b = token / a.tokens, t = token % a.tokens;
  const int c = threadIdx.x, D = a.head_dim;
  const int position = (a.positions ? a.positions[b] : 0) + t;
  const size_t dense = (static_cast<size_t>(token) * a.heads + h) * D;
  const size_t in0 = static_cast<size_t>(token) * a.x_token + static_cast<size_t>(h) * a.x_head;
  const float x = c < D ? __bfloat162float(a.x[in0 + c]) : 0.0f;
  const float inv = rsqrtf(block_sum(x * x, red) / static_cast<float>(D) + a.epsilon);
  float ng = 0.0f, weighted = 0.0f;
  if (c < D) {
    ng = a.grad[dense + c];
    if (c < a.rotary) {
      const int half = a.rotary / 2;
      const int partner = c < half ? c + half : c - half;
      const int f = c < half ? c : c - half;
      const float angle = static_cast<float>(position) *
                          expf(static_cast<float>(f) * (-2.0f * a.log_theta / static_cast<float>(a.rotary)));
      const float co = rnd(cosf(angle), a.round), si = rnd(sinf(angle), a.round);
      const float gp = a.grad[dense + partner];
      ng = ng * co + (c < half ? gp * si : -gp * si);
    }
    weighted = ng * (1.0f + a.weight[c]);
  }
  const float dot = block_sum(weighted * x, red);
  if (c < D) {
    a.dx[static_cast<size_t>(token) * a.dx_token + static_cast<size_t>(h) * a.dx_head + c] =
        inv * weighted - x * (inv * inv * inv / static_cast<float>(D)) * dot;
    if (a.parts) a.parts[dense + c] = ng * x * inv;
  }
}

// ReduceNormKernel (:228-239) in two fixed-order levels: CTA i sums rows [i*kChunk, (i+1)*kChunk)
// per column, then one CTA sums the chunk rows in order and accumulates into the gradient.
constexpr int kChunk = 1024;
__global__ void __launch_bounds__(256) norm_reduce_chunks(const float* parts, long long rows, int D,
                                                          float* chunk_sums) {
  const int c = threadIdx.x;
  if (c >= D) return;
  const long long r0 = static_cast<long long>(blockIdx.x) * kChunk;
  const long long r1 = r0 + kChunk < rows ? r0 + kChunk : rows;
  float sum = 0.0f;
  for (long long r = r0; r < r1; ++r) sum += parts[r * D + c];
  chunk_sums[static_cast<size_t>(blockIdx.x) * D + c] = sum;
}
__global__ void __launch_bounds__(256) norm_reduce_final(const float* chunk_sums, int chunks, int D,
                                                         float* dw) {
  const int c = threadIdx.x;
  if (c >= D) return;
  float sum = 0.0f;
  for (int i = 0; i < chunks; ++i) sum += chunk_sums[static_cast<size_t>(i) * D + c];
  dw[c] += sum;
}

}  // namespace

cudaError_t gqa_gate_bwd(cudaStream_t stream, const GateBwdArgs& a) {
  const long long rows = static_cast<long long>(a.batch) * a.seq * a.q_heads;
  const unsigned blocks = static_cast<unsigned>((rows + 7) / 8);
  const auto aligned = [](const void* p, size_t n) { return reinterpret_cast<uintptr_t>(p) % n == 0; };
  const bool vector = a.head_dim % 4 == 0 && a.gate_token % 4 == 0 && a.gate_head % 4 == 0 &&
                      a.dgate_token % 4 == 0 && a.dgate_head % 4 == 0 && aligned(a.gate, 8) &&
                      aligned(a.dy, 16) && aligned(a.core, 16) && aligned(a.dc, 16) &&
                      aligned(a.d_gate, 16);
  if (vector) gate_bwd_kernel<4><<<blocks, 256, 0, stream>>>(a, rows);
  else gate_bwd_kernel<1><<<blocks, 256, 0, stream>>>(a, rows);
  return cudaGetLastError();
}

size_t qk_prepare_bwd_workspace_bytes(long long rows, int head_dim) {
  const long long chunks = (rows + kChunk - 1) / kChunk;
  return static_cast<size_t>(rows + chunks) * head_dim * sizeof(float);
}

cudaError_t qk_prepare_bwd(cudaStream_t stream, NormBwdArgs a, float* d_weight, void* workspace) {
  const long long rows = static_cast<long long>(a.batch) * a.tokens * a.heads;
  a.parts = d_weight ? static_cast<float*>(workspace) : nullptr;
  norm_bwd_kernel<<<static_cast<unsigned>(rows), 256, 0, stream>>>(a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess || d_weight == nullptr) return e;
  return reduce_rows_accumulate(stream, a.parts, rows, a.head_dim,
                                a.parts + static_cast<size_t>(rows) * a.head_dim, d_weight);
}

size_t reduce_rows_scratch_floats(long long rows, int dim) {
  return static_cast<size_t>((rows + kChunk - 1) / kChunk) * dim;
}

cudaError_t reduce_rows_accumulate(cudaStream_t stream, const float* parts, long long rows, int dim,
                                   float* chunk_scratch, float* dst) {
  const int chunks = static_cast<int>((rows + kChunk - 1) / kChunk);
  norm_reduce_chunks<<<chunks, 256, 0, stream>>>(parts, rows, dim, chunk_scratch);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  norm_reduce_final<<<1, 256, 0, stream>>>(chunk_scratch, chunks, dim, dst);
  return cudaGetLastError();
}

}  // namespace pluto
