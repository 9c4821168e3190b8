// Per-head RMSNorm(1 + w) -> optional bf16 rounding -> split-half partial RoPE for queries and
// keys, plus the K/V append into the cache.  Stands in for PrepareAttentionKernel
// (src/llm/layers/util/cached_attention_ops.cc:30-79) and its sequence form PrepareKernel
// (src/llm/layers/qwen_attention.cc:30-63): the rounding sequence
//     n = R(x * inv * (1 + w));  out = R(R(n * R(cos)) + R(+-n_partner * R(sin)))
// is reproduced step by step because the reference pins sequence and cached paths to bit equality.
// One CTA of 256 threads per (token, head); token (b, t) has RoPE position positions[b] + t.
#include "common.cuh"
#include "engine.h"

namespace pluto {
namespace {

__device__ __forceinline__ float load_in(const void* p, size_t i, int is_bf16) {
  return is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i])
                 : static_cast<const float*>(p)[i];
}
__device__ __forceinline__ void store_out(void* p, size_t i, int is_bf16, float v) {
  if (is_bf16) static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else static_cast<float*>(p)[i] = v;
}
__device__ __forceinline__ float rnd(float v, int round) { return round ? bf16_round(v) : v; }

__global__ void __launch_bounds__(256) qk_prepare_kernel(PrepareArgs a) {
  const int heads = a.q_heads + a.kv_heads;
  const int token = blockIdx.x / heads, head = blockIdx.x % heads;
  const int b = token / a.tokens, t = token % a.tokens;
  const bool is_query = head < a.q_heads;
  const int h = is_query ? head : head - a.q_heads;
  const int D = a.head_dim, c = threadIdx.x;
  const int position = (a.positions ? a.positions[b] : 0) + t;
  const size_t in0 = is_query ? static_cast<size_t>(token) * a.q_token + static_cast<size_t>(h) * a.q_head
                              : (static_cast<size_t>(token) * a.kv_heads + h) * D;
  const void* in = is_query ? a.q_in : a.k_in;
  const float* norm = is_query ? a.q_norm : a.k_norm;

  const float x = c < D ? load_in(in, in0 + c, a.in_is_bf16) : 0.0f;
  __shared__ float red[8];
  float sq = x * x;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  if (c % 32 == 0) red[c / 32] = sq;
  __syncthreads();
  float total = 0.0f;
#pragma unroll
  for (int w = 0; w < 8; ++w) total += red[w];
  const float inverse = rsqrtf(total / static_cast<float>(D) + a.epsilon);

  // destination row: queries are dense [B, T, Hq, D]; keys/values go to the cache layout
  size_t kv_off = 0;
  void* k_dst = a.k_cache;
  void* v_dst = a.v_cache;
  if (!is_query && a.k_bases != nullptr) {   // separately allocated sequences
    k_dst = const_cast<void*>(a.k_bases[b]);
    v_dst = const_cast<void*>(a.v_bases[b]);
    kv_off = static_cast<size_t>(position) * a.token_stride + static_cast<size_t>(h) * D;
  } else if (!is_query) {
    const int page = a.block_table ? a.block_table[static_cast<size_t>(b) * a.max_blocks + position / a.page_size] : b;
    kv_off = static_cast<size_t>(page) * a.page_stride +
             static_cast<size_t>(position % a.page_size) * a.token_stride + static_cast<size_t>(h) * D;
  }
  if (c < D) {
    const float n = rnd(x * inverse * (1.0f + norm[c]), a.round);
    float result = n;
    if (c < a.rotary) {
      const int half = a.rotary / 2;
      const int partner = c < half ? c + half : c - half;
      float rotated = rnd(load_in(in, in0 + partner, a.in_is_bf16) * inverse * (1.0f + norm[partner]), a.round);
      if (c < half) rotated = -rotated;
      const int f = c < half ? c : c - half;
      const float angle = static_cast<float>(position) *
                          expf(static_cast<float>(f) * (-2.0f * a.log_theta / static_cast<float>(a.rotary)));
      const float cosine = rnd(cosf(angle), a.round), sine = rnd(sinf(angle), a.round);
      result = rnd(rnd(n * cosine, a.round) + rnd(rotated * sine, a.round), a.round);
    }
    if (is_query) {
      store_out(a.q_out, (static_cast<size_t>(token) * a.q_heads + h) * D + c, a.q_out_is_bf16, result);
    } else {
      store_out(k_dst, kv_off + c, a.kv_is_bf16, result);
      const float value = load_in(a.v_in, (static_cast<size_t>(token) * a.kv_heads + h) * D + c, a.in_is_bf16);
      store_out(v_dst, kv_off + c, a.kv_is_bf16, rnd(value, a.round));
    }
  }
}

}  // namespace

cudaError_t qk_prepare(cudaStream_t stream, const PrepareArgs& a) {
  const long long blocks = static_cast<long long>(a.batch) * a.tokens * (a.q_heads + a.kv_heads);
  qk_prepare_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace pluto
