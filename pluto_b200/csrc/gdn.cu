// Gated delta-net: the token-sequential recurrence with the state held on chip, plus the small
// operators either side of it.
//
// Reference kernels these stand in for:
//   DeltaRecurrenceKernel      src/llm/layers/util/cached_attention_ops.cc:205-251  (one token)
//   RecurrenceForward          src/llm/layers/sequence_delta_net.cc:55-102          (a sequence)
//   ConvolutionKernel          cached_attention_ops.cc:180-203,  ConvForward  sequence_delta_net.cc:31-51
//   DeltaOutputKernel          cached_attention_ops.cc:253-272,  OutputForward sequence_delta_net.cc:104-121
// The reference streams a [128 x 32] fp32 slice of the state through HBM for every token and, in
// the sequence layer, stores every intermediate state.  gdn_recurrent keeps a [dk x 32] slice in
// registers for the whole sequence: the state is read once and written once per launch, only the
// token vectors stream in.  The arithmetic per token is the reference's, in its order:
//     S <- g S;  delta = (v - S^T k) * beta;  S <- S + k (x) delta;  o = R(S^T q)
#include "common.cuh"
#include "engine.h"

namespace pluto {
namespace {

__device__ __forceinline__ float load_any(const void* p, size_t i, int is_bf16) {
  return is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i])
                 : static_cast<const float*>(p)[i];
}
__device__ __forceinline__ void store_any(void* p, size_t i, int is_bf16, float v) {
  if (is_bf16) static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else static_cast<float*>(p)[i] = v;
}
__device__ __forceinline__ float rnd(float v, int round) { return round ? bf16_round(v) : v; }

constexpr int kSlice = 32;    // value columns per CTA
constexpr int kRowGroups = 4; // each thread owns 32 key rows of one column
constexpr int kBlockT = 16;   // tokens staged per shared-memory block
constexpr int kRecThreads = kSlice * kRowGroups;  // 128

// grid (ceil(dv / 32), value heads, batch)
__global__ void __launch_bounds__(kRecThreads) gdn_recurrent_kernel(GdnArgs a) {
  const int slice = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int kh = h / (a.value_heads / a.key_heads);
  const int dk = a.key_dim, dv = a.value_dim;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  // lane = (column % 8) * 4 + row group, so the 4 partial sums of a column sit in one quad
  const int rg = lane & 3;
  const int col = slice * kSlice + warp * 8 + (lane >> 2);
  const bool col_ok = col < dv;

  __shared__ float sq[2][kBlockT][128];
  __shared__ float sk[2][kBlockT][128];
  __shared__ float sv[2][kBlockT][kSlice];
  __shared__ float sg[2][kBlockT], sb[2][kBlockT];

  float S[32];
  float* state = a.state + ((static_cast<size_t>(b) * a.value_heads + h) * dk) * dv;
#pragma unroll
  for (int r = 0; r < 32; ++r) {
    const int row = rg * 32 + r;
    S[r] = (col_ok && row < dk) ? state[static_cast<size_t>(row) * dv + col] : 0.0f;
  }

  auto stage = [&](int buf, int t0) {
    // q, k vectors of up to kBlockT tokens (normalised here), this slice of v, the two gates; a
    // single-token step stages one token, not sixteen
    const int n_tok = min(kBlockT, a.tokens - t0);
    for (int idx = threadIdx.x; idx < n_tok * 128; idx += kRecThreads) {
      const int tt = idx / 128, i = idx % 128, t = t0 + tt;
      float qv = 0.0f, kv = 0.0f;
      if (t < a.tokens && i < dk) {
        const size_t off = (static_cast<size_t>(b) * a.tokens + t) * a.qk_token + static_cast<size_t>(kh) * dk + i;
        qv = load_any(a.q, off, a.in_is_bf16);
        kv = load_any(a.k, off, a.in_is_bf16);
      }
      sq[buf][tt][i] = qv;
      sk[buf][tt][i] = kv;
    }
    for (int idx = threadIdx.x; idx < n_tok * kSlice; idx += kRecThreads) {
      const int tt = idx / kSlice, j = idx % kSlice, t = t0 + tt, c = slice * kSlice + j;
      float x = 0.0f;
      if (t < a.tokens && c < dv)
        x = load_any(a.v, (static_cast<size_t>(b) * a.tokens + t) * a.v_token + static_cast<size_t>(h) * dv + c,
                     a.in_is_bf16);
      sv[buf][tt][j] = x;
    }
    if (threadIdx.x < n_tok) {
      const int t = t0 + threadIdx.x;
      const size_t off = (static_cast<size_t>(b) * a.tokens + min(t, a.tokens - 1)) * a.value_heads + h;
      sg[buf][threadIdx.x] = a.g[off];
      sb[buf][threadIdx.x] = a.beta[off];
    }
  };
  auto normalise = [&](int buf, int t0) {
    // vectors 0 .. n_tok-1 are the queries, n_tok .. 2 n_tok - 1 the keys; lane covers 4 channels
    const int n_tok = min(kBlockT, a.tokens - t0);
    for (int v = warp; v < 2 * n_tok; v += 4) {
      const bool is_query = v < n_tok;
      float* vec = is_query ? sq[buf][v] : sk[buf][v - n_tok];
      float x[4], ss = 0.0f;
#pragma unroll
      for (int i = 0; i < 4; ++i) { x[i] = vec[lane + 32 * i]; ss += x[i] * x[i]; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      float f;
      if (a.normalize_qk) {
        f = rsqrtf(ss + 1e-6f);
        if (is_query) f = f / sqrtf(static_cast<float>(dk));
      } else {
        f = is_query ? a.q_scale : 1.0f;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) vec[lane + 32 * i] = x[i] * f;
    }
  };

  stage(0, 0);
  __syncthreads();
  normalise(0, 0);
  __syncthreads();
  const int blocks = (a.tokens + kBlockT - 1) / kBlockT;
  for (int blk = 0; blk < blocks; ++blk) {
    const int buf = blk & 1;
    if (blk + 1 < blocks) stage(buf ^ 1, (blk + 1) * kBlockT);
    const int count = min(kBlockT, a.tokens - blk * kBlockT);
    for (int tt = 0; tt < count; ++tt) {
      const float decay = sg[buf][tt], beta = sb[buf][tt];
      const float* kvec = &sk[buf][tt][rg * 32];
      const float* qvec = &sq[buf][tt][rg * 32];
      float prediction = 0.0f;
#pragma unroll
      for (int r = 0; r < 32; ++r) {
        S[r] *= decay;
        prediction = fmaf(S[r], kvec[r], prediction);
      }
      prediction += __shfl_xor_sync(0xffffffffu, prediction, 1);
      prediction += __shfl_xor_sync(0xffffffffu, prediction, 2);
      const float delta = (sv[buf][tt][warp * 8 + (lane >> 2)] - prediction) * beta;
      float core = 0.0f;
#pragma unroll
      for (int r = 0; r < 32; ++r) {
        S[r] = fmaf(kvec[r], delta, S[r]);
        core = fmaf(S[r], qvec[r], core);
      }
      core += __shfl_xor_sync(0xffffffffu, core, 1);
      core += __shfl_xor_sync(0xffffffffu, core, 2);
      if (rg == 0 && col_ok) {
        const int t = blk * kBlockT + tt;
        store_any(a.out, ((static_cast<size_t>(b) * a.tokens + t) * a.value_heads + h) * dv + col,
                  a.out_is_bf16, rnd(core, a.round));
      }
    }
    __syncthreads();
    if (blk + 1 < blocks) {
      normalise(buf ^ 1, (blk + 1) * kBlockT);
      __syncthreads();
    }
  }
#pragma unroll
  for (int r = 0; r < 32; ++r) {
    const int row = rg * 32 + r;
    if (col_ok && row < dk) state[static_cast<size_t>(row) * dv + col] = S[r];
  }
}

// g = exp(-exp(A_log) * softplus(a + dt_bias)),  beta = R(sigmoid(b));  one thread per (token, head)
__global__ void gdn_gates_kernel(const void* a_in, const void* b_in, const float* a_log,
                                 const float* dt_bias, int in_is_bf16, long long count, int heads,
                                 int round, float* g, float* beta) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const int h = static_cast<int>(i % heads);
  const float alpha = load_any(a_in, i, in_is_bf16) + dt_bias[h];
  const float softplus = fmaxf(alpha, 0.0f) + logf(1.0f + expf(-fabsf(alpha)));
  g[i] = expf(-expf(a_log[h]) * softplus);
  beta[i] = rnd(1.0f / (1.0f + expf(-load_any(b_in, i, in_is_bf16))), round);
}

// Causal depthwise convolution + SiLU over a sequence with an explicit history:
// `state` [B, channels, width] holds the last `width` inputs (oldest first; zero for a fresh
// sequence).  y_t = R(SiLU(R(sum_tap w[c][tap] * x[t + tap - width + 1]))) with inputs rounded
// first; on return the state holds the last `width` inputs of this call (the reference's
// shift register).  One thread per (batch, channel), sequential in t.
__global__ void gdn_conv_kernel(const void* input, const float* weight, int in_is_bf16, int batch,
                                int tokens, int channels, int width, int round, float* state,
                                void* output, int out_is_bf16) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<long long>(batch) * channels) return;
  const int b = static_cast<int>(i / channels), c = static_cast<int>(i % channels);
  float window[32], w[32];
  for (int tap = 0; tap < width; ++tap) {
    window[tap] = state[(static_cast<size_t>(b) * channels + c) * width + tap];
    w[tap] = weight[static_cast<size_t>(c) * width + tap];
  }
  for (int t = 0; t < tokens; ++t) {
    const size_t idx = (static_cast<size_t>(b) * tokens + t) * channels + c;
    float sum = 0.0f;
    for (int tap = 0; tap < width - 1; ++tap) {
      window[tap] = window[tap + 1];
      sum += window[tap] * w[tap];
    }
    const float current = rnd(load_any(input, idx, in_is_bf16), round);
    window[width - 1] = current;
    sum = rnd(sum + current * w[width - 1], round);
    store_any(output, idx, out_is_bf16, rnd(sum / (1.0f + expf(-sum)), round));
  }
  for (int tap = 0; tap < width; ++tap)
    state[(static_cast<size_t>(b) * channels + c) * width + tap] = window[tap];
}

// Per (token, head): RMSNorm * weight * SiLU(z) with the reference's rounding after every product;
// final_round = 0 leaves the last product unrounded before the store (OutputForward).
// grid = rows (token-heads), 256 threads.
__global__ void __launch_bounds__(256) gdn_output_kernel(const void* core, const void* z,
                                                         const float* norm_weight, int core_is_bf16,
                                                         int z_is_bf16, int dim, float epsilon,
                                                         int round, int final_round, void* output,
                                                         int out_is_bf16) {
  const size_t row = blockIdx.x;
  const int c = threadIdx.x;
  const float x = c < dim ? load_any(core, row * dim + c, core_is_bf16) : 0.0f;
  __shared__ float red[8];
  float sq = x * x;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  if (c % 32 == 0) red[c / 32] = sq;
  __syncthreads();
  float total = 0.0f;
#pragma unroll
  for (int w = 0; w < 8; ++w) total += red[w];
  if (c >= dim) return;
  const float inverse = rsqrtf(total / static_cast<float>(dim) + epsilon);
  const float normalized = rnd(x * inverse, round);
  const float affine = rnd(normalized * norm_weight[c], round);
  const float gate = load_any(z, row * dim + c, z_is_bf16);
  const float silu = gate / (1.0f + expf(-gate));
  store_any(output, row * dim + c, out_is_bf16, rnd(affine * silu, round && final_round));
}

}  // namespace

cudaError_t gdn_recurrent(cudaStream_t stream, const GdnArgs& a) {
  const dim3 grid((a.value_dim + kSlice - 1) / kSlice, a.value_heads, a.batch);
  gdn_recurrent_kernel<<<grid, kRecThreads, 0, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t gdn_gates(cudaStream_t stream, const void* a_in, const void* b_in, const float* a_log,
                      const float* dt_bias, int in_is_bf16, long long tokens, int heads, int round,
                      float* g, float* beta) {
  const long long count = tokens * heads;
  gdn_gates_kernel<<<static_cast<unsigned>((count + 255) / 256), 256, 0, stream>>>(
      a_in, b_in, a_log, dt_bias, in_is_bf16, count, heads, round, g, beta);
  return cudaGetLastError();
}

cudaError_t gdn_conv(cudaStream_t stream, const void* input, const float* weight, int in_is_bf16,
                     int batch, int tokens, int channels, int width, int round, float* state,
                     void* output, int out_is_bf16) {
  const long long count = static_cast<long long>(batch) * channels;
  gdn_conv_kernel<<<static_cast<unsigned>((count + 127) / 128), 128, 0, stream>>>(
      input, weight, in_is_bf16, batch, tokens, channels, width, round, state, output, out_is_bf16);
  return cudaGetLastError();
}

cudaError_t gdn_output(cudaStream_t stream, const void* core, const void* z,
                       const float* norm_weight, int core_is_bf16, int z_is_bf16, long long rows,
                       int dim, float epsilon, int round, int final_round, void* output,
                       int out_is_bf16) {
  gdn_output_kernel<<<static_cast<unsigned>(rows), 256, 0, stream>>>(
      core, z, norm_weight, core_is_bf16, z_is_bf16, dim, epsilon, round, final_round, output,
      out_is_bf16);
  return cudaGetLastError();
}

}  // namespace pluto
