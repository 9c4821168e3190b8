// Backward of the sequence gated delta-net (BPTT), any length.
//
// Reference kernels these stand in for (src/llm/layers/sequence_delta_net.cc):
//   OutputBackward :126-159 + SumNormGradient :161-171
//   RecurrenceBackward :176-258, GatherQkGradient :260-281, GatherScalarGradient :283-309
//   ConvSiluBackward :311-322, ConvInputBackward :324-341, ConvWeightBackward :343-362
// The reference saves every intermediate state S_t ((T+1) * Hv * dk * dv floats), which limits it
// to 128 tokens.  Here the recurrence pass keeps only one state per 64-token chunk: one CTA owns
// a [dk x 32] slice of one head for the whole sequence, (A) runs the recurrence forward from the
// zero state and stores the slice at every chunk boundary, then (B) walks the chunks backwards,
// re-running a chunk forward from its boundary state into a per-CTA scratch of 65 slices and
// stepping the adjoint through it.  All sums have a fixed order (no atomics): repeated runs are
// bitwise equal.  The arithmetic per token is the reference's:
//     dq = S_t dy;  dM += q dy^T;  ddelta = dM^T k;  dv = ddelta * beta;
//     dk = dM delta - (g S_{t-1}) dv;  dD = dM - k dv^T;  dg = <dD, S_{t-1}>;  dM <- g dD
#include "common.cuh"
#include "engine.h"

namespace pluto {
namespace {

__device__ __forceinline__ float load_any(const void* p, size_t i, int is_bf16) {
  return is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i])
                 : static_cast<const float*>(p)[i];
}
__device__ __forceinline__ float rnd(float v, int round) { return round ? bf16_round(v) : v; }
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ------------------------------------------------------------------------------------------------
// output norm + gate: one CTA of 256 threads per (token, head)
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gdn_out_bwd_kernel(const void* core, int core_is_bf16,
                                                          const void* z, int z_is_bf16,
                                                          const float* norm, const float* dy, int dim,
                                                          float epsilon, int round, float* dcore,
                                                          float* dz, float* parts) {
  __shared__ float red[2][8];
  const size_t row = blockIdx.x;
  const int c = threadIdx.x;
  const bool ok = c < dim;
  const float x = ok ? load_any(core, row * dim + c, core_is_bf16) : 0.0f;
  float sq = warp_sum(x * x);
  if (c % 32 == 0) red[0][c / 32] = sq;
  __syncthreads();
  float total = 0.0f;
#pragma unroll
  for (int w = 0; w < 8; ++w) total += red[0][w];
  const float inverse = rsqrtf(total / static_cast<float>(dim) + epsilon);
  const float normalized = rnd(x * inverse, round);
  const float w = ok ? norm[c] : 0.0f;
  const float affine = rnd(normalized * w, round);
  const float gate = ok ? load_any(z, row * dim + c, z_is_bf16) : 0.0f;
  const float sigmoid = 1.0f / (1.0f + expf(-gate));
  const float g = ok ? dy[row * dim + c] : 0.0f;
  const float dn = g * gate * sigmoid * w;
  float dot = warp_sum(dn * x);
  if (c % 32 == 0) red[1][c / 32] = dot;
  __syncthreads();
  dot = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) dot += red[1][i];
  if (!ok) return;
  dcore[row * dim + c] = inverse * dn - x * inverse * inverse * inverse / static_cast<float>(dim) * dot;
  dz[row * dim + c] = g * affine * sigmoid * (1.0f + gate * (1.0f - sigmoid));
  if (parts) parts[row * dim + c] = g * gate * sigmoid * normalized;
}

// ------------------------------------------------------------------------------------------------
// recurrence: grid (value tiles of 32, value heads, batch), 256 threads.
// Thread (warp w, lane l) owns rows w, w+8, ... (16 for dk = 128) of column l of the slice.
// ------------------------------------------------------------------------------------------------
constexpr int kCols = 32, kWarps = 8, kRows = 16, kChunk = 64, kBlockT = 16;
constexpr int kThreads = kCols * kWarps;

struct TokenBlock {            // kBlockT tokens staged in shared memory
  float raw_q[kBlockT][128], raw_k[kBlockT][128];
  float q[kBlockT][128], k[kBlockT][128];
  float iq[kBlockT], ik[kBlockT];
  float v[kBlockT][kCols], dy[kBlockT][kCols];
  float alpha[kBlockT], softplus[kBlockT], decay[kBlockT], sigmoid[kBlockT], beta[kBlockT];
};

__device__ __forceinline__ void stage_tokens(TokenBlock& tb, const GdnBwdArgs& a, int b, int h, int kh,
                                             int slice, int t0, int count, bool want_dy) {
  const int dk = a.key_dim, dv = a.value_dim;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  for (int idx = threadIdx.x; idx < kBlockT * 128; idx += kThreads) {
    const int tt = idx / 128, i = idx % 128;
    float qv = 0.0f, kv = 0.0f;
    if (tt < count && i < dk) {
      const size_t off = (static_cast<size_t>(b) * a.tokens + t0 + tt) * a.qk_token + static_cast<size_t>(kh) * dk + i;
      qv = load_any(a.q, off, a.in_is_bf16);
      kv = load_any(a.k, off, a.in_is_bf16);
    }
    tb.raw_q[tt][i] = qv;
    tb.raw_k[tt][i] = kv;
  }
  for (int idx = threadIdx.x; idx < kBlockT * kCols; idx += kThreads) {
    const int tt = idx / kCols, j = idx % kCols, c = slice * kCols + j;
    float x = 0.0f, g = 0.0f;
    if (tt < count && c < dv) {
      const size_t token = static_cast<size_t>(b) * a.tokens + t0 + tt;
      x = load_any(a.v, token * a.v_token + static_cast<size_t>(h) * dv + c, a.in_is_bf16);
      if (want_dy) g = a.dcore[(token * a.value_heads + h) * dv + c];
    }
    tb.v[tt][j] = x;
    tb.dy[tt][j] = g;
  }
  if (threadIdx.x < kBlockT) {
    const int tt = threadIdx.x;
    const size_t off = (static_cast<size_t>(b) * a.tokens + min(t0 + tt, a.tokens - 1)) * a.value_heads + h;
    const float alpha = load_any(a.a_in, off, a.ab_is_bf16) + a.dt_bias[h];
    const float softplus = fmaxf(alpha, 0.0f) + logf(1.0f + expf(-fabsf(alpha)));
    const float sigmoid = 1.0f / (1.0f + expf(-load_any(a.b_in, off, a.ab_is_bf16)));
    tb.alpha[tt] = alpha;
    tb.softplus[tt] = softplus;
    tb.decay[tt] = expf(-expf(a.a_log[h]) * softplus);
    tb.sigmoid[tt] = sigmoid;
    tb.beta[tt] = rnd(sigmoid, a.round);
  }
  __syncthreads();
  // norms: warp w handles vectors w, w+8, ... of the 2*kBlockT (q then k)
  const float inv_scale = rsqrtf(static_cast<float>(dk));
  for (int vec = warp; vec < 2 * kBlockT; vec += kWarps) {
    const bool is_q = vec < kBlockT;
    const int tt = is_q ? vec : vec - kBlockT;
    const float* raw = is_q ? tb.raw_q[tt] : tb.raw_k[tt];
    float x[4], ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) { x[i] = raw[lane + 32 * i]; ss += x[i] * x[i]; }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss + 1e-6f);
    float* dst = is_q ? tb.q[tt] : tb.k[tt];
#pragma unroll
    for (int i = 0; i < 4; ++i) dst[lane + 32 * i] = is_q ? x[i] * inv * inv_scale : x[i] * inv;
    if (lane == 0) (is_q ? tb.iq : tb.ik)[tt] = inv;
  }
  __syncthreads();
}

__global__ void __launch_bounds__(kThreads) gdn_recurrence_bwd_kernel(GdnBwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  TokenBlock& tb = *reinterpret_cast<TokenBlock*>(smem_raw);
  __shared__ float red[2][kWarps][kCols];     // cross-warp column sums (double-buffered)
  __shared__ float sdiff[kChunk][kCols];      // v - S^T k of the chunk being processed
  __shared__ float sdq[128], sdk[128], sdg[kWarps];

  const int slice = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tiles = gridDim.x;
  const int kh = h / (a.value_heads / a.key_heads);
  const int dk = a.key_dim, dv = a.value_dim, T = a.tokens;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int col = slice * kCols + lane;
  const int chunks = (T + kChunk - 1) / kChunk;
  const size_t cta = (static_cast<size_t>(b) * a.value_heads + h) * tiles + slice;
  const size_t slice_elems = static_cast<size_t>(kRows) * kWarps * kCols;       // 128 x 32
  float* ckpt = a.checkpoints + cta * chunks * slice_elems;
  float* scratch = a.scratch + cta * (kChunk + 1) * slice_elems;
  // element (row i = warp + 8 r, column lane) of a slice lives at (i * 32 + lane)
  auto store_slice = [&](float* dst, const float (&S)[kRows]) {
#pragma unroll
    for (int r = 0; r < kRows; ++r) dst[(warp + kWarps * r) * kCols + lane] = S[r];
  };
  auto load_slice = [&](const float* src, float (&S)[kRows]) {
#pragma unroll
    for (int r = 0; r < kRows; ++r) S[r] = src[(warp + kWarps * r) * kCols + lane];
  };
  int parity = 0;
  // one forward step on the register slice; returns v - S^T k (the same in every warp)
  auto forward_step = [&](float (&S)[kRows], int tt) -> float {
    const float decay = tb.decay[tt], beta = tb.beta[tt];
    float part = 0.0f;
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      S[r] *= decay;
      part = fmaf(S[r], tb.k[tt][warp + kWarps * r], part);
    }
    red[parity][warp][lane] = part;
    __syncthreads();
    float prediction = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) prediction += red[parity][w][lane];
    parity ^= 1;
    const float difference = tb.v[tt][lane] - prediction;
    const float delta = difference * beta;
#pragma unroll
    for (int r = 0; r < kRows; ++r) S[r] = fmaf(tb.k[tt][warp + kWarps * r], delta, S[r]);
    return difference;
  };

  // ---------------------------------------------------------------- (A) boundary states
  float S[kRows];
#pragma unroll
  for (int r = 0; r < kRows; ++r) S[r] = 0.0f;
  for (int t0 = 0; t0 < T; t0 += kBlockT) {
    const int count = min(kBlockT, T - t0);
    if (t0 % kChunk == 0) store_slice(ckpt + static_cast<size_t>(t0 / kChunk) * slice_elems, S);
    stage_tokens(tb, a, b, h, kh, slice, t0, count, false);
    for (int tt = 0; tt < count; ++tt) forward_step(S, tt);
    __syncthreads();
  }

  // ---------------------------------------------------------------- (B) chunks, last to first
  float dm[kRows];
#pragma unroll
  for (int r = 0; r < kRows; ++r) dm[r] = 0.0f;
  for (int chunk = chunks - 1; chunk >= 0; --chunk) {
    const int c0 = chunk * kChunk, ccount = min(kChunk, T - c0);
    // forward through the chunk: scratch[tt] = state before token c0 + tt, scratch[ccount] = after
    load_slice(ckpt + static_cast<size_t>(chunk) * slice_elems, S);
    for (int t0 = 0; t0 < ccount; t0 += kBlockT) {
      const int count = min(kBlockT, ccount - t0);
      stage_tokens(tb, a, b, h, kh, slice, c0 + t0, count, false);
      for (int tt = 0; tt < count; ++tt) {
        store_slice(scratch + static_cast<size_t>(t0 + tt) * slice_elems, S);
        const float difference = forward_step(S, tt);
        if (warp == 0) sdiff[t0 + tt][lane] = difference;
      }
      __syncthreads();
    }
    store_slice(scratch + static_cast<size_t>(ccount) * slice_elems, S);
    // adjoint through the chunk, token blocks last to first
    for (int t0 = (ccount - 1) / kBlockT * kBlockT; t0 >= 0; t0 -= kBlockT) {
      const int count = min(kBlockT, ccount - t0);
      stage_tokens(tb, a, b, h, kh, slice, c0 + t0, count, true);
      for (int tt = count - 1; tt >= 0; --tt) {
        const int ct = t0 + tt, t = c0 + ct;
        const float decay = tb.decay[tt], beta = tb.beta[tt];
        const float dy = tb.dy[tt][lane];
        const float difference = sdiff[ct][lane], delta = difference * beta;
        float prev[kRows], part = 0.0f;
        load_slice(scratch + static_cast<size_t>(ct) * slice_elems, prev);
        {
          const float* matrix = scratch + static_cast<size_t>(ct + 1) * slice_elems;
#pragma unroll
          for (int r = 0; r < kRows; ++r) {
            const int i = warp + kWarps * r;
            const float dq = warp_sum(matrix[i * kCols + lane] * dy);
            if (lane == 0) sdq[i] = dq;
            dm[r] = fmaf(tb.q[tt][i], dy, dm[r]);
            part = fmaf(dm[r], tb.k[tt][i], part);
          }
        }
        red[parity][warp][lane] = part;
        __syncthreads();
        float ddelta = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) ddelta += red[parity][w][lane];
        parity ^= 1;
        const float dvj = ddelta * beta;
        float dg = 0.0f;
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
          const int i = warp + kWarps * r;
          const float dk_part = dm[r] * delta - prev[r] * decay * dvj;
          const float dkv = warp_sum(dk_part);
          if (lane == 0) sdk[i] = dkv;
          const float ddecayed = dm[r] - tb.k[tt][i] * dvj;
          dg = fmaf(ddecayed, prev[r], dg);
          dm[r] = ddecayed * decay;
        }
        dg = warp_sum(dg);
        if (lane == 0) sdg[warp] = dg;
        __syncthreads();
        // per-token outputs of this (head, tile): written by the first warps
        const size_t partial = (static_cast<size_t>(b) * T + t) * a.value_heads * tiles +
                               static_cast<size_t>(h) * tiles + slice;
        if (warp < 4) {   // rows warp*32 + lane: d_raw_q, d_raw_k
          const int i = warp * 32 + lane;
          float pq = 0.0f, pk = 0.0f;
          // dot products over all rows, the same fixed order in every thread
          for (int n = 0; n < dk; ++n) {
            pq = fmaf(sdq[n], tb.raw_q[tt][n], pq);
            pk = fmaf(sdk[n], tb.raw_k[tt][n], pk);
          }
          if (i < dk) {
            const float iq = tb.iq[tt], ik = tb.ik[tt];
            const float scale = rsqrtf(static_cast<float>(dk));
            a.qk_partials[partial * 2 * dk + i] =
                (sdq[i] * iq - tb.raw_q[tt][i] * iq * iq * iq * pq) * scale;
            a.qk_partials[partial * 2 * dk + dk + i] = sdk[i] * ik - tb.raw_k[tt][i] * ik * ik * ik * pk;
          }
        } else if (warp == 4) {
          const float db_part = warp_sum(col < dv ? ddelta * difference : 0.0f);
          if (lane == 0) {
            float total = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) total += sdg[w];
            const float rate = expf(a.a_log[h]);
            const float alpha = tb.alpha[tt];
            a.scalar_partials[partial * 3 + 0] = -total * decay * rate / (1.0f + expf(-alpha));
            a.scalar_partials[partial * 3 + 1] = db_part * tb.sigmoid[tt] * (1.0f - tb.sigmoid[tt]);
            a.scalar_partials[partial * 3 + 2] = -total * decay * rate * tb.softplus[tt];
          }
        } else if (warp == 5) {
          if (col < dv)
            a.dv_out[(static_cast<size_t>(b) * T + t) * a.dv_token + static_cast<size_t>(h) * dv + col] = dvj;
        }
        __syncthreads();   // sdq / sdk / sdg are rewritten by the next token
      }
    }
  }
}

// GatherQkGradient: sum the partials of the value heads of a key head and their tiles, in order.
// grid (tokens * batch, key heads), 128 threads
__global__ void __launch_bounds__(128) gdn_gather_qk_kernel(const float* partials, int key_heads,
                                                            int value_heads, int dk, int tiles,
                                                            float* dq_out, float* dk_out,
                                                            size_t token_stride) {
  const int key_head = blockIdx.y, i = threadIdx.x;
  const size_t token = blockIdx.x;
  if (i >= dk) return;
  const int group = value_heads / key_heads;
  float dq = 0.0f, dkv = 0.0f;
  for (int h = key_head * group; h < (key_head + 1) * group; ++h)
    for (int tile = 0; tile < tiles; ++tile) {
      const size_t partial = ((token * value_heads + h) * tiles + tile) * 2 * dk;
      dq += partials[partial + i];
      dkv += partials[partial + dk + i];
    }
  dq_out[token * token_stride + static_cast<size_t>(key_head) * dk + i] = dq;
  dk_out[token * token_stride + static_cast<size_t>(key_head) * dk + i] = dkv;
}

// GatherScalarGradient: per token da, db; per head the sums over all tokens of all sequences are
// accumulated into d_a_log / d_dt_bias.  grid (value heads), 256 threads; fixed-order reduction.
__global__ void __launch_bounds__(256) gdn_gather_scalar_kernel(const float* partials, long long tokens,
                                                                int value_heads, int tiles, float* da,
                                                                float* db, float* d_a_log,
                                                                float* d_dt_bias) {
  __shared__ float red[2][256];
  const int head = blockIdx.x;
  float sum_log = 0.0f, sum_a = 0.0f;
  for (long long t = threadIdx.x; t < tokens; t += 256) {
    float ga = 0.0f, gb = 0.0f, gl = 0.0f;
    for (int tile = 0; tile < tiles; ++tile) {
      const size_t index = ((static_cast<size_t>(t) * value_heads + head) * tiles + tile) * 3;
      ga += partials[index];
      gb += partials[index + 1];
      gl += partials[index + 2];
    }
    da[t * value_heads + head] = ga;
    db[t * value_heads + head] = gb;
    sum_log += gl;
    sum_a += ga;
  }
  red[0][threadIdx.x] = sum_log;
  red[1][threadIdx.x] = sum_a;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total_log = 0.0f, total_a = 0.0f;
    for (int i = 0; i < 256; ++i) { total_log += red[0][i]; total_a += red[1][i]; }
    if (d_a_log) d_a_log[head] += total_log;
    if (d_dt_bias) d_dt_bias[head] += total_a;
  }
}

// ------------------------------------------------------------------------------------------------
// convolution + SiLU backward.  pre = R(sum_tap x w) is recomputed from the layer input.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float conv_dpre(const void* input, int in_is_bf16, const float* weight,
                                           const float* dpost, size_t seq_base, int t, int c,
                                           int channels, int width, int round) {
  float sum = 0.0f;
  for (int tap = 0; tap < width; ++tap) {
    const int source = t + tap - width + 1;
    if (source >= 0)
      sum += rnd(load_any(input, (seq_base + source) * channels + c, in_is_bf16), round) *
             weight[static_cast<size_t>(c) * width + tap];
  }
  sum = rnd(sum, round);
  const float sigmoid = 1.0f / (1.0f + expf(-sum));
  return dpost[(seq_base + t) * channels + c] * sigmoid * (1.0f + sum * (1.0f - sigmoid));
}

// dx[t, c] = sum_tap dpre[t + width - 1 - tap, c] * w[c, tap]; one thread per (token, channel)
__global__ void gdn_conv_input_bwd_kernel(const void* input, int in_is_bf16, const float* weight,
                                          const float* dpost, int tokens, int channels, int width,
                                          int round, float* dx) {
  const int blocks = (channels + 127) / 128;
  const int c = (blockIdx.x % blocks) * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int t = blockIdx.x / blocks, b = blockIdx.y;
  const size_t seq_base = static_cast<size_t>(b) * tokens;
  float sum = 0.0f;
  for (int tap = 0; tap < width; ++tap) {
    const int future = t + width - 1 - tap;
    if (future < tokens)
      sum += conv_dpre(input, in_is_bf16, weight, dpost, seq_base, future, c, channels, width, round) *
             weight[static_cast<size_t>(c) * width + tap];
  }
  dx[(seq_base + t) * channels + c] = sum;
}

// dw[c, tap] += sum over sequences and tokens of dpre[t, c] * x[t + tap - width + 1, c], in order
__global__ void gdn_conv_weight_bwd_kernel(const void* input, int in_is_bf16, const float* weight,
                                           const float* dpost, int batch, int tokens, int channels,
                                           int width, int round, float* dw) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int tap = blockIdx.y;
  float sum = 0.0f;
  for (int b = 0; b < batch; ++b) {
    const size_t seq_base = static_cast<size_t>(b) * tokens;
    for (int t = width - 1 - tap; t < tokens; ++t)
      sum += conv_dpre(input, in_is_bf16, weight, dpost, seq_base, t, c, channels, width, round) *
             rnd(load_any(input, (seq_base + t + tap - width + 1) * channels + c, in_is_bf16), round);
  }
  dw[static_cast<size_t>(c) * width + tap] += sum;
}

}  // namespace

cudaError_t gdn_out_bwd(cudaStream_t stream, const void* core, int core_is_bf16, const void* z,
                        int z_is_bf16, const float* norm, const float* dy, long long rows, int dim,
                        float epsilon, int round, float* dcore, float* dz, float* parts) {
  gdn_out_bwd_kernel<<<static_cast<unsigned>(rows), 256, 0, stream>>>(
      core, core_is_bf16, z, z_is_bf16, norm, dy, dim, epsilon, round, dcore, dz, parts);
  return cudaGetLastError();
}

size_t gdn_recurrence_bwd_workspace_bytes(int batch, int tokens, int value_heads, int key_dim,
                                          int value_dim) {
  const size_t tiles = (value_dim + kCols - 1) / kCols;
  const size_t ctas = static_cast<size_t>(batch) * value_heads * tiles;
  const size_t chunks = (tokens + kChunk - 1) / kChunk;
  const size_t slice = static_cast<size_t>(kRows) * kWarps * kCols;
  const size_t per_token = static_cast<size_t>(batch) * tokens * value_heads * tiles;
  const size_t sequential = sizeof(float) * (ctas * (chunks + kChunk + 1) * slice + per_token * (2 * key_dim + 3));
  const size_t chunked = key_dim == 128 && value_dim == 128 ? gdn_bwd_chunked_workspace_bytes(batch, tokens, value_heads) : 0;
  return sequential > chunked ? sequential : chunked;
}

cudaError_t gdn_recurrence_bwd(cudaStream_t stream, GdnBwdArgs a, float* dq_out, float* dk_out,
                               size_t dqk_token, float* da, float* db, float* d_a_log,
                               float* d_dt_bias, void* workspace) {
  if (gdn_bwd_chunked_supported(a)) {
    bool qk_direct = false;
    cudaError_t e = gdn_bwd_chunked(stream, a, dq_out, dk_out, dqk_token, workspace, kernel_status_word(), &qk_direct);
    if (e != cudaSuccess) return e;
    if (!qk_direct) {
      gdn_gather_qk_kernel<<<dim3(a.batch * a.tokens, a.key_heads), 128, 0, stream>>>(
          a.qk_partials, a.key_heads, a.value_heads, a.key_dim, 1, dq_out, dk_out, dqk_token);
      e = cudaGetLastError();
      if (e != cudaSuccess) return e;
    }
    gdn_gather_scalar_kernel<<<a.value_heads, 256, 0, stream>>>(
        a.scalar_partials, static_cast<long long>(a.batch) * a.tokens, a.value_heads, 1, da, db, d_a_log,
        d_dt_bias);
    return cudaGetLastError();
  }
  const int tiles = (a.value_dim + kCols - 1) / kCols;
  const size_t ctas = static_cast<size_t>(a.batch) * a.value_heads * tiles;
  const size_t chunks = (a.tokens + kChunk - 1) / kChunk;
  const size_t slice = static_cast<size_t>(kRows) * kWarps * kCols;
  const size_t per_token = static_cast<size_t>(a.batch) * a.tokens * a.value_heads * tiles;
  float* base = static_cast<float*>(workspace);
  a.checkpoints = base;
  a.scratch = a.checkpoints + ctas * chunks * slice;
  a.qk_partials = a.scratch + ctas * (kChunk + 1) * slice;
  a.scalar_partials = a.qk_partials + per_token * 2 * a.key_dim;
  cudaError_t e = cudaFuncSetAttribute(gdn_recurrence_bwd_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(sizeof(TokenBlock)));
  if (e != cudaSuccess) return e;
  gdn_recurrence_bwd_kernel<<<dim3(tiles, a.value_heads, a.batch), kThreads, sizeof(TokenBlock), stream>>>(a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  gdn_gather_qk_kernel<<<dim3(a.batch * a.tokens, a.key_heads), 128, 0, stream>>>(
      a.qk_partials, a.key_heads, a.value_heads, a.key_dim, tiles, dq_out, dk_out, dqk_token);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  gdn_gather_scalar_kernel<<<a.value_heads, 256, 0, stream>>>(
      a.scalar_partials, static_cast<long long>(a.batch) * a.tokens, a.value_heads, tiles, da, db,
      d_a_log, d_dt_bias);
  return cudaGetLastError();
}

cudaError_t gdn_conv_bwd(cudaStream_t stream, const void* input, int in_is_bf16, const float* weight,
                         const float* dpost, int batch, int tokens, int channels, int width, int round,
                         float* dx, float* d_weight) {
  gdn_conv_input_bwd_kernel<<<dim3(((channels + 127) / 128) * tokens, batch), 128, 0, stream>>>(
      input, in_is_bf16, weight, dpost, tokens, channels, width, round, dx);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess || d_weight == nullptr) return e;
  gdn_conv_weight_bwd_kernel<<<dim3((channels + 127) / 128, width), 128, 0, stream>>>(
      input, in_is_bf16, weight, dpost, batch, tokens, channels, width, round, d_weight);
  return cudaGetLastError();
}

}  // namespace pluto
