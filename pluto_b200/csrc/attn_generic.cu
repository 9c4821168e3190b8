// Causal multi-head attention over a packed [rows, 3E] activation -- the exact-fp32 path.
//
// Mirrors the reference layer AttentionLayer (src/llm/layers/attention.cc:98-170 forward,
// :176-230 probabilities, :235-314 query-owned backward, :319-396 key/value-owned backward) for
// every shape it accepts: any head width up to 256, fp32 storage (the reference's "FP16" compute
// policy keeps fp32 activations) or bf16 storage, ragged sequence and head tiles.  All arithmetic
// is fp32 FFMA with expf, so the fp32 policy meets a 1e-4 tolerance against the scalar CPU
// layer; the bf16 tensor-core path in attn_fwd_sm100.cu takes over for head widths 64/128.
//
// Like the reference the backward is two single-writer passes with fixed-order reductions and no
// floating-point atomics, so repeated runs are bitwise identical.
#include "common.cuh"
#include "engine.h"

namespace pluto {
namespace {

constexpr int kThreads = 256;  // 16 x 16 thread grid
constexpr float kSentinel = -3.402823466e+38f;

template <typename T>
__device__ __forceinline__ float load_as_float(const T* p);
template <>
__device__ __forceinline__ float load_as_float<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}
template <typename T>
__device__ __forceinline__ void store_from_float(T* p, float v);
template <>
__device__ __forceinline__ void store_from_float<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_from_float<__nv_bfloat16>(__nv_bfloat16* p, float v) {
  *p = __float2bfloat16_rn(v);
}

// Copies rows [row0, row0+ROWS) x head columns [0, D) of one packed section into a padded fp32
// shared tile; rows past the sequence end and columns past D become zero.
template <typename T, int ROWS, int DP>
__device__ __forceinline__ void load_tile(float (*tile)[DP + 1], const T* base, size_t row_stride,
                                          int row0, int seq, int D) {
  for (int idx = threadIdx.x; idx < ROWS * DP; idx += kThreads) {
    const int r = idx / DP, d = idx % DP;
    const int row = row0 + r;
    float v = 0.0f;
    if (row < seq && d < D) v = load_as_float(base + static_cast<size_t>(row) * row_stride + d);
    tile[r][d] = v;
  }
}

// c[i][j] = sum_d a[ty+16i][d] * b[tx+16j][d]
template <int MI, int NJ, int DP>
__device__ __forceinline__ void mm_nt(float (&c)[MI][NJ], const float (*a)[DP + 1],
                                      const float (*b)[DP + 1], int D, int ty, int tx) {
#pragma unroll
  for (int i = 0; i < MI; ++i)
#pragma unroll
    for (int j = 0; j < NJ; ++j) c[i][j] = 0.0f;
  for (int d = 0; d < D; ++d) {
    float av[MI], bv[NJ];
#pragma unroll
    for (int i = 0; i < MI; ++i) av[i] = a[ty + 16 * i][d];
#pragma unroll
    for (int j = 0; j < NJ; ++j) bv[j] = b[tx + 16 * j][d];
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
      for (int j = 0; j < NJ; ++j) c[i][j] = fmaf(av[i], bv[j], c[i][j]);
  }
}

// acc[i][c] += sum_k p[ty+16i][k] * b[k][tx+16c]        (p: [*, BN+1], b: [BN, DP+1])
template <int MI, int DC, int BN, int DP>
__device__ __forceinline__ void mm_nn(float (&acc)[MI][DC], const float (*p)[BN + 1],
                                      const float (*b)[DP + 1], int kcount, int ty, int tx) {
  for (int k = 0; k < kcount; ++k) {
    float pv[MI], bv[DC];
#pragma unroll
    for (int i = 0; i < MI; ++i) pv[i] = p[ty + 16 * i][k];
#pragma unroll
    for (int c = 0; c < DC; ++c) bv[c] = b[k][tx + 16 * c];
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
      for (int c = 0; c < DC; ++c) acc[i][c] = fmaf(pv[i], bv[c], acc[i][c]);
  }
}

// acc[i][c] += sum_q p[q][ty+16i] * b[q][tx+16c]        (transposed left operand)
template <int MI, int DC, int BN, int DP>
__device__ __forceinline__ void mm_tn(float (&acc)[MI][DC], const float (*p)[BN + 1],
                                      const float (*b)[DP + 1], int qcount, int ty, int tx) {
  for (int q = 0; q < qcount; ++q) {
    float pv[MI], bv[DC];
#pragma unroll
    for (int i = 0; i < MI; ++i) pv[i] = p[q][ty + 16 * i];
#pragma unroll
    for (int c = 0; c < DC; ++c) bv[c] = b[q][tx + 16 * c];
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
      for (int c = 0; c < DC; ++c) acc[i][c] = fmaf(pv[i], bv[c], acc[i][c]);
  }
}

__device__ __forceinline__ float group16_max(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float group16_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct Dims {
  int seq, heads, head_dim;
  float scale;
};

// Addressing of separate Q/K/V tensors for the forward kernel: element strides between tokens
// and between heads, and how many query heads share one key/value head.
struct Views {
  size_t q_token, q_head, kv_token, kv_head, out_token, out_head, gate_token, gate_head;
  int group;
};

// ------------------------------------------------------------------------------------------
// forward: grid (query tiles, heads, batch)
// ------------------------------------------------------------------------------------------
template <typename T, int DP, int BM>
__global__ void __launch_bounds__(kThreads)
attn_fwd_generic(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                 T* __restrict__ out, float* __restrict__ maxima,
                 float* __restrict__ normalizers, const T* __restrict__ gate,
                 float* __restrict__ core, int round_gate, Dims dims, Views views) {
  constexpr int BN = BM, MI = BM / 16, NJ = BN / 16, DC = DP / 16;
  extern __shared__ float smem[];
  float(*Qs)[DP + 1] = reinterpret_cast<float(*)[DP + 1]>(smem);
  float(*Ks)[DP + 1] = Qs + BM;
  float(*Vs)[DP + 1] = Ks + BN;
  float(*Ps)[BN + 1] = reinterpret_cast<float(*)[BN + 1]>(Vs + BN);

  const int S = dims.seq, H = dims.heads, D = dims.head_dim;
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
  const T* q_base = q + static_cast<size_t>(b) * S * views.q_token + h * views.q_head;
  const T* k_base = k + static_cast<size_t>(b) * S * views.kv_token + (h / views.group) * views.kv_head;
  const T* v_base = v + static_cast<size_t>(b) * S * views.kv_token + (h / views.group) * views.kv_head;

  load_tile<T, BM, DP>(Qs, q_base, views.q_token, qt * BM, S, D);
  float m[MI], l[MI], acc[MI][DC];
#pragma unroll
  for (int i = 0; i < MI; ++i) {
    m[i] = kSentinel;
    l[i] = 0.0f;
#pragma unroll
    for (int c = 0; c < DC; ++c) acc[i][c] = 0.0f;
  }
  for (int kt = 0; kt <= qt; ++kt) {
    __syncthreads();  // previous tile fully consumed (and Q visible on the first pass)
    load_tile<T, BN, DP>(Ks, k_base, views.kv_token, kt * BN, S, D);
    load_tile<T, BN, DP>(Vs, v_base, views.kv_token, kt * BN, S, D);
    __syncthreads();
    float s[MI][NJ];
    mm_nt<MI, NJ, DP>(s, Qs, Ks, D, ty, tx);
#pragma unroll
    for (int i = 0; i < MI; ++i) {
      const int query = qt * BM + ty + 16 * i;
      float tile_max = kSentinel;
      bool valid[NJ];
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const int key = kt * BN + tx + 16 * j;
        valid[j] = key <= query && key < S;
        s[i][j] = valid[j] ? s[i][j] * dims.scale : kSentinel;
        tile_max = fmaxf(tile_max, s[i][j]);
      }
      tile_max = group16_max(tile_max);
      const float next = fmaxf(m[i], tile_max);
      const float correction = expf(m[i] - next);
      float row_sum = 0.0f;
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const float p = valid[j] ? expf(s[i][j] - next) : 0.0f;
        Ps[ty + 16 * i][tx + 16 * j] = p;
        row_sum += p;
      }
      row_sum = group16_sum(row_sum);
      l[i] = l[i] * correction + row_sum;
      m[i] = next;
#pragma unroll
      for (int c = 0; c < DC; ++c) acc[i][c] *= correction;
    }
    __syncthreads();
    const int kcount = min(BN, S - kt * BN);
    mm_nn<MI, DC, BN, DP>(acc, Ps, Vs, kcount, ty, tx);
  }
#pragma unroll
  for (int i = 0; i < MI; ++i) {
    const int query = qt * BM + ty + 16 * i;
    if (query >= S) continue;
    const float inv = 1.0f / l[i];
    const size_t o_off = (static_cast<size_t>(b) * S + query) * views.out_token + h * views.out_head;
    const T* g = gate ? gate + (static_cast<size_t>(b) * S + query) * views.gate_token + h * views.gate_head
                      : nullptr;
#pragma unroll
    for (int c = 0; c < DC; ++c) {
      const int d = tx + 16 * c;
      if (d >= D) continue;
      float value = acc[i][c] * inv;
      if (core) core[o_off + d] = value;
      if (g) {
        // R(R(core) * R(sigmoid(gate))), qwen_attention.cc:103-108
        float sigmoid = 1.0f / (1.0f + expf(-load_as_float(g + d)));
        if (round_gate) {
          sigmoid = bf16_round(sigmoid);
          value = bf16_round(value);
        }
        value *= sigmoid;
      }
      store_from_float(out + o_off + d, value);
    }
    if (tx == 0 && maxima != nullptr) {
      const size_t stat = (static_cast<size_t>(b) * H + h) * S + query;
      maxima[stat] = m[i];
      normalizers[stat] = l[i];
    }
  }
}

// ------------------------------------------------------------------------------------------
// probabilities [B,H,S,S] from the saved statistics: grid (query tiles, heads, batch)
// ------------------------------------------------------------------------------------------
template <typename T, int DP, int BM>
__global__ void __launch_bounds__(kThreads)
attn_probs_generic(const T* __restrict__ qkv, const float* __restrict__ maxima,
                   const float* __restrict__ normalizers, float* __restrict__ probs, Dims dims) {
  constexpr int BN = BM, MI = BM / 16, NJ = BN / 16;
  extern __shared__ float smem[];
  float(*Qs)[DP + 1] = reinterpret_cast<float(*)[DP + 1]>(smem);
  float(*Ks)[DP + 1] = Qs + BM;
  const int S = dims.seq, H = dims.heads, D = dims.head_dim, E = H * D;
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
  const size_t stride = 3 * static_cast<size_t>(E);
  const T* base = qkv + static_cast<size_t>(b) * S * stride + static_cast<size_t>(h) * D;
  load_tile<T, BM, DP>(Qs, base, stride, qt * BM, S, D);
  float m[MI], inv[MI];
#pragma unroll
  for (int i = 0; i < MI; ++i) {
    const int query = qt * BM + ty + 16 * i;
    const size_t stat = (static_cast<size_t>(b) * H + h) * S + min(query, S - 1);
    m[i] = maxima[stat];
    inv[i] = 1.0f / normalizers[stat];
  }
  const int tiles = (S + BN - 1) / BN;
  for (int kt = 0; kt < tiles; ++kt) {
    __syncthreads();
    if (kt <= qt) load_tile<T, BN, DP>(Ks, base + E, stride, kt * BN, S, D);
    __syncthreads();
    float s[MI][NJ];
    if (kt <= qt) mm_nt<MI, NJ, DP>(s, Qs, Ks, D, ty, tx);
#pragma unroll
    for (int i = 0; i < MI; ++i) {
      const int query = qt * BM + ty + 16 * i;
      if (query >= S) continue;
      float* row = probs + ((static_cast<size_t>(b) * H + h) * S + query) * S;
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const int key = kt * BN + tx + 16 * j;
        if (key >= S) continue;
        row[key] = (kt <= qt && key <= query) ? expf(s[i][j] * dims.scale - m[i]) * inv[i] : 0.0f;
      }
    }
  }
}

// Addressing for the backward passes: element strides of the separate tensors.  `group` query
// heads share one key/value head; the packed [rows, 3E] layout is the special case with all token
// strides 3E, head strides D and group 1.
struct BwdViews {
  size_t q_token, q_head, kv_token, kv_head;      // q, and k/v (indexed by key/value head)
  size_t o_token, o_head;                         // saved output (only when deltas are computed here)
  size_t g_token, g_head;                         // upstream gradient (fp32)
  size_t dq_token, dq_head, dkv_token, dkv_head;  // gradients (fp32)
  int group;
};

// ------------------------------------------------------------------------------------------
// backward, query-owned pass: deltas and dQ.  grid (query tiles, query heads, batch)
// With `out` null the deltas were written by the caller (gate backward) and are only read.
// ------------------------------------------------------------------------------------------
template <typename T, int DP, int BM>
__global__ void __launch_bounds__(kThreads)
attn_bwd_dq_generic(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                    const T* __restrict__ out, const float* __restrict__ d_out,
                    const float* __restrict__ maxima, const float* __restrict__ normalizers,
                    float* __restrict__ dq, float* __restrict__ deltas, Dims dims, BwdViews views) {
  constexpr int BN = BM, MI = BM / 16, NJ = BN / 16, DC = DP / 16;
  extern __shared__ float smem[];
  float(*Qs)[DP + 1] = reinterpret_cast<float(*)[DP + 1]>(smem);
  float(*Gs)[DP + 1] = Qs + BM;  // upstream gradient dO
  float(*Ks)[DP + 1] = Gs + BM;
  float(*Vs)[DP + 1] = Ks + BN;
  float(*Ps)[BN + 1] = reinterpret_cast<float(*)[BN + 1]>(Vs + BN);

  const int S = dims.seq, H = dims.heads, D = dims.head_dim;
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
  const T* q_base = q + static_cast<size_t>(b) * S * views.q_token + h * views.q_head;
  const T* k_base = k + static_cast<size_t>(b) * S * views.kv_token + (h / views.group) * views.kv_head;
  const T* v_base = v + static_cast<size_t>(b) * S * views.kv_token + (h / views.group) * views.kv_head;
  const float* g_base = d_out + static_cast<size_t>(b) * S * views.g_token + h * views.g_head;

  load_tile<T, BM, DP>(Qs, q_base, views.q_token, qt * BM, S, D);
  load_tile<float, BM, DP>(Gs, g_base, views.g_token, qt * BM, S, D);
  if (out != nullptr)  // borrow Ks for the saved output
    load_tile<T, BM, DP>(Ks, out + static_cast<size_t>(b) * S * views.o_token + h * views.o_head,
                         views.o_token, qt * BM, S, D);
  __syncthreads();
  float m[MI], inv[MI], delta[MI], acc[MI][DC];
#pragma unroll
  for (int i = 0; i < MI; ++i) {
    const int r = ty + 16 * i;
    const int query = qt * BM + r;
    const size_t stat = (static_cast<size_t>(b) * H + h) * S + min(query, S - 1);
    if (out != nullptr) {
      float part = 0.0f;
      for (int d = tx; d < D; d += 16) part = fmaf(Gs[r][d], Ks[r][d], part);
      delta[i] = group16_sum(part);
      if (tx == 0 && query < S) deltas[stat] = delta[i];
    } else {
      delta[i] = deltas[stat];
    }
    m[i] = maxima[stat];
    inv[i] = 1.0f / normalizers[stat];
#pragma unroll
    for (int c = 0; c < DC; ++c) acc[i][c] = 0.0f;
  }
  for (int kt = 0; kt <= qt; ++kt) {
    __syncthreads();
    load_tile<T, BN, DP>(Ks, k_base, views.kv_token, kt * BN, S, D);
    load_tile<T, BN, DP>(Vs, v_base, views.kv_token, kt * BN, S, D);
    __syncthreads();
    float s[MI][NJ], dp[MI][NJ];
    mm_nt<MI, NJ, DP>(s, Qs, Ks, D, ty, tx);
    mm_nt<MI, NJ, DP>(dp, Gs, Vs, D, ty, tx);
#pragma unroll
    for (int i = 0; i < MI; ++i) {
      const int query = qt * BM + ty + 16 * i;
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const int key = kt * BN + tx + 16 * j;
        const bool valid = key <= query && key < S && query < S;
        const float p = valid ? expf(s[i][j] * dims.scale - m[i]) * inv[i] : 0.0f;
        Ps[ty + 16 * i][tx + 16 * j] = p * (dp[i][j] - delta[i]) * dims.scale;
      }
    }
    __syncthreads();
    mm_nn<MI, DC, BN, DP>(acc, Ps, Ks, min(BN, S - kt * BN), ty, tx);
  }
#pragma unroll
  for (int i = 0; i < MI; ++i) {
    const int query = qt * BM + ty + 16 * i;
    if (query >= S) continue;
    float* row = dq + (static_cast<size_t>(b) * S + query) * views.dq_token + h * views.dq_head;
#pragma unroll
    for (int c = 0; c < DC; ++c) {
      const int d = tx + 16 * c;
      if (d < D) row[d] = acc[i][c];
    }
  }
}

// ------------------------------------------------------------------------------------------
// backward, key/value-owned pass: dK and dV.  grid (key tiles, key/value heads, batch).  The
// query heads of the group and the query tiles are visited in a fixed order (single writer).
// ------------------------------------------------------------------------------------------
template <typename T, int DP, int BM>
__global__ void __launch_bounds__(kThreads)
attn_bwd_dkv_generic(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                     const float* __restrict__ d_out, const float* __restrict__ maxima,
                     const float* __restrict__ normalizers, const float* __restrict__ deltas,
                     float* __restrict__ dk_out, float* __restrict__ dv_out, Dims dims,
                     BwdViews views) {
  constexpr int BN = BM, MI = BM / 16, NJ = BN / 16, DC = DP / 16;
  extern __shared__ float smem[];
  float(*Qs)[DP + 1] = reinterpret_cast<float(*)[DP + 1]>(smem);
  float(*Gs)[DP + 1] = Qs + BM;
  float(*Ks)[DP + 1] = Gs + BM;
  float(*Vs)[DP + 1] = Ks + BN;
  float(*Ps)[BN + 1] = reinterpret_cast<float(*)[BN + 1]>(Vs + BN);
  float(*Ss)[BN + 1] = Ps + BM;  // dS

  const int S = dims.seq, H = dims.heads, D = dims.head_dim;
  const int kt = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
  const T* k_base = k + static_cast<size_t>(b) * S * views.kv_token + kvh * views.kv_head;
  const T* v_base = v + static_cast<size_t>(b) * S * views.kv_token + kvh * views.kv_head;

  load_tile<T, BN, DP>(Ks, k_base, views.kv_token, kt * BN, S, D);
  load_tile<T, BN, DP>(Vs, v_base, views.kv_token, kt * BN, S, D);
  float dk[MI][DC], dv[MI][DC];
#pragma unroll
  for (int i = 0; i < MI; ++i)
#pragma unroll
    for (int c = 0; c < DC; ++c) dk[i][c] = dv[i][c] = 0.0f;
  const int tiles = (S + BM - 1) / BM;
  for (int h = kvh * views.group; h < (kvh + 1) * views.group; ++h) {
    const T* q_base = q + static_cast<size_t>(b) * S * views.q_token + h * views.q_head;
    const float* g_base = d_out + static_cast<size_t>(b) * S * views.g_token + h * views.g_head;
    for (int qt = kt; qt < tiles; ++qt) {
      __syncthreads();
      load_tile<T, BM, DP>(Qs, q_base, views.q_token, qt * BM, S, D);
      load_tile<float, BM, DP>(Gs, g_base, views.g_token, qt * BM, S, D);
      __syncthreads();
      float s[MI][NJ], dp[MI][NJ];
      mm_nt<MI, NJ, DP>(s, Qs, Ks, D, ty, tx);
      mm_nt<MI, NJ, DP>(dp, Gs, Vs, D, ty, tx);
#pragma unroll
      for (int i = 0; i < MI; ++i) {
        const int query = qt * BM + ty + 16 * i;
        const size_t stat = (static_cast<size_t>(b) * H + h) * S + min(query, S - 1);
        const float m = maxima[stat], inv = 1.0f / normalizers[stat], delta = deltas[stat];
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
          const int key = kt * BN + tx + 16 * j;
          const bool valid = key <= query && key < S && query < S;
          const float p = valid ? expf(s[i][j] * dims.scale - m) * inv : 0.0f;
          Ps[ty + 16 * i][tx + 16 * j] = p;
          Ss[ty + 16 * i][tx + 16 * j] = p * (dp[i][j] - delta) * dims.scale;
        }
      }
      __syncthreads();
      const int qcount = min(BM, S - qt * BM);
      mm_tn<MI, DC, BN, DP>(dv, Ps, Gs, qcount, ty, tx);
      mm_tn<MI, DC, BN, DP>(dk, Ss, Qs, qcount, ty, tx);
    }
  }
#pragma unroll
  for (int i = 0; i < MI; ++i) {
    const int key = kt * BN + ty + 16 * i;
    if (key >= S) continue;
    const size_t off = (static_cast<size_t>(b) * S + key) * views.dkv_token + kvh * views.dkv_head;
#pragma unroll
    for (int c = 0; c < DC; ++c) {
      const int d = tx + 16 * c;
      if (d < D) {
        dk_out[off + d] = dk[i][c];
        dv_out[off + d] = dv[i][c];
      }
    }
  }
}

template <int DP, int BM>
constexpr size_t fwd_smem() { return sizeof(float) * (3 * BM * (DP + 1) + BM * (BM + 1)); }
template <int DP, int BM>
constexpr size_t probs_smem() { return sizeof(float) * (2 * BM * (DP + 1)); }
template <int DP, int BM>
constexpr size_t dq_smem() { return sizeof(float) * (4 * BM * (DP + 1) + BM * (BM + 1)); }
template <int DP, int BM>
constexpr size_t dkv_smem() { return sizeof(float) * (4 * BM * (DP + 1) + 2 * BM * (BM + 1)); }

template <typename K>
cudaError_t opt_in(K kernel, size_t bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(bytes));
}

template <typename T, int DP, int BM>
cudaError_t launch_fwd(cudaStream_t stream, const void* q, const void* k, const void* v, void* out,
                       float* maxima, float* normalizers, const void* gate, float* core,
                       int round_gate, int batch, Dims dims, Views views) {
  auto kernel = attn_fwd_generic<T, DP, BM>;
  cudaError_t e = opt_in(kernel, fwd_smem<DP, BM>());
  if (e != cudaSuccess) return e;
  dim3 grid((dims.seq + BM - 1) / BM, dims.heads, batch);
  kernel<<<grid, kThreads, fwd_smem<DP, BM>(), stream>>>(
      static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v),
      static_cast<T*>(out), maxima, normalizers, static_cast<const T*>(gate), core, round_gate,
      dims, views);
  return cudaGetLastError();
}
template <typename T, int DP, int BM>
cudaError_t launch_probs(cudaStream_t stream, const void* qkv, const float* maxima,
                         const float* normalizers, float* probs, int batch, Dims dims) {
  auto kernel = attn_probs_generic<T, DP, BM>;
  cudaError_t e = opt_in(kernel, probs_smem<DP, BM>());
  if (e != cudaSuccess) return e;
  dim3 grid((dims.seq + BM - 1) / BM, dims.heads, batch);
  kernel<<<grid, kThreads, probs_smem<DP, BM>(), stream>>>(static_cast<const T*>(qkv), maxima,
                                                           normalizers, probs, dims);
  return cudaGetLastError();
}
template <typename T, int DP, int BM>
cudaError_t launch_bwd(cudaStream_t stream, const void* q, const void* k, const void* v,
                       const void* out, const float* d_out, const float* maxima,
                       const float* normalizers, float* dq_out, float* dk_out, float* dv_out,
                       float* deltas, int batch, Dims dims, BwdViews views) {
  auto dq = attn_bwd_dq_generic<T, DP, BM>;
  auto dkv = attn_bwd_dkv_generic<T, DP, BM>;
  cudaError_t e = opt_in(dq, dq_smem<DP, BM>());
  if (e != cudaSuccess) return e;
  e = opt_in(dkv, dkv_smem<DP, BM>());
  if (e != cudaSuccess) return e;
  const int tiles = (dims.seq + BM - 1) / BM;
  dq<<<dim3(tiles, dims.heads, batch), kThreads, dq_smem<DP, BM>(), stream>>>(
      static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v),
      static_cast<const T*>(out), d_out, maxima, normalizers, dq_out, deltas, dims, views);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  // Same-stream ordering makes every delta visible to the key/value-owned pass.
  dkv<<<dim3(tiles, dims.heads / views.group, batch), kThreads, dkv_smem<DP, BM>(), stream>>>(
      static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v), d_out, maxima,
      normalizers, deltas, dk_out, dv_out, dims, views);
  return cudaGetLastError();
}

}  // namespace

// Forward over separate Q/K/V tensors.  Strides are in elements; `group` query heads share one
// key/value head.  The packed [rows, 3E] layout of AttentionLayer is the special case
// q = qkv, k = qkv + E, v = qkv + 2E with token stride 3E (see c_api.cu).
cudaError_t attn_generic_fwd(cudaStream_t stream, const void* q, const void* k, const void* v,
                             void* out, float* maxima, float* normalizers, int batch, int seq,
                             int heads, int head_dim, size_t q_token, size_t q_head,
                             size_t kv_token, size_t kv_head, size_t out_token, size_t out_head,
                             int group, const void* gate, size_t gate_token, size_t gate_head,
                             float* core, int round_gate, bool bf16) {
  Dims dims{seq, heads, head_dim, 1.0f / sqrtf(static_cast<float>(head_dim))};
  Views views{q_token, q_head, kv_token, kv_head, out_token, out_head, gate_token, gate_head, group};
#define CALL_FWD(T, DP, BM) \
  launch_fwd<T, DP, BM>(stream, q, k, v, out, maxima, normalizers, gate, core, round_gate, \
                        batch, dims, views)
  if (bf16) {
    if (head_dim <= 64) return CALL_FWD(__nv_bfloat16, 64, 64);
    if (head_dim <= 128) return CALL_FWD(__nv_bfloat16, 128, 64);
    return CALL_FWD(__nv_bfloat16, 256, 32);
  }
  if (head_dim <= 64) return CALL_FWD(float, 64, 64);
  if (head_dim <= 128) return CALL_FWD(float, 128, 64);
  return CALL_FWD(float, 256, 32);
#undef CALL_FWD
}

cudaError_t attn_generic_probs(cudaStream_t stream, const void* qkv, const float* maxima,
                               const float* normalizers, float* probs, int batch, int seq,
                               int heads, int head_dim, bool bf16) {
  Dims dims{seq, heads, head_dim, 1.0f / sqrtf(static_cast<float>(head_dim))};
#define CALL_P(T, DP, BM) launch_probs<T, DP, BM>(stream, qkv, maxima, normalizers, probs, batch, dims)
  if (bf16) {
    if (head_dim <= 64) return CALL_P(__nv_bfloat16, 64, 64);
    if (head_dim <= 128) return CALL_P(__nv_bfloat16, 128, 64);
    return CALL_P(__nv_bfloat16, 256, 32);
  }
  if (head_dim <= 64) return CALL_P(float, 64, 64);
  if (head_dim <= 128) return CALL_P(float, 128, 64);
  return CALL_P(float, 256, 32);
#undef CALL_P
}

cudaError_t attn_generic_bwd(cudaStream_t stream, const void* qkv, const void* out,
                             const float* d_out, const float* maxima, const float* normalizers,
                             float* d_qkv, float* deltas, int batch, int seq, int heads,
                             int head_dim, bool bf16) {
  const size_t E = static_cast<size_t>(heads) * head_dim, D = head_dim;
  const size_t elem = bf16 ? 2 : 4;
  const char* base = static_cast<const char*>(qkv);
  GqaBwdArgs a{};
  a.q = base;
  a.k = base + E * elem;
  a.v = base + 2 * E * elem;
  a.out = out;
  a.d_out = d_out;
  a.maxima = maxima;
  a.normalizers = normalizers;
  a.deltas = deltas;
  a.dq = d_qkv;
  a.dk = d_qkv + E;
  a.dv = d_qkv + 2 * E;
  a.batch = batch; a.seq = seq; a.q_heads = heads; a.kv_heads = heads; a.head_dim = head_dim;
  a.q_token = a.kv_token = a.dq_token = a.dkv_token = 3 * E;
  a.q_head = a.kv_head = a.dq_head = a.dkv_head = a.o_head = a.g_head = D;
  a.o_token = a.g_token = E;
  a.bf16 = bf16;
  return gqa_generic_bwd(stream, a);
}

// Backward of the attention core over separate tensors with grouped query heads (the Qwen
// sequence layer): see GqaBwdArgs in engine.h.
cudaError_t gqa_generic_bwd(cudaStream_t stream, const GqaBwdArgs& a) {
  Dims dims{a.seq, a.q_heads, a.head_dim, 1.0f / sqrtf(static_cast<float>(a.head_dim))};
  BwdViews views{a.q_token, a.q_head, a.kv_token, a.kv_head, a.o_token, a.o_head, a.g_token,
                 a.g_head, a.dq_token, a.dq_head, a.dkv_token, a.dkv_head, a.q_heads / a.kv_heads};
#define CALL_B(T, DP, BM)                                                                        \
  launch_bwd<T, DP, BM>(stream, a.q, a.k, a.v, a.out, a.d_out, a.maxima, a.normalizers, a.dq, a.dk, \
                        a.dv, a.deltas, a.batch, dims, views)
  if (a.bf16) {
    if (a.head_dim <= 64) return CALL_B(__nv_bfloat16, 64, 64);
    if (a.head_dim <= 128) return CALL_B(__nv_bfloat16, 128, 64);
    return CALL_B(__nv_bfloat16, 256, 32);
  }
  if (a.head_dim <= 64) return CALL_B(float, 64, 64);
  if (a.head_dim <= 128) return CALL_B(float, 128, 64);
  return CALL_B(float, 256, 32);
#undef CALL_B
}

}  // namespace pluto
