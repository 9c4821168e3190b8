// Chunked backward of the gated delta-net recurrence (key width = value width = 128).
//
// Reference kernels this stands in for (src/llm/layers/sequence_delta_net.cc): RecurrenceBackward
// :176-258 with GatherQkGradient :260-281 and GatherScalarGradient :283-309, which walk the
// sequence token by token.  Here the only sequential parts are two scans over 64-token chunks on
// the tensor cores (gdn_scan_sm100.cu): the forward scan leaves the state S_0 at the start of every
// chunk, the reverse scan the gradient dS_C at the end of every chunk.  Given those two, a chunk's
// gradients depend on nothing outside it, and gdn_bwd_chunk_local below computes all chunks in
// parallel, one CTA per (sequence, head, chunk), in fp32 on the CUDA cores.
//
// Chunk algebra (t, s index the chunk's tokens; b_t = running sum of log decay, c = exp(b),
// gamma = c_C; k^, q^ the normalised keys and scaled normalised queries):
//   G = k^ k^T, H = q^ k^T, A[t,s] = beta_t e^{b_t-b_s} G[t,s] (s < t), T = (I + A)^-1,
//   M[t,s] = e^{b_t-b_s} H[t,s] (s <= t), W = T (beta c . k^), U' = T (beta . v), U = U' - W S_0,
//   Kt = (gamma / c) . k^;  O = (c . q^) S_0 + M U;  S_C = gamma S_0 + Kt^T U.
// Backward, given dO, dS_C, S_0:
//   dU = M^T dO + Kt dS_C;  dM = mask(dO U^T);  dKt = U dS_C^T;  dQc = dO S_0^T;  dW = -dU S_0^T;
//   X1 = T^T dU (dv = beta . X1);  X2 = T^T dW;  dA = -mask(X1 U'^T + X2 W^T)  [= -T^T dT T^T];
//   dk^ = (dG + dG^T) k^ + dH^T q^ + (gamma/c) . dKt + (beta c) . X2,  dG = dA . beta e^{..}, dH = dM . e^{..};
//   dq^ = dH k^ + c . dQc;  dbeta = rows(X1 . v) + rows(X2 . c k^) + rows(dA . e^{..} G);
//   db  = rows(dA.A) - cols(dA.A) + rows(dM.M) - cols(dM.M) - rows(dKt.Kt) + rows(dQc . c q^)
//         + rows(X2 . beta c k^),  db_C += sum(dKt.Kt) + gamma <dS_C, S_0>;
//   d log g_s = sum over t >= s of db_t.
// Then through the L2 normalisations and the gate parametrisation exactly as the token-sequential
// kernel (gdn_bwd.cu) does.  All sums have a fixed order: repeated runs are bitwise equal.
#include "common.cuh"
#include "engine.h"
#include "gdn_records.cuh"

namespace pluto {
// gdn_chunked.cu / gdn_scan_sm100.cu
cudaError_t gdn_chunked_with_states(cudaStream_t stream, const GdnArgs& a, void* records, float* state_dump,
                                    uint32_t* status);
cudaError_t gdn_scan_bwd_launch(cudaStream_t stream, const void* dcore_bf16, const void* records, int batch,
                                int tokens, int value_heads, int chunks, float* dstate_dump, uint32_t* status);
namespace {

constexpr int kLC = 64;            // tokens per chunk
constexpr int kLD = 128;           // key width == value width
constexpr int kLP = 132;           // row pitch of the [64 x 128] matrices (floats)
constexpr int kLQ = 68;            // row pitch of the [64 x 64] matrices
constexpr int kLThreads = 256;

struct LocalSmem {
  float big[5][kLC * kLP];
  float sq[3][kLC * kLQ];
  float part[16][kLC];             // column sums: one partial per row group
  float b[kLC], beta[kLC], cdec[kLC], ik[kLC], iq[kLC];
  float alpha[kLC], softplus[kLC], sigmoid[kLC];
  float dbeta[kLC], db[kLC];
  float red[kLThreads / 32];
};

__device__ __forceinline__ float load_any(const void* p, size_t i, int is_bf16) {
  return is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i])
                 : static_cast<const float*>(p)[i];
}
__device__ __forceinline__ float4 lds4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ldg4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float comp(const float4& v, int i) { return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w)); }
// sum over the 16 lanes that share a row group (lanes with equal tid / 16)
__device__ __forceinline__ float row_sum16(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Thread (rg, cg) = (tid / 16, tid % 16) owns rows rg*4 .. +3 of every product.  Columns: eight
// neighbours cg*8 .. +7 ("dense") where the B operand is read along its rows, every 16th column
// cg + 16 j ("strided") where it is read along k -- with row pitches of 132 / 68 floats the 16
// lanes of a row group then fall into different banks.

// acc[i][j] += sum_k A[r0+i][k] B[cg+16j][k]     (A B^T, [64 x 64] result, strided columns)
template <int K>
__device__ __forceinline__ void nt_smem(const float* A, int pa, const float* B, int pb, int r0, int cg,
                                        float (&acc)[4][4]) {
#pragma unroll 2
  for (int k = 0; k < K; k += 4) {
    float4 a[4], b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = lds4(A + (r0 + i) * pa + k);
#pragma unroll
    for (int j = 0; j < 4; ++j) b[j] = lds4(B + (cg + 16 * j) * pb + k);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[i][j] = fmaf(a[i].x, b[j].x, acc[i][j]);
        acc[i][j] = fmaf(a[i].y, b[j].y, acc[i][j]);
        acc[i][j] = fmaf(a[i].z, b[j].z, acc[i][j]);
        acc[i][j] = fmaf(a[i].w, b[j].w, acc[i][j]);
      }
  }
}

// acc[i][j] += sum_k A[r0+i][k] scale[k] B[k][cg*8+j]   (A B, [64 x 128] result, dense columns)
template <int K>
__device__ __forceinline__ void nn_smem(const float* A, int pa, const float* scale, const float* B, int pb,
                                        int r0, int cg, float (&acc)[4][8]) {
#pragma unroll 2
  for (int k = 0; k < K; k += 4) {
    float4 a[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = lds4(A + (r0 + i) * pa + k);
    if (scale != nullptr) {
      const float4 s = lds4(scale + k);
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i].x *= s.x; a[i].y *= s.y; a[i].z *= s.z; a[i].w *= s.w; }
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const float4 b0 = lds4(B + (k + kk) * pb + cg * 8), b1 = lds4(B + (k + kk) * pb + cg * 8 + 4);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float av = comp(a[i], kk);
        acc[i][0] = fmaf(av, b0.x, acc[i][0]); acc[i][1] = fmaf(av, b0.y, acc[i][1]);
        acc[i][2] = fmaf(av, b0.z, acc[i][2]); acc[i][3] = fmaf(av, b0.w, acc[i][3]);
        acc[i][4] = fmaf(av, b1.x, acc[i][4]); acc[i][5] = fmaf(av, b1.y, acc[i][5]);
        acc[i][6] = fmaf(av, b1.z, acc[i][6]); acc[i][7] = fmaf(av, b1.w, acc[i][7]);
      }
    }
  }
}

// acc[i][j] += sum_k A[k][r0+i] B[k][cg*8+j]       (A^T B, dense columns)
template <int K>
__device__ __forceinline__ void tn_smem(const float* A, int pa, const float* B, int pb, int r0, int cg,
                                        float (&acc)[4][8]) {
#pragma unroll 4
  for (int k = 0; k < K; ++k) {
    const float4 a = lds4(A + k * pa + r0);
    const float4 b0 = lds4(B + k * pb + cg * 8), b1 = lds4(B + k * pb + cg * 8 + 4);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float av = comp(a, i);
      acc[i][0] = fmaf(av, b0.x, acc[i][0]); acc[i][1] = fmaf(av, b0.y, acc[i][1]);
      acc[i][2] = fmaf(av, b0.z, acc[i][2]); acc[i][3] = fmaf(av, b0.w, acc[i][3]);
      acc[i][4] = fmaf(av, b1.x, acc[i][4]); acc[i][5] = fmaf(av, b1.y, acc[i][5]);
      acc[i][6] = fmaf(av, b1.z, acc[i][6]); acc[i][7] = fmaf(av, b1.w, acc[i][7]);
    }
  }
}

// acc[i][j] += sum_k A[r0+i][k] Bg[k][cg*8+j]      (B a [128 x 128] matrix in global memory, dense columns)
__device__ __forceinline__ void nn_glob(const float* A, int pa, const float* __restrict__ Bg, int r0, int cg,
                                        float (&acc)[4][8]) {
#pragma unroll 2
  for (int k = 0; k < kLD; k += 4) {
    float4 a[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = lds4(A + (r0 + i) * pa + k);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const float4 b0 = ldg4(Bg + (k + kk) * kLD + cg * 8), b1 = ldg4(Bg + (k + kk) * kLD + cg * 8 + 4);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float av = comp(a[i], kk);
        acc[i][0] = fmaf(av, b0.x, acc[i][0]); acc[i][1] = fmaf(av, b0.y, acc[i][1]);
        acc[i][2] = fmaf(av, b0.z, acc[i][2]); acc[i][3] = fmaf(av, b0.w, acc[i][3]);
        acc[i][4] = fmaf(av, b1.x, acc[i][4]); acc[i][5] = fmaf(av, b1.y, acc[i][5]);
        acc[i][6] = fmaf(av, b1.z, acc[i][6]); acc[i][7] = fmaf(av, b1.w, acc[i][7]);
      }
    }
  }
}

// acc[i][j] += sum_k A[r0+i][k] Bg[cg+16j][k]      (A Bg^T, strided columns)
__device__ __forceinline__ void nt_glob(const float* A, int pa, const float* __restrict__ Bg, int r0, int cg,
                                        float (&acc)[4][8]) {
#pragma unroll 1
  for (int k = 0; k < kLD; k += 4) {
    float4 a[4], b[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = lds4(A + (r0 + i) * pa + k);
#pragma unroll
    for (int j = 0; j < 8; ++j) b[j] = ldg4(Bg + (cg + 16 * j) * kLD + k);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        acc[i][j] = fmaf(a[i].x, b[j].x, acc[i][j]);
        acc[i][j] = fmaf(a[i].y, b[j].y, acc[i][j]);
        acc[i][j] = fmaf(a[i].z, b[j].z, acc[i][j]);
        acc[i][j] = fmaf(a[i].w, b[j].w, acc[i][j]);
      }
  }
}

template <int N>
__device__ __forceinline__ void zero(float (&acc)[4][N]) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < N; ++j) acc[i][j] = 0.0f;
}
// dense tile -> [64 x 128] matrix in shared memory
__device__ __forceinline__ void store_dense(float* dst, int r0, int cg, const float (&acc)[4][8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    *reinterpret_cast<float4*>(dst + (r0 + i) * kLP + cg * 8) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    *reinterpret_cast<float4*>(dst + (r0 + i) * kLP + cg * 8 + 4) = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
  }
}

struct LocalArgs {
  GdnBwdArgs a;
  const float* states;    // [sequence, head, chunk, value column, key]: state at each chunk's start
  const float* dstates;   // same shape: state gradient at each chunk's end
  int chunks;
};

__global__ void __launch_bounds__(kLThreads, 1) gdn_bwd_chunk_local(LocalArgs la) {
  extern __shared__ uint8_t local_raw[];
  LocalSmem& sm = *reinterpret_cast<LocalSmem*>(local_raw);
  const GdnBwdArgs& a = la.a;
  const int chunk = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int kh = h / (a.value_heads / a.key_heads);
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int rg = tid >> 4, cg = tid & 15, r0 = rg * 4;
  const int t0 = chunk * kLC, count = min(kLC, a.tokens - t0);
  const size_t unit = static_cast<size_t>(b) * a.value_heads + h;
  const float* S0 = la.states + (unit * la.chunks + chunk) * kLD * kLD;     // [value column][key]
  const float* dS = la.dstates + (unit * la.chunks + chunk) * kLD * kLD;
  float* Kh = sm.big[0];
  const float q_scale = rsqrtf(static_cast<float>(kLD));

  // ---- gates
  if (tid < kLC) {
    float lg = 0.0f, be = 0.0f, alpha = 0.0f, softplus = 0.0f, sigmoid = 0.0f;
    if (tid < count) {
      const size_t off = (static_cast<size_t>(b) * a.tokens + t0 + tid) * a.value_heads + h;
      alpha = load_any(a.a_in, off, a.ab_is_bf16) + a.dt_bias[h];
      softplus = fmaxf(alpha, 0.0f) + logf(1.0f + expf(-fabsf(alpha)));
      sigmoid = 1.0f / (1.0f + expf(-load_any(a.b_in, off, a.ab_is_bf16)));
      lg = -expf(a.a_log[h]) * softplus;
      be = a.round ? bf16_round(sigmoid) : sigmoid;
    }
    sm.alpha[tid] = alpha;
    sm.softplus[tid] = softplus;
    sm.sigmoid[tid] = sigmoid;
    sm.beta[tid] = be;
    sm.b[tid] = lg;          // log decay, summed below
    sm.dbeta[tid] = 0.0f;
    sm.db[tid] = 0.0f;
  }
  __syncthreads();
  if (tid == 0) {
    float run = 0.0f;
    for (int t = 0; t < kLC; ++t) { run += sm.b[t]; sm.b[t] = run; }
  }
  __syncthreads();
  if (tid < kLC) sm.cdec[tid] = expf(sm.b[tid]);

  // ---- keys and queries, normalised: k^ -> big[0], q^ -> big[1]
  for (int idx = tid; idx < 2 * kLC * (kLD / 4); idx += kLThreads) {
    const int which = idx / (kLC * (kLD / 4)), rest = idx % (kLC * (kLD / 4));
    const int t = rest / (kLD / 4), c4 = rest % (kLD / 4);
    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (t < count) {
      const size_t off = (static_cast<size_t>(b) * a.tokens + t0 + t) * a.qk_token + static_cast<size_t>(kh) * kLD + c4 * 4;
      const void* src = which ? a.q : a.k;
      v = make_float4(load_any(src, off, a.in_is_bf16), load_any(src, off + 1, a.in_is_bf16),
                      load_any(src, off + 2, a.in_is_bf16), load_any(src, off + 3, a.in_is_bf16));
    }
    *reinterpret_cast<float4*>(sm.big[which] + t * kLP + c4 * 4) = v;
  }
  __syncthreads();
  for (int vec = warp; vec < 2 * kLC; vec += kLThreads / 32) {
    const int which = vec / kLC, t = vec % kLC;
    float* row = sm.big[which] + t * kLP;
    const float4 v = lds4(row + lane * 4);
    float ss = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = rsqrtf(ss + 1e-6f);
    const float f = which ? inv * q_scale : inv;
    *reinterpret_cast<float4*>(row + lane * 4) = make_float4(v.x * f, v.y * f, v.z * f, v.w * f);
    if (lane == 0) (which ? sm.iq : sm.ik)[t] = inv;
  }
  __syncthreads();

  // ---- A (transposed, for the substitution) -> sq[0];  M -> sq[1]
  {
    float g[4][4], hh[4][4];
    zero(g);
    zero(hh);
    nt_smem<kLD>(Kh, kLP, Kh, kLP, r0, cg, g);
    nt_smem<kLD>(sm.big[1], kLP, Kh, kLP, r0, cg, hh);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int t = r0 + i, s = cg + 16 * j;
        const float ratio = s <= t ? expf(sm.b[t] - sm.b[s]) : 0.0f;
        sm.sq[0][s * kLQ + t] = s < t ? sm.beta[t] * ratio * g[i][j] : 0.0f;
        sm.sq[1][t * kLQ + s] = ratio * hh[i][j];
      }
  }
  __syncthreads();

  // ---- T = (I + A)^-1 -> sq[2], one thread per column, right-looking forward substitution
  if (tid < kLC) {
    float x[kLC];
#pragma unroll
    for (int t = 0; t < kLC; ++t) x[t] = t == tid ? 1.0f : 0.0f;
#pragma unroll
    for (int s = 0; s < kLC - 1; ++s) {
      const float xs = x[s];
#pragma unroll
      for (int t4 = (s + 1) / 4; t4 < kLC / 4; ++t4) {
        const float4 av = lds4(sm.sq[0] + s * kLQ + t4 * 4);   // A[t][s], zero for t <= s
        x[t4 * 4 + 0] = fmaf(-av.x, xs, x[t4 * 4 + 0]);
        x[t4 * 4 + 1] = fmaf(-av.y, xs, x[t4 * 4 + 1]);
        x[t4 * 4 + 2] = fmaf(-av.z, xs, x[t4 * 4 + 2]);
        x[t4 * 4 + 3] = fmaf(-av.w, xs, x[t4 * 4 + 3]);
      }
    }
#pragma unroll
    for (int t = 0; t < kLC; ++t) sm.sq[2][t * kLQ + tid] = x[t];
  }
  __syncthreads();
  const float* Tm = sm.sq[2];
  const float* Mm = sm.sq[1];

  // ---- W = T (beta c . k^) -> big[1] (the queries are read again later)
  if (tid < kLC) sm.part[0][tid] = sm.beta[tid] * sm.cdec[tid];
  __syncthreads();
  {
    float acc[4][8];
    zero(acc);
    nn_smem<kLC>(Tm, kLQ, sm.part[0], Kh, kLP, r0, cg, acc);
    store_dense(sm.big[1], r0, cg, acc);
  }
  // ---- v -> big[2];  U' = T (beta . v) -> big[3]
  for (int idx = tid; idx < kLC * (kLD / 4); idx += kLThreads) {
    const int t = idx / (kLD / 4), c4 = idx % (kLD / 4);
    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (t < count) {
      const size_t off = (static_cast<size_t>(b) * a.tokens + t0 + t) * a.v_token + static_cast<size_t>(h) * kLD + c4 * 4;
      v = make_float4(load_any(a.v, off, a.in_is_bf16), load_any(a.v, off + 1, a.in_is_bf16),
                      load_any(a.v, off + 2, a.in_is_bf16), load_any(a.v, off + 3, a.in_is_bf16));
    }
    *reinterpret_cast<float4*>(sm.big[2] + t * kLP + c4 * 4) = v;
  }
  __syncthreads();
  {
    float acc[4][8];
    zero(acc);
    nn_smem<kLC>(Tm, kLQ, sm.beta, sm.big[2], kLP, r0, cg, acc);
    store_dense(sm.big[3], r0, cg, acc);
  }
  __syncthreads();
  // ---- U = U' - W S_0 -> big[4] (strided columns)
  {
    float acc[4][8];
    zero(acc);
    nt_glob(sm.big[1], kLP, S0, r0, cg, acc);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int e = (r0 + i) * kLP + cg + 16 * j;
        sm.big[4][e] = sm.big[3][e] - acc[i][j];
      }
  }
  __syncthreads();
  // ---- dO -> big[2]
  for (int idx = tid; idx < kLC * (kLD / 4); idx += kLThreads) {
    const int t = idx / (kLD / 4), c4 = idx % (kLD / 4);
    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (t < count)
      v = ldg4(a.dcore + ((static_cast<size_t>(b) * a.tokens + t0 + t) * a.value_heads + h) * kLD + c4 * 4);
    *reinterpret_cast<float4*>(sm.big[2] + t * kLP + c4 * 4) = v;
  }
  __syncthreads();

  // row sums into sm.db / sm.dbeta are added by the lane with cg == 0 of the row's group; column
  // sums go through sm.part
  auto add_rows = [&](float* dst, const float (&v)[4], float sign) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float total = row_sum16(v[i]);
      if (cg == 0) dst[r0 + i] += sign * total;
    }
  };

  // ---- dM = mask(dO U^T): M-bar = dM . M into db, dH = dM . ratio -> sq[0]
  {
    float acc[4][4];
    zero(acc);
    nt_smem<kLD>(sm.big[2], kLP, sm.big[4], kLP, r0, cg, acc);
    float rows[4] = {0.0f, 0.0f, 0.0f, 0.0f}, cols[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int t = r0 + i, s = cg + 16 * j;
        const float dm = s <= t ? acc[i][j] : 0.0f;
        const float bar = dm * Mm[t * kLQ + s];
        rows[i] += bar;
        cols[j] += bar;
        sm.sq[0][t * kLQ + s] = s <= t ? dm * expf(sm.b[t] - sm.b[s]) : 0.0f;
      }
    add_rows(sm.db, rows, 1.0f);
#pragma unroll
    for (int j = 0; j < 4; ++j) sm.part[rg][cg + 16 * j] = cols[j];
  }
  __syncthreads();
  if (tid < kLC) {
    float total = 0.0f;
#pragma unroll
    for (int g = 0; g < 16; ++g) total += sm.part[g][tid];
    sm.db[tid] -= total;
  }
  __syncthreads();

  float dk_acc[4][8], dq_acc[4][8];
  zero(dk_acc);
  zero(dq_acc);
  float kt_total = 0.0f;   // sum of dKt . Kt over the chunk (thread partial)
  const float gamma = sm.cdec[kLC - 1];

  // ---- dKt = U dS^T (dense columns = keys)
  {
    float acc[4][8];
    zero(acc);
    nn_glob(sm.big[4], kLP, dS, r0, cg, acc);
    float rows[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float f = gamma / sm.cdec[r0 + i];
      float rs = 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        dk_acc[i][j] = fmaf(f, acc[i][j], dk_acc[i][j]);
        rs = fmaf(acc[i][j] * f, Kh[(r0 + i) * kLP + cg * 8 + j], rs);
      }
      rows[i] = rs;
      kt_total += rs;
    }
    add_rows(sm.db, rows, -1.0f);
  }
  __syncthreads();   // every read of U is done
  // ---- dU = M^T dO + Kt dS -> big[4]
  {
    float acc[4][8];
    zero(acc);
    tn_smem<kLC>(Mm, kLQ, sm.big[2], kLP, r0, cg, acc);
    store_dense(sm.big[4], r0, cg, acc);
  }
  __syncthreads();
  {
    float acc[4][8];
    zero(acc);
    nt_glob(Kh, kLP, dS, r0, cg, acc);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float f = gamma / sm.cdec[r0 + i];
#pragma unroll
      for (int j = 0; j < 8; ++j) sm.big[4][(r0 + i) * kLP + cg + 16 * j] += f * acc[i][j];
    }
  }
  // ---- dQc = dO S_0^T: dq^ += c . dQc, db += rows(dQc . c q^)
  {
    float acc[4][8];
    zero(acc);
    nn_glob(sm.big[2], kLP, S0, r0, cg, acc);
    float rows[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = r0 + i;
      const float c = sm.cdec[t];
      float rs = 0.0f;
      const size_t off = (static_cast<size_t>(b) * a.tokens + t0 + t) * a.qk_token + static_cast<size_t>(kh) * kLD + cg * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        dq_acc[i][j] = fmaf(c, acc[i][j], dq_acc[i][j]);
        const float qh = t < count ? load_any(a.q, off + j, a.in_is_bf16) * sm.iq[t] * q_scale : 0.0f;
        rs = fmaf(acc[i][j] * c, qh, rs);
      }
      rows[i] = rs;
    }
    add_rows(sm.db, rows, 1.0f);
  }
  __syncthreads();   // dU complete; dO no longer needed
  // ---- dW = -dU S_0^T -> big[2]
  {
    float acc[4][8];
    zero(acc);
    nn_glob(sm.big[4], kLP, S0, r0, cg, acc);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[i][j] = -acc[i][j];
    store_dense(sm.big[2], r0, cg, acc);
  }
  // ---- X1 = T^T dU: dv = beta . X1, dbeta += rows(X1 . v); X1 replaces dU
  {
    float acc[4][8];
    zero(acc);
    tn_smem<kLC>(Tm, kLQ, sm.big[4], kLP, r0, cg, acc);
    float rows[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = r0 + i;
      float rs = 0.0f;
      if (t < count) {
        const size_t voff = (static_cast<size_t>(b) * a.tokens + t0 + t) * a.v_token + static_cast<size_t>(h) * kLD + cg * 8;
        float* dv = a.dv_out + (static_cast<size_t>(b) * a.tokens + t0 + t) * a.dv_token + static_cast<size_t>(h) * kLD + cg * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          rs = fmaf(acc[i][j], load_any(a.v, voff + j, a.in_is_bf16), rs);
          dv[j] = sm.beta[t] * acc[i][j];
        }
      }
      rows[i] = rs;
    }
    add_rows(sm.dbeta, rows, 1.0f);
    __syncthreads();   // every read of dU is done (and dW is complete)
    store_dense(sm.big[4], r0, cg, acc);
  }
  // ---- X2 = T^T dW: dk^ += beta c . X2, dbeta += rows(X2 . c k^), db += rows(X2 . beta c k^); X2 replaces dW
  {
    float acc[4][8];
    zero(acc);
    tn_smem<kLC>(Tm, kLQ, sm.big[2], kLP, r0, cg, acc);
    float rows_beta[4], rows_b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = r0 + i;
      const float c = sm.cdec[t], be = sm.beta[t];
      float rs = 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        dk_acc[i][j] = fmaf(be * c, acc[i][j], dk_acc[i][j]);
        rs = fmaf(acc[i][j] * c, Kh[t * kLP + cg * 8 + j], rs);
      }
      rows_beta[i] = rs;
      rows_b[i] = rs * be;
    }
    add_rows(sm.dbeta, rows_beta, 1.0f);
    add_rows(sm.db, rows_b, 1.0f);
    __syncthreads();   // every read of dW is done
    store_dense(sm.big[2], r0, cg, acc);
  }
  __syncthreads();
  // ---- dA = -mask(X1 U'^T + X2 W^T); with G again: A-bar into db, dbeta; dG + dG^T -> sq[1]
  {
    float acc[4][4], g[4][4];
    zero(acc);
    zero(g);
    nt_smem<kLD>(sm.big[4], kLP, sm.big[3], kLP, r0, cg, acc);
    nt_smem<kLD>(sm.big[2], kLP, sm.big[1], kLP, r0, cg, acc);
    nt_smem<kLD>(Kh, kLP, Kh, kLP, r0, cg, g);
    float rows_beta[4] = {0.0f, 0.0f, 0.0f, 0.0f}, rows_b[4] = {0.0f, 0.0f, 0.0f, 0.0f}, cols[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    // (M was last read by the dU product, two barriers ago)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int t = r0 + i, s = cg + 16 * j;
        if (s < t) {
          const float e = expf(sm.b[t] - sm.b[s]);
          const float per_beta = -acc[i][j] * e * g[i][j];   // dA . dA/dbeta_t
          const float bar = per_beta * sm.beta[t];            // dA . A
          const float dg = -acc[i][j] * e * sm.beta[t];       // dA . dA/dG
          rows_beta[i] += per_beta;
          rows_b[i] += bar;
          cols[j] += bar;
          sm.sq[1][t * kLQ + s] = dg;
          sm.sq[1][s * kLQ + t] = dg;
        } else if (s == t) {
          sm.sq[1][t * kLQ + s] = 0.0f;
        }
      }
    add_rows(sm.dbeta, rows_beta, 1.0f);
    add_rows(sm.db, rows_b, 1.0f);
#pragma unroll
    for (int j = 0; j < 4; ++j) sm.part[rg][cg + 16 * j] = cols[j];
  }
  __syncthreads();
  if (tid < kLC) {
    float total = 0.0f;
#pragma unroll
    for (int g = 0; g < 16; ++g) total += sm.part[g][tid];
    sm.db[tid] -= total;
  }
  // ---- dk^ += (dG + dG^T) k^ + dH^T q^;  dq^ += dH k^   (q^ is staged again, into big[3])
  for (int idx = tid; idx < kLC * (kLD / 4); idx += kLThreads) {
    const int t = idx / (kLD / 4), c4 = idx % (kLD / 4);
    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (t < count) {
      const size_t off = (static_cast<size_t>(b) * a.tokens + t0 + t) * a.qk_token + static_cast<size_t>(kh) * kLD + c4 * 4;
      const float f = sm.iq[t] * q_scale;
      v = make_float4(load_any(a.q, off, a.in_is_bf16) * f, load_any(a.q, off + 1, a.in_is_bf16) * f,
                      load_any(a.q, off + 2, a.in_is_bf16) * f, load_any(a.q, off + 3, a.in_is_bf16) * f);
    }
    *reinterpret_cast<float4*>(sm.big[3] + t * kLP + c4 * 4) = v;
  }
  __syncthreads();
  nn_smem<kLC>(sm.sq[1], kLQ, nullptr, Kh, kLP, r0, cg, dk_acc);
  nn_smem<kLC>(sm.sq[0], kLQ, nullptr, Kh, kLP, r0, cg, dq_acc);
  tn_smem<kLC>(sm.sq[0], kLQ, sm.big[3], kLP, r0, cg, dk_acc);

  // ---- through the normalisations: per-token partials in the layout of the gather kernels (one tile)
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = r0 + i;
    float pk = 0.0f, pq = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      pk = fmaf(dk_acc[i][j], Kh[t * kLP + cg * 8 + j], pk);
      pq = fmaf(dq_acc[i][j], sm.big[3][t * kLP + cg * 8 + j], pq);
    }
    pk = row_sum16(pk);
    pq = row_sum16(pq) / (q_scale * q_scale);   // q^ = scale . unit vector
    if (t < count) {
      const size_t partial = (static_cast<size_t>(b) * a.tokens + t0 + t) * a.value_heads + h;
      float* out = a.qk_partials + partial * 2 * kLD + cg * 8;
      const float ikt = sm.ik[t], iqt = sm.iq[t] * q_scale;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        out[j] = iqt * (dq_acc[i][j] - sm.big[3][t * kLP + cg * 8 + j] * pq);
        out[kLD + j] = ikt * (dk_acc[i][j] - Kh[t * kLP + cg * 8 + j] * pk);
      }
    }
  }

  // ---- the chunk-end terms of db: sum(dKt . Kt) + gamma <dS_C, S_0>
  {
    float dot = 0.0f;
    for (int e = tid * 4; e < kLD * kLD; e += kLThreads * 4) {
      const float4 x = ldg4(S0 + e), y = ldg4(dS + e);
      dot = fmaf(x.x, y.x, dot); dot = fmaf(x.y, y.y, dot); dot = fmaf(x.z, y.z, dot); dot = fmaf(x.w, y.w, dot);
    }
    float total = kt_total + gamma * dot;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    if (lane == 0) sm.red[warp] = total;
  }
  __syncthreads();
  if (tid == 0) {
    float total = 0.0f;
    for (int w = 0; w < kLThreads / 32; ++w) total += sm.red[w];
    sm.db[kLC - 1] += total;
    // d log g_s = sum of db_t over t >= s
    float run = 0.0f;
    for (int t = kLC - 1; t >= 0; --t) { run += sm.db[t]; sm.db[t] = run; }
  }
  __syncthreads();
  if (tid < count) {
    const size_t partial = (static_cast<size_t>(b) * a.tokens + t0 + tid) * a.value_heads + h;
    const float rate = expf(a.a_log[h]);
    const float dlog = sm.db[tid];
    a.scalar_partials[partial * 3 + 0] = -dlog * rate / (1.0f + expf(-sm.alpha[tid]));
    a.scalar_partials[partial * 3 + 1] = sm.dbeta[tid] * sm.sigmoid[tid] * (1.0f - sm.sigmoid[tid]);
    a.scalar_partials[partial * 3 + 2] = -dlog * rate * sm.softplus[tid];
  }
}

__global__ void cast_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, size_t count) {
  const size_t i = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (i + 3 < count) {
    const float4 v = ldg4(src + i);
    *reinterpret_cast<uint2*>(dst + i) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
  } else {
    for (size_t e = i; e < count; ++e) dst[e] = __float2bfloat16_rn(src[e]);
  }
}

size_t align_up(size_t n) { return (n + 1023) / 1024 * 1024; }

}  // namespace

bool gdn_bwd_chunked_supported(const GdnBwdArgs& a) {
  return a.key_dim == kLD && a.value_dim == kLD && a.in_is_bf16 && a.tokens >= 4 * kLC &&
         (reinterpret_cast<uintptr_t>(a.q) & 15u) == 0 && (reinterpret_cast<uintptr_t>(a.k) & 15u) == 0 &&
         (reinterpret_cast<uintptr_t>(a.v) & 15u) == 0 && a.qk_token % 8 == 0 && a.v_token % 8 == 0;
}

// Layout of the workspace: records | g, beta | dcore as bf16 | forward output (bf16, unused) |
// states | state gradients | q/k partials | scalar partials
struct ChunkedBwdLayout {
  size_t records, gates, dcore16, out16, states, dstates, qk_partials, scalar_partials, total;
};
static ChunkedBwdLayout chunked_bwd_layout(int batch, int tokens, int value_heads) {
  const size_t chunks = (tokens + kLC - 1) / kLC, units = static_cast<size_t>(batch) * value_heads;
  const size_t rows = static_cast<size_t>(batch) * tokens * value_heads;
  ChunkedBwdLayout l;
  size_t at = 0;
  l.records = at; at += align_up(gdn_chunked_workspace_bytes(batch, tokens, value_heads, kLD));
  l.gates = at; at += align_up(rows * 2 * sizeof(float));
  l.dcore16 = at; at += align_up(rows * kLD * 2);
  l.out16 = at; at += align_up(rows * kLD * 2);
  l.states = at; at += align_up(units * chunks * kLD * kLD * sizeof(float));
  l.dstates = at; at += align_up(units * chunks * kLD * kLD * sizeof(float));
  l.qk_partials = at; at += align_up(rows * 2 * kLD * sizeof(float));
  l.scalar_partials = at; at += align_up(rows * 3 * sizeof(float));
  l.total = at + 1024;   // room to align the base
  return l;
}
size_t gdn_bwd_chunked_workspace_bytes(int batch, int tokens, int value_heads) {
  return chunked_bwd_layout(batch, tokens, value_heads).total;
}

// Fills a.qk_partials / a.scalar_partials (one tile per head) and a.dv_out; the caller runs the
// gather kernels over them.
cudaError_t gdn_bwd_chunked(cudaStream_t stream, GdnBwdArgs& a, void* workspace, uint32_t* status) {
  const ChunkedBwdLayout l = chunked_bwd_layout(a.batch, a.tokens, a.value_heads);
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(workspace) + 1023) & ~static_cast<uintptr_t>(1023));
  const int chunks = (a.tokens + kLC - 1) / kLC;
  const size_t rows = static_cast<size_t>(a.batch) * a.tokens * a.value_heads;
  float* g = reinterpret_cast<float*>(base + l.gates);
  float* beta = g + rows;
  __nv_bfloat16* dcore16 = reinterpret_cast<__nv_bfloat16*>(base + l.dcore16);
  float* states = reinterpret_cast<float*>(base + l.states);
  float* dstates = reinterpret_cast<float*>(base + l.dstates);
  a.qk_partials = reinterpret_cast<float*>(base + l.qk_partials);
  a.scalar_partials = reinterpret_cast<float*>(base + l.scalar_partials);

  cudaError_t e = gdn_gates(stream, a.a_in, a.b_in, a.a_log, a.dt_bias, a.ab_is_bf16,
                            static_cast<long long>(a.batch) * a.tokens, a.value_heads, a.round, g, beta);
  if (e != cudaSuccess) return e;
  const size_t count = rows * kLD;
  cast_to_bf16_kernel<<<static_cast<unsigned>((count / 4 + 255) / 256 + 1), 256, 0, stream>>>(a.dcore, dcore16, count);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  // forward: records and the state at every chunk's start (from a zero state, as the layer's
  // sequence mode runs); its outputs are not needed
  GdnArgs f{};
  f.q = a.q; f.k = a.k; f.v = a.v;
  f.in_is_bf16 = 1;
  f.qk_token = a.qk_token; f.v_token = a.v_token;
  f.g = g; f.beta = beta;
  f.out = base + l.out16; f.out_is_bf16 = 1;
  f.batch = a.batch; f.tokens = a.tokens; f.key_heads = a.key_heads; f.value_heads = a.value_heads;
  f.key_dim = kLD; f.value_dim = kLD;
  f.normalize_qk = 1; f.q_scale = 1.0f; f.round = a.round;
  // the scan reads its initial state from and leaves its final state in f.state: the last chunk's
  // slot of the state-gradient area is free until the reverse scan runs
  f.state = dstates;
  e = cudaMemsetAsync(dstates, 0, static_cast<size_t>(a.batch) * a.value_heads * kLD * kLD * sizeof(float), stream);
  if (e != cudaSuccess) return e;
  e = gdn_chunked_with_states(stream, f, base + l.records, states, status);
  if (e != cudaSuccess) return e;
  e = gdn_scan_bwd_launch(stream, dcore16, base + l.records, a.batch, a.tokens, a.value_heads, chunks, dstates, status);
  if (e != cudaSuccess) return e;
  LocalArgs la{a, states, dstates, chunks};
  e = cudaFuncSetAttribute(gdn_bwd_chunk_local, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(sizeof(LocalSmem)));
  if (e != cudaSuccess) return e;
  gdn_bwd_chunk_local<<<dim3(chunks, a.value_heads, a.batch), kLThreads, sizeof(LocalSmem), stream>>>(la);
  return cudaGetLastError();
}

}  // namespace pluto
