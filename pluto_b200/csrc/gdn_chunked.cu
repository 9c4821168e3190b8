// Chunked gated delta-net prefill (chunk = 64 tokens, key width 128).
//
// The reference runs the recurrence token by token (RecurrenceForward,
// src/llm/layers/sequence_delta_net.cc:55-102: 16384 dependent steps for the benchmark sequence).
// With decay g_t, write strength beta_t, normalised keys k_t and queries q_t the update is
//     S_t = g_t S_{t-1} + k_t d_t^T,   d_t = beta_t (v_t - (g_t S_{t-1})^T k_t),   o_t = S_t^T q_t.
// Inside a chunk with cumulative decay c_t = prod_{s<=t} g_s and chunk-start state S_0 this is
//     (I + A) D = beta.V - (beta.c.K) S_0,      A[t,s] = beta_t (c_t/c_s) (k_t.k_s)  for s < t
//     O = (c.Q) S_0 + M D,                      M[t,s] = (c_t/c_s) (q_t.k_s)         for s <= t
//     S_C = c_C S_0 + (K . c_C/c)^T D
// so with T = (I + A)^-1, W = T (beta.c.K), U = T (beta.V):   D = U - W S_0.
// Every decay factor used is a ratio c_t/c_s <= 1 computed as exp(b_t - b_s) from the running sum
// of log g, so nothing overflows however small the decays get.
//
// Two kernels:
//   gdn_chunk_prepare     one CTA per (sequence, head, chunk), all chunks in parallel: norms, A, M,
//                         the triangular inverse in fp32 (forward substitution), W, U, c.Q, K.c_C/c.
//                         Matrix products on the tensor cores (mma.sync bf16, fp32 accumulate;
//                         T is applied as a bf16 high part plus a bf16 remainder).
//   gdn_chunk_recurrence  one CTA per (sequence, head, 32 value columns) walks the chunks in
//                         order.  The transposed state slice S^T [16 columns x 128 keys] lives in
//                         each warp's MMA accumulator registers for the whole sequence, is re-used
//                         directly as the A operand of the next products (accumulator fragments
//                         repack to A fragments without leaving registers), and so does D: no
//                         shared-memory or TMEM round trip sits on the sequential path.  The
//                         per-chunk operand tiles arrive through 16-byte-aligned bulk copies into a
//                         two-stage ring; their rows are stored pre-padded in the workspace so
//                         ldmatrix is bank-conflict free.
#include "common.cuh"
#include "engine.h"
#include "gdn_records.cuh"

#include <mutex>

namespace pluto {
// gdn_scan_sm100.cu
size_t gdn_scan_smem_bytes();
cudaError_t gdn_scan_launch(cudaStream_t stream, const GdnArgs& a, const void* records, int first_chunk,
                            int chunks, int all_chunks, float* state_dump, uint32_t* status);
// gdn_prepare_sm100.cu
bool gdn_prepare_sm100_supported(const GdnArgs& a);
bool gdn_prepare_sm100_maps(const GdnArgs& a, CUtensorMap maps[3]);
cudaError_t gdn_prepare_sm100_launch(cudaStream_t stream, const CUtensorMap maps[3], const GdnArgs& a,
                                     void* records, int first_pair, int pairs, int chunks, uint32_t* status);
namespace {

// The scan walks a sequence's chunks one after another on (sequences x heads x slices) SMs -- 32 of
// 148 at batch 2 with 16 heads -- while the prepare kernel fills all of them.  Cut into pieces, the
// two overlap: the scan of piece i runs on a second, higher-priority stream beside the prepare of
// piece i + 1, each piece's scan ordered after its prepare by an event, and the caller's stream
// joins the second one at the end.
constexpr int kGdnMaxPieces = 16;
constexpr int kGdnMaxDevices = 64;
struct GdnLanes {
  cudaStream_t scan = nullptr;
  cudaEvent_t prepared[kGdnMaxPieces] = {}, scanned = nullptr;
  bool ok = false;
  std::mutex enqueue;   // one call at a time records and waits on the events
};
GdnLanes g_gdn_lanes[kGdnMaxDevices];
std::once_flag g_gdn_once[kGdnMaxDevices];

GdnLanes* gdn_lanes_for_current_device() {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kGdnMaxDevices) return nullptr;
  std::call_once(g_gdn_once[device], [device] {
    GdnLanes& l = g_gdn_lanes[device];
    int least = 0, greatest = 0;
    bool ok = cudaDeviceGetStreamPriorityRange(&least, &greatest) == cudaSuccess &&
              cudaStreamCreateWithPriority(&l.scan, cudaStreamNonBlocking, greatest) == cudaSuccess &&
              cudaEventCreateWithFlags(&l.scanned, cudaEventDisableTiming) == cudaSuccess;
    for (int i = 0; i < kGdnMaxPieces && ok; ++i)
      ok = cudaEventCreateWithFlags(&l.prepared[i], cudaEventDisableTiming) == cudaSuccess;
    l.ok = ok;
  });
  return g_gdn_lanes[device].ok ? &g_gdn_lanes[device] : nullptr;
}

// Chunk pairs per piece.  Measured at batch 2, 16 heads, 16384 tokens (128 pairs, 32 scan CTAs):
// 0.81 ms as one piece, 0.69 ms with 32 or 43 pairs per piece, 0.72 / 0.75 / 0.82 ms with 24 / 16 /
// 12 -- every piece costs the scan a state round trip through global memory and a cold record
// ring, and the prepare grid a partial last wave.  So: pieces of about a thousand prepare CTAs
// (seven waves), and one piece when the scan itself fills most of the GPU or the sequence is short.
int gdn_piece_pairs(const GdnArgs& a, int pairs) {
  const int units = a.batch * a.value_heads;
  const int scan_ctas = units * (a.value_dim / kGdnSliceCols);
  if (scan_ctas > 96) return pairs;
  int per_piece = max(8, (1024 + units - 1) / units);
  if (pairs < 2 * per_piece) return pairs;
  while ((pairs + per_piece - 1) / per_piece > kGdnMaxPieces) per_piece *= 2;
  return per_piece;
}

// after_prepare (optional): recorded on `stream` behind the last prepare launch -- what only needs
// the records (the reverse scan of the backward pass) can start there, beside the scan.
cudaError_t gdn_prepare_and_scan(cudaStream_t stream, const GdnArgs& a, uint8_t* records, int chunks,
                                 float* state_dump, uint32_t* status, cudaEvent_t after_prepare = nullptr) {
  CUtensorMap maps[3];
  if (!gdn_prepare_sm100_maps(a, maps)) return cudaErrorInvalidValue;
  const int pairs = (chunks + 1) / 2;
  const int per_piece = gdn_piece_pairs(a, pairs);
  if (per_piece >= pairs) {
    cudaError_t e = gdn_prepare_sm100_launch(stream, maps, a, records, 0, pairs, chunks, status);
    if (e == cudaSuccess && after_prepare != nullptr) e = cudaEventRecord(after_prepare, stream);
    if (e != cudaSuccess) return e;
    return gdn_scan_launch(stream, a, records, 0, chunks, chunks, state_dump, status);
  }
  GdnLanes* l = gdn_lanes_for_current_device();
  if (l == nullptr) return cudaErrorInitializationError;
  std::lock_guard<std::mutex> lock(l->enqueue);
  cudaError_t e = cudaSuccess;
  int piece = 0;
  for (int first = 0; first < pairs && e == cudaSuccess; first += per_piece, ++piece) {
    const int n = min(per_piece, pairs - first);
    e = gdn_prepare_sm100_launch(stream, maps, a, records, first, n, chunks, status);
    if (e == cudaSuccess) e = cudaEventRecord(l->prepared[piece], stream);
    if (e == cudaSuccess && after_prepare != nullptr && first + per_piece >= pairs) e = cudaEventRecord(after_prepare, stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(l->scan, l->prepared[piece], 0);
    if (e == cudaSuccess)
      e = gdn_scan_launch(l->scan, a, records, first * 2, min(n * 2, chunks - first * 2), chunks, state_dump, status);
  }
  // (joined even after a failed launch, so that nothing of this call is left running unordered)
  cudaError_t joined = cudaEventRecord(l->scanned, l->scan);
  if (joined == cudaSuccess) joined = cudaStreamWaitEvent(stream, l->scanned, 0);
  return e != cudaSuccess ? e : joined;
}

constexpr int kC = 64;           // tokens per chunk
constexpr int kDK = 128;         // key width handled by this path
constexpr int kPitch = 136;      // bf16 elements per padded row of a [64 x 128] tile (272 bytes)
constexpr int kMPitch = 72;      // bf16 elements per padded row of the [64 x 64] M tile (144 bytes)
constexpr int kUPitch = 68;      // fp32 elements per padded row of U^T (272 bytes)
constexpr int kTileBytes = kC * kPitch * 2;     // 17408
constexpr int kMBytes = kC * kMPitch * 2;       // 9216
constexpr float kMinLogDecay = -60.0f;
// bf16 remainders ("lo" parts) used on the sequential path.  W S feeds the difference
// D = U - W S, so the state enters that product as high part + remainder; the output products
// and the state increment take the high parts only (their results are rounded to bf16 anyway or
// decay away), which halves the dependent MMA stream of every chunk.
constexpr bool kStateLoForWS = true;
constexpr bool kStateLoForOut = false;
constexpr bool kDeltaLo = false;

// Workspace record of one (sequence, head, chunk); offsets in bytes.
struct Record {
  static constexpr size_t kW = 0;
  static constexpr size_t kQ = kW + kTileBytes;
  static constexpr size_t kK = kQ + kTileBytes;
  static constexpr size_t kM = kK + kTileBytes;
  static constexpr size_t kU = kM + kMBytes;  // U^T: [value_dim][kUPitch] fp32
  static __host__ __device__ size_t gamma(int dv) { return kU + static_cast<size_t>(dv) * kUPitch * 4; }
  static __host__ __device__ size_t bytes(int dv) { return gamma(dv) + 256; }
};

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// A fragment of a row-major [rows][pitch] bf16 tile: rows row0..row0+15, columns k0..k0+15.
__device__ __forceinline__ void load_a(uint32_t (&a)[4], const __nv_bfloat16* tile, int pitch,
                                       int row0, int k0, int lane) {
  ldsm_x4(a, tile + (row0 + lane % 16) * pitch + k0 + (lane / 16) * 8);
}
// B fragments for two k-steps (k0..k0+31) of an operand stored [n][k]: n0..n0+7.
__device__ __forceinline__ void load_b_nk(uint32_t (&b)[4], const __nv_bfloat16* tile, int pitch,
                                          int n0, int k0, int lane) {
  ldsm_x4(b, tile + (n0 + lane % 8) * pitch + k0 + (lane / 8) * 8);
}
// B fragments for two n-tiles (n0..n0+15) of an operand stored [k][n]: k0..k0+15.
__device__ __forceinline__ void load_b_kn(uint32_t (&b)[4], const __nv_bfloat16* tile, int pitch,
                                          int k0, int n0, int lane) {
  ldsm_x4_t(b, tile + (k0 + ((lane / 8) & 1) * 8 + lane % 8) * pitch + n0 + (lane / 16) * 8);
}

// -------------------------------------------------------------------------------------------
// prepare: grid (chunks, value heads, batch), 128 threads
// -------------------------------------------------------------------------------------------
struct PrepareSmem {
  __nv_bfloat16 kb[kC][kPitch];   // normalised keys
  __nv_bfloat16 qb[kC][kPitch];   // normalised, scaled queries
  __nv_bfloat16 x1[kC][kPitch];   // beta * c * k
  __nv_bfloat16 x2[kC][kPitch];   // beta * v (value columns in blocks of 128)
  float a[kC][kC + 1];            // strictly lower triangular A
  __nv_bfloat16 t_hi[kC][kMPitch];
  __nv_bfloat16 t_lo[kC][kMPitch];
  float b[kC], beta[kC];
};

__global__ void __launch_bounds__(128) gdn_chunk_prepare(GdnArgs a, uint8_t* workspace, int chunks) {
  extern __shared__ __align__(16) uint8_t prepare_raw[];
  PrepareSmem& s = *reinterpret_cast<PrepareSmem*>(prepare_raw);
  const int chunk = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int kh = h / (a.value_heads / a.key_heads);
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int dv = a.value_dim;
  const int t0 = chunk * kC;
  uint8_t* rec = workspace + ((static_cast<size_t>(b) * a.value_heads + h) * chunks + chunk) * Record::bytes(dv);
  const __nv_bfloat16* qg = static_cast<const __nv_bfloat16*>(a.q);
  const __nv_bfloat16* kg = static_cast<const __nv_bfloat16*>(a.k);
  const __nv_bfloat16* vg = static_cast<const __nv_bfloat16*>(a.v);

  // ---- gates: running sum of log decay (tokens past the sequence end: g = 1, beta = 0)
  if (threadIdx.x < kC) {
    const int t = t0 + threadIdx.x;
    float lg = 0.0f, be = 0.0f;
    if (t < a.tokens) {
      const size_t off = (static_cast<size_t>(b) * a.tokens + t) * a.value_heads + h;
      lg = fmaxf(logf(a.g[off]), kMinLogDecay);
      be = a.beta[off];
    }
    s.b[threadIdx.x] = lg;
    s.beta[threadIdx.x] = be;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float run = 0.0f;
    for (int t = 0; t < kC; ++t) { run += s.b[t]; s.b[t] = run; }
  }
  // ---- q, k: 16-byte loads issued up front (8 per thread each); 16 threads share a token row,
  //      so the norms reduce inside a half-warp and the raw values never touch shared memory
  const int sub = threadIdx.x % 16, rbase = threadIdx.x / 16;   // row = rbase + 8 * i
  uint4 qraw[8], kraw[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int t = t0 + rbase + 8 * i;
    qraw[i] = kraw[i] = make_uint4(0, 0, 0, 0);
    if (t < a.tokens) {
      const size_t off = (static_cast<size_t>(b) * a.tokens + t) * a.qk_token + static_cast<size_t>(kh) * kDK + sub * 8;
      qraw[i] = __ldg(reinterpret_cast<const uint4*>(qg + off));
      kraw[i] = __ldg(reinterpret_cast<const uint4*>(kg + off));
    }
  }
  __syncthreads();  // running sums of log decay are in place
  const float b_last = s.b[kC - 1];
  __nv_bfloat16* q_out = reinterpret_cast<__nv_bfloat16*>(rec + Record::kQ);
  __nv_bfloat16* k_out = reinterpret_cast<__nv_bfloat16*>(rec + Record::kK);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int tt = rbase + 8 * i;
    const uint32_t qw[4] = {qraw[i].x, qraw[i].y, qraw[i].z, qraw[i].w};
    const uint32_t kw[4] = {kraw[i].x, kraw[i].y, kraw[i].z, kraw[i].w};
    float qf[8], kf[8], qs = 0.0f, ks = 0.0f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      qf[2 * e] = bf16_lo(qw[e]); qf[2 * e + 1] = bf16_hi(qw[e]);
      kf[2 * e] = bf16_lo(kw[e]); kf[2 * e + 1] = bf16_hi(kw[e]);
      qs += qf[2 * e] * qf[2 * e] + qf[2 * e + 1] * qf[2 * e + 1];
      ks += kf[2 * e] * kf[2 * e] + kf[2 * e + 1] * kf[2 * e + 1];
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) {
      qs += __shfl_xor_sync(0xffffffffu, qs, o);
      ks += __shfl_xor_sync(0xffffffffu, ks, o);
    }
    const float qn = a.normalize_qk ? rsqrtf(qs + 1e-6f) / sqrtf(static_cast<float>(kDK)) : a.q_scale;
    const float kn = a.normalize_qk ? rsqrtf(ks + 1e-6f) : 1.0f;
    const float decay = __expf(s.b[tt]), tail = __expf(b_last - s.b[tt]), bd = s.beta[tt] * decay;
    uint32_t kbw[4], qbw[4], x1w[4], qow[4], kow[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float q0 = qf[2 * e] * qn, q1 = qf[2 * e + 1] * qn;
      const float k0 = kf[2 * e] * kn, k1 = kf[2 * e + 1] * kn;
      kbw[e] = pack_bf16(k0, k1);
      qbw[e] = pack_bf16(q0, q1);
      x1w[e] = pack_bf16(bd * k0, bd * k1);
      qow[e] = pack_bf16(decay * q0, decay * q1);
      kow[e] = pack_bf16(tail * k0, tail * k1);
    }
    *reinterpret_cast<uint4*>(&s.kb[tt][sub * 8]) = make_uint4(kbw[0], kbw[1], kbw[2], kbw[3]);
    *reinterpret_cast<uint4*>(&s.qb[tt][sub * 8]) = make_uint4(qbw[0], qbw[1], qbw[2], qbw[3]);
    *reinterpret_cast<uint4*>(&s.x1[tt][sub * 8]) = make_uint4(x1w[0], x1w[1], x1w[2], x1w[3]);
    *reinterpret_cast<uint4*>(q_out + tt * kPitch + sub * 8) = make_uint4(qow[0], qow[1], qow[2], qow[3]);
    *reinterpret_cast<uint4*>(k_out + tt * kPitch + sub * 8) = make_uint4(kow[0], kow[1], kow[2], kow[3]);
  }
  if (threadIdx.x == 0) *reinterpret_cast<float*>(rec + Record::gamma(dv)) = __expf(b_last);
  __syncthreads();

  // ---- A = beta_t e^{b_t-b_s} (k_t.k_s) [s<t],  M = e^{b_t-b_s} (q_t.k_s) [s<=t]
  {
    float kk[8][4], qk[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) kk[n][i] = qk[n][i] = 0.0f;
#pragma unroll
    for (int kp = 0; kp < kDK / 32; ++kp) {
      uint32_t ak0[4], ak1[4], aq0[4], aq1[4];
      load_a(ak0, &s.kb[0][0], kPitch, warp * 16, kp * 32, lane);
      load_a(ak1, &s.kb[0][0], kPitch, warp * 16, kp * 32 + 16, lane);
      load_a(aq0, &s.qb[0][0], kPitch, warp * 16, kp * 32, lane);
      load_a(aq1, &s.qb[0][0], kPitch, warp * 16, kp * 32 + 16, lane);
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        uint32_t bf[4];
        load_b_nk(bf, &s.kb[0][0], kPitch, n * 8, kp * 32, lane);
        mma16816(kk[n], ak0, bf[0], bf[1]);
        mma16816(kk[n], ak1, bf[2], bf[3]);
        mma16816(qk[n], aq0, bf[0], bf[1]);
        mma16816(qk[n], aq1, bf[2], bf[3]);
      }
    }
    __nv_bfloat16* m_out = reinterpret_cast<__nv_bfloat16*>(rec + Record::kM);
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int t = warp * 16 + lane / 4 + half * 8;
        const int s0 = n * 8 + (lane % 4) * 2;
        float av[2], mv[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int sc = s0 + e;
          const float ratio = sc <= t ? __expf(s.b[t] - s.b[sc]) : 0.0f;
          av[e] = sc < t ? s.beta[t] * ratio * kk[n][half * 2 + e] : 0.0f;
          mv[e] = ratio * qk[n][half * 2 + e];
          s.a[t][sc] = av[e];
        }
        *reinterpret_cast<uint32_t*>(m_out + t * kMPitch + s0) = pack_bf16(mv[0], mv[1]);
      }
  }
  __syncthreads();

  // ---- T = (I + A)^-1 by forward substitution; thread j owns column j
  if (threadIdx.x < kC) {
    const int j = threadIdx.x;
    float col[kC];
#pragma unroll
    for (int t = 0; t < kC; ++t) {
      float acc = t == j ? 1.0f : 0.0f;
#pragma unroll
      for (int sc = 0; sc < t; ++sc) acc = fmaf(-s.a[t][sc], col[sc], acc);
      col[t] = acc;
    }
#pragma unroll
    for (int t = 0; t < kC; ++t) {
      const __nv_bfloat16 hi = __float2bfloat16_rn(col[t]);
      s.t_hi[t][j] = hi;
      s.t_lo[t][j] = __float2bfloat16_rn(col[t] - __bfloat162float(hi));
    }
  }
  __syncthreads();

  // ---- W = T x1  -> workspace (bf16, padded rows)
  uint32_t th[4][4], tl[4][4];
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    load_a(th[ks], &s.t_hi[0][0], kMPitch, warp * 16, ks * 16, lane);
    load_a(tl[ks], &s.t_lo[0][0], kMPitch, warp * 16, ks * 16, lane);
  }
  {
    __nv_bfloat16* w_out = reinterpret_cast<__nv_bfloat16*>(rec + Record::kW);
#pragma unroll
    for (int np = 0; np < kDK / 16; ++np) {
      float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        uint32_t bf[4];
        load_b_kn(bf, &s.x1[0][0], kPitch, ks * 16, np * 16, lane);
        mma16816(acc[0], th[ks], bf[0], bf[1]);
        mma16816(acc[0], tl[ks], bf[0], bf[1]);
        mma16816(acc[1], th[ks], bf[2], bf[3]);
        mma16816(acc[1], tl[ks], bf[2], bf[3]);
      }
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int t = warp * 16 + lane / 4 + half * 8;
          const int i = np * 16 + n * 8 + (lane % 4) * 2;
          *reinterpret_cast<uint32_t*>(w_out + t * kPitch + i) =
              pack_bf16(acc[n][half * 2], acc[n][half * 2 + 1]);
        }
    }
  }
  // ---- U = T (beta v), value columns in blocks of 128 -> workspace as U^T fp32
  float* u_out = reinterpret_cast<float*>(rec + Record::kU);
  for (int j0 = 0; j0 < dv; j0 += kDK) {
    __syncthreads();
    uint4 vraw[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int t = t0 + rbase + 8 * i, j = j0 + sub * 8;
      vraw[i] = make_uint4(0, 0, 0, 0);
      if (t < a.tokens && j < dv)
        vraw[i] = __ldg(reinterpret_cast<const uint4*>(
            vg + (static_cast<size_t>(b) * a.tokens + t) * a.v_token + static_cast<size_t>(h) * dv + j));
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int tt = rbase + 8 * i;
      const float be = s.beta[tt];
      const uint32_t vw[4] = {vraw[i].x, vraw[i].y, vraw[i].z, vraw[i].w};
      uint32_t xw[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) xw[e] = pack_bf16(be * bf16_lo(vw[e]), be * bf16_hi(vw[e]));
      *reinterpret_cast<uint4*>(&s.x2[tt][sub * 8]) = make_uint4(xw[0], xw[1], xw[2], xw[3]);
    }
    __syncthreads();
#pragma unroll
    for (int np = 0; np < kDK / 16; ++np) {
      if (j0 + np * 16 >= dv) break;
      float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        uint32_t bf[4];
        load_b_kn(bf, &s.x2[0][0], kPitch, ks * 16, np * 16, lane);
        mma16816(acc[0], th[ks], bf[0], bf[1]);
        mma16816(acc[0], tl[ks], bf[0], bf[1]);
        mma16816(acc[1], th[ks], bf[2], bf[3]);
        mma16816(acc[1], tl[ks], bf[2], bf[3]);
      }
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int half = 0; half < 2; ++half)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int t = warp * 16 + lane / 4 + half * 8;
            const int j = j0 + np * 16 + n * 8 + (lane % 4) * 2 + e;
            if (j < dv) u_out[static_cast<size_t>(j) * kUPitch + t] = acc[n][half * 2 + e];
          }
    }
  }
}

// -------------------------------------------------------------------------------------------
// recurrence: grid (value_dim / 32, value heads, batch); warps 0-1 compute 16 value columns
// each, warp 2 feeds the ring.
// -------------------------------------------------------------------------------------------
constexpr int kRecStages = 2;
constexpr int kSliceCols = 32;
constexpr int kUSliceBytes = kSliceCols * kUPitch * 4;  // 8704
constexpr int kStageBytes = 3 * kTileBytes + kMBytes + kUSliceBytes + 16;  // + gamma
struct RecBarriers {
  uint64_t full[kRecStages];
  uint64_t empty[kRecStages];
};

__global__ void __launch_bounds__(96) gdn_chunk_recurrence(GdnArgs a, const uint8_t* workspace,
                                                           int chunks, uint32_t* status) {
  extern __shared__ __align__(128) uint8_t rec_smem[];
  RecBarriers* bar = reinterpret_cast<RecBarriers*>(rec_smem + kRecStages * kStageBytes);
  const int slice = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int dv = a.value_dim;
  const size_t rec_bytes = Record::bytes(dv);
  const uint8_t* rec0 = workspace + (static_cast<size_t>(b) * a.value_heads + h) * chunks * rec_bytes;

  if (threadIdx.x == 0) {
    for (int st = 0; st < kRecStages; ++st) {
      mbar_init(&bar->full[st], 1);
      mbar_init(&bar->empty[st], 2);
    }
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == 2) {
    if (lane == 0) {
      bool ok = true;
      for (int c = 0; c < chunks && ok; ++c) {
        const int st = c % kRecStages, use = c / kRecStages;
        if (use > 0) ok = mbar_wait(&bar->empty[st], (use - 1) & 1, status, 40);
        if (!ok) break;
        uint8_t* dst = rec_smem + st * kStageBytes;
        const uint8_t* rec = rec0 + static_cast<size_t>(c) * rec_bytes;
        mbar_expect_tx(&bar->full[st], 3 * kTileBytes + kMBytes + kUSliceBytes + 16);
        bulk_load(dst, rec + Record::kW, kTileBytes, &bar->full[st]);
        bulk_load(dst + kTileBytes, rec + Record::kQ, kTileBytes, &bar->full[st]);
        bulk_load(dst + 2 * kTileBytes, rec + Record::kK, kTileBytes, &bar->full[st]);
        bulk_load(dst + 3 * kTileBytes, rec + Record::kM, kMBytes, &bar->full[st]);
        bulk_load(dst + 3 * kTileBytes + kMBytes,
                  rec + Record::kU + static_cast<size_t>(slice) * kUSliceBytes, kUSliceBytes,
                  &bar->full[st]);
        bulk_load(dst + 3 * kTileBytes + kMBytes + kUSliceBytes, rec + Record::gamma(dv), 16,
                  &bar->full[st]);
      }
      for (int c = max(0, chunks - kRecStages); c < chunks; ++c)
        mbar_wait(&bar->full[c % kRecStages], (c / kRecStages) & 1, status, 41);
    }
    return;
  }

  // ---- compute warps: value columns j0..j0+15, state kept transposed: st[n][.] covers keys 8n..8n+7
  const int j0 = slice * kSliceCols + warp * 16;
  const int r0 = lane / 4, c0 = (lane % 4) * 2;
  float* state = a.state + (static_cast<size_t>(b) * a.value_heads + h) * kDK * dv;
  float sf[16][4];
#pragma unroll
  for (int n = 0; n < 16; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int j = j0 + r0 + (e >> 1) * 8, i = n * 8 + c0 + (e & 1);
      sf[n][e] = j < dv ? state[static_cast<size_t>(i) * dv + j] : 0.0f;
    }
  bool ok = true;
  for (int c = 0; c < chunks && ok; ++c) {
    const int st = c % kRecStages;
    ok = mbar_wait(&bar->full[st], (c / kRecStages) & 1, status, 42);
    if (!ok) break;
    const uint8_t* base = rec_smem + st * kStageBytes;
    const __nv_bfloat16* w_t = reinterpret_cast<const __nv_bfloat16*>(base);
    const __nv_bfloat16* q_t = reinterpret_cast<const __nv_bfloat16*>(base + kTileBytes);
    const __nv_bfloat16* k_t = reinterpret_cast<const __nv_bfloat16*>(base + 2 * kTileBytes);
    const __nv_bfloat16* m_t = reinterpret_cast<const __nv_bfloat16*>(base + 3 * kTileBytes);
    const float* u_t = reinterpret_cast<const float*>(base + 3 * kTileBytes + kMBytes) + warp * 16 * kUPitch;
    const float gamma = *reinterpret_cast<const float*>(base + 3 * kTileBytes + kMBytes + kUSliceBytes);

    // (W S)^T and (c.Q S)^T : [16 columns x 64 tokens].  The state enters as the A operand
    // (keys = contraction dimension) as a bf16 high part plus a bf16 remainder, repacked from the
    // accumulator fragments 32 keys at a time.
    float ws[8][4], os[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) ws[n][e] = os[n][e] = 0.0f;
#pragma unroll
    for (int kp = 0; kp < 4; ++kp) {
      uint32_t sa[2][4], sl[2][4];
#pragma unroll
      for (int q = 0; q < 2; ++q)
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          const int n = 2 * (2 * kp + q) + (p >> 1);
          const float x = sf[n][(p & 1) * 2], y = sf[n][(p & 1) * 2 + 1];
          sa[q][p] = pack_bf16(x, y);
          sl[q][p] = pack_bf16(x - bf16_lo(sa[q][p]), y - bf16_hi(sa[q][p]));
        }
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        uint32_t bw[4], bq[4];
        load_b_nk(bw, w_t, kPitch, n * 8, kp * 32, lane);
        load_b_nk(bq, q_t, kPitch, n * 8, kp * 32, lane);
        mma16816(ws[n], sa[0], bw[0], bw[1]);
        mma16816(ws[n], sa[1], bw[2], bw[3]);
        if (kStateLoForWS) {
          mma16816(ws[n], sl[0], bw[0], bw[1]);
          mma16816(ws[n], sl[1], bw[2], bw[3]);
        }
        mma16816(os[n], sa[0], bq[0], bq[1]);
        mma16816(os[n], sa[1], bq[2], bq[3]);
        if (kStateLoForOut) {
          mma16816(os[n], sl[0], bq[0], bq[1]);
          mma16816(os[n], sl[1], bq[2], bq[3]);
        }
      }
    }
    // D^T = U^T - (W S)^T, repacked as A operand (tokens = contraction dimension), hi + remainder
    uint32_t da[4][4], dl[4][4];
#pragma unroll
    for (int kt = 0; kt < 4; ++kt)
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const int n = 2 * kt + (p >> 1), half = p & 1;
        const int row = r0 + half * 8, t = n * 8 + c0;
        const float x = u_t[row * kUPitch + t] - ws[n][half * 2];
        const float y = u_t[row * kUPitch + t + 1] - ws[n][half * 2 + 1];
        da[kt][p] = pack_bf16(x, y);
        dl[kt][p] = pack_bf16(x - bf16_lo(da[kt][p]), y - bf16_hi(da[kt][p]));
      }
    // O^T += D^T M^T
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int kp = 0; kp < 2; ++kp) {
        uint32_t bm[4];
        load_b_nk(bm, m_t, kMPitch, n * 8, kp * 32, lane);
        mma16816(os[n], da[2 * kp], bm[0], bm[1]);
        mma16816(os[n], da[2 * kp + 1], bm[2], bm[3]);
        if (kDeltaLo) {
          mma16816(os[n], dl[2 * kp], bm[0], bm[1]);
          mma16816(os[n], dl[2 * kp + 1], bm[2], bm[3]);
        }
      }
    // S^T <- c_C S^T + D^T (K . c_C/c)
#pragma unroll
    for (int n = 0; n < 16; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) sf[n][e] *= gamma;
#pragma unroll
    for (int np = 0; np < 8; ++np)
#pragma unroll
      for (int kt = 0; kt < 4; ++kt) {
        uint32_t bk[4];
        load_b_kn(bk, k_t, kPitch, kt * 16, np * 16, lane);
        mma16816(sf[2 * np], da[kt], bk[0], bk[1]);
        mma16816(sf[2 * np + 1], da[kt], bk[2], bk[3]);
        if (kDeltaLo) {
          mma16816(sf[2 * np], dl[kt], bk[0], bk[1]);
          mma16816(sf[2 * np + 1], dl[kt], bk[2], bk[3]);
        }
      }
    __syncwarp();
    if (lane == 0) mbar_arrive(&bar->empty[st]);
    // store O^T (round as the reference does before its bf16 store)
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int t = c * kC + n * 8 + c0 + (e & 1), j = j0 + r0 + (e >> 1) * 8;
        if (t < a.tokens && j < dv) {
          const size_t off = ((static_cast<size_t>(b) * a.tokens + t) * a.value_heads + h) * dv + j;
          const float value = a.round ? bf16_round(os[n][e]) : os[n][e];
          if (a.out_is_bf16) static_cast<__nv_bfloat16*>(a.out)[off] = __float2bfloat16_rn(value);
          else static_cast<float*>(a.out)[off] = value;
        }
      }
  }
#pragma unroll
  for (int n = 0; n < 16; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int j = j0 + r0 + (e >> 1) * 8, i = n * 8 + c0 + (e & 1);
      if (j < dv) state[static_cast<size_t>(i) * dv + j] = sf[n][e];
    }
}

// -------------------------------------------------------------------------------------------
// Rewrites a (sequence, head, chunk) record of gdn_chunk_prepare into the swizzled operand tiles
// the tcgen05 scan kernel reads (gdn_records.cuh), computing the two chunk-local products that
// take the dependent pair of state products off the sequential path:
//     Pn = -(Kt^T W)   and   Qt = c.Q - M W.
// grid (chunks, value heads, batch), 256 threads; plain fp32 arithmetic.
// -------------------------------------------------------------------------------------------
struct ConvertSmem {
  __nv_bfloat16 w[kC][kDK + 2];
  __nv_bfloat16 kt[kC][kDK + 2];
  __nv_bfloat16 m[kC][kC + 2];
};

__global__ void __launch_bounds__(256) gdn_chunk_convert(const uint8_t* __restrict__ old_records,
                                                         uint8_t* __restrict__ new_records, int chunks,
                                                         int value_heads, int dv) {
  extern __shared__ __align__(16) uint8_t convert_raw[];
  ConvertSmem& s = *reinterpret_cast<ConvertSmem*>(convert_raw);
  const size_t index = (static_cast<size_t>(blockIdx.z) * value_heads + blockIdx.y) * chunks + blockIdx.x;
  const uint8_t* src = old_records + index * Record::bytes(dv);
  uint8_t* dst = new_records + index * GdnRecord::bytes(dv);
  const __nv_bfloat16* w_in = reinterpret_cast<const __nv_bfloat16*>(src + Record::kW);
  const __nv_bfloat16* q_in = reinterpret_cast<const __nv_bfloat16*>(src + Record::kQ);
  const __nv_bfloat16* k_in = reinterpret_cast<const __nv_bfloat16*>(src + Record::kK);
  const __nv_bfloat16* m_in = reinterpret_cast<const __nv_bfloat16*>(src + Record::kM);
  const float* u_in = reinterpret_cast<const float*>(src + Record::kU);
  for (int e = threadIdx.x; e < kC * kDK; e += 256) {
    const int t = e / kDK, i = e % kDK;
    s.w[t][i] = w_in[t * kPitch + i];
    const __nv_bfloat16 k = k_in[t * kPitch + i];
    s.kt[t][i] = k;
    *reinterpret_cast<__nv_bfloat16*>(dst + GdnRecord::kKT + gdn_swizzled_offset(kC, t, i)) = k;
  }
  for (int e = threadIdx.x; e < kC * kC; e += 256) {
    const int t = e / kC, sc = e % kC;
    const __nv_bfloat16 v = m_in[t * kMPitch + sc];
    s.m[t][sc] = v;
    *reinterpret_cast<__nv_bfloat16*>(dst + GdnRecord::kMM + gdn_swizzled_offset(kC, t, sc)) = v;
  }
  if (threadIdx.x == 0)
    *reinterpret_cast<float*>(dst + GdnRecord::kGM) = *reinterpret_cast<const float*>(src + Record::gamma(dv));
  __syncthreads();
  // Pn[i_out][i_in] = -sum_t Kt[t][i_out] W[t][i_in]
  for (int e = threadIdx.x; e < kDK * kDK; e += 256) {
    const int io = e / kDK, ii = e % kDK;
    float acc = 0.0f;
    for (int t = 0; t < kC; ++t) acc = fmaf(__bfloat162float(s.kt[t][io]), __bfloat162float(s.w[t][ii]), acc);
    *reinterpret_cast<__nv_bfloat16*>(dst + GdnRecord::kPN + gdn_swizzled_offset(kDK, io, ii)) =
        __float2bfloat16_rn(-acc);
  }
  // Qt[t][i] = (c.Q)[t][i] - sum_s M[t][s] W[s][i]
  for (int e = threadIdx.x; e < kC * kDK; e += 256) {
    const int t = e / kDK, i = e % kDK;
    float acc = __bfloat162float(q_in[t * kPitch + i]);
    for (int sc = 0; sc < kC; ++sc) acc = fmaf(-__bfloat162float(s.m[t][sc]), __bfloat162float(s.w[sc][i]), acc);
    *reinterpret_cast<__nv_bfloat16*>(dst + GdnRecord::kQT + gdn_swizzled_offset(kC, t, i)) = __float2bfloat16_rn(acc);
  }
  // U [token][value column] in bf16, one tile per 128-column slice
  for (int e = threadIdx.x; e < kC * dv; e += 256) {
    const int j = e / kC, t = e % kC;
    const float u = u_in[static_cast<size_t>(j) * kUPitch + t];
    uint8_t* tile = dst + GdnRecord::kCommon + static_cast<size_t>(j / kGdnSliceCols) * GdnRecord::kSlice;
    *reinterpret_cast<__nv_bfloat16*>(tile + GdnRecord::kUH + gdn_swizzled_offset(kC, t, j % kGdnSliceCols)) =
        __float2bfloat16_rn(u);
  }
}

}  // namespace

bool gdn_chunked_supported(const GdnArgs& a) {
  return a.in_is_bf16 && a.key_dim == kDK && a.value_dim % kSliceCols == 0 && a.value_dim <= 256 &&
         a.tokens >= kC && a.qk_token % 8 == 0 && a.v_token % 8 == 0 &&
         (reinterpret_cast<uintptr_t>(a.q) & 15u) == 0 && (reinterpret_cast<uintptr_t>(a.k) & 15u) == 0 &&
         (reinterpret_cast<uintptr_t>(a.v) & 15u) == 0;
}

// Value widths that are whole 128-column slices take the tcgen05 scan kernel.
static bool scan_on_tensor_memory(int value_dim) { return value_dim % kGdnSliceCols == 0; }

static size_t old_record_bytes(int batch, int tokens, int value_heads, int value_dim) {
  const size_t chunks = (static_cast<size_t>(tokens) + kC - 1) / kC;
  return (static_cast<size_t>(batch) * value_heads * chunks * Record::bytes(value_dim) + 1023) / 1024 * 1024;
}

// One 128-column slice: both kernels are tcgen05 and only the swizzled records exist.  Several
// slices: the mma.sync prepare writes its records, a conversion kernel rewrites them, tcgen05 scan.
// Other widths: the mma.sync pair of kernels.
size_t gdn_chunked_workspace_bytes(int batch, int tokens, int value_heads, int value_dim) {
  const size_t chunks = (static_cast<size_t>(tokens) + kC - 1) / kC;
  const size_t swizzled = static_cast<size_t>(batch) * value_heads * chunks * GdnRecord::bytes(value_dim) + 1024;
  if (value_dim == kGdnSliceCols) return swizzled;
  size_t bytes = old_record_bytes(batch, tokens, value_heads, value_dim);
  if (scan_on_tensor_memory(value_dim)) bytes += swizzled;
  return bytes;
}

cudaError_t gdn_chunked(cudaStream_t stream, const GdnArgs& a, void* workspace, uint32_t* status) {
  const int chunks = (a.tokens + kC - 1) / kC;
  if (gdn_prepare_sm100_supported(a)) {
    uint8_t* records = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(workspace) + 1023) &
                                                  ~static_cast<uintptr_t>(1023));
    return gdn_prepare_and_scan(stream, a, records, chunks, nullptr, status);
  }
  cudaError_t e = cudaFuncSetAttribute(gdn_chunk_prepare, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(sizeof(PrepareSmem)));
  if (e != cudaSuccess) return e;
  gdn_chunk_prepare<<<dim3(chunks, a.value_heads, a.batch), 128, sizeof(PrepareSmem), stream>>>(
      a, static_cast<uint8_t*>(workspace), chunks);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  if (scan_on_tensor_memory(a.value_dim)) {
    uint8_t* base = static_cast<uint8_t*>(workspace) + old_record_bytes(a.batch, a.tokens, a.value_heads, a.value_dim);
    uint8_t* records = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(base) + 1023) & ~static_cast<uintptr_t>(1023));
    e = cudaFuncSetAttribute(gdn_chunk_convert, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(sizeof(ConvertSmem)));
    if (e != cudaSuccess) return e;
    gdn_chunk_convert<<<dim3(chunks, a.value_heads, a.batch), 256, sizeof(ConvertSmem), stream>>>(
        static_cast<const uint8_t*>(workspace), records, chunks, a.value_heads, a.value_dim);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    return gdn_scan_launch(stream, a, records, 0, chunks, chunks, nullptr, status);
  }
  const size_t smem = kRecStages * kStageBytes + sizeof(RecBarriers);
  e = cudaFuncSetAttribute(gdn_chunk_recurrence, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  gdn_chunk_recurrence<<<dim3(a.value_dim / kSliceCols, a.value_heads, a.batch), 96, smem, stream>>>(
      a, static_cast<const uint8_t*>(workspace), chunks, status);
  return cudaGetLastError();
}

// The tcgen05 prefill (value width 128) with the state at every chunk's start written out as
// well: the forward half of the chunked backward pass.  `records` is 1024-byte aligned and holds
// gdn_chunked_workspace_bytes(...) bytes.
cudaError_t gdn_chunked_with_states(cudaStream_t stream, const GdnArgs& a, void* records, float* state_dump,
                                    uint32_t* status, cudaEvent_t after_prepare) {
  if (!gdn_prepare_sm100_supported(a)) return cudaErrorInvalidValue;
  return gdn_prepare_and_scan(stream, a, static_cast<uint8_t*>(records), (a.tokens + kC - 1) / kC, state_dump, status,
                              after_prepare);
}

}  // namespace pluto
