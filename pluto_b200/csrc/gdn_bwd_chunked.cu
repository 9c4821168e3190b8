// Chunked backward of the gated delta-net recurrence (key width = value width = 128).
//
// Reference kernels this stands in for (src/llm/layers/sequence_delta_net.cc): RecurrenceBackward
// :176-258 with GatherQkGradient :260-281 and GatherScalarGradient :283-309, which walk the
// sequence token by token.  Here the only sequential parts are two scans over 64-token chunks on
// the tensor cores (gdn_scan_sm100.cu): the forward scan leaves the state S_0 at the start of every
// chunk, the reverse scan the gradient dS_C at the end of every chunk.  Given those two, a chunk's
// gradients depend on nothing outside it, and gdn_bwd_chunk_local below computes all chunks in
// parallel, one CTA per (sequence, head, chunk), with fp32-level accuracy: its long products on
// mma.sync with every operand split into a bf16 high part and remainder, the short ones and all
// element-wise work in fp32 on the CUDA cores.
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

#include <mutex>

namespace pluto {
// gdn_chunked.cu / gdn_scan_sm100.cu
cudaError_t gdn_chunked_with_states(cudaStream_t stream, const GdnArgs& a, void* records, float* state_dump,
                                    uint32_t* status, cudaEvent_t after_prepare);
cudaError_t gdn_scan_bwd_launch(cudaStream_t stream, const void* dcore_bf16, const void* records, int batch,
                                int tokens, int value_heads, int chunks, float* dstate_dump, uint32_t* status);
namespace {

constexpr int kLC = 64;            // tokens per chunk
constexpr int kLD = 128;           // key width == value width
constexpr int kLP = 132;           // row pitch of the [64 x 128] matrices (floats)
constexpr int kLQ = 68;            // row pitch of the [64 x 64] matrices
constexpr int kLThreads = 512;

struct LocalSmem {
  float big[5][kLC * kLP];
  float sq[3][kLC * kLQ];
  float part[16][kLC];             // column sums: one partial per row group
  float b[kLC], beta[kLC], cdec[kLC], ik[kLC], iq[kLC];
  float alpha[kLC], softplus[kLC], sigmoid[kLC];
  float dbeta[2][kLC], db[2][kLC];   // row sums, one slot per column half (summed at the end)
  float dots[2][2][kLC];             // per column half: <dq^, q^> and <dk^, k^> of every row
  float red[kLThreads / 32];
};

__device__ __forceinline__ float load_any(const void* p, size_t i, int is_bf16) {
  return is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i])
                 : static_cast<const float*>(p)[i];
}
// four consecutive activations (the offset is a multiple of four elements; bf16 rows are 8-byte aligned)
__device__ __forceinline__ float4 load_any4(const void* p, size_t i, int is_bf16) {
  if (is_bf16) {
    const uint2 w = __ldg(reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(p) + i));
    return make_float4(bf16_lo(w.x), bf16_hi(w.x), bf16_lo(w.y), bf16_hi(w.y));
  }
  return __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(p) + i));
}
__device__ __forceinline__ float4 lds4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ldg4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float comp(const float4& v, int i) { return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w)); }
// sum over the 16 lanes that share a row group (the two halves of a warp)
__device__ __forceinline__ float row_sum16(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// 512 threads = 16 warps.  The epilogues and the short products (64 contraction steps, two-lane
// fp32 FMAs) use a tile per thread: warp w covers the column half ch = w & 1 of the row groups
// 2 (w >> 1) and 2 (w >> 1) + 1 (one per half warp); thread (rg, ch, cg) owns rows rg*4 .. +3 and
//   "dense"   columns ch*64 + cg*4 .. +3 of a [64 x 128] matrix (the 16 lanes of a row group read
//             256 contiguous bytes per 16-byte load, the two row groups of a warp the same ones),
//   "strided" columns cg + 16 j + 32 ch (j < 2) of a [64 x 64] matrix (row pitches of 132 / 68
//             floats keep those lanes in different banks).
// The long products (128 contraction steps) run on mma.sync in warp blocks of their own and hand
// their results to these tiles through shared memory.
struct Lane {
  int rg, ch, cg, r0, c0;   // c0: first dense column
};

__device__ __forceinline__ void to_pairs(const float (&acc)[4][4], uint64_t (&pair)[4][2]) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) pair[i][j] = f2_pack(acc[i][2 * j], acc[i][2 * j + 1]);
}
__device__ __forceinline__ void from_pairs(const uint64_t (&pair)[4][2], float (&acc)[4][4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) f2_unpack(pair[i][j], acc[i][2 * j], acc[i][2 * j + 1]);
}
// pair[i][.] += a . (b.x, b.y), (b.z, b.w)
__device__ __forceinline__ void dense_step(float av, const float4& bv, uint64_t (&pair)[2]) {
  const uint64_t av2 = f2_pack(av, av);
  pair[0] = f2_fma(av2, f2_pack(bv.x, bv.y), pair[0]);
  pair[1] = f2_fma(av2, f2_pack(bv.z, bv.w), pair[1]);
}

// acc[i][j] += sum_k A[k][r0+i] B[k][c0+j]       (A^T B, dense columns)
template <int K>
__device__ __forceinline__ void tn_smem(const float* A, int pa, const float* B, int pb, const Lane& l,
                                        float (&acc)[4][4]) {
  uint64_t pair[4][2];
  to_pairs(acc, pair);
#pragma unroll 8
  for (int k = 0; k < K; ++k) {
    const float4 a = lds4(A + k * pa + l.r0);
    const float4 bv = lds4(B + k * pb + l.c0);
#pragma unroll
    for (int i = 0; i < 4; ++i) dense_step(comp(a, i), bv, pair[i]);
  }
  from_pairs(pair, acc);
}

// Pairs of products that share an operand, in one pass (the shared fragments are loaded once):
// acc1 += A1 B, acc2 += A2 B                                                (two A B, dense columns)
template <int K>
__device__ __forceinline__ void nn_smem2(const float* A1, const float* A2, int pa, const float* B, int pb,
                                         const Lane& l, float (&acc1)[4][4], float (&acc2)[4][4]) {
  uint64_t p1[4][2], p2[4][2];
  to_pairs(acc1, p1);
  to_pairs(acc2, p2);
#pragma unroll 2
  for (int k = 0; k < K; k += 4) {
    float4 a1[4], a2[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      a1[i] = lds4(A1 + (l.r0 + i) * pa + k);
      a2[i] = lds4(A2 + (l.r0 + i) * pa + k);
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const float4 bv = lds4(B + (k + kk) * pb + l.c0);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        dense_step(comp(a1[i], kk), bv, p1[i]);
        dense_step(comp(a2[i], kk), bv, p2[i]);
      }
    }
  }
  from_pairs(p1, acc1);
  from_pairs(p2, acc2);
}
// acc1 += A^T B1, acc2 += A^T B2                                            (two A^T B, dense columns)
template <int K>
__device__ __forceinline__ void tn_smem2(const float* A, int pa, const float* B1, const float* B2, int pb,
                                         const Lane& l, float (&acc1)[4][4], float (&acc2)[4][4]) {
  uint64_t p1[4][2], p2[4][2];
  to_pairs(acc1, p1);
  to_pairs(acc2, p2);
#pragma unroll 4
  for (int k = 0; k < K; ++k) {
    const float4 a = lds4(A + k * pa + l.r0);
    const float4 b1 = lds4(B1 + k * pb + l.c0), b2 = lds4(B2 + k * pb + l.c0);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      dense_step(comp(a, i), b1, p1[i]);
      dense_step(comp(a, i), b2, p2[i]);
    }
  }
  from_pairs(p1, acc1);
  from_pairs(p2, acc2);
}

__device__ __forceinline__ void cp_async16(float* smem_dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void to_array(const float4& v, float (&x)[4]) { x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w; }

// ---- products on the tensor cores -----------------------------------------------------------------
// fp32 operands as bf16 high part + bf16 remainder, three mma.sync products per pair of fragments
// (high x high, high x remainder, remainder x high; the remainder x remainder term is 2^-16 of
// the product), fp32 accumulation.  The results go to a matrix in shared memory, from where the
// threads pick up their usual tiles.
__device__ __forceinline__ void split_pair(float x0, float x1, uint32_t& hi, uint32_t& lo) {
  hi = pack_bf16(x0, x1);
  lo = pack_bf16(x0 - bf16_lo(hi), x1 - bf16_hi(hi));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
constexpr int kMmaRingPitch = 132;                       // floats per staged row: conflict-free fragment loads
constexpr int kMmaStageFloats = 16 * kMmaRingPitch;      // 16 rows = one k step; 4 stages = one [64 x 132] buffer
// A fragment (16 rows x 16 k) of a row-major fp32 matrix, split
__device__ __forceinline__ void load_a_fragment(const float* A, int pa, int m0, int k0, int g, int t,
                                                uint32_t (&hi)[4], uint32_t (&lo)[4]) {
  const float2 x0 = *reinterpret_cast<const float2*>(A + (m0 + g) * pa + k0 + 2 * t);
  const float2 x1 = *reinterpret_cast<const float2*>(A + (m0 + g + 8) * pa + k0 + 2 * t);
  const float2 x2 = *reinterpret_cast<const float2*>(A + (m0 + g) * pa + k0 + 2 * t + 8);
  const float2 x3 = *reinterpret_cast<const float2*>(A + (m0 + g + 8) * pa + k0 + 2 * t + 8);
  split_pair(x0.x, x0.y, hi[0], lo[0]);
  split_pair(x1.x, x1.y, hi[1], lo[1]);
  split_pair(x2.x, x2.y, hi[2], lo[2]);
  split_pair(x3.x, x3.y, hi[3], lo[3]);
}
// out1 = A1 Bg (and out2 = sign2 A2 Bg when kTwo) for a [128 x 128] matrix Bg in global memory, whose
// rows pass through `ring` ([4 stages][16 rows][132] floats, one 16-byte asynchronous copy per thread
// and stage, three stages in flight).  Warp w owns the 16 x 32 block (rows 16 (w / 4), columns
// 32 (w % 4)) of the [64 x 128] results.  out2 may be the matrix A1 lives in: the results are
// written after the last read of the operands.  All 512 threads call this together; on return the
// results are visible to every thread and the ring is free.
template <bool kTwo>
__device__ __forceinline__ void nn_ring_mma(const float* A1, const float* A2, int pa, const float* __restrict__ Bg,
                                            float* ring, int tid, float* out1, float* out2, float sign2) {
  const int warp = tid >> 5, lane = tid & 31;
  const int m0 = (warp >> 2) * 16, n0 = (warp & 3) * 32, g = lane >> 2, t = lane & 3;
  float c1[4][4], c2[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) c1[i][j] = c2[i][j] = 0.0f;
  const int row = tid >> 5, c4 = tid & 31;   // this thread's 16 bytes of a stage
  auto issue = [&](int s) {
    cp_async16(ring + (s % 4) * kMmaStageFloats + row * kMmaRingPitch + c4 * 4, Bg + (s * 16 + row) * kLD + c4 * 4);
  };
#pragma unroll
  for (int s = 0; s < 3; ++s) {
    issue(s);
    cp_async_commit();
  }
#pragma unroll 1
  for (int s = 0; s < kLD / 16; ++s) {
    cp_async_wait<2>();
    __syncthreads();   // stage s has landed for every thread; the slot refilled below was read in step s - 1
    if (s + 3 < kLD / 16) issue(s + 3);
    cp_async_commit();
    const float* Bs = ring + (s % 4) * kMmaStageFloats;
    uint32_t a1h[4], a1l[4], a2h[4], a2l[4];
    load_a_fragment(A1, pa, m0, s * 16, g, t, a1h, a1l);
    if (kTwo) load_a_fragment(A2, pa, m0, s * 16, g, t, a2h, a2l);
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const float* col = Bs + n0 + nt * 8 + g;
      uint32_t bh0, bl0, bh1, bl1;
      split_pair(col[(2 * t) * kMmaRingPitch], col[(2 * t + 1) * kMmaRingPitch], bh0, bl0);
      split_pair(col[(2 * t + 8) * kMmaRingPitch], col[(2 * t + 9) * kMmaRingPitch], bh1, bl1);
      mma16816(c1[nt], a1h, bh0, bh1);
      mma16816(c1[nt], a1h, bl0, bl1);
      mma16816(c1[nt], a1l, bh0, bh1);
      if (kTwo) {
        mma16816(c2[nt], a2h, bh0, bh1);
        mma16816(c2[nt], a2h, bl0, bl1);
        mma16816(c2[nt], a2l, bh0, bh1);
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();   // every operand read is done
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) {
    const int col = n0 + nt * 8 + 2 * t;
    *reinterpret_cast<float2*>(out1 + (m0 + g) * kLP + col) = make_float2(c1[nt][0], c1[nt][1]);
    *reinterpret_cast<float2*>(out1 + (m0 + g + 8) * kLP + col) = make_float2(c1[nt][2], c1[nt][3]);
    if (kTwo) {
      *reinterpret_cast<float2*>(out2 + (m0 + g) * kLP + col) = make_float2(sign2 * c2[nt][0], sign2 * c2[nt][1]);
      *reinterpret_cast<float2*>(out2 + (m0 + g + 8) * kLP + col) = make_float2(sign2 * c2[nt][2], sign2 * c2[nt][3]);
    }
  }
  __syncthreads();   // the results are there for every thread
}
// out1 = A1 B^T (and out2 = A2 B^T when kTwo) for [64 x K] matrices in shared memory, the same way;
// warp w owns the 16 x 16 block (rows 16 (w / 4), columns 16 (w % 4)) of the [64 x 64] results, which
// go to matrices of pitch kLQ.  The caller synchronises before the results are read.
template <int K, bool kTwo>
__device__ __forceinline__ void nt_mma(const float* A1, const float* A2, int pa, const float* B, int pb, int tid,
                                       float* out1, float* out2) {
  const int warp = tid >> 5, lane = tid & 31;
  const int m0 = (warp >> 2) * 16, n0 = (warp & 3) * 16, g = lane >> 2, t = lane & 3;
  float c1[2][4], c2[2][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) c1[i][j] = c2[i][j] = 0.0f;
#pragma unroll 2
  for (int k0 = 0; k0 < K; k0 += 16) {
    uint32_t a1h[4], a1l[4], a2h[4], a2l[4];
    load_a_fragment(A1, pa, m0, k0, g, t, a1h, a1l);
    if (kTwo) load_a_fragment(A2, pa, m0, k0, g, t, a2h, a2l);
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const float* rowp = B + (n0 + nt * 8 + g) * pb + k0 + 2 * t;
      const float2 y0 = *reinterpret_cast<const float2*>(rowp), y1 = *reinterpret_cast<const float2*>(rowp + 8);
      uint32_t bh0, bl0, bh1, bl1;
      split_pair(y0.x, y0.y, bh0, bl0);
      split_pair(y1.x, y1.y, bh1, bl1);
      mma16816(c1[nt], a1h, bh0, bh1);
      mma16816(c1[nt], a1h, bl0, bl1);
      mma16816(c1[nt], a1l, bh0, bh1);
      if (kTwo) {
        mma16816(c2[nt], a2h, bh0, bh1);
        mma16816(c2[nt], a2h, bl0, bl1);
        mma16816(c2[nt], a2l, bh0, bh1);
      }
    }
  }
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
    const int col = n0 + nt * 8 + 2 * t;
    *reinterpret_cast<float2*>(out1 + (m0 + g) * kLQ + col) = make_float2(c1[nt][0], c1[nt][1]);
    *reinterpret_cast<float2*>(out1 + (m0 + g + 8) * kLQ + col) = make_float2(c1[nt][2], c1[nt][3]);
    if (kTwo) {
      *reinterpret_cast<float2*>(out2 + (m0 + g) * kLQ + col) = make_float2(c2[nt][0], c2[nt][1]);
      *reinterpret_cast<float2*>(out2 + (m0 + g + 8) * kLQ + col) = make_float2(c2[nt][2], c2[nt][3]);
    }
  }
}
// out1 (+)= op(A) diag(sc1) B1  (and out2 = op(A) diag(sc2) B2 when kTwoB) for A [64 x K] (or, kTransA,
// stored [K x 64]) and B [K x 128] in shared memory; sc: optional factor per k.  Warp blocks and result
// matrices as nn_ring_mma; kAccumulate adds to what out1 holds.  No barrier inside.
template <int K, bool kTransA, bool kTwoB, bool kAccumulate>
__device__ __forceinline__ void nn_mma(const float* A, int pa, const float* B1, const float* sc1, const float* B2,
                                       const float* sc2, int pb, int tid, float* out1, float* out2) {
  const int warp = tid >> 5, lane = tid & 31;
  const int m0 = (warp >> 2) * 16, n0 = (warp & 3) * 32, g = lane >> 2, t = lane & 3;
  float c1[4][4], c2[4][4];
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) {
    const int col = n0 + nt * 8 + 2 * t;
    float2 lo = make_float2(0.0f, 0.0f), hi = make_float2(0.0f, 0.0f);
    if (kAccumulate) {
      lo = *reinterpret_cast<const float2*>(out1 + (m0 + g) * kLP + col);
      hi = *reinterpret_cast<const float2*>(out1 + (m0 + g + 8) * kLP + col);
    }
    c1[nt][0] = lo.x; c1[nt][1] = lo.y; c1[nt][2] = hi.x; c1[nt][3] = hi.y;
    c2[nt][0] = c2[nt][1] = c2[nt][2] = c2[nt][3] = 0.0f;
  }
#pragma unroll 2
  for (int k0 = 0; k0 < K; k0 += 16) {
    uint32_t ah[4], al[4];
    if (kTransA) {
      const float* colp = A + m0 + g;
      split_pair(colp[(k0 + 2 * t) * pa], colp[(k0 + 2 * t + 1) * pa], ah[0], al[0]);
      split_pair(colp[(k0 + 2 * t) * pa + 8], colp[(k0 + 2 * t + 1) * pa + 8], ah[1], al[1]);
      split_pair(colp[(k0 + 2 * t + 8) * pa], colp[(k0 + 2 * t + 9) * pa], ah[2], al[2]);
      split_pair(colp[(k0 + 2 * t + 8) * pa + 8], colp[(k0 + 2 * t + 9) * pa + 8], ah[3], al[3]);
    } else {
      load_a_fragment(A, pa, m0, k0, g, t, ah, al);
    }
    float s1[4] = {1.0f, 1.0f, 1.0f, 1.0f}, s2[4] = {1.0f, 1.0f, 1.0f, 1.0f};   // factors of rows 2t, 2t+1, 2t+8, 2t+9
    if (sc1 != nullptr) { s1[0] = sc1[k0 + 2 * t]; s1[1] = sc1[k0 + 2 * t + 1]; s1[2] = sc1[k0 + 2 * t + 8]; s1[3] = sc1[k0 + 2 * t + 9]; }
    if (kTwoB && sc2 != nullptr) { s2[0] = sc2[k0 + 2 * t]; s2[1] = sc2[k0 + 2 * t + 1]; s2[2] = sc2[k0 + 2 * t + 8]; s2[3] = sc2[k0 + 2 * t + 9]; }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const float* col = B1 + k0 * pb + n0 + nt * 8 + g;
      uint32_t bh0, bl0, bh1, bl1;
      split_pair(col[(2 * t) * pb] * s1[0], col[(2 * t + 1) * pb] * s1[1], bh0, bl0);
      split_pair(col[(2 * t + 8) * pb] * s1[2], col[(2 * t + 9) * pb] * s1[3], bh1, bl1);
      mma16816(c1[nt], ah, bh0, bh1);
      mma16816(c1[nt], ah, bl0, bl1);
      mma16816(c1[nt], al, bh0, bh1);
      if (kTwoB) {
        const float* col2 = B2 + k0 * pb + n0 + nt * 8 + g;
        split_pair(col2[(2 * t) * pb] * s2[0], col2[(2 * t + 1) * pb] * s2[1], bh0, bl0);
        split_pair(col2[(2 * t + 8) * pb] * s2[2], col2[(2 * t + 9) * pb] * s2[3], bh1, bl1);
        mma16816(c2[nt], ah, bh0, bh1);
        mma16816(c2[nt], ah, bl0, bl1);
        mma16816(c2[nt], al, bh0, bh1);
      }
    }
  }
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) {
    const int col = n0 + nt * 8 + 2 * t;
    *reinterpret_cast<float2*>(out1 + (m0 + g) * kLP + col) = make_float2(c1[nt][0], c1[nt][1]);
    *reinterpret_cast<float2*>(out1 + (m0 + g + 8) * kLP + col) = make_float2(c1[nt][2], c1[nt][3]);
    if (kTwoB) {
      *reinterpret_cast<float2*>(out2 + (m0 + g) * kLP + col) = make_float2(c2[nt][0], c2[nt][1]);
      *reinterpret_cast<float2*>(out2 + (m0 + g + 8) * kLP + col) = make_float2(c2[nt][2], c2[nt][3]);
    }
  }
}
// out (+)= A (diag(f) B)^T with f[n] = fa[n] (* fb[n] when given): row n of B scaled; otherwise as nt_mma.
template <int K, bool kAccumulate>
__device__ __forceinline__ void nt_mma_scaled(const float* A, int pa, const float* B, int pb, const float* fa,
                                              const float* fb, int tid, float* out) {
  const int warp = tid >> 5, lane = tid & 31;
  const int m0 = (warp >> 2) * 16, n0 = (warp & 3) * 16, g = lane >> 2, t = lane & 3;
  float c[2][4], f[2];
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
    const int n = n0 + nt * 8 + g, col = n0 + nt * 8 + 2 * t;
    f[nt] = fa[n] * (fb != nullptr ? fb[n] : 1.0f);
    float2 lo = make_float2(0.0f, 0.0f), hi = make_float2(0.0f, 0.0f);
    if (kAccumulate) {
      lo = *reinterpret_cast<const float2*>(out + (m0 + g) * kLQ + col);
      hi = *reinterpret_cast<const float2*>(out + (m0 + g + 8) * kLQ + col);
    }
    c[nt][0] = lo.x; c[nt][1] = lo.y; c[nt][2] = hi.x; c[nt][3] = hi.y;
  }
#pragma unroll 2
  for (int k0 = 0; k0 < K; k0 += 16) {
    uint32_t ah[4], al[4];
    load_a_fragment(A, pa, m0, k0, g, t, ah, al);
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const float* rowp = B + (n0 + nt * 8 + g) * pb + k0 + 2 * t;
      const float2 y0 = *reinterpret_cast<const float2*>(rowp), y1 = *reinterpret_cast<const float2*>(rowp + 8);
      uint32_t bh0, bl0, bh1, bl1;
      split_pair(y0.x * f[nt], y0.y * f[nt], bh0, bl0);
      split_pair(y1.x * f[nt], y1.y * f[nt], bh1, bl1);
      mma16816(c[nt], ah, bh0, bh1);
      mma16816(c[nt], ah, bl0, bl1);
      mma16816(c[nt], al, bh0, bh1);
    }
  }
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
    const int col = n0 + nt * 8 + 2 * t;
    *reinterpret_cast<float2*>(out + (m0 + g) * kLQ + col) = make_float2(c[nt][0], c[nt][1]);
    *reinterpret_cast<float2*>(out + (m0 + g + 8) * kLQ + col) = make_float2(c[nt][2], c[nt][3]);
  }
}
// this thread's 4 x 2 tile (strided columns) of a [64 x 64] matrix of pitch kLQ
__device__ __forceinline__ void load_strided(const float* src, const Lane& l, float (&acc)[4][2]) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) acc[i][j] = src[(l.r0 + i) * kLQ + l.cg + 16 * j + 32 * l.ch];
}
// this thread's 4 x 4 tile of a [64 x 128] matrix
__device__ __forceinline__ void load_dense(const float* src, const Lane& l, float (&acc)[4][4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) to_array(lds4(src + (l.r0 + i) * kLP + l.c0), acc[i]);
}

template <int N>
__device__ __forceinline__ void zero(float (&acc)[4][N]) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < N; ++j) acc[i][j] = 0.0f;
}
// dense tile -> [64 x 128] matrix in shared memory
__device__ __forceinline__ void store_dense(float* dst, const Lane& l, const float (&acc)[4][4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
    *reinterpret_cast<float4*>(dst + (l.r0 + i) * kLP + l.c0) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
}

struct LocalArgs {
  GdnBwdArgs a;
  const float* states;      // [sequence, head, chunk, key, value column]: state at each chunk's start
  const float* states_t;    // the same matrices transposed, [.., value column, key]
  const float* dstates;     // [sequence, head, chunk, key, value column]: state gradient at each chunk's end
  const float* dstates_t;
  int chunks;
  // Where the q / k gradients of a token's head go: rows of 2 x 128 floats (q then k) in the
  // partials when several value heads share a key head (the gather kernel sums them), or the
  // final dq / dk rows themselves when every value head has its own key head.
  float* dq_rows;
  float* dk_rows;
  size_t row_stride, head_stride;
};

__global__ void __launch_bounds__(kLThreads, 1) gdn_bwd_chunk_local(LocalArgs la) {
  extern __shared__ uint8_t local_raw[];
  LocalSmem& sm = *reinterpret_cast<LocalSmem*>(local_raw);
  const GdnBwdArgs& a = la.a;
  const int chunk = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int kh = h / (a.value_heads / a.key_heads);
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  Lane l;
  l.ch = warp & 1;
  l.rg = (warp >> 1) * 2 + (lane >> 4);
  l.cg = lane & 15;
  l.r0 = l.rg * 4;
  l.c0 = l.ch * 64 + l.cg * 4;
  const int r0 = l.r0, c0 = l.c0;
  const int t0 = chunk * kLC, count = min(kLC, a.tokens - t0);
  const size_t unit = static_cast<size_t>(b) * a.value_heads + h;
  const size_t matrix = (unit * la.chunks + chunk) * kLD * kLD;
  const float* S0 = la.states + matrix;        // [key][value column]
  const float* S0t = la.states_t + matrix;     // [value column][key]
  const float* dS = la.dstates + matrix;
  const float* dSt = la.dstates_t + matrix;
  float* Kh = sm.big[0];
  const float q_scale = rsqrtf(static_cast<float>(kLD));
  const size_t token0 = static_cast<size_t>(b) * a.tokens + t0;   // first token of the chunk

  // The four state matrices are first needed tens of microseconds from now and would come from
  // DRAM then: ask for them in L2 now.
  if (tid < 4) {
    const float* m = tid == 0 ? S0 : (tid == 1 ? dS : (tid == 2 ? S0t : dSt));
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(m), "r"(kLD * kLD * 4) : "memory");
  }
  // ---- gates
  if (tid < kLC) {
    float lg = 0.0f, be = 0.0f, alpha = 0.0f, softplus = 0.0f, sigmoid = 0.0f;
    if (tid < count) {
      const size_t off = (token0 + tid) * a.value_heads + h;
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
    sm.dbeta[0][tid] = sm.dbeta[1][tid] = 0.0f;
    sm.db[0][tid] = sm.db[1][tid] = 0.0f;
  }
  // ---- keys and queries: k -> big[0], q -> big[1] (normalised below)
  for (int idx = tid; idx < 2 * kLC * (kLD / 4); idx += kLThreads) {
    const int which = idx / (kLC * (kLD / 4)), rest = idx % (kLC * (kLD / 4));
    const int t = rest / (kLD / 4), c4 = rest % (kLD / 4);
    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (t < count)
      v = load_any4(which ? a.q : a.k, (token0 + t) * a.qk_token + static_cast<size_t>(kh) * kLD + c4 * 4, a.in_is_bf16);
    *reinterpret_cast<float4*>(sm.big[which] + t * kLP + c4 * 4) = v;
  }
  __syncthreads();
  if (tid == 0) {
    float run = 0.0f;
    for (int t = 0; t < kLC; ++t) { run += sm.b[t]; sm.b[t] = run; }
  }
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
  if (tid < kLC) sm.cdec[tid] = expf(sm.b[tid]);

  // ---- A (transposed, for the substitution) -> sq[0];  M -> sq[1]
  {
    float g[4][2], hh[4][2];
    nt_mma<kLD, true>(Kh, sm.big[1], kLP, Kh, kLP, tid, sm.big[3], sm.big[4]);   // (big[3], big[4] are still free)
    __syncthreads();
    load_strided(sm.big[3], l, g);
    load_strided(sm.big[4], l, hh);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int t = r0 + i, s = l.cg + 16 * j + 32 * l.ch;
        const float ratio = s <= t ? expf(sm.b[t] - sm.b[s]) : 0.0f;
        sm.sq[0][s * kLQ + t] = s < t ? sm.beta[t] * ratio * g[i][j] : 0.0f;
        sm.sq[1][t * kLQ + s] = ratio * hh[i][j];
      }
  }
  __syncthreads();

  // ---- T = (I + A)^-1 -> sq[2], one thread per column, right-looking forward substitution;
  //      meanwhile the other warps stage v -> big[2]
  if (tid < kLC) {
    uint64_t x[kLC / 2];
#pragma unroll
    for (int t = 0; t < kLC / 2; ++t) x[t] = f2_pack(2 * t == tid ? 1.0f : 0.0f, 2 * t + 1 == tid ? 1.0f : 0.0f);
#pragma unroll
    for (int s = 0; s < kLC - 1; ++s) {
      float lo, hi;
      f2_unpack(x[s >> 1], lo, hi);
      const float xs = s & 1 ? hi : lo;
      const uint64_t minus = f2_pack(-xs, -xs);
#pragma unroll
      for (int t4 = (s + 1) / 4; t4 < kLC / 4; ++t4) {
        const float4 av = lds4(sm.sq[0] + s * kLQ + t4 * 4);   // A[t][s], zero for t <= s
        x[2 * t4] = f2_fma(f2_pack(av.x, av.y), minus, x[2 * t4]);
        x[2 * t4 + 1] = f2_fma(f2_pack(av.z, av.w), minus, x[2 * t4 + 1]);
      }
    }
#pragma unroll
    for (int t = 0; t < kLC / 2; ++t) {
      float lo, hi;
      f2_unpack(x[t], lo, hi);
      sm.sq[2][(2 * t) * kLQ + tid] = lo;
      sm.sq[2][(2 * t + 1) * kLQ + tid] = hi;
    }
  } else {
    for (int idx = tid - kLC; idx < kLC * (kLD / 4); idx += kLThreads - kLC) {
      const int t = idx / (kLD / 4), c4 = idx % (kLD / 4);
      float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (t < count)
        v = load_any4(a.v, (token0 + t) * a.v_token + static_cast<size_t>(h) * kLD + c4 * 4, a.in_is_bf16);
      *reinterpret_cast<float4*>(sm.big[2] + t * kLP + c4 * 4) = v;
    }
  }
  if (tid < kLC) sm.part[0][tid] = sm.beta[tid] * sm.cdec[tid];
  __syncthreads();
  const float* Tm = sm.sq[2];
  const float* Mm = sm.sq[1];

  // ---- W = T (beta c . k^) -> big[1] (the queries are read again later);  U' = T (beta . v) -> big[3]
  nn_mma<kLC, false, true, false>(Tm, kLQ, Kh, sm.part[0], sm.big[2], sm.beta, kLP, tid, sm.big[1], sm.big[3]);
  __syncthreads();
  // ---- U = U' - W S_0 -> big[4]
  {
    float acc[4][4];
    nn_ring_mma<false>(sm.big[1], nullptr, kLP, S0, sm.big[2], tid, sm.big[4], nullptr, 0.0f);   // (v in big[2] is dead: U' is complete)
    load_dense(sm.big[4], l, acc);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 up = lds4(sm.big[3] + (r0 + i) * kLP + c0);
      *reinterpret_cast<float4*>(sm.big[4] + (r0 + i) * kLP + c0) =
          make_float4(up.x - acc[i][0], up.y - acc[i][1], up.z - acc[i][2], up.w - acc[i][3]);
    }
  }
  // ---- dO -> big[2] (the ring is free: nn_ring ends with a barrier)
  for (int idx = tid; idx < kLC * (kLD / 4); idx += kLThreads) {
    const int t = idx / (kLD / 4), c4 = idx % (kLD / 4);
    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (t < count) v = ldg4(a.dcore + ((token0 + t) * a.value_heads + h) * kLD + c4 * 4);
    *reinterpret_cast<float4*>(sm.big[2] + t * kLP + c4 * 4) = v;
  }
  __syncthreads();

  // row sums into sm.db / sm.dbeta: added by the lane with cg == 0 of the row's group, into the
  // slot of its column half; column sums go through sm.part
  auto add_rows = [&](float (*dst)[kLC], const float (&v)[4], float sign) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float total = row_sum16(v[i]);
      if (l.cg == 0) dst[l.ch][r0 + i] += sign * total;
    }
  };

  // ---- dM = mask(dO U^T): M-bar = dM . M into db, dH = dM . ratio -> sq[0]
  {
    float acc[4][2];
    nt_mma<kLD, false>(sm.big[2], nullptr, kLP, sm.big[4], kLP, tid, sm.big[1], nullptr);   // (W in big[1] is dead)
    __syncthreads();
    load_strided(sm.big[1], l, acc);
    float rows[4] = {0.0f, 0.0f, 0.0f, 0.0f}, cols[2] = {0.0f, 0.0f};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int t = r0 + i, s = l.cg + 16 * j + 32 * l.ch;
        const float dm = s <= t ? acc[i][j] : 0.0f;
        const float bar = dm * Mm[t * kLQ + s];
        rows[i] += bar;
        cols[j] += bar;
        sm.sq[0][t * kLQ + s] = s <= t ? dm * expf(sm.b[t] - sm.b[s]) : 0.0f;
      }
    add_rows(sm.db, rows, 1.0f);
#pragma unroll
    for (int j = 0; j < 2; ++j) sm.part[l.rg][l.cg + 16 * j + 32 * l.ch] = cols[j];
  }
  __syncthreads();
  if (tid < kLC) {
    float total = 0.0f;
#pragma unroll
    for (int g = 0; g < 16; ++g) total += sm.part[g][tid];
    sm.part[0][tid] = total;   // (own column of row 0 only: no other thread reads it)
  }
  __syncthreads();
  if (tid < kLC) sm.db[0][tid] -= sm.part[0][tid];   // cg == 0 lanes add to db only after later barriers

  // The two contributions that are known early -- (gamma/c) . dKt to dk^ and c . dQc to dq^ -- wait
  // in this chunk's rows of the output partials (each thread its own elements) until the last
  // products, so that no accumulator tile stays live across the phases in between.
  float kt_total = 0.0f;   // sum of dKt . Kt over the chunk (thread partial)
  const float gamma = sm.cdec[kLC - 1];

  // ---- dKt = U dS^T (dense columns = keys)
  {
    float acc[4][4];
    nn_ring_mma<false>(sm.big[4], nullptr, kLP, dSt, sm.big[3], tid, sm.big[1], nullptr, 0.0f);   // (W and U' are dead from here on: big[1], big[3])
    load_dense(sm.big[1], l, acc);
    float rows[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float f = gamma / sm.cdec[r0 + i];
      float kv[4];
      to_array(lds4(Kh + (r0 + i) * kLP + c0), kv);
      float rs = 0.0f, scaled[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        scaled[j] = acc[i][j] * f;
        rs = fmaf(scaled[j], kv[j], rs);
      }
      if (r0 + i < count)
        *reinterpret_cast<float4*>(la.dk_rows + (token0 + r0 + i) * la.row_stride + h * la.head_stride + c0) =
            make_float4(scaled[0], scaled[1], scaled[2], scaled[3]);
      rows[i] = rs;
      kt_total += rs;
    }
    add_rows(sm.db, rows, -1.0f);
  }
  // ---- dU = M^T dO + Kt dS -> big[4]   (every read of U is done: nn_ring ends with a barrier)
  {
    float acc[4][4], from_state[4][4];
    nn_mma<kLC, true, false, false>(Mm, kLQ, sm.big[2], nullptr, nullptr, nullptr, kLP, tid, sm.big[4], nullptr);   // M^T dO (U is dead)
    nn_ring_mma<false>(Kh, nullptr, kLP, dS, sm.big[3], tid, sm.big[1], nullptr, 0.0f);   // (starts with a barrier: the dKt tiles are out of big[1])
    load_dense(sm.big[4], l, acc);
    load_dense(sm.big[1], l, from_state);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float f = gamma / sm.cdec[r0 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(f, from_state[i][j], acc[i][j]);
    }
    store_dense(sm.big[4], l, acc);
  }
  // ---- dQc = dO S_0^T: dq^ += c . dQc, db += rows(dQc . c q^);  dW = -dU S_0^T -> big[2] in the same pass
  //      over S_0^T (dU is complete: the pass starts with a barrier; dO is read for the last time)
  {
    float4 qraw[4];   // requested before the product, used after it
#pragma unroll
    for (int i = 0; i < 4; ++i)
      qraw[i] = r0 + i < count ? load_any4(a.q, (token0 + r0 + i) * a.qk_token + static_cast<size_t>(kh) * kLD + c0, a.in_is_bf16)
                               : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float acc[4][4];
    __syncthreads();   // every thread has its tile of the dU product's state term out of big[1]; dU is stored
    nn_ring_mma<true>(sm.big[2], sm.big[4], kLP, S0t, sm.big[3], tid, sm.big[1], sm.big[2], -1.0f);
    load_dense(sm.big[1], l, acc);
    float rows[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = r0 + i;
      const float c = sm.cdec[t], f = sm.iq[t] * q_scale;
      float qv[4], scaled[4], rs = 0.0f;
      to_array(qraw[i], qv);
      // (this thread's piece of q^, kept for the last products: big[1] is free since U)
      *reinterpret_cast<float4*>(sm.big[1] + t * kLP + c0) = make_float4(qv[0] * f, qv[1] * f, qv[2] * f, qv[3] * f);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        scaled[j] = acc[i][j] * c;
        rs = fmaf(scaled[j], qv[j] * f, rs);
      }
      if (t < count)
        *reinterpret_cast<float4*>(la.dq_rows + (token0 + t) * la.row_stride + h * la.head_stride + c0) =
            make_float4(scaled[0], scaled[1], scaled[2], scaled[3]);
      rows[i] = rs;
    }
    add_rows(sm.db, rows, 1.0f);
  }
  // ---- X1 = T^T dU: dv = beta . X1, dbeta += rows(X1 . v); X1 replaces dU
  //      X2 = T^T dW: dk^ += beta c . X2 (at the end), dbeta += rows(X2 . c k^), db += rows(X2 . beta c k^);
  //      X2 replaces dW.  One pass over T for both.
  {
    float4 vraw[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      vraw[i] = r0 + i < count ? load_any4(a.v, (token0 + r0 + i) * a.v_token + static_cast<size_t>(h) * kLD + c0, a.in_is_bf16)
                               : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float acc[4][4], acc2[4][4];
    zero(acc);
    zero(acc2);
    __syncthreads();   // dW (stored after the pass over S_0^T) is complete
    tn_smem2<kLC>(Tm, kLQ, sm.big[4], sm.big[2], kLP, l, acc, acc2);
    float rows[4], rows_beta[4], rows_b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = r0 + i;
      float vv[4], kv[4], rs = 0.0f, rs2 = 0.0f;
      to_array(vraw[i], vv);
      to_array(lds4(Kh + t * kLP + c0), kv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        rs = fmaf(acc[i][j], vv[j], rs);
        rs2 = fmaf(acc2[i][j], kv[j], rs2);
      }
      if (t < count) {
        const float be = sm.beta[t];
        *reinterpret_cast<float4*>(a.dv_out + (token0 + t) * a.dv_token + static_cast<size_t>(h) * kLD + c0) =
            make_float4(be * acc[i][0], be * acc[i][1], be * acc[i][2], be * acc[i][3]);
      }
      rows[i] = rs;
      rows_beta[i] = rs2 * sm.cdec[t];
      rows_b[i] = rows_beta[i] * sm.beta[t];
    }
    add_rows(sm.dbeta, rows, 1.0f);
    add_rows(sm.dbeta, rows_beta, 1.0f);
    add_rows(sm.db, rows_b, 1.0f);
    // (this thread's piece of v, for R below: big[3] is free since the last ring product)
#pragma unroll
    for (int i = 0; i < 4; ++i) *reinterpret_cast<float4*>(sm.big[3] + (r0 + i) * kLP + c0) = vraw[i];
    __syncthreads();   // every read of dU and dW is done
    store_dense(sm.big[4], l, acc);
    store_dense(sm.big[2], l, acc2);
  }
  __syncthreads();
  // ---- dA = -mask(X1 U'^T + X2 W^T) = -mask(R T^T),  R = X1 (beta . v)^T + X2 (beta c . k^)^T: U' and W
  //      need not be kept (v came into big[3] with X1, the barrier after X2 covers it); R -> sq[1] (M is dead)
  nt_mma_scaled<kLD, false>(sm.big[4], kLP, sm.big[3], kLP, sm.beta, nullptr, tid, sm.sq[1]);
  nt_mma_scaled<kLD, true>(sm.big[2], kLP, Kh, kLP, sm.beta, sm.cdec, tid, sm.sq[1]);   // (same lanes, same elements)
  __syncthreads();
  {
    float acc[4][2], g[4][2];
    nt_mma<kLC, false>(sm.sq[1], nullptr, kLQ, Tm, kLQ, tid, sm.big[3], nullptr);   // R T^T (v and X1 are dead)
    nt_mma<kLD, false>(Kh, nullptr, kLP, Kh, kLP, tid, sm.big[4], nullptr);        // G once more
    __syncthreads();   // every read of R is done: dG + dG^T goes over it
    load_strided(sm.big[3], l, acc);
    load_strided(sm.big[4], l, g);
    float rows_beta[4] = {0.0f, 0.0f, 0.0f, 0.0f}, rows_b[4] = {0.0f, 0.0f, 0.0f, 0.0f}, cols[2] = {0.0f, 0.0f};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int t = r0 + i, s = l.cg + 16 * j + 32 * l.ch;
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
    for (int j = 0; j < 2; ++j) sm.part[l.rg][l.cg + 16 * j + 32 * l.ch] = cols[j];
  }
  __syncthreads();
  if (tid < kLC) {
    float total = 0.0f;
#pragma unroll
    for (int g = 0; g < 16; ++g) total += sm.part[g][tid];
    sm.part[0][tid] = total;
  }
  // ---- dk^ = stashed + beta c . X2 + (dG + dG^T) k^ + dH^T q^;  dq^ = stashed + dH k^   (q^ in big[1] since dQc)
  float dk_acc[4][4], dq_acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = r0 + i;
    const size_t row = (token0 + min(t, count - 1)) * la.row_stride + h * la.head_stride + c0;
    const float bc = sm.beta[t] * sm.cdec[t];
    float x2[4], sq_[4] = {0.0f, 0.0f, 0.0f, 0.0f}, sk_[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    to_array(lds4(sm.big[2] + t * kLP + c0), x2);
    if (t < count) {
      to_array(*reinterpret_cast<const float4*>(la.dq_rows + row), sq_);
      to_array(*reinterpret_cast<const float4*>(la.dk_rows + row), sk_);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      dq_acc[i][j] = sq_[j];
      dk_acc[i][j] = sk_[j] + bc * x2[j];
    }
  }
  nn_smem2<kLC>(sm.sq[1], sm.sq[0], kLQ, Kh, kLP, l, dk_acc, dq_acc);
  tn_smem<kLC>(sm.sq[0], kLQ, sm.big[1], kLP, l, dk_acc);

  // ---- through the normalisations: per-token partials in the layout of the gather kernels (one
  //      tile).  The row dot products span both column halves: exchanged through sm.dots.
  float kv[4][4], qv[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = r0 + i;
    to_array(lds4(Kh + t * kLP + c0), kv[i]);
    to_array(lds4(sm.big[1] + t * kLP + c0), qv[i]);
    float pk = 0.0f, pq = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      pk = fmaf(dk_acc[i][j], kv[i][j], pk);
      pq = fmaf(dq_acc[i][j], qv[i][j], pq);
    }
    pk = row_sum16(pk);
    pq = row_sum16(pq);
    if (l.cg == 0) {
      sm.dots[l.ch][0][t] = pq;
      sm.dots[l.ch][1][t] = pk;
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
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = r0 + i;
    if (t < count) {
      const float pq = (sm.dots[0][0][t] + sm.dots[1][0][t]) / (q_scale * q_scale);   // q^ = scale . unit vector
      const float pk = sm.dots[0][1][t] + sm.dots[1][1][t];
      const float ikt = sm.ik[t], iqt = sm.iq[t] * q_scale;
      const size_t row = (token0 + t) * la.row_stride + h * la.head_stride + c0;
      *reinterpret_cast<float4*>(la.dq_rows + row) =
          make_float4(iqt * (dq_acc[i][0] - qv[i][0] * pq), iqt * (dq_acc[i][1] - qv[i][1] * pq),
                      iqt * (dq_acc[i][2] - qv[i][2] * pq), iqt * (dq_acc[i][3] - qv[i][3] * pq));
      *reinterpret_cast<float4*>(la.dk_rows + row) =
          make_float4(ikt * (dk_acc[i][0] - kv[i][0] * pk), ikt * (dk_acc[i][1] - kv[i][1] * pk),
                      ikt * (dk_acc[i][2] - kv[i][2] * pk), ikt * (dk_acc[i][3] - kv[i][3] * pk));
    }
  }
  if (tid == 0) {
    float total = 0.0f;
    for (int w = 0; w < kLThreads / 32; ++w) total += sm.red[w];
    // d log g_s = sum of db_t over t >= s (db: both column halves, minus the column sums of A-bar)
    float run = 0.0f;
    for (int t = kLC - 1; t >= 0; --t) {
      run += sm.db[0][t] + sm.db[1][t] - sm.part[0][t] + (t == kLC - 1 ? total : 0.0f);
      sm.db[0][t] = run;
    }
  }
  __syncthreads();
  if (tid < count) {
    const size_t partial = (token0 + tid) * a.value_heads + h;
    const float rate = expf(a.a_log[h]);
    const float dlog = sm.db[0][tid];
    a.scalar_partials[partial * 3 + 0] = -dlog * rate / (1.0f + expf(-sm.alpha[tid]));
    a.scalar_partials[partial * 3 + 1] = (sm.dbeta[0][tid] + sm.dbeta[1][tid]) * sm.sigmoid[tid] * (1.0f - sm.sigmoid[tid]);
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

// out[m] = in[m]^T for a batch of [128 x 128] fp32 matrices; one CTA of 256 threads per matrix
__global__ void __launch_bounds__(256) transpose_128_kernel(const float* __restrict__ in, float* __restrict__ out) {
  __shared__ float tile[32][129];
  const size_t base = static_cast<size_t>(blockIdx.x) * kLD * kLD;
  for (int strip = 0; strip < 4; ++strip) {   // rows strip*32 .. +31 of the input
    for (int e = threadIdx.x; e < 32 * kLD; e += 256) {
      const int r = e / kLD, c = e % kLD;
      tile[r][c] = in[base + static_cast<size_t>(strip * 32 + r) * kLD + c];
    }
    __syncthreads();
    for (int e = threadIdx.x; e < 32 * kLD; e += 256) {
      const int c = e / 32, r = e % 32;
      out[base + static_cast<size_t>(c) * kLD + strip * 32 + r] = tile[r][c];
    }
    __syncthreads();
  }
}

// A second stream per device: the reverse scan needs the forward's records but not its states, so
// it runs beside the forward scan (both fill only sequences x heads SMs), with the bf16 copy of the
// output gradient made there too; the caller's stream joins before the transposes.
struct BwdLanes {
  cudaStream_t aux = nullptr;
  cudaEvent_t forked = nullptr, prepared = nullptr, aux_done = nullptr;
  bool ok = false;
  std::mutex enqueue;
};
BwdLanes g_bwd_lanes[64];
std::once_flag g_bwd_once[64];
BwdLanes* bwd_lanes_for_current_device() {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return nullptr;
  std::call_once(g_bwd_once[device], [device] {
    BwdLanes& l = g_bwd_lanes[device];
    l.ok = cudaStreamCreateWithFlags(&l.aux, cudaStreamNonBlocking) == cudaSuccess &&
           cudaEventCreateWithFlags(&l.forked, cudaEventDisableTiming) == cudaSuccess &&
           cudaEventCreateWithFlags(&l.prepared, cudaEventDisableTiming) == cudaSuccess &&
           cudaEventCreateWithFlags(&l.aux_done, cudaEventDisableTiming) == cudaSuccess;
  });
  return g_bwd_lanes[device].ok ? &g_bwd_lanes[device] : nullptr;
}

size_t align_up(size_t n) { return (n + 1023) / 1024 * 1024; }

}  // namespace

bool gdn_bwd_chunked_supported(const GdnBwdArgs& a) {
  return a.key_dim == kLD && a.value_dim == kLD && a.in_is_bf16 && a.tokens >= 4 * kLC &&
         (reinterpret_cast<uintptr_t>(a.q) & 15u) == 0 && (reinterpret_cast<uintptr_t>(a.k) & 15u) == 0 &&
         (reinterpret_cast<uintptr_t>(a.v) & 15u) == 0 && a.qk_token % 8 == 0 && a.v_token % 8 == 0;
}

// Layout of the workspace: records | g, beta | dcore as bf16 | forward output (bf16, unused) |
// states, their transposes | state gradients, their transposes | q/k partials | scalar partials
struct ChunkedBwdLayout {
  size_t records, gates, dcore16, out16, states, states_t, dstates, dstates_t, qk_partials, scalar_partials, total;
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
  l.states_t = at; at += align_up(units * chunks * kLD * kLD * sizeof(float));
  l.dstates = at; at += align_up(units * chunks * kLD * kLD * sizeof(float));
  l.dstates_t = at; at += align_up(units * chunks * kLD * kLD * sizeof(float));
  l.qk_partials = at; at += align_up(rows * 2 * kLD * sizeof(float));
  l.scalar_partials = at; at += align_up(rows * 3 * sizeof(float));
  l.total = at + 1024;   // room to align the base
  return l;
}
size_t gdn_bwd_chunked_workspace_bytes(int batch, int tokens, int value_heads) {
  return chunked_bwd_layout(batch, tokens, value_heads).total;
}

// Fills a.scalar_partials (one tile per head) and a.dv_out, and either a.qk_partials (several value
// heads per key head: *qk_direct = false, the caller runs the q/k gather over them) or dq_out /
// dk_out themselves.
cudaError_t gdn_bwd_chunked(cudaStream_t stream, GdnBwdArgs& a, float* dq_out, float* dk_out, size_t dqk_token,
                            void* workspace, uint32_t* status, bool* qk_direct) {
  const ChunkedBwdLayout l = chunked_bwd_layout(a.batch, a.tokens, a.value_heads);
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(workspace) + 1023) & ~static_cast<uintptr_t>(1023));
  const int chunks = (a.tokens + kLC - 1) / kLC;
  const size_t rows = static_cast<size_t>(a.batch) * a.tokens * a.value_heads;
  float* g = reinterpret_cast<float*>(base + l.gates);
  float* beta = g + rows;
  __nv_bfloat16* dcore16 = reinterpret_cast<__nv_bfloat16*>(base + l.dcore16);
  float* states = reinterpret_cast<float*>(base + l.states);
  float* dstates = reinterpret_cast<float*>(base + l.dstates);
  float* states_t = reinterpret_cast<float*>(base + l.states_t);
  float* dstates_t = reinterpret_cast<float*>(base + l.dstates_t);
  a.qk_partials = reinterpret_cast<float*>(base + l.qk_partials);
  a.scalar_partials = reinterpret_cast<float*>(base + l.scalar_partials);

  BwdLanes* lanes = bwd_lanes_for_current_device();
  if (lanes == nullptr) return cudaErrorInitializationError;
  std::lock_guard<std::mutex> lock(lanes->enqueue);
  cudaError_t e = gdn_gates(stream, a.a_in, a.b_in, a.a_log, a.dt_bias, a.ab_is_bf16,
                            static_cast<long long>(a.batch) * a.tokens, a.value_heads, a.round, g, beta);
  if (e != cudaSuccess) return e;
  // second stream: the output gradient as bf16 now, the reverse scan once the records are there
  e = cudaEventRecord(lanes->forked, stream);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(lanes->aux, lanes->forked, 0);
  if (e != cudaSuccess) return e;
  const size_t count = rows * kLD;
  cast_to_bf16_kernel<<<static_cast<unsigned>((count / 4 + 255) / 256 + 1), 256, 0, lanes->aux>>>(a.dcore, dcore16, count);
  e = cudaGetLastError();
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
  // the scan reads its initial state from and leaves its final state in f.state: the transposed
  // state-gradient area is free until the transposes run
  f.state = dstates_t;
  if (e == cudaSuccess)
    e = cudaMemsetAsync(dstates_t, 0, static_cast<size_t>(a.batch) * a.value_heads * kLD * kLD * sizeof(float), stream);
  if (e == cudaSuccess) e = gdn_chunked_with_states(stream, f, base + l.records, states, status, lanes->prepared);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(lanes->aux, lanes->prepared, 0);
  if (e == cudaSuccess)
    e = gdn_scan_bwd_launch(lanes->aux, dcore16, base + l.records, a.batch, a.tokens, a.value_heads, chunks, dstates, status);
  // (joined even after a failed launch, so that nothing of this call is left running unordered)
  cudaError_t joined = cudaEventRecord(lanes->aux_done, lanes->aux);
  const unsigned matrices = static_cast<unsigned>(a.batch) * a.value_heads * chunks;
  if (e == cudaSuccess && joined == cudaSuccess) {
    transpose_128_kernel<<<matrices, 256, 0, stream>>>(states, states_t);   // (needs the forward only)
    e = cudaGetLastError();
  }
  if (joined == cudaSuccess) joined = cudaStreamWaitEvent(stream, lanes->aux_done, 0);
  if (e != cudaSuccess) return e;
  if (joined != cudaSuccess) return joined;
  transpose_128_kernel<<<matrices, 256, 0, stream>>>(dstates, dstates_t);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  LocalArgs la{a, states, states_t, dstates, dstates_t, chunks, nullptr, nullptr, 0, 0};
  *qk_direct = a.value_heads == a.key_heads && dqk_token % 4 == 0 && (reinterpret_cast<uintptr_t>(dq_out) & 15u) == 0 &&
               (reinterpret_cast<uintptr_t>(dk_out) & 15u) == 0;
  if (*qk_direct) {
    la.dq_rows = dq_out; la.dk_rows = dk_out; la.row_stride = dqk_token; la.head_stride = kLD;
  } else {
    la.dq_rows = a.qk_partials; la.dk_rows = a.qk_partials + kLD;
    la.row_stride = static_cast<size_t>(a.value_heads) * 2 * kLD; la.head_stride = 2 * kLD;
  }
  e = cudaFuncSetAttribute(gdn_bwd_chunk_local, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(sizeof(LocalSmem)));
  if (e != cudaSuccess) return e;
  gdn_bwd_chunk_local<<<dim3(chunks, a.value_heads, a.batch), kLThreads, sizeof(LocalSmem), stream>>>(la);
  return cudaGetLastError();
}

}  // namespace pluto
