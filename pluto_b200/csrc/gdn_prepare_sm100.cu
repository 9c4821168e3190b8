// Chunked gated delta-net prefill on the 5th-generation tensor cores: the chunk-parallel part.
//
// For every chunk of 64 tokens (notation of gdn_chunked.cu; b_t = running sum of log decay inside
// the chunk, c_t = e^{b_t}, k^, q^ the normalised key / scaled query):
//     A[t,s] = beta_t e^{b_t-b_s} (k^_t.k^_s)  (s < t),   T = (I + A)^-1
//     M[t,s] = e^{b_t-b_s} (q^_t.k^_s)         (s <= t)
//     W = T (beta c k^),   U = T (beta v),   Kt = k^ . c_C/c
//     Pn = -(Kt^T W),      Qt = c q^ - M W
// and the record of gdn_records.cuh (Pn, Kt, Qt, M, gamma = c_C, U; all bf16) goes to the scan kernel.
//
// One CTA takes TWO consecutive chunks of a (sequence, head): 128 tokens = the 128 rows of a
// tcgen05.mma tile = the 128 lanes of TMEM, so every product below is a full M128 instruction and
// every thread owns one token row from the raw scores to the records (two threads per row, one per
// half of the columns):
//   * raw q, k, v tiles arrive by TMA straight from the activations (128-byte swizzle, zero fill
//     past the sequence end); no register staging, no normalised copies: the row scalings (norms,
//     decays, beta) are applied to the small matrices instead of the 128-wide operands;
//   * K K^T and Q K^T for both chunks in two M128 N128 K128 products (the cross-chunk blocks are
//     ignored); the key norms are the diagonal of K K^T;
//   * (I + A)^-1 in fp32 on the CUDA cores from shared memory;
//   * W = (T . col-scale) K and U = (T . beta) V as block-diagonal products: the A tiles are laid
//     out [T_a][zero block][T_b] so that "rows 0-63 = T_a, rest zero" and "rows 64-127 = T_b, rest
//     zero" are two overlapping 128-row views sharing the zero block; U's T enters as bf16 high
//     part plus remainder;
//   * Pn (per chunk) and M W from the bf16 W written back to shared memory, then the records are
//     written from registers in the swizzled operand order (16-byte pieces, 128 contiguous bytes
//     per row and slab).
// TMEM columns: K K^T 0-127 | Q K^T 128-255 | W 256-383 | U 384-511, then Pn(a) 0-127 |
// Pn(b) 128-255 | M W 256-383.
#include <stddef.h>

#include "common.cuh"
#include "engine.h"
#include "gdn_records.cuh"

namespace pluto {
namespace {

constexpr int kPrepThreads = 256;
constexpr float kMinLogDecay = -60.0f;
constexpr bool kULoFromT = true;   // U = (T_hi + T_lo)(beta v): the remainder costs 8 more MMAs

// shared-memory regions, byte offsets from the 1024-aligned base
constexpr uint32_t kRegK = 0;          // raw keys [128 tokens][128]: 2 slabs x 16384   -> Kt in place
constexpr uint32_t kRegQ = 32768;      // raw queries                                   -> fp32 scratch [128][64]
constexpr uint32_t kRegV = 65536;      // raw values                                    -> W (bf16)
constexpr uint32_t kRegT1 = 98304;     // T . (beta c kn)        [T_a 8192][zero 8192][T_b 8192]
constexpr uint32_t kRegT2H = 122880;   // T . beta, high parts
constexpr uint32_t kRegT2L = 147456;   // T . beta, remainders
constexpr uint32_t kRegM = 172032;     // M                      same three-block layout
constexpr uint32_t kRegSmall = 196608;

struct PrepSmall {
  float b[128], beta[128], kn[128], scale1[128], qsq[2][128];
  uint64_t loaded, loaded_v, mma_done;   // keys and queries; values (needed later); products
  uint32_t tmem_base;
};


// The fp32 scratch holds, per chunk, first A TRANSPOSED ([s][t] with the even rows t before the odd
// ones: the substitution's two threads per column own the even and the odd rows and read four of
// their rows of one column s as one broadcast 16-byte load), then T row-major with the 16-byte pieces of row t permuted by (piece ^ (t & 15)):
// the column owners write conflict-free and the row owners read 16-byte pieces almost so.
__device__ __forceinline__ int a_transposed_index(int chunk, int s, int t) {
  // even rows, then odd rows, of column s; the odd half is rotated by 16 banks, so that the two
  // 16-byte pieces one substitution step reads (one per parity) and the 32 elements a warp writes
  // fall into different banks
  return chunk * 4096 + s * 64 + (t & 1) * 32 + ((t >> 1) ^ ((t & 1) << 4));
}
__device__ __forceinline__ int t_index(int row, int s) {
  return row * 64 + ((((s >> 2) ^ (row & 15)) << 2) | (s & 3));
}

__global__ void __launch_bounds__(kPrepThreads, 1)
gdn_prepare_sm100(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                  const __grid_constant__ CUtensorMap map_v, GdnArgs a, uint8_t* __restrict__ records,
                  int first_pair, int chunks, uint32_t* status) {
  extern __shared__ uint8_t prep_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(prep_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  PrepSmall& sm = *reinterpret_cast<PrepSmall*>(smem + kRegSmall);   // (barriers; the arrays go through lds/sts)
  // Every access to shared memory below uses a 32-bit shared address and ld.shared / st.shared:
  // `smem` is a generic pointer to the compiler (the alignment arithmetic hides its address
  // space), and generic accesses made the phases that live on shared memory several times slower.
  const uint32_t base = smem_u32(smem);
  const uint32_t scratch = base + kRegQ;                       // fp32 [2 chunks][64][64]
  const uint32_t sm_b = base + kRegSmall + offsetof(PrepSmall, b);
  const uint32_t sm_beta = base + kRegSmall + offsetof(PrepSmall, beta);
  const uint32_t sm_kn = base + kRegSmall + offsetof(PrepSmall, kn);
  const uint32_t sm_scale1 = base + kRegSmall + offsetof(PrepSmall, scale1);
  const uint32_t sm_qsq = base + kRegSmall + offsetof(PrepSmall, qsq);
  const int pair = first_pair + blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int kh = h / (a.value_heads / a.key_heads);
  const int warp = uniform_warp_index(), lane = threadIdx.x % 32;
  const int quarter = warp & 3, half = warp >> 2;     // TMEM lane quarter; column half of the row
  const int r = quarter * 32 + lane;                  // token row of the pair == TMEM lane
  const int cb = r >> 6, rl = r & 63;                 // chunk of the pair, row inside the chunk
  const int t0 = pair * 128;
  const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
  const int dv = a.value_dim;
  const int chunk = pair * 2 + cb;
  uint8_t* rec = records + ((static_cast<size_t>(b) * a.value_heads + h) * chunks + chunk) * GdnRecord::bytes(dv);
  const bool live_chunk = chunk < chunks;

  if (threadIdx.x == 0) {
    mbar_init(&sm.loaded, 1);
    mbar_init(&sm.loaded_v, 1);
    mbar_init(&sm.mma_done, 1);
    mbar_fence_init();
    // the raw tiles are requested first: everything up to the first product hides their latency
    // (measured without effect: pulling the tiles of the CTA one wave later into L2 with bulk
    // prefetches from here, 0.698 ms against 0.689 ms for the whole prefill; so the wait for the
    // tiles is the memory system's load, not one CTA's round trip)
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
    mbar_expect_tx(&sm.loaded, 2 * 32768);
    for (int s = 0; s < 2; ++s) {
      tma_load_3d(smem + kRegK + s * 16384, &map_k, kh * kGdnKeyDim + s * 64, t0, b, &sm.loaded);
      tma_load_3d(smem + kRegQ + s * 16384, &map_q, kh * kGdnKeyDim + s * 64, t0, b, &sm.loaded);
    }
    // the values are first read by the U product, after the inversion: their own barrier
    mbar_expect_tx(&sm.loaded_v, 32768);
    for (int s = 0; s < 2; ++s)
      tma_load_3d(smem + kRegV + s * 16384, &map_v, h * dv + s * 64, t0, b, &sm.loaded_v);
  }
  if (warp == 1) {
    tmem_alloc(&sm.tmem_base, 512);
    tmem_relinquish();
  }
  // the zero blocks shared by the two 128-row views of every three-block tile
  for (int i = threadIdx.x; i < 4 * 512; i += kPrepThreads) {
    const uint32_t region = i / 512 == 0 ? kRegT1 : (i / 512 == 1 ? kRegT2H : (i / 512 == 2 ? kRegT2L : kRegM));
    sts_b32x4(base + region + 8192 + (i % 512) * 16, 0, 0, 0, 0);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;

  // ---- gates: running sum of log decay inside each chunk (past the sequence end: g = 1, beta = 0)
  float run = 0.0f, be = 0.0f;
  if (half == 0) {
    const int t = t0 + r;
    if (t < a.tokens) {
      const size_t off = (static_cast<size_t>(b) * a.tokens + t) * a.value_heads + h;
      run = fmaxf(logf(a.g[off]), kMinLogDecay);
      be = a.beta[off];
    }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float v = __shfl_up_sync(0xffffffffu, run, o);
      if (lane >= o) run += v;
    }
    if (lane == 31) sts_f32(sm_kn + quarter * 4, run);   // (kn is free until the key norms are known)
  }
  __syncthreads();
  if (half == 0) {
    if (quarter & 1) run += lds_f32(sm_kn + (quarter - 1) * 4);
    sts_f32(sm_b + r * 4, run);
    sts_f32(sm_beta + r * 4, be);
  }
  __syncthreads();

  // ---- raw scores on the tensor cores; meanwhile every thread takes its half of its query row
  bool ok = __all_sync(0xffffffffu, mbar_wait(&sm.loaded, 0, status, 60));
  constexpr uint32_t kIdescKK = umma_idesc_bf16_majors(128, 128, false, false);
  constexpr uint32_t kIdescTB = umma_idesc_bf16_majors(128, 128, false, true);    // K-major A, token-major B
  constexpr uint32_t kIdescTT = umma_idesc_bf16_majors(128, 128, true, true);     // both token-major
  if (warp == 0 && ok) {
    if (elect_one()) {
      const uint64_t kd = umma_desc_sw128(base + kRegK, 16, 1024), qd = umma_desc_sw128(base + kRegQ, 16, 1024);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t off = ((ks / 4) * 16384 + (ks % 4) * 32) >> 4;
        umma_ss(tmem + 0, kd + off, kd + off, kIdescKK, ks > 0);
      }
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t off = ((ks / 4) * 16384 + (ks % 4) * 32) >> 4;
        umma_ss(tmem + 128, qd + off, kd + off, kIdescKK, ks > 0);
      }
      tc_commit(&sm.mma_done);
    }
    __syncwarp();
  }
  {
    // |q|^2 of this thread's half of its query row (the row itself is read again for Qt at the end:
    // holding it in registers across the inversion pushed that phase's column into local memory)
    const uint32_t row = base + kRegQ + half * 16384 + r * 128;
    float ss = 0.0f;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint4 v = lds_b32x4(row + ((c ^ (r & 7)) * 16));
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) ss += bf16_lo(w[e]) * bf16_lo(w[e]) + bf16_hi(w[e]) * bf16_hi(w[e]);
    }
    sts_f32(sm_qsq + (half * 128 + r) * 4, ss);
  }
  __syncthreads();
  const float qn = a.normalize_qk
                       ? rsqrtf(lds_f32(sm_qsq + r * 4) + lds_f32(sm_qsq + (128 + r) * 4) + 1e-6f) / sqrtf(static_cast<float>(kGdnKeyDim))
                       : a.q_scale;

  ok = __all_sync(0xffffffffu, ok && mbar_wait(&sm.mma_done, 0, status, 61));
  tc_fence_after();
  uint32_t kk[32], qk[32];
  if (ok) {
    tmem_ld32(tmem + lane_base + 0 + cb * 64 + half * 32, kk);
    tmem_ld32(tmem + lane_base + 128 + cb * 64 + half * 32, qk);
    tmem_wait_ld();
    if ((rl >> 5) == half) {   // the diagonal of K K^T is |k|^2
      float diagonal = 0.0f;
#pragma unroll
      for (int i = 0; i < 32; ++i)   // (a register array must not be indexed with a runtime value)
        if (i == (rl & 31)) diagonal = __uint_as_float(kk[i]);
      sts_f32(sm_kn + r * 4, a.normalize_qk ? rsqrtf(diagonal + 1e-6f) : 1.0f);
    }
  }
  __syncthreads();
  const float br = lds_f32(sm_b + r * 4), betar = lds_f32(sm_beta + r * 4), knr = lds_f32(sm_kn + r * 4);
  if (half == 0) sts_f32(sm_scale1 + r * 4, betar * __expf(br) * knr);
  if (ok) {
    // ---- A (fp32, to the scratch) and M (bf16, to its operand tile) for this thread's 32 columns
    uint32_t mrow[16];
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      float mv[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int s = half * 32 + i + e, sg = cb * 64 + s;
        const float ratio = s <= rl ? __expf(br - lds_f32(sm_b + sg * 4)) : 0.0f;
        const float kns = lds_f32(sm_kn + sg * 4);
        sts_f32(scratch + a_transposed_index(cb, s, rl) * 4,
                s < rl ? betar * ratio * knr * kns * __uint_as_float(kk[i + e]) : 0.0f);
        mv[e] = ratio * qn * kns * __uint_as_float(qk[i + e]);
      }
      mrow[i / 2] = pack_bf16(mv[0], mv[1]);
    }
    const uint32_t mtile = base + kRegM + r * 128 + (cb ? 8192 : 0);
#pragma unroll
    for (int q = 0; q < 4; ++q)
      sts_b32x4(mtile + (((half * 4 + q) ^ (r & 7)) * 16), mrow[4 * q], mrow[4 * q + 1], mrow[4 * q + 2],
                mrow[4 * q + 3]);
  }
  __syncthreads();

  // ---- T = (I + A)^-1 by forward substitution, right-looking: as soon as entry s of a column is
  //      final it is folded into every later entry (independent FMAs, one of them on the chain to
  //      the next step).  Two threads per (chunk, column), neighbouring lanes: one owns the even
  //      rows, the other the odd ones; the pivot of step s comes from the lane that owns row s by a
  //      shuffle.  All threads of a chunk read the same elements of A, four rows at a time.
  {
    // rows 2 i + parity of column jj, as 16 pairs (i even, i odd) for two-lane fp32 FMAs
    uint64_t col[16];
    const int c2 = threadIdx.x >> 7, jj = (threadIdx.x >> 1) & 63, parity = threadIdx.x & 1;
#pragma unroll
    for (int p2 = 0; p2 < 16; ++p2)
      col[p2] = f2_pack(4 * p2 + parity == jj ? 1.0f : 0.0f, 4 * p2 + 2 + parity == jj ? 1.0f : 0.0f);
    // The elements of A for step s + 1 are requested before step s waits for its pivot, so the
    // chain from one step to the next is shuffle -> FMA -> select and never a shared-memory load.
    // pieces 0-3 and 4-7 of this thread's half of a column (the odd half has them exchanged)
    const uint32_t a_lo = scratch + (c2 * 4096 + parity * 48) * 4, a_hi = scratch + (c2 * 4096 + parity * 16) * 4;
    float4 ahead[8];
#pragma unroll
    for (int i4 = 0; i4 < 8; ++i4) ahead[i4] = lds_f32x4((i4 < 4 ? a_lo : a_hi) + i4 * 16);
#pragma unroll
    for (int sc = 0; sc < 63; ++sc) {
      float4 now[8];
#pragma unroll
      for (int i4 = sc / 8; i4 < 8; ++i4) now[i4] = ahead[i4];
      if (sc + 1 < 63) {
#pragma unroll
        for (int i4 = (sc + 1) / 8; i4 < 8; ++i4)
          ahead[i4] = lds_f32x4((i4 < 4 ? a_lo : a_hi) + (sc + 1) * 256 + i4 * 16);
      }
      float lo, hi;
      f2_unpack(col[sc >> 2], lo, hi);
      const float mine = (sc >> 1) & 1 ? hi : lo;   // entry i = sc >> 1 of this thread
      const float c = __shfl_sync(0xffffffffu, mine, (lane & ~1) | (sc & 1));
      const uint64_t minus_c = f2_pack(-c, -c);
      // own rows t = 2 i + parity > sc; A is zero at and above the pivot (strictly lower
      // triangular), so whole groups of four rows are folded in from the pivot's group on
#pragma unroll
      for (int i4 = sc / 8; i4 < 8; ++i4) {
        col[2 * i4] = f2_fma(f2_pack(now[i4].x, now[i4].y), minus_c, col[2 * i4]);
        col[2 * i4 + 1] = f2_fma(f2_pack(now[i4].z, now[i4].w), minus_c, col[2 * i4 + 1]);
      }
    }
    __syncthreads();
#pragma unroll
    for (int p2 = 0; p2 < 16; ++p2) {
      float lo, hi;
      f2_unpack(col[p2], lo, hi);
      sts_f32(scratch + t_index(c2 * 64 + 4 * p2 + parity, jj) * 4, lo);
      sts_f32(scratch + t_index(c2 * 64 + 4 * p2 + 2 + parity, jj) * 4, hi);
    }
  }
  __syncthreads();

  // ---- T . column scales -> bf16 operand tiles
  {
    uint32_t t1[16], t2h[16], t2l[16];
#pragma unroll
    for (int v = 0; v < 8; ++v) {
      const int piece = half * 8 + v;   // columns piece*4 .. +3 of this row
      const float4 t4 = lds_f32x4(scratch + (r * 64 + ((piece ^ (r & 15)) << 2)) * 4);
      const float tv[4] = {t4.x, t4.y, t4.z, t4.w};
      float x1[4], x2[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int sg = cb * 64 + piece * 4 + e;
        x1[e] = tv[e] * lds_f32(sm_scale1 + sg * 4);
        x2[e] = tv[e] * lds_f32(sm_beta + sg * 4);
      }
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        t1[v * 2 + e] = pack_bf16(x1[2 * e], x1[2 * e + 1]);
        t2h[v * 2 + e] = pack_bf16(x2[2 * e], x2[2 * e + 1]);
        t2l[v * 2 + e] = pack_bf16(x2[2 * e] - bf16_lo(t2h[v * 2 + e]), x2[2 * e + 1] - bf16_hi(t2h[v * 2 + e]));
      }
    }
    const uint32_t row_off = r * 128 + (cb ? 8192 : 0);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint32_t piece = ((half * 4 + q) ^ (r & 7)) * 16;
      sts_b32x4(base + kRegT1 + row_off + piece, t1[4 * q], t1[4 * q + 1], t1[4 * q + 2], t1[4 * q + 3]);
      sts_b32x4(base + kRegT2H + row_off + piece, t2h[4 * q], t2h[4 * q + 1], t2h[4 * q + 2], t2h[4 * q + 3]);
      sts_b32x4(base + kRegT2L + row_off + piece, t2l[4 * q], t2l[4 * q + 1], t2l[4 * q + 2], t2l[4 * q + 3]);
    }
  }
  fence_proxy_async();
  __syncthreads();

  // ---- W = (T . scale1) K and U = (T . beta) V, each chunk through its 128-row view
  ok = __all_sync(0xffffffffu, ok && mbar_wait(&sm.loaded_v, 0, status, 59));
  if (warp == 0 && ok) {
    if (elect_one()) {
#pragma unroll
      for (int view = 0; view < 2; ++view) {
        const uint64_t t1d = umma_desc_sw128(base + kRegT1 + view * 8192, 16, 1024);
        const uint64_t kd = umma_desc_sw128(base + kRegK + view * 8192, 16384, 1024);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_ss(tmem + 256, t1d + ks * 2, kd + ks * 128, kIdescTB, view > 0 || ks > 0);
      }
#pragma unroll
      for (int part = 0; part < (kULoFromT ? 2 : 1); ++part)
#pragma unroll
        for (int view = 0; view < 2; ++view) {
          const uint64_t t2d = umma_desc_sw128(base + (part ? kRegT2L : kRegT2H) + view * 8192, 16, 1024);
          const uint64_t vd = umma_desc_sw128(base + kRegV + view * 8192, 16384, 1024);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_ss(tmem + 384, t2d + ks * 2, vd + ks * 128, kIdescTB, part > 0 || view > 0 || ks > 0);
        }
      tc_commit(&sm.mma_done);
    }
    __syncwarp();
  }
  ok = __all_sync(0xffffffffu, ok && mbar_wait(&sm.mma_done, 1, status, 62));
  tc_fence_after();
  const float tail = __expf(lds_f32(sm_b + (cb * 64 + 63) * 4) - br) * knr;   // Kt = k . (c_C / c) . kn
  if (ok) {
    // W row -> bf16 operand tile (over the raw values, which the U products no longer need)
    uint32_t x[2][32];
    tmem_ld32(tmem + lane_base + 256 + half * 64, x[0]);
    tmem_ld32(tmem + lane_base + 256 + half * 64 + 32, x[1]);
    tmem_wait_ld();
    const uint32_t wrow = base + kRegV + half * 16384 + r * 128;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = c * 8 + e * 2;
        w[e] = pack_bf16(__uint_as_float(x[i / 32][i % 32]), __uint_as_float(x[i / 32][i % 32 + 1]));
      }
      sts_b32x4(wrow + ((c ^ (r & 7)) * 16), w[0], w[1], w[2], w[3]);
    }
    // U row -> staging tile in record order (over the scratch, which nobody reads any more)
    tmem_ld32(tmem + lane_base + 384 + half * 64, x[0]);
    tmem_ld32(tmem + lane_base + 384 + half * 64 + 32, x[1]);
    tmem_wait_ld();
    {
      const uint32_t urow = base + kRegQ + cb * 16384 + half * 8192 + rl * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = c * 8 + e * 2;
          w[e] = pack_bf16(__uint_as_float(x[i / 32][i % 32]), __uint_as_float(x[i / 32][i % 32 + 1]));
        }
        sts_b32x4(urow + ((c ^ (rl & 7)) * 16), w[0], w[1], w[2], w[3]);
      }
    }
    // Kt row: scaled keys, in place (operand of Pn, and the record's tile)
    const uint32_t krow = base + kRegK + half * 16384 + r * 128;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint32_t piece = (c ^ (r & 7)) * 16;
      uint4 v = lds_b32x4(krow + piece);
      v.x = pack_bf16(bf16_lo(v.x) * tail, bf16_hi(v.x) * tail);
      v.y = pack_bf16(bf16_lo(v.y) * tail, bf16_hi(v.y) * tail);
      v.z = pack_bf16(bf16_lo(v.z) * tail, bf16_hi(v.z) * tail);
      v.w = pack_bf16(bf16_lo(v.w) * tail, bf16_hi(v.w) * tail);
      sts_b32x4(krow + piece, v.x, v.y, v.z, v.w);
    }
  }
  tc_fence_before();
  fence_proxy_async();
  __syncthreads();
  tc_fence_after();

  // ---- Pn(chunk) = Kt^T W over the chunk's 64 tokens; M W through the two views of M
  if (warp == 0 && ok) {
    if (elect_one()) {
#pragma unroll
      for (int view = 0; view < 2; ++view) {
        const uint64_t ktd = umma_desc_sw128(base + kRegK + view * 8192, 16384, 1024);
        const uint64_t wd = umma_desc_sw128(base + kRegV + view * 8192, 16384, 1024);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_ss(tmem + view * 128, ktd + ks * 128, wd + ks * 128, kIdescTT, ks > 0);
      }
#pragma unroll
      for (int view = 0; view < 2; ++view) {
        const uint64_t md = umma_desc_sw128(base + kRegM + view * 8192, 16, 1024);
        const uint64_t wd = umma_desc_sw128(base + kRegV + view * 8192, 16384, 1024);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_ss(tmem + 256, md + ks * 2, wd + ks * 128, kIdescTB, view > 0 || ks > 0);
      }
      tc_commit(&sm.mma_done);
    }
    __syncwarp();
  }
  // the raw query row again for Qt, from global memory (the TMA load pulled it through L2 a few
  // microseconds ago), requested before the wait for the last products so that it hides there
  uint4 qraw[8];
  {
    const bool live_token = t0 + r < a.tokens;
    const uint4* qsrc = reinterpret_cast<const uint4*>(
        static_cast<const __nv_bfloat16*>(a.q) + (static_cast<size_t>(b) * a.tokens + (live_token ? t0 + r : 0)) * a.qk_token +
        static_cast<size_t>(kh) * kGdnKeyDim + half * 64);
#pragma unroll
    for (int c = 0; c < 8; ++c) qraw[c] = live_token ? __ldg(qsrc + c) : make_uint4(0, 0, 0, 0);
  }
  ok = __all_sync(0xffffffffu, ok && mbar_wait(&sm.mma_done, 0, status, 63));
  tc_fence_after();
  // The tiles that are final leave now, as linear bulk copies from shared memory -- after the
  // last products, not before them: bulk copies in flight made those products twice as slow.
  uint8_t* pair_rec = records + ((static_cast<size_t>(b) * a.value_heads + h) * chunks + pair * 2) * GdnRecord::bytes(dv);
  if (threadIdx.x == 32 && ok) {
    for (int v = 0; v < 2 && pair * 2 + v < chunks; ++v) {
      uint8_t* out = pair_rec + static_cast<size_t>(v) * GdnRecord::bytes(dv);
      bulk_store(out + GdnRecord::kCommon + GdnRecord::kUH, smem + kRegQ + v * 16384, 16384);
      bulk_store(out + GdnRecord::kKT, smem + kRegK + v * 8192, 8192);
      bulk_store(out + GdnRecord::kKT + 8192, smem + kRegK + 16384 + v * 8192, 8192);
      bulk_store(out + GdnRecord::kMM, smem + kRegM + v * 16384, 8192);
    }
    bulk_store_commit();
  }

  if (ok) {
    uint32_t x[2][32];
    // Pn rows: row r = key index of the output, this thread's 64 input keys, for both chunks; staged
    // in record order over the T tiles (72 KB, dead since the W / U products)
#pragma unroll
    for (int view = 0; view < 2; ++view) {
      tmem_ld32(tmem + lane_base + view * 128 + half * 64, x[0]);
      tmem_ld32(tmem + lane_base + view * 128 + half * 64 + 32, x[1]);
      tmem_wait_ld();
      const uint32_t prow = base + kRegT1 + view * 32768 + half * 16384 + r * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = c * 8 + e * 2;
          w[e] = pack_bf16(-__uint_as_float(x[i / 32][i % 32]), -__uint_as_float(x[i / 32][i % 32 + 1]));
        }
        sts_b32x4(prow + ((c ^ (r & 7)) * 16), w[0], w[1], w[2], w[3]);
      }
    }
    // Qt = c q^ - M W, staged over W (dead since the last products)
    tmem_ld32(tmem + lane_base + 256 + half * 64, x[0]);
    tmem_ld32(tmem + lane_base + 256 + half * 64 + 32, x[1]);
    tmem_wait_ld();
    {
      const float cq = __expf(br) * qn;
      const uint32_t qrow_out = base + kRegV + cb * 16384 + half * 8192 + rl * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint32_t qw[4] = {qraw[c].x, qraw[c].y, qraw[c].z, qraw[c].w};
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = c * 8 + e * 2;
          const uint32_t q2 = qw[e];
          w[e] = pack_bf16(cq * bf16_lo(q2) - __uint_as_float(x[i / 32][i % 32]),
                           cq * bf16_hi(q2) - __uint_as_float(x[i / 32][i % 32 + 1]));
        }
        sts_b32x4(qrow_out + ((c ^ (rl & 7)) * 16), w[0], w[1], w[2], w[3]);
      }
    }
    if (live_chunk && rl == 63 && half == 0) *reinterpret_cast<float*>(rec + GdnRecord::kGM) = __expf(br);
  }
  fence_proxy_async();
  __syncthreads();
  if (threadIdx.x == 32) {
    if (ok) {
      for (int v = 0; v < 2 && pair * 2 + v < chunks; ++v) {
        uint8_t* out = pair_rec + static_cast<size_t>(v) * GdnRecord::bytes(dv);
        bulk_store(out + GdnRecord::kPN, smem + kRegT1 + v * 32768, 32768);
        bulk_store(out + GdnRecord::kQT, smem + kRegV + v * 16384, 16384);
      }
      bulk_store_commit();
    }
    bulk_store_wait_read();   // shared memory may go away only after the copies have read it
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace

bool gdn_prepare_sm100_supported(const GdnArgs& a) { return a.value_dim == kGdnSliceCols; }

bool gdn_prepare_sm100_maps(const GdnArgs& a, CUtensorMap maps[3]) {
  return make_token_map(&maps[0], a.q, a.key_heads * kGdnKeyDim, a.tokens, a.batch, a.qk_token, 128) &&
         make_token_map(&maps[1], a.k, a.key_heads * kGdnKeyDim, a.tokens, a.batch, a.qk_token, 128) &&
         make_token_map(&maps[2], a.v, a.value_heads * a.value_dim, a.tokens, a.batch, a.v_token, 128);
}

// Chunk pairs first_pair .. first_pair + pairs - 1 of every (sequence, head); `chunks` is the whole
// sequence's chunk count (the stride of the record array).
cudaError_t gdn_prepare_sm100_launch(cudaStream_t stream, const CUtensorMap maps[3], const GdnArgs& a,
                                     void* records, int first_pair, int pairs, int chunks, uint32_t* status) {
  const size_t smem = 1024 + kRegSmall + sizeof(PrepSmall);
  if (first_pair == 0) {   // (every call starts with the piece at pair 0)
    cudaError_t e = cudaFuncSetAttribute(gdn_prepare_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return e;
  }
  gdn_prepare_sm100<<<dim3(pairs, a.value_heads, a.batch), kPrepThreads, smem, stream>>>(
      maps[0], maps[1], maps[2], a, static_cast<uint8_t*>(records), first_pair, chunks, status);
  return cudaGetLastError();
}

}  // namespace pluto
