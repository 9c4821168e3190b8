// Causal multi-head attention backward on the Blackwell tensor cores (bf16 operands, fp32
// accumulation, head width 64 or 128) for the packed [rows, 3E] layout of AttentionLayer.
//
// Same decomposition as the reference (src/llm/layers/attention.cc:235-314 query-owned pass,
// :319-396 key/value-owned pass): two passes that each own their output tile, so every dQ, dK
// and dV element has one writer and a fixed summation order -- no floating-point atomics, runs
// are bitwise repeatable.  Probabilities are rebuilt from the statistics the forward saved:
//     P = exp(s*scale - max) / l,   dP = dO V^T,   dS = P (dP - delta) scale,   delta = sum dO.O
//     dQ = dS K                     dK = dS^T Q,                                dV = P^T dO
//
//   attn_bwd_prep          delta per row (fp32, from the stored O like the reference), the upstream
//                          gradient rounded to bf16 for the tensor cores, and per-row statistics
//                          x = -(max*log2e + log2 l) (so that P = exp2(s*scale*log2e + x)) and delta.
//   attn_bwd_dq_sm100      head width 64, one CTA per 128-query tile, two CTAs per SM; per 64-key step:
//                          S and dP by tcgen05.mma into TMEM (the CTA's Q and dO rows are TMEM A
//                          operands), the row threads turn them into dS (bf16, written over S in
//                          TMEM), dQ += dS K with dS as the TMEM operand and K MN-major from smem.
//   attn_bwd_dkv_sm100     head width 64, one CTA per 128-key tile; per 64-query step: S^T = K Q^T and
//                          dP^T = V dO^T, the row threads build P^T and dS^T, then dV += P^T dO and
//                          dK += dS^T Q.
//   attn_bwd_dq128_sm100,  head width 128 in steps of 128 opposite-side rows (an N64 instruction costs
//   attn_bwd_dkv128_sm100  more than half an N128 one); all 512 TMEM columns single-buffered, four
//                          warpgroups of row threads working in two phases; see above each kernel.
// dS carries no softmax scale: dQ and dK are scaled once when they are written.  The Q/dO rows of a
// dQ CTA arrive by TMA and every gradient tile leaves as bulk copies of rows staged in shared
// memory.  All copies are tiled TMA loads without multicast; all waits are bounded.
#include <type_traits>

#include "common.cuh"
#include "engine.h"

namespace pluto {
namespace {

constexpr int kRowTile = 128;   // rows owned by a CTA (TMEM lanes)
constexpr int kColTile = 64;    // opposite-side rows consumed per step
constexpr int kBwdStages = 4;
constexpr int kRowGroups = 2;   // warpgroups of row threads; group g takes columns [32 g, 32 g + 32) of a step
constexpr int kBwdThreads = 64 + 128 * kRowGroups;   // warp 0 loads, warp 1 issues MMAs, then the row warps
constexpr float kLog2e = 1.4426950408889634f;

struct BwdParams {
  int seq, heads, head_dim;   // heads = query heads
  int group;                  // query heads per key/value head
  int q_col0, k_col0, v_col0; // column of head 0 inside a token row of the q / k / v tensor maps
  float scale, scale_log2;
  // Row statistics, one float4 per pair of rows: [(b*H+h) * seq_pad/2 + s/2] = (x_even, x_odd,
  // delta_even, delta_odd) with x = -(max*log2e + log2 l), so that P = exp2(s*scale*log2e + x);
  // the two-lane arithmetic of the dK/dV pass takes both halves as they lie.  Past the sequence
  // end x = -1e30 (P = 0) and delta = 0.
  const float* stats;
  // The same two values as plain arrays, [(b*H+h) * seq_pad + s] each, for the passes that fetch
  // them at different times.
  const float* shifts;
  const float* deltas_pad;
  int seq_pad;   // even
  const __nv_bfloat16* q;        // query rows as the dQ pass reads them itself: token stride q_token
  const __nv_bfloat16* d_out16;  // upstream gradient rounded to bf16, [token, head, D]
  size_t q_token;
  float *dq, *dk, *dv;   // fp32; token strides dq_token / dkv_token elements, head stride D
  size_t dq_token, dkv_token;
  uint32_t* status;
};

// ---------------------------------------------------------------------------------------------
// prep: a stream over the (token, head) rows of dO and O, which are contiguous in that order.
// D / 8 lanes share a row (8 channels a lane: two 16-byte gradient loads, one 16-byte output
// load, one 16-byte bf16 store), so a warp covers 4 (D = 64) or 2 (D = 128) rows per step and
// the row sum needs 3 or 4 shuffles; two steps are in flight per warp.
// The row statistics live head-major ([sequence, head, token]) while the rows stream token-major,
// so a CTA owns `block_tokens` consecutive tokens of one sequence with all their heads and passes
// the statistics through shared memory: read and written per head as runs of consecutive tokens.
// (One 4-byte access per row and array, 32 KB apart, made 24 of this kernel's 58 us at the prefill
// shape.)  Dynamic shared memory: 2 * heads * block_tokens floats.
// ---------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(256)
attn_bwd_prep(const __nv_bfloat16* __restrict__ out, const float* __restrict__ d_out,  // out may be null
              const float* __restrict__ maxima, const float* __restrict__ normalizers,
              __nv_bfloat16* __restrict__ d_out_bf16, float* __restrict__ stats,
              float* __restrict__ shifts, float* __restrict__ deltas_pad,
              float* __restrict__ deltas, int seq, int seq_pad, int heads, int block_tokens) {
  constexpr int kLanes = D / 8;              // lanes per row
  constexpr int kRowsPerWarp = 32 / kLanes;
  constexpr int kUnroll = 2;
  extern __shared__ float prep_smem[];
  float* shift_s = prep_smem;                          // [head][token of the block]
  float* delta_s = prep_smem + heads * block_tokens;
  pdl_launch_dependents();   // the dQ kernel may set itself up (barriers, TMEM) while this one runs
  const int blocks_per_seq = (seq + block_tokens - 1) / block_tokens;
  const int b = blockIdx.x / blocks_per_seq, t0 = (blockIdx.x % blocks_per_seq) * block_tokens;
  const int tokens = min(block_tokens, seq - t0);
  const size_t stat_seq = static_cast<size_t>(b) * heads;   // (sequence, head) index of head 0
  // x = -(max*log2e + log2 l), so that P = exp2(s*scale*log2e + x): the division by l is folded in
  for (int idx = threadIdx.x; idx < heads * block_tokens; idx += blockDim.x) {
    const int h = idx / block_tokens, tk = idx % block_tokens;
    if (tk >= tokens) continue;
    const size_t stat = (stat_seq + h) * seq + t0 + tk;
    shift_s[idx] = -(maxima[stat] * kLog2e + log2f(normalizers[stat]));
    if (out == nullptr) delta_s[idx] = deltas[stat];   // the caller's deltas are the input
  }
  __syncthreads();

  const int lane = threadIdx.x % 32, sub = lane % kLanes, warp = threadIdx.x / 32;
  const int n_rows = tokens * heads;
  const size_t row0 = (static_cast<size_t>(b) * seq + t0) * heads;
  for (int first = warp * kRowsPerWarp; first < n_rows; first += 8 * kRowsPerWarp * kUnroll) {
    float4 g0[kUnroll], g1[kUnroll];
    uint4 o[kUnroll];
    int row[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      row[u] = first + u * 8 * kRowsPerWarp + lane / kLanes;
      const int r = row[u] < n_rows ? row[u] : n_rows - 1;   // past the end: a valid row, not stored
      const size_t base = (row0 + r) * D + sub * 8;
      g0[u] = *reinterpret_cast<const float4*>(d_out + base);
      g1[u] = *reinterpret_cast<const float4*>(d_out + base + 4);
      o[u] = out != nullptr ? *reinterpret_cast<const uint4*>(out + base) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      float part = g0[u].x * bf16_lo(o[u].x) + g0[u].y * bf16_hi(o[u].x) + g0[u].z * bf16_lo(o[u].y) +
                   g0[u].w * bf16_hi(o[u].y) + g1[u].x * bf16_lo(o[u].z) + g1[u].y * bf16_hi(o[u].z) +
                   g1[u].z * bf16_lo(o[u].w) + g1[u].w * bf16_hi(o[u].w);
#pragma unroll
      for (int off = kLanes / 2; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
      if (row[u] >= n_rows) continue;
      *reinterpret_cast<uint4*>(d_out_bf16 + (row0 + row[u]) * D + sub * 8) =
          make_uint4(pack_bf16(g0[u].x, g0[u].y), pack_bf16(g0[u].z, g0[u].w), pack_bf16(g1[u].x, g1[u].y),
                     pack_bf16(g1[u].z, g1[u].w));
      if (sub == 0 && out != nullptr) delta_s[(row[u] % heads) * block_tokens + row[u] / heads] = part;
    }
  }
  __syncthreads();

  for (int idx = threadIdx.x; idx < heads * block_tokens; idx += blockDim.x) {
    const int h = idx / block_tokens, tk = idx % block_tokens;
    if (tk >= tokens) continue;
    const int t = t0 + tk;
    const float shift = shift_s[idx], delta = delta_s[idx];
    if (out != nullptr) deltas[(stat_seq + h) * seq + t] = delta;
    const size_t padded = (stat_seq + h) * seq_pad;
    float* record = stats + (padded + (t & ~1)) * 2 + (t & 1);   // (x_even, x_odd, delta_even, delta_odd)
    record[0] = shift;
    record[2] = delta;
    shifts[padded + t] = shift;
    deltas_pad[padded + t] = delta;
  }
  // records of the padding past the sequence end (probability 0, delta 0): the sequence's last block
  if (t0 + block_tokens >= seq) {
    const int pad = seq_pad - seq;
    for (int idx = threadIdx.x; idx < heads * pad; idx += blockDim.x) {
      const int h = idx / pad, t = seq + idx % pad;
      const size_t padded = (stat_seq + h) * seq_pad;
      float* record = stats + (padded + (t & ~1)) * 2 + (t & 1);
      record[0] = -1.0e30f;
      record[2] = 0.0f;
      shifts[padded + t] = -1.0e30f;
      deltas_pad[padded + t] = 0.0f;
    }
  }
}

// One row of a TMA-written [rows x 64 bf16] slab (128-byte swizzle) into 32 registers: the 16-byte
// chunk c of row r lies at chunk position c ^ (r & 7).
__device__ __forceinline__ void load_swizzled_row(uint32_t slab, int row, uint32_t (&w)[32]) {
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint4 v = lds_b32x4(slab + row * 128 + ((c ^ (row & 7)) << 4));
    w[4 * c] = v.x; w[4 * c + 1] = v.y; w[4 * c + 2] = v.z; w[4 * c + 3] = v.w;
  }
}

// 32 accumulator columns of one row, scaled, into the row's slot of a staging tile in shared
// memory.  The tiles leave as one linear bulk copy per row: a thread writing its own row to global
// memory touches 32 different lines per warp instruction, which cost 4 to 5 us per CTA.  Rows
// are kStagePad bytes apart beyond their length, so that the 16-byte stores of a warp (one row
// per lane) spread over the banks.
constexpr int kStagePad = 16;
__device__ __forceinline__ void stage_columns(uint32_t slot, const uint32_t (&o)[32], float factor) {
#pragma unroll
  for (int i = 0; i < 32; i += 4)
    sts_b32x4(slot + i * 4, __float_as_uint(__uint_as_float(o[i]) * factor),
              __float_as_uint(__uint_as_float(o[i + 1]) * factor),
              __float_as_uint(__uint_as_float(o[i + 2]) * factor),
              __float_as_uint(__uint_as_float(o[i + 3]) * factor));
}

struct DqBarriers {
  uint64_t qdo_full, rows_ready, k_full[kBwdStages], v_full[kBwdStages], kv_empty[kBwdStages];
  uint64_t s_full[2], ds_full[2], dq_done;
  uint32_t tmem_base;
};

// ---------------------------------------------------------------------------------------------
// dQ: grid (query tiles of 128, heads, batch)
// ---------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(kBwdThreads, D == 64 ? 2 : 1)
attn_bwd_dq_sm100(const __grid_constant__ CUtensorMap map_k64,
                  const __grid_constant__ CUtensorMap map_v64,
                  const __grid_constant__ CUtensorMap map_q128,
                  const __grid_constant__ CUtensorMap map_do128, BwdParams p) {
  static_assert(D == 64, "the staging below fits head width 64; head width 128 has its own pass");
  constexpr int kSlabs = D / 64;
  constexpr int kColTileBytes = kSlabs * kColTile * 128;   // [64 x D] bf16
  // The CTA's own Q and dO rows live in TMEM (D / 2 columns each, two bf16 per column) as the A
  // operands of S = Q K^T and dP = dO V^T: an A operand in shared memory would be fetched again by
  // every MMA (4 KB against the 2 KB of a 64-key B operand), and shared-memory bandwidth, not the
  // tensor pipe, then sets the pace.  Head width 128 (one CTA per SM): then two (S, dP) buffers of
  // 64 + 64 columns and dQ, 512 columns in all; the MMA warp computes step j+1's S and dP while the
  // row threads turn step j's into dS.  Head width 64: one buffer and 256 columns, so that two
  // CTAs share an SM and overlap each other instead.
  constexpr bool kPipe = D == 128;
  constexpr uint32_t kTmemCols = kPipe ? 512 : 256;
  constexpr uint32_t kColQ = 0, kColDO = D / 2, kFirstBuf = D;
  constexpr uint32_t kColS = 0, kColDP = 64, kBuf = kPipe ? 128 : 0;
  constexpr uint32_t kColDQ = kFirstBuf + (kPipe ? 256 : 128);
  constexpr uint32_t kIdescS = umma_idesc_bf16(kRowTile, kColTile, false);
  constexpr uint32_t kIdescDQ = umma_idesc_bf16(kRowTile, D, true);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* k_smem = smem;
  uint8_t* v_smem = k_smem + kBwdStages * kColTileBytes;
  DqBarriers* bar = reinterpret_cast<DqBarriers*>(v_smem + kBwdStages * kColTileBytes);

  const int warp = uniform_warp_index(), lane = threadIdx.x % 32;
  // (sequence, head) varies fastest and the tile index slowest: longest tiles start first
  const int q_tile = gridDim.y - 1 - blockIdx.y, head = blockIdx.x % p.heads, batch = blockIdx.x / p.heads;
  const int kv_head = head / p.group;
  const int col_tiles = (p.seq + kColTile - 1) / kColTile;
  const int n_steps = min(2 * q_tile + 2, col_tiles);   // key tiles that hold a visible key

  if (threadIdx.x == 0) {
    mbar_init(&bar->qdo_full, 1);
    mbar_init(&bar->rows_ready, 4 * kRowGroups);
    for (int s = 0; s < kBwdStages; ++s) {
      mbar_init(&bar->k_full[s], 1);
      mbar_init(&bar->v_full[s], 1);
      mbar_init(&bar->kv_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bar->s_full[s], 1);
      mbar_init(&bar->ds_full[s], 4 * kRowGroups);   // one arrival per row warp
    }
    mbar_init(&bar->dq_done, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&bar->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bar->tmem_base;
  // Launched with programmatic stream serialisation: everything above overlapped the prep kernel;
  // its records and the bf16 gradient are read, and dQ is written, only after it has completed.
  // The dK/dV kernel reads nothing this kernel writes, so it may start as soon as every CTA of
  // this grid has got here (prep is then complete) and fill the SMs this grid's last CTAs leave.
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&map_k64);
      tma_prefetch_desc(&map_v64);
      tma_prefetch_desc(&map_q128);
      tma_prefetch_desc(&map_do128);
      // The CTA's Q and dO rows pass through the last two stages of the K and V rings on their way
      // into TMEM; those stages take key tiles only after the row threads have read them.
      mbar_expect_tx(&bar->qdo_full, 2 * kRowTile * 128);
      tma_load_3d(k_smem + 2 * kColTileBytes, &map_q128, p.q_col0 + head * D, q_tile * kRowTile, batch,
                  &bar->qdo_full);
      tma_load_3d(v_smem + 2 * kColTileBytes, &map_do128, head * D, q_tile * kRowTile, batch, &bar->qdo_full);
      bool ok = true;
      for (int j = 0; j < n_steps && ok; ++j) {
        const int st = j % kBwdStages, use = j / kBwdStages;
        if (j == 2) ok = mbar_wait(&bar->rows_ready, 0, p.status, 51);
        if (!ok) break;
        if (use > 0) ok = mbar_wait(&bar->kv_empty[st], (use - 1) & 1, p.status, 50);
        if (!ok) break;
        mbar_expect_tx(&bar->k_full[st], kColTileBytes);
        mbar_expect_tx(&bar->v_full[st], kColTileBytes);
        for (int s = 0; s < kSlabs; ++s) {
          tma_load_3d(k_smem + st * kColTileBytes + s * kColTile * 128, &map_k64,
                      p.k_col0 + kv_head * D + s * 64, j * kColTile, batch, &bar->k_full[st]);
          tma_load_3d(v_smem + st * kColTileBytes + s * kColTile * 128, &map_v64,
                      p.v_col0 + kv_head * D + s * 64, j * kColTile, batch, &bar->v_full[st]);
        }
      }
      for (int j = max(0, n_steps - kBwdStages); j < n_steps; ++j) {
        mbar_wait(&bar->k_full[j % kBwdStages], (j / kBwdStages) & 1, p.status, 52);
        mbar_wait(&bar->v_full[j % kBwdStages], (j / kBwdStages) & 1, p.status, 53);
      }
    }
  } else if (warp == 1) {
    {
      // The whole warp walks the schedule (uniform control flow); one elected lane issues.
      bool ok = __all_sync(0xffffffffu, mbar_wait(&bar->rows_ready, 0, p.status, 54));
      auto issue_scores = [&](int j) -> bool {   // S(j) = Q K_j^T, dP(j) = dO V_j^T into buffer j & 1
        const int st = j % kBwdStages;
        if (!__all_sync(0xffffffffu,
                        mbar_wait(&bar->k_full[st], (j / kBwdStages) & 1, p.status, 55) &&
                            mbar_wait(&bar->v_full[st], (j / kBwdStages) & 1, p.status, 56)))
          return false;
        tc_fence_after();
        if (elect_one()) {
          const uint64_t k_desc = umma_desc_sw128(smem_u32(k_smem + st * kColTileBytes), 16, 1024);
          const uint64_t v_desc = umma_desc_sw128(smem_u32(v_smem + st * kColTileBytes), 16, 1024);
          const uint32_t buf = tmem + kFirstBuf + (j & 1) * kBuf;
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {   // 16 channels = 8 TMEM columns of the A operand
            const uint32_t b_off = ((ks / 4) * kColTile * 128 + (ks % 4) * 32) >> 4;
            umma_ts(buf + kColS, tmem + kColQ + ks * 8, k_desc + b_off, kIdescS, ks > 0);
          }
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t b_off = ((ks / 4) * kColTile * 128 + (ks % 4) * 32) >> 4;
            umma_ts(buf + kColDP, tmem + kColDO + ks * 8, v_desc + b_off, kIdescS, ks > 0);
          }
          tc_commit(&bar->s_full[j & 1]);
        }
        __syncwarp();
        return true;
      };
      if (ok && n_steps > 0) ok = issue_scores(0);
      for (int j = 0; j < n_steps && ok; ++j) {
        const int st = j % kBwdStages;
        // buffer (j+1) & 1 was last read by the dQ instructions of step j-1, issued before these
        if (kPipe && j + 1 < n_steps) ok = issue_scores(j + 1);
        if (!ok) break;
        ok = __all_sync(0xffffffffu, mbar_wait(&bar->ds_full[j & 1], (j >> 1) & 1, p.status, 57));
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
          const uint64_t k_mn = umma_desc_sw128(smem_u32(k_smem + st * kColTileBytes), kColTile * 128, 1024);
#pragma unroll
          for (int ks = 0; ks < kColTile / 16; ++ks)   // dQ += dS K: 16 keys per step, K MN-major
            umma_ts(tmem + kColDQ, tmem + kFirstBuf + (j & 1) * kBuf + kColS + (ks >> 1) * 32 + (ks & 1) * 8,
                    k_mn + ks * (2048 >> 4), kIdescDQ, j > 0 || ks > 0);
          tc_commit(&bar->kv_empty[st]);
        }
        __syncwarp();
        if (!kPipe && j + 1 < n_steps) ok = issue_scores(j + 1);
      }
      if (ok && elect_one()) tc_commit(&bar->dq_done);
      __syncwarp();
    }
  } else if (warp >= 2) {
    // Row threads: TMEM lane quarter = warp % 4; warps 2..5 are group 0, warps 6..9 group 1.
    const int group = (warp - 2) >> 2, quarter = warp & 3, row = quarter * 32 + lane;
    const int query = q_tile * kRowTile + row;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const int stat_row = min(query, p.seq_pad - 1);
    const float* record = p.stats + ((static_cast<size_t>(batch) * p.heads + head) * p.seq_pad +
                                     (stat_row & ~1)) * 2 + (stat_row & 1);
    const float shift = record[0], delta = record[2];
    // dS here is P (dP - delta) without the softmax scale: dQ is scaled once when it is written.
    const uint64_t scale2 = f2_pack(p.scale_log2, p.scale_log2);
    const uint64_t shift2 = f2_pack(shift, shift), delta2 = f2_pack(delta, delta);
    {
      // group 0 brings the Q rows into TMEM, group 1 the dO rows: one row of D bf16 per thread
      uint32_t w[32];
      mbar_wait(&bar->qdo_full, 0, p.status, 53);
      load_swizzled_row(smem_u32(group == 0 ? k_smem : v_smem) + 2 * kColTileBytes, row, w);
      tmem_st32(tmem + lane_base + (group == 0 ? kColQ : kColDO), w);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->rows_ready);
    }
    bool ok = true;
    for (int j = 0; j < n_steps && ok; ++j) {
      const uint32_t buf = tmem + kFirstBuf + (j & 1) * kBuf + lane_base + group * 32;
      ok = mbar_wait(&bar->s_full[j & 1], (j >> 1) & 1, p.status, 58);
      if (!ok) break;
      tc_fence_after();
      const bool masked = (j + 1) * kColTile - 1 > q_tile * kRowTile;  // tile may cross the diagonal
      const int key0 = j * kColTile + group * 32;
      uint32_t s[32], dp[32], packed[16];
#ifdef BWD_EXP_NOROW
      if (lane == 0) mbar_arrive(&bar->ds_full[j & 1]);
      continue;
#endif
      tmem_ld32(buf + kColS, s);
      tmem_ld32(buf + kColDP, dp);
      tmem_wait_ld();
      auto build = [&](auto masked_tag) {
#ifdef BWD_EXP_NOMATH
        for (int i = 0; i < 16; ++i) packed[i] = s[2 * i] ^ dp[2 * i + 1];
        return;
#endif
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0, p1, d0, d1;
          f2_unpack(f2_fma(f2_pack(__uint_as_float(s[i]), __uint_as_float(s[i + 1])), scale2, shift2), p0, p1);
          p0 = fast_exp2(p0);
          p1 = fast_exp2(p1);
          if (decltype(masked_tag)::value) {
            if (key0 + i > query) p0 = 0.0f;
            if (key0 + i + 1 > query) p1 = 0.0f;
          }
          const uint64_t t2 = f2_sub(f2_pack(__uint_as_float(dp[i]), __uint_as_float(dp[i + 1])), delta2);
          f2_unpack(f2_mul(f2_pack(p0, p1), t2), d0, d1);
          packed[i / 2] = pack_bf16(d0, d1);
        }
      };
      if (masked) build(std::true_type{});
      else build(std::false_type{});
      tmem_st16(buf + kColS, packed);   // over the first half of this group's own S columns
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->ds_full[j & 1]);
    }
    if (ok) ok = mbar_wait(&bar->dq_done, 0, p.status, 59);
    // dQ leaves through the K and V rings, which lie one behind the other (every key tile has been
    // consumed by now): [128 rows x D] fp32
    static_assert(2 * kBwdStages * kColTileBytes >= kRowTile * (D * 4 + kStagePad), "staging tile");
    if (ok) {
      tc_fence_after();
#pragma unroll
      for (int c = group; c < D / 32; c += kRowGroups) {
        uint32_t o[32];
        tmem_ld32(tmem + lane_base + kColDQ + c * 32, o);
        tmem_wait_ld();
        stage_columns(smem_u32(k_smem) + row * (D * 4 + kStagePad) + c * 128, o, p.scale);
      }
    }
    fence_proxy_async();
    named_barrier_sync(1, 128 * kRowGroups);   // every row thread gets here, whatever `ok` says
    if (ok && group == 0 && query < p.seq) {
      bulk_store(p.dq + (static_cast<size_t>(batch) * p.seq + query) * p.dq_token + head * D,
                 k_smem + row * (D * 4 + kStagePad), D * 4);
      bulk_store_commit();
      bulk_store_wait_read();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// dQ for head width 128 in steps of 128 keys.
//
// An MMA of 64 columns takes as long as one of 128 on this tensor pipe, so the passes for head
// width 128 consume 128 opposite-side rows per step.  All 512 TMEM columns are then in use (Q and
// dO as A operands 64 + 64, S 128, dP 128, dQ 128) and nothing is double-buffered; the pipe is
// kept busy by the order of work instead:
//   row threads, step j    phase 1: S(j) -> registers, release the S columns, P = exp2(...)
//                          phase 2: dP(j) -> registers, dS = P (dP - delta) over the dP columns
//   tensor pipe            dQ(j) after phase 2 of step j, then dP(j+1), then S(j+2)
// so that phase 1 of step j+1 runs beside dQ(j) and dP(j+1), and S(j+2) beside phase 2.
// Sixteen row warps: group g (warps 2+4g .. 5+4g) takes key columns [32 g, 32 g + 32) of a step.
// ---------------------------------------------------------------------------------------------
constexpr int kWideGroups = 4;
constexpr int kWideThreads = 64 + 128 * kWideGroups;
constexpr int kWideKStages = 4, kWideVStages = 3;
constexpr int kWideTileBytes = 2 * kRowTile * 128;   // [128 x 128] bf16, two 64-channel slabs

struct DqWideBarriers {
  uint64_t qdo_full, rows_ready, k_full[kWideKStages], k_empty[kWideKStages], v_full[kWideVStages], v_empty[kWideVStages];
  uint64_t s_full, dp_full, s_free, stored, dq_done;
  uint32_t tmem_base;
};

__global__ void __launch_bounds__(kWideThreads, 1)
attn_bwd_dq128_sm100(const __grid_constant__ CUtensorMap map_k128,
                     const __grid_constant__ CUtensorMap map_v128,
                     const __grid_constant__ CUtensorMap map_q128,
                     const __grid_constant__ CUtensorMap map_do128, BwdParams p) {
  constexpr int D = 128;
  constexpr uint32_t kColQ = 0, kColDO = 64, kColS = 128, kColDP = 256, kColDQ = 384;
  constexpr uint32_t kIdescS = umma_idesc_bf16(kRowTile, kRowTile, false);
  constexpr uint32_t kIdescDQ = umma_idesc_bf16(kRowTile, D, true);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* k_smem = smem;
  uint8_t* v_smem = k_smem + kWideKStages * kWideTileBytes;
  DqWideBarriers* bar = reinterpret_cast<DqWideBarriers*>(v_smem + kWideVStages * kWideTileBytes);

  const int warp = uniform_warp_index(), lane = threadIdx.x % 32;
  const int q_tile = gridDim.y - 1 - blockIdx.y, head = blockIdx.x % p.heads, batch = blockIdx.x / p.heads;
  const int kv_head = head / p.group;
  const int n_steps = min(q_tile + 1, (p.seq + kRowTile - 1) / kRowTile);   // key tiles with a visible key

  if (threadIdx.x == 0) {
    mbar_init(&bar->qdo_full, 1);
    mbar_init(&bar->rows_ready, 4 * kWideGroups);
    for (int s = 0; s < kWideKStages; ++s) {
      mbar_init(&bar->k_full[s], 1);
      mbar_init(&bar->k_empty[s], 1);
    }
    for (int s = 0; s < kWideVStages; ++s) {
      mbar_init(&bar->v_full[s], 1);
      mbar_init(&bar->v_empty[s], 1);
    }
    mbar_init(&bar->s_full, 1);
    mbar_init(&bar->dp_full, 1);
    mbar_init(&bar->s_free, 4 * kWideGroups);
    mbar_init(&bar->stored, 4 * kWideGroups);
    mbar_init(&bar->dq_done, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&bar->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bar->tmem_base;
  pdl_wait();   // the prep kernel's records and bf16 gradient are read below
  pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&map_k128);
      tma_prefetch_desc(&map_v128);
      tma_prefetch_desc(&map_q128);
      tma_prefetch_desc(&map_do128);
      // The CTA's Q and dO rows pass through the last stage of the K and of the V ring on their way
      // into TMEM; those stages take key tiles only after the row threads have read them.
      mbar_expect_tx(&bar->qdo_full, 2 * kWideTileBytes);
      for (int s = 0; s < 2; ++s) {
        tma_load_3d(k_smem + (kWideKStages - 1) * kWideTileBytes + s * kRowTile * 128, &map_q128,
                    p.q_col0 + head * D + s * 64, q_tile * kRowTile, batch, &bar->qdo_full);
        tma_load_3d(v_smem + (kWideVStages - 1) * kWideTileBytes + s * kRowTile * 128, &map_do128,
                    head * D + s * 64, q_tile * kRowTile, batch, &bar->qdo_full);
      }
      bool ok = true;
      for (int j = 0; j < n_steps && ok; ++j) {
        const int ks = j % kWideKStages, vs = j % kWideVStages;
        if (j == kWideVStages - 1) ok = mbar_wait(&bar->rows_ready, 0, p.status, 69);
        if (!ok) break;
        if (j >= kWideKStages) ok = mbar_wait(&bar->k_empty[ks], (j / kWideKStages - 1) & 1, p.status, 70);
        if (!ok) break;
        mbar_expect_tx(&bar->k_full[ks], kWideTileBytes);
        for (int s = 0; s < 2; ++s)
          tma_load_3d(k_smem + ks * kWideTileBytes + s * kRowTile * 128, &map_k128,
                      p.k_col0 + kv_head * D + s * 64, j * kRowTile, batch, &bar->k_full[ks]);
        if (j >= kWideVStages) ok = mbar_wait(&bar->v_empty[vs], (j / kWideVStages - 1) & 1, p.status, 71);
        if (!ok) break;
        mbar_expect_tx(&bar->v_full[vs], kWideTileBytes);
        for (int s = 0; s < 2; ++s)
          tma_load_3d(v_smem + vs * kWideTileBytes + s * kRowTile * 128, &map_v128,
                      p.v_col0 + kv_head * D + s * 64, j * kRowTile, batch, &bar->v_full[vs]);
      }
      // no copy may still be in flight when the CTA leaves
      for (int j = max(0, n_steps - kWideKStages); j < n_steps; ++j)
        mbar_wait(&bar->k_full[j % kWideKStages], (j / kWideKStages) & 1, p.status, 72);
      for (int j = max(0, n_steps - kWideVStages); j < n_steps; ++j)
        mbar_wait(&bar->v_full[j % kWideVStages], (j / kWideVStages) & 1, p.status, 73);
    }
  } else if (warp == 1) {
    // The whole warp walks the schedule (uniform control flow); one elected lane issues.
    auto issue_s = [&](int j) -> bool {   // S(j) = Q K_j^T
      const int st = j % kWideKStages;
      if (!__all_sync(0xffffffffu, mbar_wait(&bar->k_full[st], (j / kWideKStages) & 1, p.status, 74))) return false;
      tc_fence_after();
      if (elect_one()) {
        const uint64_t k_desc = umma_desc_sw128(smem_u32(k_smem + st * kWideTileBytes), 16, 1024);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          umma_ts(tmem + kColS, tmem + kColQ + ks * 8,
                  k_desc + (((ks / 4) * kRowTile * 128 + (ks % 4) * 32) >> 4), kIdescS, ks > 0);
        tc_commit(&bar->s_full);
      }
      __syncwarp();
      return true;
    };
    auto issue_dp = [&](int j) -> bool {   // dP(j) = dO V_j^T
      const int st = j % kWideVStages;
      if (!__all_sync(0xffffffffu, mbar_wait(&bar->v_full[st], (j / kWideVStages) & 1, p.status, 75))) return false;
      tc_fence_after();
      if (elect_one()) {
        const uint64_t v_desc = umma_desc_sw128(smem_u32(v_smem + st * kWideTileBytes), 16, 1024);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          umma_ts(tmem + kColDP, tmem + kColDO + ks * 8,
                  v_desc + (((ks / 4) * kRowTile * 128 + (ks % 4) * 32) >> 4), kIdescS, ks > 0);
        tc_commit(&bar->dp_full);
        tc_commit(&bar->v_empty[st]);
      }
      __syncwarp();
      return true;
    };
    bool ok = __all_sync(0xffffffffu, mbar_wait(&bar->rows_ready, 0, p.status, 76));
    if (ok) ok = issue_s(0);
    if (ok) ok = issue_dp(0);
    if (ok && n_steps > 1) {
      ok = __all_sync(0xffffffffu, mbar_wait(&bar->s_free, 0, p.status, 77));
      if (ok) ok = issue_s(1);
    }
    for (int j = 0; j < n_steps && ok; ++j) {
      ok = __all_sync(0xffffffffu, mbar_wait(&bar->stored, j & 1, p.status, 78));
      if (!ok) break;
      tc_fence_after();
      if (elect_one()) {
        const int st = j % kWideKStages;
        const uint64_t k_mn = umma_desc_sw128(smem_u32(k_smem + st * kWideTileBytes), kRowTile * 128, 1024);
#pragma unroll
        for (int ks = 0; ks < kRowTile / 16; ++ks)   // dQ += dS K: 16 keys per instruction, K MN-major
          umma_ts(tmem + kColDQ, tmem + kColDP + (ks >> 1) * 32 + (ks & 1) * 8, k_mn + ks * (2048 >> 4),
                  kIdescDQ, j > 0 || ks > 0);
        tc_commit(&bar->k_empty[st]);
      }
      __syncwarp();
      if (j + 1 < n_steps) ok = issue_dp(j + 1);   // the pipe runs in order: dQ(j) has read dS(j) by then
      if (ok && j + 2 < n_steps) {
        ok = __all_sync(0xffffffffu, mbar_wait(&bar->s_free, (j + 1) & 1, p.status, 79));
        if (ok) ok = issue_s(j + 2);
      }
    }
    if (ok && elect_one()) tc_commit(&bar->dq_done);
    __syncwarp();
  } else {
    const int group = (warp - 2) >> 2, quarter = warp & 3, row = quarter * 32 + lane;
    const int query = q_tile * kRowTile + row;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const int stat_row = min(query, p.seq_pad - 1);
    const float* record = p.stats + ((static_cast<size_t>(batch) * p.heads + head) * p.seq_pad +
                                     (stat_row & ~1)) * 2 + (stat_row & 1);
    const float shift = record[0], delta = record[2];
    const uint64_t scale2 = f2_pack(p.scale_log2, p.scale_log2);
    const uint64_t shift2 = f2_pack(shift, shift), delta2 = f2_pack(delta, delta);
    {
      // groups 0, 1 bring the two 64-channel halves of the Q rows into TMEM, groups 2, 3 those of dO
      uint32_t w[32];
      mbar_wait(&bar->qdo_full, 0, p.status, 68);
      load_swizzled_row(smem_u32(group < 2 ? k_smem + (kWideKStages - 1) * kWideTileBytes
                                           : v_smem + (kWideVStages - 1) * kWideTileBytes) +
                            (group & 1) * kRowTile * 128, row, w);
      tmem_st32(tmem + lane_base + (group < 2 ? kColQ : kColDO) + (group & 1) * 32, w);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->rows_ready);
    }
    bool ok = true;
    for (int j = 0; j < n_steps && ok; ++j) {
      const uint32_t cols = tmem + lane_base + group * 32;
      const int key0 = j * kRowTile + group * 32;
      uint32_t s[32], dp[32], packed[16];
      ok = mbar_wait(&bar->s_full, j & 1, p.status, 80);
      if (!ok) break;
      tc_fence_after();
      tmem_ld32(cols + kColS, s);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->s_free);
      const bool masked = j == q_tile;   // the step on the diagonal
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        float p0, p1;
        f2_unpack(f2_fma(f2_pack(__uint_as_float(s[i]), __uint_as_float(s[i + 1])), scale2, shift2), p0, p1);
        p0 = fast_exp2(p0);
        p1 = fast_exp2(p1);
        if (masked) {
          if (key0 + i > query) p0 = 0.0f;
          if (key0 + i + 1 > query) p1 = 0.0f;
        }
        s[i] = __float_as_uint(p0);
        s[i + 1] = __float_as_uint(p1);
      }
      ok = mbar_wait(&bar->dp_full, j & 1, p.status, 81);
      if (!ok) break;
      tc_fence_after();
      tmem_ld32(cols + kColDP, dp);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        float d0, d1;
        const uint64_t t2 = f2_sub(f2_pack(__uint_as_float(dp[i]), __uint_as_float(dp[i + 1])), delta2);
        f2_unpack(f2_mul(f2_pack(__uint_as_float(s[i]), __uint_as_float(s[i + 1])), t2), d0, d1);
        packed[i / 2] = pack_bf16(d0, d1);
      }
      tmem_st16(cols + kColDP, packed);   // dS over the first half of this group's own dP columns
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->stored);
    }
    if (ok) ok = mbar_wait(&bar->dq_done, 0, p.status, 82);
    // dQ leaves through the K ring (every key tile has been consumed by now): [128 rows x 128] fp32
    if (ok) {
      tc_fence_after();
      uint32_t o[32];
      tmem_ld32(tmem + lane_base + kColDQ + group * 32, o);
      tmem_wait_ld();
      stage_columns(smem_u32(k_smem) + row * (D * 4 + kStagePad) + group * 128, o, p.scale);
    }
    fence_proxy_async();
    named_barrier_sync(1, 128 * kWideGroups);   // every row thread gets here, whatever `ok` says
    if (ok && group == 0 && query < p.seq) {
      bulk_store(p.dq + (static_cast<size_t>(batch) * p.seq + query) * p.dq_token + head * D,
                 k_smem + row * (D * 4 + kStagePad), D * 4);
      bulk_store_commit();
      bulk_store_wait_read();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

struct DkvBarriers {
  uint64_t kv_full, q_full[kBwdStages], q_empty[kBwdStages];
  uint64_t s_full[2], ds_full[2], done;
  uint32_t tmem_base;
};

// ---------------------------------------------------------------------------------------------
// dK, dV: grid (key tiles of 128, heads, batch)
// ---------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(kBwdThreads, D == 64 ? 2 : 1)
attn_bwd_dkv_sm100(const __grid_constant__ CUtensorMap map_k128,
                   const __grid_constant__ CUtensorMap map_v128,
                   const __grid_constant__ CUtensorMap map_q64,
                   const __grid_constant__ CUtensorMap map_do64, BwdParams p) {
  constexpr int kSlabs = D / 64;
  constexpr int kRowTileBytes = kSlabs * kRowTile * 128;
  constexpr int kColTileBytes = kSlabs * kColTile * 128;
  constexpr int kStatsBytes = kColTile * 8;
  constexpr int kStageBytes = 2 * kColTileBytes + 1024;   // Q_i, dO_i, stats (tiles stay 1024-byte aligned)
  static_assert(D == 64, "the staging below fits head width 64; head width 128 has its own pass");
  constexpr int kStageTile = kRowTile * (D * 4 + kStagePad);   // one staged output tile
  static_assert(kBwdStages * kStageBytes >= 2 * kStageTile, "the output tiles are staged in the ring");
  // as in the dQ kernel: two (S^T, dP^T) buffers for head width 128 (256 + 2 D = 512 columns),
  // one buffer and 256 columns for head width 64
  constexpr bool kPipe = D == 128;
  constexpr uint32_t kTmemCols = kPipe ? 512 : 256;
  constexpr uint32_t kColS = 0, kColDP = 64, kBuf = kPipe ? 128 : 0;
  constexpr uint32_t kColDV = kPipe ? 256 : 128, kColDK = kColDV + D;
  constexpr uint32_t kIdescS = umma_idesc_bf16(kRowTile, kColTile, false);
  constexpr uint32_t kIdescAcc = umma_idesc_bf16(kRowTile, D, true);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* k_smem = smem;
  uint8_t* v_smem = k_smem + kRowTileBytes;
  uint8_t* stage_smem = v_smem + kRowTileBytes;   // per stage: Q_i | dO_i | stats
  DkvBarriers* bar = reinterpret_cast<DkvBarriers*>(stage_smem + kBwdStages * kStageBytes);

  const int warp = uniform_warp_index(), lane = threadIdx.x % 32;
  // key tile 0 is seen by every query tile: the lowest tile index is the longest, and it starts first
  const int kv_heads = p.heads / p.group;
  const int k_tile = blockIdx.y, kv_head = blockIdx.x % kv_heads, batch = blockIdx.x / kv_heads;
  const int col_tiles = (p.seq + kColTile - 1) / kColTile;
  const int first = 2 * k_tile;                    // first query tile that can see these keys
  const int per_head = max(0, col_tiles - first);  // steps per query head of the group
  const int n_steps = per_head * p.group;          // heads of the group one after the other

  if (threadIdx.x == 0) {
    mbar_init(&bar->kv_full, 1);
    for (int s = 0; s < kBwdStages; ++s) {
      mbar_init(&bar->q_full[s], 1);
      mbar_init(&bar->q_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bar->s_full[s], 1);
      mbar_init(&bar->ds_full[s], 4 * kRowGroups);   // one arrival per row warp
    }
    mbar_init(&bar->done, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&bar->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bar->tmem_base;
  const float* stats_group =
      p.stats + (static_cast<size_t>(batch) * p.heads + kv_head * p.group) * p.seq_pad * 2;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&map_k128);
      tma_prefetch_desc(&map_v128);
      tma_prefetch_desc(&map_q64);
      tma_prefetch_desc(&map_do64);
      mbar_expect_tx(&bar->kv_full, 2 * kRowTileBytes);
      for (int s = 0; s < kSlabs; ++s) {
        tma_load_3d(k_smem + s * kRowTile * 128, &map_k128, p.k_col0 + kv_head * D + s * 64,
                    k_tile * kRowTile, batch, &bar->kv_full);
        tma_load_3d(v_smem + s * kRowTile * 128, &map_v128, p.v_col0 + kv_head * D + s * 64,
                    k_tile * kRowTile, batch, &bar->kv_full);
      }
      bool ok = true;
      for (int i = 0; i < n_steps && ok; ++i) {
        const int st = i % kBwdStages, use = i / kBwdStages;
        const int in_group = i / per_head, tile = first + i % per_head;
        const int head = kv_head * p.group + in_group;
        if (use > 0) ok = mbar_wait(&bar->q_empty[st], (use - 1) & 1, p.status, 60);
        if (!ok) break;
        uint8_t* dst = stage_smem + st * kStageBytes;
        mbar_expect_tx(&bar->q_full[st], 2 * kColTileBytes + kStatsBytes);
        for (int s = 0; s < kSlabs; ++s) {
          tma_load_3d(dst + s * kColTile * 128, &map_q64, p.q_col0 + head * D + s * 64,
                      tile * kColTile, batch, &bar->q_full[st]);
          tma_load_3d(dst + kColTileBytes + s * kColTile * 128, &map_do64, head * D + s * 64,
                      tile * kColTile, batch, &bar->q_full[st]);
        }
        bulk_load(dst + 2 * kColTileBytes,
                  stats_group + (static_cast<size_t>(in_group) * p.seq_pad + tile * kColTile) * 2,
                  kStatsBytes, &bar->q_full[st]);
      }
      mbar_wait(&bar->kv_full, 0, p.status, 61);
      for (int i = max(0, n_steps - kBwdStages); i < n_steps; ++i)
        mbar_wait(&bar->q_full[i % kBwdStages], (i / kBwdStages) & 1, p.status, 62);
    }
  } else if (warp == 1) {
    {
      bool ok = __all_sync(0xffffffffu, mbar_wait(&bar->kv_full, 0, p.status, 63));
      const uint64_t k_desc = umma_desc_sw128(smem_u32(k_smem), 16, 1024);
      const uint64_t v_desc = umma_desc_sw128(smem_u32(v_smem), 16, 1024);
      auto issue_scores = [&](int i) -> bool {   // S^T = K Q_i^T, dP^T = V dO_i^T into buffer i & 1
        const int st = i % kBwdStages;
        if (!__all_sync(0xffffffffu, mbar_wait(&bar->q_full[st], (i / kBwdStages) & 1, p.status, 64)))
          return false;
        tc_fence_after();
        if (elect_one()) {
          const uint32_t q_addr = smem_u32(stage_smem + st * kStageBytes);
          const uint64_t q_desc = umma_desc_sw128(q_addr, 16, 1024);
          const uint64_t do_desc = umma_desc_sw128(q_addr + kColTileBytes, 16, 1024);
          const uint32_t buf = tmem + (i & 1) * kBuf;
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t a_off = ((ks / 4) * kRowTile * 128 + (ks % 4) * 32) >> 4;
            const uint32_t b_off = ((ks / 4) * kColTile * 128 + (ks % 4) * 32) >> 4;
            umma_ss(buf + kColS, k_desc + a_off, q_desc + b_off, kIdescS, ks > 0);
          }
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t a_off = ((ks / 4) * kRowTile * 128 + (ks % 4) * 32) >> 4;
            const uint32_t b_off = ((ks / 4) * kColTile * 128 + (ks % 4) * 32) >> 4;
            umma_ss(buf + kColDP, v_desc + a_off, do_desc + b_off, kIdescS, ks > 0);
          }
          tc_commit(&bar->s_full[i & 1]);
        }
        __syncwarp();
        return true;
      };
      if (ok && n_steps > 0) ok = issue_scores(0);
      for (int i = 0; i < n_steps && ok; ++i) {
        const int st = i % kBwdStages;
        if (kPipe && i + 1 < n_steps) ok = issue_scores(i + 1);
        if (!ok) break;
        ok = __all_sync(0xffffffffu, mbar_wait(&bar->ds_full[i & 1], (i >> 1) & 1, p.status, 65));
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
          const uint32_t q_addr = smem_u32(stage_smem + st * kStageBytes);
          const uint64_t do_mn = umma_desc_sw128(q_addr + kColTileBytes, kColTile * 128, 1024);
          const uint64_t q_mn = umma_desc_sw128(q_addr, kColTile * 128, 1024);
          const uint32_t buf = tmem + (i & 1) * kBuf;
#pragma unroll
          for (int ks = 0; ks < kColTile / 16; ++ks) {   // 16 queries per step, operands MN-major
            const uint32_t col = (ks >> 1) * 32 + (ks & 1) * 8;   // where the row group left these 16 queries
            umma_ts(tmem + kColDV, buf + kColS + col, do_mn + ks * (2048 >> 4), kIdescAcc, i > 0 || ks > 0);
            umma_ts(tmem + kColDK, buf + kColDP + col, q_mn + ks * (2048 >> 4), kIdescAcc, i > 0 || ks > 0);
          }
          tc_commit(&bar->q_empty[st]);
        }
        __syncwarp();
        if (!kPipe && i + 1 < n_steps) ok = issue_scores(i + 1);
      }
      if (ok && elect_one()) tc_commit(&bar->done);
      __syncwarp();
    }
  } else if (warp >= 2) {
    const int group = (warp - 2) >> 2, quarter = warp & 3, row = quarter * 32 + lane;
    const int key = k_tile * kRowTile + row;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint64_t scale2 = f2_pack(p.scale_log2, p.scale_log2);
    bool ok = true;
    for (int i = 0; i < n_steps && ok; ++i) {
      const int st = i % kBwdStages, tile = first + i % per_head;
      const uint32_t buf = tmem + (i & 1) * kBuf + lane_base + group * 32;
      ok = mbar_wait(&bar->s_full[i & 1], (i >> 1) & 1, p.status, 66) &&
           mbar_wait(&bar->q_full[st], (i / kBwdStages) & 1, p.status, 68);  // stats landed (acquire)
      if (!ok) break;
      tc_fence_after();
      const uint32_t pair_stats = smem_u32(stage_smem + st * kStageBytes + 2 * kColTileBytes) + group * 256;
      const bool masked = tile * kColTile < k_tile * kRowTile + kRowTile;  // some query may precede a key
      const int query0 = tile * kColTile + group * 32;
      uint32_t s[32], dp[32], pp[16], dsp[16];
#ifdef BWD_EXP_NOROW
      if (lane == 0) mbar_arrive(&bar->ds_full[i & 1]);
      continue;
#endif
      tmem_ld32(buf + kColS, s);
      tmem_ld32(buf + kColDP, dp);
      tmem_wait_ld();
      // dS^T here is P^T (dP^T - delta) without the softmax scale: dK is scaled once when it is written.
      auto build = [&](auto masked_tag) {
#ifdef BWD_EXP_NOMATH
        for (int c = 0; c < 16; ++c) { pp[c] = s[2 * c] ^ dp[2 * c + 1]; dsp[c] = s[2 * c + 1] ^ dp[2 * c]; }
        return;
#endif
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          const float4 q4 = lds_f32x4(pair_stats + c * 8);   // same address for the whole warp
          float p0, p1, d0, d1;
          f2_unpack(f2_fma(f2_pack(__uint_as_float(s[c]), __uint_as_float(s[c + 1])), scale2,
                           f2_pack(q4.x, q4.y)), p0, p1);
          p0 = fast_exp2(p0);
          p1 = fast_exp2(p1);
          if (decltype(masked_tag)::value) {
            if (query0 + c < key) p0 = 0.0f;
            if (query0 + c + 1 < key) p1 = 0.0f;
          }
          const uint64_t t2 = f2_sub(f2_pack(__uint_as_float(dp[c]), __uint_as_float(dp[c + 1])),
                                     f2_pack(q4.z, q4.w));
          f2_unpack(f2_mul(f2_pack(p0, p1), t2), d0, d1);
          pp[c / 2] = pack_bf16(p0, p1);
          dsp[c / 2] = pack_bf16(d0, d1);
        }
      };
      if (masked) build(std::true_type{});
      else build(std::false_type{});
      // P^T and dS^T over the first half of this group's own S^T and dP^T columns
      tmem_st16(buf + kColS, pp);
      tmem_st16(buf + kColDP, dsp);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->ds_full[i & 1]);
    }
    if (ok && n_steps > 0) ok = mbar_wait(&bar->done, 0, p.status, 67);
    // dV and dK leave through the stage ring (every stage has been consumed by now): two
    // [128 rows x D] fp32 tiles
    if (ok) {
      tc_fence_after();
#pragma unroll
      for (int idx = group; idx < 2 * (D / 32); idx += kRowGroups) {
        const int which = idx / (D / 32), c = idx % (D / 32);   // 0: dV, 1: dK
        uint32_t o[32];
        if (n_steps > 0) {
          tmem_ld32(tmem + lane_base + (which == 0 ? kColDV : kColDK) + c * 32, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        stage_columns(smem_u32(stage_smem) + which * kStageTile + row * (D * 4 + kStagePad) + c * 128, o,
                      which == 0 ? 1.0f : p.scale);
      }
    }
    fence_proxy_async();
    named_barrier_sync(1, 128 * kRowGroups);   // every row thread gets here, whatever `ok` says
    if (ok && key < p.seq && group < 2) {   // group 0 sends the dV rows, group 1 the dK rows
      const size_t dst = (static_cast<size_t>(batch) * p.seq + key) * p.dkv_token + kv_head * D;
      bulk_store((group == 0 ? p.dv : p.dk) + dst, stage_smem + group * kStageTile + row * (D * 4 + kStagePad),
                 D * 4);
      bulk_store_commit();
      bulk_store_wait_read();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// dK, dV for head width 128 in steps of 128 queries: grid (key tiles of 128, kv heads, batch).
//
// With 64-query steps the S^T and dP^T instructions re-read their 128-row A operand (the K or V
// tile, 4 KB per instruction) from shared memory for 64 columns of output, and shared-memory
// bandwidth held them to two thirds of the tensor pipe's rate; 128 columns per instruction halve
// that traffic.  All 512 TMEM columns are in use (S^T 128, dP^T 128, dV 128, dK 128) with no
// second buffer, so, as in the wide dQ pass, the order of work keeps the pipe busy:
//   row threads, step i    phase 1: S^T(i) -> registers, release its columns, P^T = exp2(...)
//                          phase 2: dP^T(i) -> registers; dS^T and P^T (bf16) over the dP^T columns
//   tensor pipe            dV(i), dK(i) after phase 2 of step i, then dP^T(i+1), then S^T(i+2)
// Group g of the sixteen row warps takes query columns [32 g, 32 g + 32) of a step and leaves
// dS^T in the first 16 and P^T in the last 16 of its own dP^T columns.
// Shared memory is used to the last kilobyte (K, V, three Q stages, two dO stages, the row
// statistics: the shifts travel with the Q stages because phase 1 needs them early, the deltas
// with the dO stages), so there is no slack for aligning the base: a base off the 1024-byte
// boundary is reported through the status word and the CTA returns.
// ---------------------------------------------------------------------------------------------
constexpr int kWideQStages = 3, kWideDoStages = 2;
constexpr int kWideStatBytes = kRowTile * 4;   // one float per query of a step

struct DkvWideBarriers {
  uint64_t kv_full, q_full[kWideQStages], q_empty[kWideQStages], do_full[kWideDoStages], do_empty[kWideDoStages];
  uint64_t s_full, dp_full, s_free, stored, done;
  uint32_t tmem_base;
};
constexpr int kDkvWideSmem = (2 + kWideQStages + kWideDoStages) * kWideTileBytes +
                             (kWideQStages + kWideDoStages) * kWideStatBytes + 256;
static_assert(sizeof(DkvWideBarriers) <= 256, "barrier block");
static_assert(kDkvWideSmem <= 232448, "dynamic shared memory of one CTA");

__global__ void __launch_bounds__(kWideThreads, 1)
attn_bwd_dkv128_sm100(const __grid_constant__ CUtensorMap map_k128,
                      const __grid_constant__ CUtensorMap map_v128,
                      const __grid_constant__ CUtensorMap map_q128,
                      const __grid_constant__ CUtensorMap map_do128, BwdParams p) {
  constexpr int D = 128;
  constexpr uint32_t kColS = 0, kColDP = 128, kColDV = 256, kColDK = 384;
  constexpr uint32_t kIdescS = umma_idesc_bf16(kRowTile, kRowTile, false);
  constexpr uint32_t kIdescAcc = umma_idesc_bf16(kRowTile, D, true);

  extern __shared__ uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {   // uniform over the CTA: nothing has been set up yet
    if (threadIdx.x == 0) report_status(p.status, 83, kBadSmemBase);
    return;
  }
  uint8_t* k_smem = smem;
  uint8_t* v_smem = k_smem + kWideTileBytes;
  uint8_t* q_ring = v_smem + kWideTileBytes;
  uint8_t* do_ring = q_ring + kWideQStages * kWideTileBytes;
  uint8_t* shift_ring = do_ring + kWideDoStages * kWideTileBytes;
  uint8_t* delta_ring = shift_ring + kWideQStages * kWideStatBytes;
  DkvWideBarriers* bar = reinterpret_cast<DkvWideBarriers*>(delta_ring + kWideDoStages * kWideStatBytes);

  const int warp = uniform_warp_index(), lane = threadIdx.x % 32;
  const int kv_heads = p.heads / p.group;
  const int k_tile = blockIdx.y, kv_head = blockIdx.x % kv_heads, batch = blockIdx.x / kv_heads;
  const int tiles = (p.seq + kRowTile - 1) / kRowTile;
  const int per_head = tiles - k_tile;        // query tiles that can see these keys
  const int n_steps = per_head * p.group;     // heads of the group one after the other

  if (threadIdx.x == 0) {
    mbar_init(&bar->kv_full, 1);
    for (int s = 0; s < kWideQStages; ++s) {
      mbar_init(&bar->q_full[s], 1);
      mbar_init(&bar->q_empty[s], 1);
    }
    for (int s = 0; s < kWideDoStages; ++s) {
      mbar_init(&bar->do_full[s], 1);
      mbar_init(&bar->do_empty[s], 1);
    }
    mbar_init(&bar->s_full, 1);
    mbar_init(&bar->dp_full, 1);
    mbar_init(&bar->s_free, 4 * kWideGroups);
    mbar_init(&bar->stored, 4 * kWideGroups);
    mbar_init(&bar->done, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&bar->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bar->tmem_base;
  const size_t stat_group = (static_cast<size_t>(batch) * p.heads + kv_head * p.group) * p.seq_pad;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&map_k128);
      tma_prefetch_desc(&map_v128);
      tma_prefetch_desc(&map_q128);
      tma_prefetch_desc(&map_do128);
      mbar_expect_tx(&bar->kv_full, 2 * kWideTileBytes);
      for (int s = 0; s < 2; ++s) {
        tma_load_3d(k_smem + s * kRowTile * 128, &map_k128, p.k_col0 + kv_head * D + s * 64,
                    k_tile * kRowTile, batch, &bar->kv_full);
        tma_load_3d(v_smem + s * kRowTile * 128, &map_v128, p.v_col0 + kv_head * D + s * 64,
                    k_tile * kRowTile, batch, &bar->kv_full);
      }
      // The two rings advance independently: each copy starts as soon as its own stage is free.
      // (Pulling tiles into L2 two steps ahead was measured without effect.)
      bool ok = true;
      int qi = 0, di = 0;
      uint32_t spins = 0;
      const uint64_t start = global_timer_ns();
      while ((qi < n_steps || di < n_steps) && ok) {
        bool progress = false;
        if (qi < n_steps && (qi < kWideQStages ||
                             mbar_poll(&bar->q_empty[qi % kWideQStages], (qi / kWideQStages - 1) & 1))) {
          const int qs = qi % kWideQStages, in_group = qi / per_head, tile = k_tile + qi % per_head;
          const int head = kv_head * p.group + in_group;
          mbar_expect_tx(&bar->q_full[qs], kWideTileBytes + kWideStatBytes);
          for (int s = 0; s < 2; ++s)
            tma_load_3d(q_ring + qs * kWideTileBytes + s * kRowTile * 128, &map_q128,
                        p.q_col0 + head * D + s * 64, tile * kRowTile, batch, &bar->q_full[qs]);
          bulk_load(shift_ring + qs * kWideStatBytes,
                    p.shifts + stat_group + static_cast<size_t>(in_group) * p.seq_pad + tile * kRowTile,
                    kWideStatBytes, &bar->q_full[qs]);
          ++qi;
          progress = true;
        }
        if (di < n_steps && (di < kWideDoStages ||
                             mbar_poll(&bar->do_empty[di % kWideDoStages], (di / kWideDoStages - 1) & 1))) {
          const int ds = di % kWideDoStages, in_group = di / per_head, tile = k_tile + di % per_head;
          const int head = kv_head * p.group + in_group;
          mbar_expect_tx(&bar->do_full[ds], kWideTileBytes + kWideStatBytes);
          for (int s = 0; s < 2; ++s)
            tma_load_3d(do_ring + ds * kWideTileBytes + s * kRowTile * 128, &map_do128, head * D + s * 64,
                        tile * kRowTile, batch, &bar->do_full[ds]);
          bulk_load(delta_ring + ds * kWideStatBytes,
                    p.deltas_pad + stat_group + static_cast<size_t>(in_group) * p.seq_pad + tile * kRowTile,
                    kWideStatBytes, &bar->do_full[ds]);
          ++di;
          progress = true;
        }
        if (!progress && (++spins & 0x3ffu) == 0) {   // bounded like every other wait
          if (*reinterpret_cast<volatile uint32_t*>(p.status) != 0) ok = false;
          else if (global_timer_ns() - start > kWaitLimitNs) {
            report_status(p.status, 84, kWaitTimeout);
            ok = false;
          }
        }
      }
      // no copy may still be in flight when the CTA leaves
      mbar_wait(&bar->kv_full, 0, p.status, 86);
      for (int i = max(0, n_steps - kWideQStages); i < n_steps; ++i)
        mbar_wait(&bar->q_full[i % kWideQStages], (i / kWideQStages) & 1, p.status, 87);
      for (int i = max(0, n_steps - kWideDoStages); i < n_steps; ++i)
        mbar_wait(&bar->do_full[i % kWideDoStages], (i / kWideDoStages) & 1, p.status, 88);
    }
  } else if (warp == 1) {
    const uint64_t k_desc = umma_desc_sw128(smem_u32(k_smem), 16, 1024);
    const uint64_t v_desc = umma_desc_sw128(smem_u32(v_smem), 16, 1024);
    auto issue_s = [&](int i) -> bool {   // S^T(i) = K Q_i^T
      const int st = i % kWideQStages;
      if (!__all_sync(0xffffffffu, mbar_wait(&bar->q_full[st], (i / kWideQStages) & 1, p.status, 89))) return false;
      tc_fence_after();
      if (elect_one()) {
        const uint64_t q_desc = umma_desc_sw128(smem_u32(q_ring + st * kWideTileBytes), 16, 1024);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = ((ks / 4) * kRowTile * 128 + (ks % 4) * 32) >> 4;
          umma_ss(tmem + kColS, k_desc + off, q_desc + off, kIdescS, ks > 0);
        }
        tc_commit(&bar->s_full);
      }
      __syncwarp();
      return true;
    };
    auto issue_dp = [&](int i) -> bool {   // dP^T(i) = V dO_i^T
      const int st = i % kWideDoStages;
      if (!__all_sync(0xffffffffu, mbar_wait(&bar->do_full[st], (i / kWideDoStages) & 1, p.status, 90))) return false;
      tc_fence_after();
      if (elect_one()) {
        const uint64_t do_desc = umma_desc_sw128(smem_u32(do_ring + st * kWideTileBytes), 16, 1024);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = ((ks / 4) * kRowTile * 128 + (ks % 4) * 32) >> 4;
          umma_ss(tmem + kColDP, v_desc + off, do_desc + off, kIdescS, ks > 0);
        }
        tc_commit(&bar->dp_full);
      }
      __syncwarp();
      return true;
    };
    bool ok = __all_sync(0xffffffffu, mbar_wait(&bar->kv_full, 0, p.status, 91));
    if (ok && n_steps > 0) ok = issue_s(0);
    if (ok && n_steps > 0) ok = issue_dp(0);
    if (ok && n_steps > 1) {
      ok = __all_sync(0xffffffffu, mbar_wait(&bar->s_free, 0, p.status, 92));
      if (ok) ok = issue_s(1);
    }
    for (int i = 0; i < n_steps && ok; ++i) {
      ok = __all_sync(0xffffffffu, mbar_wait(&bar->stored, i & 1, p.status, 93));
      if (!ok) break;
      tc_fence_after();
      if (elect_one()) {
        const uint64_t do_mn = umma_desc_sw128(smem_u32(do_ring + (i % kWideDoStages) * kWideTileBytes),
                                               kRowTile * 128, 1024);
        const uint64_t q_mn = umma_desc_sw128(smem_u32(q_ring + (i % kWideQStages) * kWideTileBytes),
                                              kRowTile * 128, 1024);
        // 16 queries per instruction, operands MN-major; dS^T starts at `col`, P^T 16 columns on.
        // dV goes first: the dO ring is the shorter one, and its stage is free after these.
#pragma unroll
        for (int ks = 0; ks < kRowTile / 16; ++ks) {
          const uint32_t col = tmem + kColDP + (ks >> 1) * 32 + (ks & 1) * 8;
          umma_ts(tmem + kColDV, col + 16, do_mn + ks * (2048 >> 4), kIdescAcc, i > 0 || ks > 0);
        }
        tc_commit(&bar->do_empty[i % kWideDoStages]);
#pragma unroll
        for (int ks = 0; ks < kRowTile / 16; ++ks) {
          const uint32_t col = tmem + kColDP + (ks >> 1) * 32 + (ks & 1) * 8;
          umma_ts(tmem + kColDK, col, q_mn + ks * (2048 >> 4), kIdescAcc, i > 0 || ks > 0);
        }
        tc_commit(&bar->q_empty[i % kWideQStages]);
      }
      __syncwarp();
      if (i + 1 < n_steps) ok = issue_dp(i + 1);   // the pipe runs in order: the products above have read by then
      if (ok && i + 2 < n_steps) {
        ok = __all_sync(0xffffffffu, mbar_wait(&bar->s_free, (i + 1) & 1, p.status, 94));
        if (ok) ok = issue_s(i + 2);
      }
    }
    if (ok && elect_one()) tc_commit(&bar->done);
    __syncwarp();
  } else {
    const int group = (warp - 2) >> 2, quarter = warp & 3, row = quarter * 32 + lane;
    const int key = k_tile * kRowTile + row;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t cols = tmem + lane_base + group * 32;
    const uint64_t scale2 = f2_pack(p.scale_log2, p.scale_log2);
    bool ok = true;
    for (int i = 0; i < n_steps && ok; ++i) {
      const int tile = k_tile + i % per_head;
      const int query0 = tile * kRowTile + group * 32;
      const bool masked = tile == k_tile;   // the step on the diagonal: a query may precede a key
      uint32_t s[32], pp[16];
      ok = mbar_wait(&bar->s_full, i & 1, p.status, 95) &&
           mbar_wait(&bar->q_full[i % kWideQStages], (i / kWideQStages) & 1, p.status, 96);   // shifts landed
      if (!ok) break;
      tc_fence_after();
      tmem_ld32(cols + kColS, s);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->s_free);
      const uint32_t shifts = smem_u32(shift_ring + (i % kWideQStages) * kWideStatBytes) + group * 128;
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        float p0, p1;
        f2_unpack(f2_fma(f2_pack(__uint_as_float(s[c]), __uint_as_float(s[c + 1])), scale2,
                         lds_b64(shifts + c * 4)), p0, p1);   // same address for the whole warp
        p0 = fast_exp2(p0);
        p1 = fast_exp2(p1);
        if (masked) {
          if (query0 + c < key) p0 = 0.0f;
          if (query0 + c + 1 < key) p1 = 0.0f;
        }
        s[c] = __float_as_uint(p0);
        s[c + 1] = __float_as_uint(p1);
        pp[c / 2] = pack_bf16(p0, p1);
      }
      ok = mbar_wait(&bar->dp_full, i & 1, p.status, 97) &&
           mbar_wait(&bar->do_full[i % kWideDoStages], (i / kWideDoStages) & 1, p.status, 98);   // deltas landed
      if (!ok) break;
      tc_fence_after();
      const uint32_t deltas = smem_u32(delta_ring + (i % kWideDoStages) * kWideStatBytes) + group * 128;
      // dS^T here is P^T (dP^T - delta) without the softmax scale: dK is scaled once when it is written.
      uint32_t dp_lo[16], dp_hi[16], ds_lo[8], ds_hi[8];
      tmem_ld16(cols + kColDP, dp_lo);
      tmem_ld16(cols + kColDP + 16, dp_hi);
      tmem_wait_ld();
#pragma unroll
      for (int c = 0; c < 16; c += 2) {
        float d0, d1;
        const uint64_t t2 = f2_sub(f2_pack(__uint_as_float(dp_lo[c]), __uint_as_float(dp_lo[c + 1])),
                                   lds_b64(deltas + c * 4));
        f2_unpack(f2_mul(f2_pack(__uint_as_float(s[c]), __uint_as_float(s[c + 1])), t2), d0, d1);
        ds_lo[c / 2] = pack_bf16(d0, d1);
      }
      tmem_st8(cols + kColDP, ds_lo);
#pragma unroll
      for (int c = 0; c < 16; c += 2) {
        float d0, d1;
        const uint64_t t2 = f2_sub(f2_pack(__uint_as_float(dp_hi[c]), __uint_as_float(dp_hi[c + 1])),
                                   lds_b64(deltas + (16 + c) * 4));
        f2_unpack(f2_mul(f2_pack(__uint_as_float(s[16 + c]), __uint_as_float(s[16 + c + 1])), t2), d0, d1);
        ds_hi[c / 2] = pack_bf16(d0, d1);
      }
      tmem_st8(cols + kColDP + 8, ds_hi);
      tmem_st16(cols + kColDP + 16, pp);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->stored);
    }
    if (ok && n_steps > 0) ok = mbar_wait(&bar->done, 0, p.status, 99);
    // dV and dK leave through the Q and dO rings, which lie one behind the other (every stage has
    // been consumed by now): two [128 rows x 128] fp32 tiles
    constexpr int kStageTile = kRowTile * (D * 4 + kStagePad);
    static_assert((kWideQStages + kWideDoStages) * kWideTileBytes >= 2 * kStageTile, "staging tiles");
    if (ok) {
      tc_fence_after();
#pragma unroll
      for (int which = 0; which < 2; ++which) {   // 0: dV, 1: dK
        uint32_t o[32];
        if (n_steps > 0) {
          tmem_ld32(tmem + lane_base + (which == 0 ? kColDV : kColDK) + group * 32, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        stage_columns(smem_u32(q_ring) + which * kStageTile + row * (D * 4 + kStagePad) + group * 128, o,
                      which == 0 ? 1.0f : p.scale);
      }
    }
    fence_proxy_async();
    named_barrier_sync(1, 128 * kWideGroups);   // every row thread gets here, whatever `ok` says
    if (ok && key < p.seq && group < 2) {   // group 0 sends the dV rows, group 1 the dK rows
      const size_t dst = (static_cast<size_t>(batch) * p.seq + key) * p.dkv_token + kv_head * D;
      bulk_store((group == 0 ? p.dv : p.dk) + dst, q_ring + group * kStageTile + row * (D * 4 + kStagePad), D * 4);
      bulk_store_commit();
      bulk_store_wait_read();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

struct BwdMaps {
  CUtensorMap q128, q64, k128, k64, v128, v64, do128, do64;
};

template <int D>
cudaError_t launch_bwd_tc(cudaStream_t stream, const BwdMaps& m, const BwdParams& p, int batch) {
  constexpr int kSlabs = D / 64;
  const size_t dq_smem = 1024 + 2 * kBwdStages * kSlabs * kColTile * 128 + sizeof(DqBarriers);
  const size_t dkv_smem = 1024 + 2 * kSlabs * kRowTile * 128 +
                          kBwdStages * (2 * kSlabs * kColTile * 128 + 1024) + sizeof(DkvBarriers);
  const size_t dq_wide_smem = 1024 + (kWideKStages + kWideVStages) * kWideTileBytes + sizeof(DqWideBarriers);
  cudaError_t e;
  if constexpr (D == 128)
    e = cudaFuncSetAttribute(attn_bwd_dq128_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(dq_wide_smem));
  else
    e = cudaFuncSetAttribute(attn_bwd_dq_sm100<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(dq_smem));
  if (e != cudaSuccess) return e;
  if constexpr (D == 128)
    e = cudaFuncSetAttribute(attn_bwd_dkv128_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize, kDkvWideSmem);
  else
    e = cudaFuncSetAttribute(attn_bwd_dkv_sm100<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(dkv_smem));
  if (e != cudaSuccess) return e;
  const int tiles = (p.seq + kRowTile - 1) / kRowTile;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t config = {};
  config.blockDim = dim3(kBwdThreads);
  config.stream = stream;
  config.attrs = &attribute;
  config.numAttrs = 1;
  config.gridDim = dim3(p.heads * batch, tiles);
  if constexpr (D == 128) {
    config.blockDim = dim3(kWideThreads);
    config.dynamicSmemBytes = dq_wide_smem;
    e = cudaLaunchKernelEx(&config, attn_bwd_dq128_sm100, m.k128, m.v128, m.q128, m.do128, p);
  } else {
    config.dynamicSmemBytes = dq_smem;
    e = cudaLaunchKernelEx(&config, attn_bwd_dq_sm100<D>, m.k64, m.v64, m.q128, m.do128, p);
  }
  if (e != cudaSuccess) return e;
  config.gridDim = dim3((p.heads / p.group) * batch, tiles);
  if constexpr (D == 128) {
    config.dynamicSmemBytes = kDkvWideSmem;
    return cudaLaunchKernelEx(&config, attn_bwd_dkv128_sm100, m.k128, m.v128, m.q128, m.do128, p);
  } else {
    config.blockDim = dim3(kBwdThreads);
    config.dynamicSmemBytes = dkv_smem;
    return cudaLaunchKernelEx(&config, attn_bwd_dkv_sm100<D>, m.k128, m.v128, m.q64, m.do64, p);
  }
}

}  // namespace

size_t attn_bwd_tc_workspace_bytes(int batch, int seq, int heads, int head_dim) {
  const size_t seq_pad = (static_cast<size_t>(seq) + kColTile - 1) / kColTile * kColTile + kColTile;
  const size_t do_bytes = (static_cast<size_t>(batch) * seq * heads * head_dim * 2 + 255) / 256 * 256;
  return do_bytes + static_cast<size_t>(batch) * heads * seq_pad * sizeof(float4);
}

// See engine.h for the contract.
cudaError_t gqa_bwd_tc(cudaStream_t stream, const GqaBwdTcArgs& a) {
  const int D = a.head_dim, E = a.q_heads * D;
  const int seq_pad = (a.seq + kColTile - 1) / kColTile * kColTile + kColTile;
  const size_t do_bytes = (static_cast<size_t>(a.batch) * a.seq * E * 2 + 255) / 256 * 256;
  auto* do_bf16 = static_cast<__nv_bfloat16*>(a.workspace);
  // 16 bytes per (sequence, head, padded row): 8 of pair records, then the two plain arrays
  auto* stats = reinterpret_cast<float*>(static_cast<uint8_t*>(a.workspace) + do_bytes);
  const size_t stat_rows = static_cast<size_t>(a.batch) * a.q_heads * seq_pad;
  float* shifts = stats + 2 * stat_rows;
  float* deltas_pad = stats + 3 * stat_rows;
  {
    // tokens per CTA: 8 (one 32-byte sector of every statistics array per head; more tokens per
    // CTA leave too few CTAs in flight to fill the memory pipe), fewer when many heads would not
    // fit 32 KB of shared memory
    int block_tokens = 8;
    while (block_tokens > 1 && static_cast<long long>(a.q_heads) * block_tokens * 8 > 32768) block_tokens /= 2;
    if (static_cast<long long>(a.q_heads) * block_tokens * 8 > 48 * 1024) return cudaErrorInvalidValue;
    const unsigned blocks = static_cast<unsigned>(a.batch) * ((a.seq + block_tokens - 1) / block_tokens);
    const size_t prep_smem = static_cast<size_t>(a.q_heads) * block_tokens * 8;
    auto prep = D == 128 ? attn_bwd_prep<128> : attn_bwd_prep<64>;
    prep<<<blocks, 256, prep_smem, stream>>>(static_cast<const __nv_bfloat16*>(a.out), a.d_out, a.maxima,
                                            a.normalizers, do_bf16, stats, shifts, deltas_pad, a.deltas, a.seq,
                                            seq_pad, a.q_heads, block_tokens);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  BwdMaps m;
  if (!make_token_map(&m.q128, a.q, a.q_cols, a.seq, a.batch, a.q_token, kRowTile) ||
      !make_token_map(&m.do128, do_bf16, E, a.seq, a.batch, E, kRowTile) ||
      !make_token_map(&m.q64, a.q, a.q_cols, a.seq, a.batch, a.q_token, kColTile) ||
      !make_token_map(&m.k128, a.k, a.kv_cols, a.seq, a.batch, a.kv_token, kRowTile) ||
      !make_token_map(&m.k64, a.k, a.kv_cols, a.seq, a.batch, a.kv_token, kColTile) ||
      !make_token_map(&m.v128, a.v, a.kv_cols, a.seq, a.batch, a.kv_token, kRowTile) ||
      !make_token_map(&m.v64, a.v, a.kv_cols, a.seq, a.batch, a.kv_token, kColTile) ||
      !make_token_map(&m.do64, do_bf16, E, a.seq, a.batch, E, kColTile))
    return cudaErrorInvalidValue;
  BwdParams p;
  p.seq = a.seq;
  p.heads = a.q_heads;
  p.head_dim = D;
  p.group = a.q_heads / a.kv_heads;
  p.q_col0 = a.q_col0;
  p.k_col0 = a.k_col0;
  p.v_col0 = a.v_col0;
  p.scale = 1.0f / sqrtf(static_cast<float>(D));
  p.scale_log2 = p.scale * kLog2e;
  p.stats = stats;
  p.shifts = shifts;
  p.deltas_pad = deltas_pad;
  p.q = static_cast<const __nv_bfloat16*>(a.q);
  p.d_out16 = do_bf16;
  p.q_token = a.q_token;
  p.seq_pad = seq_pad;
  p.dq = a.dq;
  p.dk = a.dk;
  p.dv = a.dv;
  p.dq_token = a.dq_token;
  p.dkv_token = a.dkv_token;
  p.status = a.status;
  if (D == 64) return launch_bwd_tc<64>(stream, m, p, a.batch);
  if (D == 128) return launch_bwd_tc<128>(stream, m, p, a.batch);
  return cudaErrorInvalidValue;
}

// Packed [rows, 3E] layout of AttentionLayer: q, k, v are column ranges of one tensor.
cudaError_t attn_bwd_tc(cudaStream_t stream, const void* qkv, const void* out, const float* d_out,
                        const float* maxima, const float* normalizers, float* d_qkv, float* deltas,
                        void* workspace, int batch, int seq, int heads, int head_dim,
                        uint32_t* status) {
  const int E = heads * head_dim;
  GqaBwdTcArgs a{};
  a.q = a.k = a.v = qkv;
  a.q_cols = a.kv_cols = 3 * E;
  a.q_token = a.kv_token = 3 * static_cast<size_t>(E);
  a.q_col0 = 0; a.k_col0 = E; a.v_col0 = 2 * E;
  a.out = out; a.d_out = d_out; a.maxima = maxima; a.normalizers = normalizers; a.deltas = deltas;
  a.dq = d_qkv; a.dk = d_qkv + E; a.dv = d_qkv + 2 * E;
  a.dq_token = a.dkv_token = 3 * static_cast<size_t>(E);
  a.workspace = workspace;
  a.batch = batch; a.seq = seq; a.q_heads = heads; a.kv_heads = heads; a.head_dim = head_dim;
  a.status = status;
  return gqa_bwd_tc(stream, a);
}

}  // namespace pluto
