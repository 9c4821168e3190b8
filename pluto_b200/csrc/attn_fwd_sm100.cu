// Causal softmax attention forward on the Blackwell tensor cores (bf16 operands, fp32
// accumulation), head width 64 or 128.  One kernel serves both layers on the hot path:
//   * AttentionLayer forward over the packed [rows, 3E] activation
//     (reference: src/llm/layers/attention.cc:98-170, 418-507), writing O plus the row maximum
//     and row normaliser the backward pass reuses;
//   * the attention core of QwenAttentionLayer's sequence forward with grouped query heads
//     (reference: src/llm/layers/qwen_attention.cc:68-119), with the optional sigmoid output gate
//     and its rounding sequence R(R(core) * R(sigmoid(gate))).
//
// Structure of one CTA (256 threads) = one 128-row query tile of one (sequence, query head):
//   warp 0      TMA producer: Q once, then K_j / V_j tiles of 128 keys into a 2-stage ring
//               (128-byte swizzled boxes of 64 columns; no multicast).
//   warp 1      tcgen05.mma issuer: S_j = Q K_j^T into one of two 128-column TMEM buffers,
//               then O += P_j V_j with P_j read straight from TMEM (it overwrites S_j in place
//               as packed bf16) and V_j as an MN-major shared-memory operand.
//   warps 4-7   one thread per query row (TMEM lane): tcgen05.ld the score row, online softmax
//               in fp32 with exp2, lazy rescaling of the O accumulator (only when the running
//               maximum grew by more than 2^8), tcgen05.st of P, final normalise and store.
// QK^T of tile j+1 is issued before PV of tile j, so the tensor pipe works on the next score tile
// while the softmax warps are busy with the current one.
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "engine.h"

namespace pluto {
namespace {

constexpr int kBM = 128;          // query rows per CTA
constexpr int kBN = 128;          // keys per tile
constexpr int kStages = 2;        // K/V ring depth
constexpr int kThreadsFwd = 256;
constexpr int kSlabBytes = 128 * 64 * 2;  // one [128 rows x 64 bf16] swizzled slab
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct FwdParams {
  // column (innermost) coordinate of head 0 in each tensor map, and per-head column step
  int q_col0, k_col0, v_col0;
  int q_head_cols, kv_head_cols;
  int seq, heads, group;
  float scale_log2;  // softmax scale * log2(e)
  float scale;
  // outputs
  __nv_bfloat16* out;          // [batch*seq, heads, D] with out_token/out_head element strides
  size_t out_token, out_head;
  float* maxima;               // optional, [(b*H+h)*S + s]
  float* normalizers;          // optional
  float* core;                 // optional fp32 copy of the ungated result, same indexing as out
  const __nv_bfloat16* gate;   // optional, indexed like q: token stride gate_token, head stride gate_head
  size_t gate_token, gate_head;
  int round_gate;              // apply bf16 rounding inside the gate product (reference behaviour)
  // key/value split (pair kernel only): the CTAs of one tile pair each walk a contiguous part of the
  // key blocks and write an unnormalised partial; attn_fwd_merge combines them.  How many parts a
  // pair has comes with the schedule (PairSchedule); split_pairs says whether any pair is split.
  int split_pairs;
  float* part_o;               // [split][batch*seq tokens][heads][D] accumulator relative to part_m.x
  float4* part_m;              // [split][batch][heads][seq] = (max used * scale_log2, true max *
                               //  scale_log2, sum relative to max used, 0)
  uint32_t* status;
  int tile_end;                // one past the last query tile this launch computes
};

struct Barriers {
  uint64_t q_full;
  uint64_t k_full[kStages], k_empty[kStages];
  uint64_t v_full[kStages], v_empty[kStages];
  uint64_t s_full[2], p_full[2], pv_done[2];
  uint32_t tmem_base;
};

template <int D>
__global__ void __launch_bounds__(kThreadsFwd, 1)
attn_fwd_sm100(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, FwdParams p) {
  constexpr int kSlabs = D / 64;
  constexpr int kTileBytes = kSlabs * kSlabBytes;  // one Q, K or V tile
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColS = 0, kColO = 256;
  constexpr uint32_t kIdescQK = umma_idesc_bf16(kBM, kBN, false);
  constexpr uint32_t kIdescPV = umma_idesc_bf16(kBM, D, true);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* q_smem = smem;
  uint8_t* k_smem = q_smem + kTileBytes;
  uint8_t* v_smem = k_smem + kStages * kTileBytes;
  Barriers* bar = reinterpret_cast<Barriers*>(v_smem + kStages * kTileBytes);

  const int warp = uniform_warp_index(), lane = threadIdx.x % 32;
  // (sequence, head) varies fastest, the tile index slowest: the longest tiles of every head start
  // first and the shortest fill the tail.
  // The grid's y extent may cover only the query tiles [tile_end - gridDim.y, tile_end).
  const int q_tile = p.tile_end - 1 - blockIdx.y;
  const int head = blockIdx.x % p.heads, batch = blockIdx.x / p.heads;
  const int n_tiles = q_tile + 1;                 // causal: key tiles 0..q_tile

  if (threadIdx.x == 0) {
    mbar_init(&bar->q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bar->k_full[s], 1);
      mbar_init(&bar->k_empty[s], 1);
      mbar_init(&bar->v_full[s], 1);
      mbar_init(&bar->v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bar->s_full[s], 1);
      mbar_init(&bar->p_full[s], 128);
      mbar_init(&bar->pv_done[s], 1);
    }
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

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      const int kv_head = head / p.group;
      mbar_expect_tx(&bar->q_full, kTileBytes);
      for (int s = 0; s < kSlabs; ++s)
        tma_load_3d(q_smem + s * kSlabBytes, &map_q, p.q_col0 + head * p.q_head_cols + s * 64,
                    q_tile * kBM, batch, &bar->q_full);
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j % kStages, use = j / kStages;
        if (use > 0) ok = mbar_wait(&bar->k_empty[st], (use - 1) & 1, p.status, 1);
        if (!ok) break;
        mbar_expect_tx(&bar->k_full[st], kTileBytes);
        for (int s = 0; s < kSlabs; ++s)
          tma_load_3d(k_smem + st * kTileBytes + s * kSlabBytes, &map_k,
                      p.k_col0 + kv_head * p.kv_head_cols + s * 64, j * kBN, batch,
                      &bar->k_full[st]);
        if (use > 0) ok = mbar_wait(&bar->v_empty[st], (use - 1) & 1, p.status, 2);
        if (!ok) break;
        mbar_expect_tx(&bar->v_full[st], kTileBytes);
        for (int s = 0; s < kSlabs; ++s)
          tma_load_3d(v_smem + st * kTileBytes + s * kSlabBytes, &map_v,
                      p.v_col0 + kv_head * p.kv_head_cols + s * 64, j * kBN, batch,
                      &bar->v_full[st]);
      }
      // Before leaving, make sure every copy this thread started has landed (bounded): nothing
      // may still be writing this CTA's shared memory when it exits.
      mbar_wait(&bar->q_full, 0, p.status, 3);
      for (int j = max(0, n_tiles - kStages); j < n_tiles; ++j) {
        mbar_wait(&bar->k_full[j % kStages], (j / kStages) & 1, p.status, 4);
        mbar_wait(&bar->v_full[j % kStages], (j / kStages) & 1, p.status, 5);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    {
      // The whole warp walks the schedule (uniform control flow); one elected lane issues.
      bool ok = __all_sync(0xffffffffu, mbar_wait(&bar->q_full, 0, p.status, 10));
      tc_fence_after();
      const uint32_t q_base = smem_u32(q_smem), k_base = smem_u32(k_smem), v_base = smem_u32(v_smem);
      auto issue_pv = [&](int i) -> bool {
        const int sb = i & 1, st = i % kStages;
        if (!__all_sync(0xffffffffu, mbar_wait(&bar->p_full[sb], (i >> 1) & 1, p.status, 11)))
          return false;
        if (!__all_sync(0xffffffffu, mbar_wait(&bar->v_full[st], (i / kStages) & 1, p.status, 12)))
          return false;
        tc_fence_after();
        if (elect_one()) {
          // B = V tile, MN-major: 16 key rows per step (2048 bytes), 64-column slabs kBN*128 apart
          const uint64_t v_desc = umma_desc_sw128(v_base + st * kTileBytes, kSlabBytes, 1024);
#pragma unroll
          for (int ks = 0; ks < kBN / 16; ++ks)
            umma_ts(tmem + kColO, tmem + kColS + sb * 128 + ks * 8, v_desc + ks * (2048 >> 4),
                    kIdescPV, i > 0 || ks > 0);
          tc_commit(&bar->pv_done[sb]);
          tc_commit(&bar->v_empty[st]);
        }
        __syncwarp();
        return true;
      };
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int sb = j & 1, st = j % kStages;
        ok = __all_sync(0xffffffffu, mbar_wait(&bar->k_full[st], (j / kStages) & 1, p.status, 13));
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
          const uint64_t q_desc = umma_desc_sw128(q_base, 16, 1024);
          const uint64_t k_desc = umma_desc_sw128(k_base + st * kTileBytes, 16, 1024);
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t off = ((ks / 4) * kSlabBytes + (ks % 4) * 32) >> 4;
            umma_ss(tmem + kColS + sb * 128, q_desc + off, k_desc + off, kIdescQK, ks > 0);
          }
          tc_commit(&bar->s_full[sb]);
          tc_commit(&bar->k_empty[st]);
        }
        __syncwarp();
        if (j > 0) ok = issue_pv(j - 1);
      }
      if (ok) issue_pv(n_tiles - 1);
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ softmax / epilogue
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;             // row inside the query tile == TMEM lane
    const int query = q_tile * kBM + row;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    float m_used = -INFINITY;   // maximum the accumulators are expressed against (raw scores)
    float m_true = -INFINITY;   // true running maximum (raw scores)
    float l = 0.0f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int sb = j & 1;
      ok = mbar_wait(&bar->s_full[sb], (j >> 1) & 1, p.status, 20);
      if (!ok) break;
      tc_fence_after();
      uint32_t s[4][32];
      const uint32_t s_addr = tmem + lane_base + kColS + sb * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(s_addr + c * 32, s[c]);
      tmem_wait_ld();
      float tile_max = -INFINITY;
      if (j == q_tile) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (c * 32 + i > row) s[c][i] = 0xff800000u;  // -inf above the diagonal
            tile_max = fmaxf(tile_max, __uint_as_float(s[c][i]));
          }
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) tile_max = fmaxf(tile_max, __uint_as_float(s[c][i]));
      }
      m_true = fmaxf(m_true, tile_max);
      const bool grow = (m_true - m_used) * p.scale_log2 > kRescaleThreshold;
      if (__any_sync(0xffffffffu, grow)) {
        const float factor = grow ? fast_exp2((m_used - m_true) * p.scale_log2) : 1.0f;
        if (grow) m_used = m_true;
        l *= factor;
        if (j > 0) {
          // the previous PV must have landed in O before O is rescaled
          ok = mbar_wait(&bar->pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, p.status, 21);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(tmem + lane_base + kColO + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
            tmem_st32(tmem + lane_base + kColO + c * 32, o);
          }
        }
      }
      const float neg_m = -m_used * p.scale_log2;
      float row_sum = 0.0f;
      uint32_t packed[2][32];
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(s[c][i]), p.scale_log2, neg_m));
          const float p1 = fast_exp2(fmaf(__uint_as_float(s[c][i + 1]), p.scale_log2, neg_m));
          row_sum += p0 + p1;
          packed[c / 2][(c % 2) * 16 + i / 2] = pack_bf16(p0, p1);
        }
      l += row_sum;
      tmem_st32(s_addr, packed[0]);
      tmem_st32(s_addr + 32, packed[1]);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&bar->p_full[sb]);
    }
    if (ok) ok = mbar_wait(&bar->pv_done[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1, p.status, 22);
    if (ok) {
      tc_fence_after();
      const float inv = 1.0f / l;
      const bool live = query < p.seq;
      const size_t token = static_cast<size_t>(batch) * p.seq + query;
      __nv_bfloat16* out = p.out + token * p.out_token + head * p.out_head;
      float* core = p.core ? p.core + token * p.out_token + head * p.out_head : nullptr;
      const __nv_bfloat16* gate =
          p.gate ? p.gate + token * p.gate_token + head * p.gate_head : nullptr;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(tmem + lane_base + kColO + c * 32, o);
        tmem_wait_ld();
        if (live) {
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float a = __uint_as_float(o[i]) * inv, b = __uint_as_float(o[i + 1]) * inv;
            if (core) {
              core[c * 32 + i] = a;
              core[c * 32 + i + 1] = b;
            }
            if (gate) {
              const float g0 = __bfloat162float(gate[c * 32 + i]);
              const float g1 = __bfloat162float(gate[c * 32 + i + 1]);
              float s0 = 1.0f / (1.0f + expf(-g0)), s1 = 1.0f / (1.0f + expf(-g1));
              if (p.round_gate) {
                s0 = bf16_round(s0);
                s1 = bf16_round(s1);
                a = bf16_round(a);
                b = bf16_round(b);
              }
              a *= s0;
              b *= s1;
            }
            w[i / 2] = pack_bf16(a, b);
          }
          uint4* dst = reinterpret_cast<uint4*>(out + c * 32);
#pragma unroll
          for (int i = 0; i < 4; ++i) dst[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
        }
      }
      if (live && p.maxima) {
        const size_t stat = (static_cast<size_t>(batch) * p.heads + head) * p.seq + query;
        p.maxima[stat] = m_true * p.scale;
        p.normalizers[stat] = l * fast_exp2((m_used - m_true) * p.scale_log2);
      }
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
// Two query tiles per CTA in ping-pong (sequences longer than one tile).
//
// A CTA owns the query tiles 2i and 2i+1 of one (sequence, head) and shares every K/V tile
// between them.  Warps 4-7 run the softmax of tile A, warps 8-11 of tile B; the MMA warp issues
//     ... PV_A(j), QK_A(j+1), PV_B(j), QK_B(j+1), PV_A(j+1), ...
// so while one tile's rows are in the exp2 unit the tensor pipe works on the other tile, and the
// two units overlap instead of alternating.  Each tile has one score buffer in TMEM (P overwrites
// S in place; the next QK^T of that tile is issued behind the PV that reads P, and the tensor pipe
// runs its instructions in order) and its own O accumulator: 2 x 128 + 2 x D <= 512 columns.
// The copy/MMA warpgroup hands registers to the softmax warpgroups (setmaxnreg), so a softmax
// thread can hold its whole 128-entry score row and read TMEM once per tile.
// ---------------------------------------------------------------------------------------------
constexpr int kThreadsPair = 384;
constexpr int kEarly = 6;     // PV instructions (of 8) issued on the early hand-off of P
constexpr int kPolyOf4 = 1;  // pairs per four whose exp2 runs on the FMA pipe

struct PairBarriers {
  uint64_t q_full;
  uint64_t k_full[kStages], k_empty[kStages];
  uint64_t v_full[kStages], v_empty[kStages];
  uint64_t s_full[2], p_full[2], p_early[2], pv_done[2];
  uint32_t tmem_base;
};

// The pair kernel's work list, longest item first (CTAs are handed to SMs in blockIdx order, so this
// is longest-processing-time-first scheduling): item i of every (sequence, head) is part
// (meta & 15) of (meta >> 4) of tile pair `pair`.  A causal prompt's pairs differ in length by two
// orders of magnitude; when a GPU holds few heads the longest pair alone exceeds an SM's fair share
// of the whole problem, and only the pairs above that share are cut (2 to 4 parts), not all of them.
constexpr int kMaxPairItems = 512;
constexpr int kMaxPairs = 128;
struct PairSchedule {
  uint16_t pair[kMaxPairItems];
  uint8_t meta[kMaxPairItems];
  uint8_t parts_of[kMaxPairs];   // per pair, for the merge
};

template <int D>
__global__ void __launch_bounds__(kThreadsPair, 1)
attn_fwd_sm100_pair(const __grid_constant__ CUtensorMap map_q,
                    const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, FwdParams p,
                    const __grid_constant__ PairSchedule schedule) {
  constexpr int kSlabs = D / 64;
  constexpr int kTileBytes = kSlabs * kSlabBytes;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kIdescQK = umma_idesc_bf16(kBM, kBN, false);
  constexpr uint32_t kIdescPV = umma_idesc_bf16(kBM, D, true);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* q_smem = smem;                              // two query tiles
  uint8_t* k_smem = q_smem + 2 * kTileBytes;
  uint8_t* v_smem = k_smem + kStages * kTileBytes;
  PairBarriers* bar = reinterpret_cast<PairBarriers*>(v_smem + kStages * kTileBytes);

  const int warp = uniform_warp_index(), lane = threadIdx.x % 32;
  // CTAs are handed to SMs in blockIdx.x-major order: (sequence, head) varies fastest and the pair
  // index slowest, so every head's longest pairs start first and the shortest ones fill the tail
  // (longest-processing-time-first over the whole grid, not per head).
  // blockIdx.y indexes the schedule (pairs below the launch's range are not in it).
  pdl_launch_dependents();   // a merge kernel behind this launch may be placed as SMs free up
  const int pair = schedule.pair[blockIdx.y];
  const int part = schedule.meta[blockIdx.y] & 15, parts = schedule.meta[blockIdx.y] >> 4;
  const int head = blockIdx.x % p.heads, batch = blockIdx.x / p.heads;
  const int q_tiles = (p.seq + kBM - 1) / kBM;
  const int tile_of[2] = {2 * pair, 2 * pair + 1};
  const int blocks_of[2] = {tile_of[0] + 1, tile_of[1] < q_tiles ? tile_of[1] + 1 : 0};
  // this CTA's key blocks [jb, je); tile x takes the ones below its own count n_of[x]
  const int chunk = (max(blocks_of[0], blocks_of[1]) + parts - 1) / parts;
  const int jb = part * chunk;
  const int n_of[2] = {max(jb, min(blocks_of[0], jb + chunk)), max(jb, min(blocks_of[1], jb + chunk))};
  const int n_max = max(n_of[0], n_of[1]);

  if (threadIdx.x == 0) {
    mbar_init(&bar->q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bar->k_full[s], 1);
      mbar_init(&bar->k_empty[s], 1);
      mbar_init(&bar->v_full[s], 1);
      mbar_init(&bar->v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bar->s_full[s], 1);
      mbar_init(&bar->p_full[s], 4);  // one arrival per softmax warp
      mbar_init(&bar->p_early[s], 4);
      mbar_init(&bar->pv_done[s], 1);
    }
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

  // Register file: 384 threads x 168 at launch.  The warpgroup of the copy/MMA warps gives most of
  // its registers back so that the two softmax warpgroups can keep a whole score row each.

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (lane == 0) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      const int kv_head = head / p.group;
      mbar_expect_tx(&bar->q_full, 2 * kTileBytes);  // a tile past the sequence end reads zeros
      for (int x = 0; x < 2; ++x)
        for (int s = 0; s < kSlabs; ++s)
          tma_load_3d(q_smem + x * kTileBytes + s * kSlabBytes, &map_q,
                      p.q_col0 + head * p.q_head_cols + s * 64, tile_of[x] * kBM, batch,
                      &bar->q_full);
      bool ok = true;
      for (int j = jb; j < n_max && ok; ++j) {
        const int st = (j - jb) % kStages, use = (j - jb) / kStages;
        if (use > 0) ok = mbar_wait(&bar->k_empty[st], (use - 1) & 1, p.status, 1);
        if (!ok) break;
        mbar_expect_tx(&bar->k_full[st], kTileBytes);
        for (int s = 0; s < kSlabs; ++s)
          tma_load_3d(k_smem + st * kTileBytes + s * kSlabBytes, &map_k,
                      p.k_col0 + kv_head * p.kv_head_cols + s * 64, j * kBN, batch,
                      &bar->k_full[st]);
        if (use > 0) ok = mbar_wait(&bar->v_empty[st], (use - 1) & 1, p.status, 2);
        if (!ok) break;
        mbar_expect_tx(&bar->v_full[st], kTileBytes);
        for (int s = 0; s < kSlabs; ++s)
          tma_load_3d(v_smem + st * kTileBytes + s * kSlabBytes, &map_v,
                      p.v_col0 + kv_head * p.kv_head_cols + s * 64, j * kBN, batch,
                      &bar->v_full[st]);
      }
      mbar_wait(&bar->q_full, 0, p.status, 3);
      for (int j = max(jb, n_max - kStages); j < n_max; ++j) {
        mbar_wait(&bar->k_full[(j - jb) % kStages], ((j - jb) / kStages) & 1, p.status, 4);
        mbar_wait(&bar->v_full[(j - jb) % kStages], ((j - jb) / kStages) & 1, p.status, 5);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    {
      // The whole warp walks the schedule (uniform control flow); one elected lane issues.
      bool ok = __all_sync(0xffffffffu, mbar_wait(&bar->q_full, 0, p.status, 10));
      tc_fence_after();
      const uint32_t q_base = smem_u32(q_smem), k_base = smem_u32(k_smem), v_base = smem_u32(v_smem);
      auto issue_qk = [&](int x, int j) -> bool {
        const int st = (j - jb) % kStages;
        if (!__all_sync(0xffffffffu, mbar_wait(&bar->k_full[st], ((j - jb) / kStages) & 1, p.status, 13)))
          return false;
        tc_fence_after();
        if (elect_one()) {
          const uint64_t q_desc = umma_desc_sw128(q_base + x * kTileBytes, 16, 1024);
          const uint64_t k_desc = umma_desc_sw128(k_base + st * kTileBytes, 16, 1024);
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            // advancing the start-address field (bytes >> 4) of a descriptor is a 32-bit add
            const uint32_t off = ((ks / 4) * kSlabBytes + (ks % 4) * 32) >> 4;
            umma_ss(tmem + x * 128, q_desc + off, k_desc + off, kIdescQK, ks > 0);
          }
          tc_commit(&bar->s_full[x]);
        }
        __syncwarp();
        return true;
      };
      auto issue_pv = [&](int x, int j) -> bool {
        const int st = (j - jb) % kStages;
        // P arrives in two parts (96 + 32 keys): the first kEarly PV instructions run while the
        // softmax warps still work on the rest of the row.
        if (!__all_sync(0xffffffffu, mbar_wait(&bar->p_early[x], (j - jb) & 1, p.status, 14))) return false;
        if (!__all_sync(0xffffffffu, mbar_wait(&bar->v_full[st], ((j - jb) / kStages) & 1, p.status, 12)))
          return false;
        tc_fence_after();
        const uint64_t v_desc = umma_desc_sw128(v_base + st * kTileBytes, kSlabBytes, 1024);
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < kEarly; ++ks)
            umma_ts(tmem + 256 + x * 128, tmem + x * 128 + ks * 8, v_desc + ks * (2048 >> 4),
                    kIdescPV, j > jb || ks > 0);
        }
        __syncwarp();
        if (!__all_sync(0xffffffffu, mbar_wait(&bar->p_full[x], (j - jb) & 1, p.status, 11))) return false;
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int ks = kEarly; ks < kBN / 16; ++ks)
            umma_ts(tmem + 256 + x * 128, tmem + x * 128 + ks * 8, v_desc + ks * (2048 >> 4),
                    kIdescPV, true);
          tc_commit(&bar->pv_done[x]);
        }
        __syncwarp();
        return true;
      };
#pragma unroll
      for (int x = 0; x < 2; ++x)
        if (ok && n_of[x] > jb) ok = issue_qk(x, jb);
      if (ok && elect_one()) tc_commit(&bar->k_empty[0]);
      __syncwarp();
      for (int j = jb; j < n_max && ok; ++j) {
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          if (!ok || j >= n_of[x]) continue;
          ok = issue_pv(x, j);
          if (ok && j + 1 < n_of[x]) ok = issue_qk(x, j + 1);
        }
        if (!ok) break;
        if (elect_one()) {
          tc_commit(&bar->v_empty[(j - jb) % kStages]);
          if (j + 1 < n_max) tc_commit(&bar->k_empty[(j + 1 - jb) % kStages]);
        }
        __syncwarp();
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ softmax / epilogue
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    const int x = (warp - 4) / 4;                    // which query tile this warpgroup serves
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int q_tile = tile_of[x];
    const int query = q_tile * kBM + row;
    const int n_tiles = n_of[x];
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_addr = tmem + lane_base + x * 128;
    const uint32_t o_addr = tmem + lane_base + 256 + x * 128;
    float m_used = -INFINITY, m_true = -INFINITY, l = 0.0f;
    bool ok = true;
    for (int j = jb; j < n_tiles && ok; ++j) {
      ok = mbar_wait(&bar->s_full[x], (j - jb) & 1, p.status, 20);
      if (!ok) break;
      tc_fence_after();
      const bool diagonal = j == q_tile;
      // the whole score row in registers (this warpgroup raised its register allowance)
      uint32_t s[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(s_addr + c * 32, s[c]);
      tmem_wait_ld();
      if (diagonal) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i > row) s[c][i] = 0xff800000u;  // -inf above the diagonal
      }
      float mx[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) mx[i] = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 2)
          mx[(i >> 1) & 7] = max3(mx[(i >> 1) & 7], __uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1]));
      m_true = fmaxf(m_true, fmaxf(max3(mx[0], mx[1], mx[2]), max3(mx[3], mx[4], mx[5])));
      m_true = max3(m_true, mx[6], mx[7]);
      const bool grow = (m_true - m_used) * p.scale_log2 > kRescaleThreshold;
      if (__any_sync(0xffffffffu, grow)) {
        const float factor = grow ? fast_exp2((m_used - m_true) * p.scale_log2) : 1.0f;
        if (grow) m_used = m_true;
        l *= factor;
        if (j > jb) {
          ok = mbar_wait(&bar->pv_done[x], (j - 1 - jb) & 1, p.status, 21);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(o_addr + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
            tmem_st32(o_addr + c * 32, o);
          }
        }
      }
      // exp2 of the row: the special-function unit (16 results per clock and SM) would need as
      // long for the two tiles as the tensor pipe needs for their MMAs, so kPolyOf4 of every four
      // pairs are evaluated on the FMA pipe instead.
      const uint64_t scale2 = f2_pack(p.scale_log2, p.scale_log2);
      const uint64_t neg_m2 = f2_pack(-m_used * p.scale_log2, -m_used * p.scale_log2);
      uint64_t sum2[2] = {0ull, 0ull};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const uint64_t x2 = f2_fma(f2_pack(__uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1])),
                                     scale2, neg_m2);
          uint64_t p2;
          float p0, p1;
          if (((i >> 1) & 3) < kPolyOf4) {
            p2 = f2_exp2_poly(x2);
            f2_unpack(p2, p0, p1);
          } else {
            f2_unpack(x2, p0, p1);
            p0 = fast_exp2(p0);
            p1 = fast_exp2(p1);
            p2 = f2_pack(p0, p1);
          }
          sum2[(i >> 1) & 1] = f2_add(sum2[(i >> 1) & 1], p2);
          packed[i / 2] = pack_bf16(p0, p1);
        }
        tmem_st16(s_addr + c * 16, packed);
        if (c == kEarly / 2 - 1) {
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bar->p_early[x]);
        }
      }
      {
        float a0, a1, b0, b1;
        f2_unpack(sum2[0], a0, a1);
        f2_unpack(sum2[1], b0, b1);
        l += (a0 + a1) + (b0 + b1);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->p_full[x]);
    }
    const bool any = n_tiles > jb;             // this part holds key blocks of this tile
    if (ok && any) ok = mbar_wait(&bar->pv_done[x], (n_tiles - 1 - jb) & 1, p.status, 22);
    if (parts > 1 && blocks_of[x] > 0) {   // (uniform over the warpgroup: the other branch holds a barrier)
      // Unnormalised partial of this part (accumulator and sums are relative to m_used), staged like
      // the normalised rows below: fp32 rows go through this tile's query buffer half a row at a
      // time (16-byte chunk c of row r at chunk position c ^ (r & (chunks - 1))), and the warpgroup
      // copies each half out with 16 threads per row.
      constexpr int kRoundCols = kTileBytes / (kBM * 4);   // fp32 columns of a row per round: 64 (D 128) or 32
      constexpr int kChunks = kRoundCols / 4;              // 16-byte chunks per row and round
      uint8_t* stage = q_smem + x * kTileBytes;
      const bool live = query < p.seq;
      const size_t tokens = static_cast<size_t>(gridDim.x / p.heads) * p.seq;
      float* dst_tile = p.part_o + ((static_cast<size_t>(part) * tokens + static_cast<size_t>(batch) * p.seq +
                                     static_cast<size_t>(q_tile) * kBM) * p.heads + head) * D;
      const int t128 = threadIdx.x - (4 + 4 * x) * 32;
      if (ok && any) tc_fence_after();
#pragma unroll 1
      for (int round = 0; round < D / kRoundCols; ++round) {
        if (ok) {
#pragma unroll
          for (int c = 0; c < kRoundCols / 32; ++c) {
            uint32_t o[32];
            if (any) {
              tmem_ld32(o_addr + round * kRoundCols + c * 32, o);
              tmem_wait_ld();
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = 0u;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i)
              sts_b32x4(smem_u32(stage) + row * (kRoundCols * 4) + (((c * 8 + i) ^ (row & (kChunks - 1))) * 16),
                        o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
          }
        }
        // all 128 threads of this tile's warpgroup, whatever their waits returned
        asm volatile("bar.sync %0, 128;" ::"r"(1 + x) : "memory");
        if (ok) {
#pragma unroll 4
          for (int e = t128; e < kBM * kChunks; e += 128) {
            const int r = e / kChunks, piece = e % kChunks;
            if (q_tile * kBM + r < p.seq)
              *reinterpret_cast<uint4*>(dst_tile + static_cast<size_t>(r) * p.heads * D + round * kRoundCols + piece * 4) =
                  lds_b32x4(smem_u32(stage) + r * (kRoundCols * 4) + ((piece ^ (r & (kChunks - 1))) * 16));
          }
        }
        asm volatile("bar.sync %0, 128;" ::"r"(1 + x) : "memory");   // the next round reuses the buffer
      }
      if (ok && live)
        p.part_m[((static_cast<size_t>(part) * (gridDim.x / p.heads) + batch) * p.heads + head) * p.seq + query] =
            make_float4(any ? m_used * p.scale_log2 : -INFINITY, any ? m_true * p.scale_log2 : -INFINITY,
                        any ? l : 0.0f, 0.0f);
    } else if (any) {
      // The normalised rows leave through shared memory: each thread writes its row, as bf16, into
      // this tile's query buffer (free: the tile's last Q K^T has completed) in the swizzled slab
      // layout, then the warpgroup's 128 threads copy the tile out in 16-byte pieces, 16 threads
      // per 256-byte row.  (Written straight from the row's thread, every store instruction of a
      // warp touched 32 rows: 11 to 17 thousand cycles per tile against two thousand this way.)
      uint8_t* stage = q_smem + x * kTileBytes;
      const bool live = query < p.seq;
      const size_t token = static_cast<size_t>(batch) * p.seq + query;
      if (ok) {
        tc_fence_after();
        const float inv = 1.0f / l;
        float* core = p.core ? p.core + token * p.out_token + head * p.out_head : nullptr;
        const __nv_bfloat16* gate =
            p.gate ? p.gate + token * p.gate_token + head * p.gate_head : nullptr;
        // (not unrolled: this code runs once per CTA, so every instruction of it is fetched cold)
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(o_addr + c * 32, o);
          tmem_wait_ld();
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float a = __uint_as_float(o[i]) * inv, b = __uint_as_float(o[i + 1]) * inv;
            if (core && live) {
              core[c * 32 + i] = a;
              core[c * 32 + i + 1] = b;
            }
            if (gate && live) {
              const float g0 = __bfloat162float(gate[c * 32 + i]);
              const float g1 = __bfloat162float(gate[c * 32 + i + 1]);
              float s0 = 1.0f / (1.0f + expf(-g0)), s1 = 1.0f / (1.0f + expf(-g1));
              if (p.round_gate) {
                s0 = bf16_round(s0);
                s1 = bf16_round(s1);
                a = bf16_round(a);
                b = bf16_round(b);
              }
              a *= s0;
              b *= s1;
            }
            w[i / 2] = pack_bf16(a, b);
          }
          // (st.shared by address: a store through the generic `stage` pointer took four times as long)
          const uint32_t slab_row = smem_u32(stage) + (c / 2) * kSlabBytes + row * 128;
#pragma unroll
          for (int i = 0; i < 4; ++i)
            sts_b32x4(slab_row + ((((c & 1) * 4 + i) ^ (row & 7)) * 16), w[4 * i], w[4 * i + 1], w[4 * i + 2],
                      w[4 * i + 3]);
        }
      }
      // all 128 threads of this tile's warpgroup, whatever their waits returned (`any` is uniform)
      asm volatile("bar.sync %0, 128;" ::"r"(1 + x) : "memory");
      if (ok) {
        constexpr int kPieces = D / 8;   // 16-byte pieces per row
        const int t128 = threadIdx.x - (4 + 4 * x) * 32;
#pragma unroll 4
        for (int e = t128; e < kBM * kPieces; e += 128) {
          const int r = e / kPieces, piece = e % kPieces;
          const int q_row = q_tile * kBM + r;
          if (q_row < p.seq) {
            const uint4 v = lds_b32x4(smem_u32(stage) + (piece / 8) * kSlabBytes + r * 128 +
                                      (((piece & 7) ^ (r & 7)) * 16));
            *reinterpret_cast<uint4*>(p.out + (static_cast<size_t>(batch) * p.seq + q_row) * p.out_token +
                                      head * p.out_head + piece * 8) = v;
          }
        }
      }
      if (ok && live && p.maxima) {
        const size_t stat = (static_cast<size_t>(batch) * p.heads + head) * p.seq + query;
        p.maxima[stat] = m_true * p.scale;
        p.normalizers[stat] = l * fast_exp2((m_used - m_true) * p.scale_log2);
      }
    }
  } else {
    // warps 2-3 idle, but every warp of a warpgroup has to give its registers back together
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

// Combines the key/value parts of the pair kernel: one warp per (token, head), a lane owns D / 32
// consecutive channels.  With M = max over parts of the maximum each part's numbers are relative
// to:  O = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M); then the same epilogue as the kernel
// (fp32 core, gate with the reference's rounding sequence, bf16 output, statistics).
template <int D>
__global__ void __launch_bounds__(256) attn_fwd_merge(FwdParams p, int batch, int first_token,
                                                      const __grid_constant__ PairSchedule schedule) {
  pdl_wait();   // the pair kernel's partials are complete and visible from here on
  // rows (token, head) of the tokens from first_token on (the first token of the first pair that
  // was cut: the plan cuts the long pairs, i.e. the late ones)
  constexpr int kPer = D / 32;
  const int span = p.seq - first_token;
  const long long row = static_cast<long long>(blockIdx.x) * 8 + threadIdx.x / 32;
  const long long rows = static_cast<long long>(batch) * span * p.heads;
  if (row >= rows) return;
  const int lane = threadIdx.x % 32;
  const int head = static_cast<int>(row % p.heads);
  const long long local = row / p.heads;
  const int b = static_cast<int>(local / span), s = first_token + static_cast<int>(local % span);
  const size_t token = static_cast<size_t>(b) * p.seq + s;
  const size_t tokens = static_cast<size_t>(batch) * p.seq;
  const int parts = schedule.parts_of[s / (2 * kBM)];
  if (parts <= 1) return;   // the pair's only CTA wrote the final rows itself
  // every load of the row is requested before any is used: one memory round trip
  float4 rec[4];
  float4 val[4];
  static_assert(kPer == 4 || kPer == 2, "a lane owns two or four channels");
#pragma unroll
  for (int part = 0; part < 4; ++part) {
    if (part < parts) {
      rec[part] = p.part_m[((static_cast<size_t>(part) * batch + b) * p.heads + head) * p.seq + s];
      const float* src = p.part_o + ((static_cast<size_t>(part) * tokens + token) * p.heads + head) * D + lane * kPer;
      if (kPer == 4) val[part] = *reinterpret_cast<const float4*>(src);
      else {
        const float2 v2 = *reinterpret_cast<const float2*>(src);
        val[part] = make_float4(v2.x, v2.y, 0.0f, 0.0f);
      }
    } else {
      rec[part] = make_float4(-INFINITY, -INFINITY, 0.0f, 0.0f);
      val[part] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
  }
  float m_used = -INFINITY, m_true = -INFINITY;
#pragma unroll
  for (int part = 0; part < 4; ++part) {
    m_used = fmaxf(m_used, rec[part].x);
    m_true = fmaxf(m_true, rec[part].y);
  }
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, l = 0.0f;
#pragma unroll
  for (int part = 0; part < 4; ++part) {
    const float w = part < parts ? fast_exp2(rec[part].x - m_used) : 0.0f;      // 0 for a part without key blocks
    l = fmaf(rec[part].z, w, l);
    acc[0] = fmaf(val[part].x, w, acc[0]);
    acc[1] = fmaf(val[part].y, w, acc[1]);
    acc[2] = fmaf(val[part].z, w, acc[2]);
    acc[3] = fmaf(val[part].w, w, acc[3]);
  }
  const float inv = 1.0f / l;
  __nv_bfloat16* out = p.out + token * p.out_token + head * p.out_head + lane * kPer;
  float* core = p.core ? p.core + token * p.out_token + head * p.out_head + lane * kPer : nullptr;
  const __nv_bfloat16* gate = p.gate ? p.gate + token * p.gate_token + head * p.gate_head + lane * kPer : nullptr;
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    float a = acc[i] * inv;
    if (core) core[i] = a;
    if (gate) {
      float g = 1.0f / (1.0f + expf(-__bfloat162float(gate[i])));
      if (p.round_gate) {
        g = bf16_round(g);
        a = bf16_round(a);
      }
      a *= g;
    }
    out[i] = __float2bfloat16_rn(a);
  }
  if (lane == 0 && p.maxima) {
    const size_t stat = (static_cast<size_t>(b) * p.heads + head) * p.seq + s;
    p.maxima[stat] = m_true * 0.6931471805599453f;       // back from log2 units
    p.normalizers[stat] = l * fast_exp2(m_used - m_true);
  }
}

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                 const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
  static EncodeTiled fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &result) !=
            cudaSuccess ||
        result != cudaDriverEntryPointSuccess)
      return static_cast<EncodeTiled>(nullptr);
    return reinterpret_cast<EncodeTiled>(sym);
  }();
  return fn;
}

}  // namespace

// bf16 tensor [batch][seq][cols] with `token_stride` elements between tokens; box = 64 columns x
// `box_rows` tokens, 128-byte swizzle, out-of-range reads return zero.
bool make_token_map(CUtensorMap* map, const void* base, int cols, int seq, int batch,
                    size_t token_stride, int box_rows) {
  EncodeTiled encode = encode_fn();
  if (encode == nullptr) return false;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(seq),
                              static_cast<cuuint64_t>(batch)};
  const cuuint64_t strides[2] = {token_stride * 2, token_stride * 2 * static_cast<cuuint64_t>(seq)};
  const cuuint32_t box[3] = {64, static_cast<cuuint32_t>(box_rows), 1};
  const cuuint32_t elem[3] = {1, 1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) ==
         CUDA_SUCCESS;
}

// How a launch over query tiles [tile_begin, tile_begin + q_tiles) of (batch x heads) causal
// sequences is cut into CTAs.
//   pairs: two query tiles per CTA in ping-pong (each tile runs faster, but the units are coarser);
//   split: some or all pairs are cut along their keys into parts_of[pair] CTAs (needs the workspace);
//   pairs_without_split: what to do when split is wanted but no workspace was given.
// Work is counted in key blocks: pair p (tiles 2p, 2p + 1) has (2p + 1) + (2p + 2) of them.
//   * Few units (no more tiles than SMs): every pair in 2 or 4 parts.  Measured at S = 8192,
//     D = 128: 1 head 74 -> 50 us, 2 heads 76 -> 62 us.
//   * Otherwise a pair is cut into ceil(work / (f . fair share)) parts, the fair share being the
//     whole problem's work over the SMs and f the best of a few values in a simulation of the
//     launch (below); no cut at all is one of the candidates.  Measured at S = 8192, D = 128
//     (without -> with cuts): 3 heads 111 -> 79 us, 4 heads 113 -> 87, 5 heads 102 -> 99,
//     6 heads 123 -> 118, 8 heads 150 -> 128, 10 heads 152 -> 150; from 12 heads on nothing is cut.
//   * Without a workspace nothing is cut: pairs where there are at least two per SM (or exactly
//     one wave of them), the single-tile kernel otherwise.
static int fill_pair_schedule(PairSchedule* schedule, int tile_begin, int q_tiles, const uint8_t* parts_of,
                              int* work_of);
struct AttnFwdPlan {
  bool pairs, split, pairs_without_split;
  uint8_t parts_of[kMaxPairs];
};
static AttnFwdPlan attn_fwd_plan_uncached(int batch, int seq, int heads, int tile_begin, int q_tiles, int sms) {
  AttnFwdPlan plan{};
  const int all_tiles = (seq + kBM - 1) / kBM;
  const bool whole = tile_begin == 0 && q_tiles == all_tiles;
  // a partial range runs as pairs only when it starts on a pair and ends on one (or at the end)
  const bool pairable = tile_begin % 2 == 0 && (q_tiles % 2 == 0 || tile_begin + q_tiles == all_tiles);
  const long long units = static_cast<long long>(heads) * batch;
  const int n_pairs = (q_tiles + 1) / 2;
  const long long pair_units = n_pairs * units;
  for (int i = 0; i < kMaxPairs; ++i) plan.parts_of[i] = 1;
  // Pairs also win when they fit the SMs in one wave and the single tiles would not (measured at
  // B 16, H 6, S 256, D 64: 16.3 against 20.5 us).
  const bool one_wave_of_pairs = pair_units <= sms && static_cast<long long>(q_tiles) * units > sms;
  plan.pairs_without_split = q_tiles >= 2 && pairable && (pair_units >= 2LL * sms || one_wave_of_pairs);
  plan.pairs = q_tiles >= 2 && pairable && n_pairs <= kMaxPairItems;
  plan.pairs_without_split = plan.pairs_without_split && n_pairs <= kMaxPairItems;
  if (!plan.pairs || !whole || n_pairs > kMaxPairs || q_tiles < 8) {
    plan.pairs = plan.pairs_without_split;
    return plan;
  }
  if (static_cast<long long>(q_tiles) * units <= sms) {
    const int parts = pair_units * 2 >= 2LL * sms ? 2 : 4;
    for (int i = 0; i < n_pairs; ++i) plan.parts_of[i] = static_cast<uint8_t>(parts);
    plan.split = true;
    return plan;
  }
  long long total = 0;
  for (int i = 0; i < n_pairs; ++i) total += (2 * i + 1) + (2 * i + 1 < q_tiles ? 2 * i + 2 : 0);
  const double fair = static_cast<double>(total) * units / sms;
  // A pair is cut into ceil(work / (f . fair share)) parts; f is chosen by simulating the launch
  // (CTAs in schedule order onto the earliest free SM) with a CTA costing its key blocks plus a
  // fixed 11 blocks' worth of set-up and epilogue (13 when it writes partials), which reproduces
  // the measured times of 3 to 8 heads at S = 8192 within a few per cent.  Cutting at the fair
  // share itself leaves a second wave of half-length CTAs behind a first wave of full-length ones;
  // a somewhat finer cut fills the tail better, a much finer one pays too many fixed costs.
  // f = 0 stands for no cut at all; a plan with cuts also pays for the merge kernel (about 11 blocks).
  static const double kCuts[] = {0.0, 1.0, 0.85, 0.7, 0.6, 0.5};
  double best_time = 0.0;
  bool first = true;
  for (double f : kCuts) {
    uint8_t parts_of[kMaxPairs];
    bool any = false;
    for (int i = 0; i < n_pairs; ++i) {
      const int work = (2 * i + 1) + (2 * i + 1 < q_tiles ? 2 * i + 2 : 0);
      const int parts = f > 0.0 ? static_cast<int>((work + f * fair - 1e-9) / (f * fair)) : 1;
      parts_of[i] = static_cast<uint8_t>(parts < 1 ? 1 : (parts > 4 ? 4 : parts));
      any = any || parts_of[i] > 1;
    }
    if (!any && f > 0.0) continue;
    PairSchedule schedule;
    int work_of[kMaxPairItems];
    const int items = fill_pair_schedule(&schedule, tile_begin, q_tiles, parts_of, work_of);
    // earliest-free-SM simulation, CTAs in launch order: item-major, (sequence, head) fastest
    double free_at[256];
    const int machines = sms < 256 ? sms : 256;
    for (int m = 0; m < machines; ++m) free_at[m] = 0.0;
    auto place = [&](double cost) {
      for (long long u = 0; u < units; ++u) {
        int at = 0;
        for (int m = 1; m < machines; ++m)
          if (free_at[m] < free_at[at]) at = m;
        free_at[at] += cost;
      }
    };
    if (f == 0.0 && !plan.pairs_without_split) {
      // what runs without cuts here is the single-tile kernel: a key block costs 1.4 times as much
      // without the second tile to alternate with (5 heads at S = 8192: 102 us)
      for (int t = q_tiles - 1; t >= 0; --t) place(1.4 * (t + 1) + 11.0);
    } else {
      for (int i = 0; i < items; ++i) place(work_of[i] + ((schedule.meta[i] >> 4) > 1 ? 13.0 : 11.0));
    }
    double time = any ? 11.0 : 0.0;
    for (int m = 0; m < machines; ++m) time = free_at[m] > time ? free_at[m] + (any ? 11.0 : 0.0) : time;
    if (first || time < best_time) {
      first = false;
      best_time = time;
      plan.split = any;
      for (int i = 0; i < kMaxPairs; ++i) plan.parts_of[i] = i < n_pairs ? parts_of[i] : 1;
    }
  }
  if (!plan.split) plan.pairs = plan.pairs_without_split;
  return plan;
}

// The plan of a shape is computed once (the simulation above costs tens of microseconds).
static AttnFwdPlan attn_fwd_plan(int batch, int seq, int heads, int tile_begin, int q_tiles, int sms) {
  struct Entry { int key[6]; AttnFwdPlan plan; };
  static std::mutex mutex;
  static Entry cache[16];
  static int used = 0, next = 0;
  const int key[6] = {batch, seq, heads, tile_begin, q_tiles, sms};
  std::lock_guard<std::mutex> lock(mutex);
  for (int i = 0; i < used; ++i)
    if (memcmp(cache[i].key, key, sizeof(key)) == 0) return cache[i].plan;
  Entry& e = cache[next];
  memcpy(e.key, key, sizeof(key));
  e.plan = attn_fwd_plan_uncached(batch, seq, heads, tile_begin, q_tiles, sms);
  next = (next + 1) % 16;
  used = used < 16 ? used + 1 : 16;
  return e.plan;
}

// Items of pairs [tile_begin / 2, ...) sorted by length, longest first; returns their number.
static int fill_pair_schedule(PairSchedule* schedule, int tile_begin, int q_tiles, const uint8_t* parts_of,
                              int* work_of) {
  const int first = tile_begin / 2, last = (tile_begin + q_tiles + 1) / 2;   // pairs [first, last)
  struct Item { int work, pair, part, parts; };
  Item items[kMaxPairItems];
  int n = 0;
  for (int pair = last - 1; pair >= first && n < kMaxPairItems; --pair) {
    const int parts = parts_of != nullptr && pair < kMaxPairs ? parts_of[pair] : 1;
    const int blocks = 2 * pair + 2;
    const int chunk = (blocks + parts - 1) / parts;
    for (int part = 0; part < parts && n < kMaxPairItems; ++part) {
      const int lo = part * chunk, hi = lo + chunk < blocks ? lo + chunk : blocks;
      // key blocks of the two tiles inside [lo, hi): tile 2p has 2p + 1 of them, tile 2p + 1 has 2p + 2
      const int a0 = (hi < blocks - 1 ? hi : blocks - 1) - lo, a1 = hi - lo;
      items[n++] = Item{(a0 > 0 ? a0 : 0) + (a1 > 0 ? a1 : 0), pair, part, parts};
    }
  }
  for (int i = 1; i < n; ++i) {   // insertion sort, stable, descending by work
    const Item x = items[i];
    int j = i - 1;
    for (; j >= 0 && items[j].work < x.work; --j) items[j + 1] = items[j];
    items[j + 1] = x;
  }
  for (int i = 0; i < n; ++i) {
    schedule->pair[i] = static_cast<uint16_t>(items[i].pair);
    schedule->meta[i] = static_cast<uint8_t>(items[i].part | (items[i].parts << 4));
    if (work_of != nullptr) work_of[i] = items[i].work;
  }
  for (int i = 0; i < kMaxPairs; ++i) schedule->parts_of[i] = parts_of != nullptr ? parts_of[i] : 1;
  return n;
}

// Bytes of scratch attn_fwd_tc can use for this shape, 0 when it would not cut any pair.
size_t attn_fwd_tc_split_workspace_bytes(int batch, int seq, int heads, int head_dim) {
  int sms = 148, device = 0;
  if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const AttnFwdPlan plan = attn_fwd_plan(batch, seq, heads, 0, (seq + kBM - 1) / kBM, sms);
  return plan.split ? attn_fwd_tc_workspace_bytes(batch, seq, heads, head_dim) : 0;
}

// Partials of the key/value-split mode: a float4 record and D floats per (part, token, head), 4 parts.
size_t attn_fwd_tc_workspace_bytes(int batch, int seq, int heads, int head_dim) {
  const size_t units = static_cast<size_t>(batch) * seq * heads;
  return 4 * units * (sizeof(float4) + static_cast<size_t>(head_dim) * sizeof(float));
}

// See engine.h for the contract.  Returns cudaErrorInvalidValue when a tensor map cannot be
// encoded (misaligned base or stride).
cudaError_t attn_fwd_tc(cudaStream_t stream, const AttnFwdArgs& a) {
  CUtensorMap map_q, map_k, map_v;
  if (!make_token_map(&map_q, a.q, a.q_cols, a.seq, a.batch, a.q_token, kBM) ||
      !make_token_map(&map_k, a.k, a.kv_cols, a.seq, a.batch, a.kv_token, kBN) ||
      !make_token_map(&map_v, a.v, a.kv_cols, a.seq, a.batch, a.kv_token, kBN))
    return cudaErrorInvalidValue;
  FwdParams p;
  p.q_col0 = a.q_col0;
  p.k_col0 = a.k_col0;
  p.v_col0 = a.v_col0;
  p.q_head_cols = a.q_head_cols;
  p.kv_head_cols = a.head_dim;
  p.seq = a.seq;
  p.heads = a.heads;
  p.group = a.group;
  p.scale = 1.0f / sqrtf(static_cast<float>(a.head_dim));
  p.scale_log2 = p.scale * 1.4426950408889634f;
  p.out = static_cast<__nv_bfloat16*>(a.out);
  p.out_token = a.out_token;
  p.out_head = a.out_head;
  p.maxima = a.maxima;
  p.normalizers = a.normalizers;
  p.core = a.core;
  p.gate = static_cast<const __nv_bfloat16*>(a.gate);
  p.gate_token = a.gate_token;
  p.gate_head = a.gate_head;
  p.round_gate = a.round_gate;
  p.status = a.status;
  const int all_tiles = (a.seq + kBM - 1) / kBM;
  // a caller may ask for the query tiles [tile_begin, tile_begin + tile_count) only (rows of a
  // longer causal problem whose earlier rows were, or later rows will be, computed by other calls)
  const int tile_begin = a.tile_count > 0 ? a.tile_begin : 0;
  const int q_tiles = a.tile_count > 0 ? a.tile_count : all_tiles;
  if (tile_begin < 0 || tile_begin + q_tiles > all_tiles) return cudaErrorInvalidValue;
  p.tile_end = tile_begin + q_tiles;
  const size_t tile = static_cast<size_t>(a.head_dim / 64) * kSlabBytes;
  cudaError_t e;
  if (a.head_dim != 128 && a.head_dim != 64) return cudaErrorInvalidValue;
  // Two query tiles per CTA (ping-pong) run each tile faster but make coarser work units: the
  // longest unit of a causal sequence is then ~1/16 of one head's work.  With few heads per GPU
  // (head-sharded across 8 GPUs) that unit alone would exceed an SM's fair share, so the
  // single-tile kernel takes over when there are fewer than two units per SM.
  int sms = 148;
  {
    int device = 0;
    if (cudaGetDevice(&device) == cudaSuccess)
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  }
  const AttnFwdPlan plan = attn_fwd_plan(a.batch, a.seq, a.heads, tile_begin, q_tiles, sms);
  const bool split = plan.split && a.workspace != nullptr;
  p.split_pairs = split ? 1 : 0;
  p.part_o = nullptr;
  p.part_m = nullptr;
  if (split) {
    const size_t tokens = static_cast<size_t>(a.batch) * a.seq;
    p.part_m = static_cast<float4*>(a.workspace);
    p.part_o = reinterpret_cast<float*>(p.part_m + 4 * tokens * a.heads);
  }
  if (plan.pairs && (split || !plan.split || plan.pairs_without_split)) {
    // two query tiles per CTA in ping-pong
    PairSchedule schedule;
    const int items = fill_pair_schedule(&schedule, tile_begin, q_tiles, split ? plan.parts_of : nullptr, nullptr);
    const dim3 grid(a.heads * a.batch, items);
    const size_t smem = 1024 + tile * (2 + 2 * kStages) + sizeof(PairBarriers);
    auto kernel = a.head_dim == 128 ? attn_fwd_sm100_pair<128> : attn_fwd_sm100_pair<64>;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    kernel<<<grid, kThreadsPair, smem, stream>>>(map_q, map_k, map_v, p, schedule);
    if (split) {
      e = cudaGetLastError();
      if (e != cudaSuccess) return e;
      int first_pair = 0;
      while (first_pair < kMaxPairs && plan.parts_of[first_pair] <= 1) ++first_pair;
      const int first_token = first_pair * 2 * kBM;
      const long long rows = static_cast<long long>(a.batch) * (a.seq - first_token) * a.heads;
      const unsigned blocks = static_cast<unsigned>((rows + 7) / 8);
      // launched with programmatic stream serialisation: its CTAs are placed while the pair
      // kernel's last CTAs still run and wait for that grid before they read a partial
      cudaLaunchAttribute attribute;
      attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attribute.val.programmaticStreamSerializationAllowed = 1;
      cudaLaunchConfig_t config = {};
      config.gridDim = dim3(blocks);
      config.blockDim = dim3(256);
      config.stream = stream;
      config.attrs = &attribute;
      config.numAttrs = 1;
      if (a.head_dim == 128) return cudaLaunchKernelEx(&config, attn_fwd_merge<128>, p, a.batch, first_token, schedule);
      return cudaLaunchKernelEx(&config, attn_fwd_merge<64>, p, a.batch, first_token, schedule);
    }
  } else {
    const dim3 grid(a.heads * a.batch, q_tiles);
    const size_t smem = 1024 + tile * (1 + 2 * kStages) + sizeof(Barriers);
    auto kernel = a.head_dim == 128 ? attn_fwd_sm100<128> : attn_fwd_sm100<64>;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    kernel<<<grid, kThreadsFwd, smem, stream>>>(map_q, map_k, map_v, p);
  }
  return cudaGetLastError();
}

}  // namespace pluto
