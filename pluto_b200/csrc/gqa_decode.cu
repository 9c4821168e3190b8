// Grouped-query attention decode: one new query token per sequence against a KV cache.
//
// Stands in for FullAttentionKernel and the cached AttentionProbabilitiesKernel of the reference
// (src/llm/layers/util/cached_attention_ops.cc:83-126, :131-178), which run one program per query
// head (24-40 CTAs), re-read each KV head once per query head and keep the cache in fp32.  Here:
//   * the cache is read exactly once: all query heads of a KV head are the rows of one MMA tile;
//   * the sequence is split into fixed chunks across CTAs (split-KV); every CTA produces a
//     partial (max, sum, accumulator), the four consumer warps of a CTA merge through shared
//     memory, and a second kernel merges the chunks in a fixed order (deterministic, no atomics,
//     no inter-CTA waits);
//   * K/V tiles travel global -> shared as tiled TMA loads (no multicast) over a 4-D map of the
//     page pool (column, kv head, token in page, page): one elected thread issues a handful of
//     box copies per 64-token stage into a 3-stage ring guarded by mbarriers, 128-byte swizzled
//     so ldmatrix is bank-conflict free.  (Per-row bulk copies were tried first: at 256 bytes
//     per instruction the copy engine's per-instruction cost capped the kernel near 2 TB/s.)
//   * the arithmetic is bf16 mma.sync (m16n8k16) with fp32 accumulation -- the kernel is bound by
//     HBM bandwidth, the tensor path only has to stay out of the way.
// The cache is a page pool: token t of sequence b lives in page block_table[b][t / page_size]
// (or page b when there is no table: one contiguous region per sequence).
//
// A plain fp32 kernel covers every other case (fp32 cache, head widths other than 64/128,
// unrounded operands) with the same split/merge structure.
#include "common.cuh"
#include "engine.h"

namespace pluto {
namespace {

constexpr int kTile = 64;          // tokens per pipeline stage
constexpr int kDecodeStages = 3;
constexpr int kConsumerWarps = 4;  // 16 tokens of every tile each
constexpr int kDecodeThreads = (kConsumerWarps + 1) * 32;

// Sequence length as the kernels use it: the device value clamped into what the host sized the
// grid and the workspace for, [0, decode_chunk_capacity(splits, split_tokens)].  A value outside is a caller error; it
// is reported through the status word and the launch stays inside its buffers.
__device__ __forceinline__ int bounded_length(const DecodeArgs& a, int b, uint32_t site) {
  const int length = a.seq_lens[b];
  const long long limit = decode_chunk_capacity(a.splits, a.split_tokens);
  if (length < 0 || length > limit) {
    report_status(a.status, site, kBadLength);
    return length < 0 ? 0 : static_cast<int>(limit);
  }
  return length;
}

__device__ __forceinline__ const char* kv_row(const DecodeArgs& a, bool value, int b, int t,
                                              int kv_head, size_t element) {
  const void* base = value ? a.v_base : a.k_base;
  if (a.k_bases != nullptr) {   // separately allocated sequences
    const void* own = (value ? a.v_bases : a.k_bases)[b];
    return static_cast<const char*>(own) +
           (static_cast<size_t>(t) * a.token_stride + static_cast<size_t>(kv_head) * a.head_dim) * element;
  }
  int page = a.block_table ? a.block_table[static_cast<size_t>(b) * a.max_blocks + t / a.page_size]
                           : b;
  if (a.block_table && a.num_pages > 0 && (page < 0 || page >= a.num_pages)) {
    report_status(a.status, 35, kBadPage);   // the tiled-TMA path reads zeros there instead
    page = 0;
  }
  const size_t offset = static_cast<size_t>(page) * a.page_stride +
                        static_cast<size_t>(t % a.page_size) * a.token_stride +
                        static_cast<size_t>(kv_head) * a.head_dim;
  return static_cast<const char*>(base) + offset * element;
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct DecodeBarriers {
  uint64_t full[kDecodeStages];
  uint64_t empty[kDecodeStages];
};

// grid (kv_heads, batch, splits), chunks in decreasing index order.  Partials: acc [B, Hq, splits, D], ml [B, Hq, splits, 2].
template <int D>
__global__ void __launch_bounds__(kDecodeThreads, 2)
gqa_decode_tc(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
              DecodeArgs a) {
  constexpr int kHalves = D / 64;                 // 64-column (128-byte) swizzled slabs per row
  constexpr int kHalfBytes = kTile * 128;         // one slab of a tile
  constexpr int kTileBytes = kHalves * kHalfBytes;
  constexpr int kStageBytes = 2 * kTileBytes;     // K tile then V tile
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  DecodeBarriers* bar = reinterpret_cast<DecodeBarriers*>(smem + kDecodeStages * kStageBytes);

  pdl_launch_dependents();   // the merge may be placed as SMs free up; it waits for this grid itself
  // chunks in decreasing index order, (KV head, sequence) fastest: the four short chunks of every
  // sequence are the last CTAs of the launch
  const int split = gridDim.z - 1 - blockIdx.z, kv_head = blockIdx.x, b = blockIdx.y;
  const int length = bounded_length(a, b, 36);
  const int begin = decode_chunk_begin(split, a.split_tokens);
  if (begin >= length) return;  // whole CTA leaves before touching any barrier
  const int end = min(length, begin + decode_chunk_tokens(split, a.split_tokens));
  const int tiles = (end - begin + kTile - 1) / kTile;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int group = a.q_heads / a.kv_heads;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kDecodeStages; ++s) {
      mbar_init(&bar->full[s], 1);
      mbar_init(&bar->empty[s], kConsumerWarps);
    }
    mbar_fence_init();
  }
  __syncthreads();

  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
  float o[D / 8][4];

  if (warp == kConsumerWarps) {
    // ---------------------------------------------------------------- producer warp
    if (lane == 0) {
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      bool ok = true;
      const int rows = a.box_rows;  // tokens per box: divides both the tile and the page size
      for (int it = 0; it < tiles && ok; ++it) {
        const int st = it % kDecodeStages, use = it / kDecodeStages;
        if (use > 0) ok = mbar_wait(&bar->empty[st], (use - 1) & 1, a.status, 30);
        if (!ok) break;
        const int t0 = begin + it * kTile;
        const int boxes = min(kTile, end - t0 + rows - 1) / rows;  // boxes that hold a live token
        mbar_expect_tx(&bar->full[st], static_cast<uint32_t>(boxes) * rows * D * 2 * 2);
        uint8_t* k_tile = smem + st * kStageBytes;
        uint8_t* v_tile = k_tile + kTileBytes;
        for (int bx = 0; bx < boxes; ++bx) {
          const int t = t0 + bx * rows;
          const int page = a.block_table
                               ? a.block_table[static_cast<size_t>(b) * a.max_blocks + t / a.page_size]
                               : b;
          const int in_page = t % a.page_size;
#pragma unroll
          for (int h = 0; h < kHalves; ++h) {
            tma_load_4d(k_tile + h * kHalfBytes + bx * rows * 128, &map_k, h * 64, kv_head, in_page,
                        page, &bar->full[st]);
            tma_load_4d(v_tile + h * kHalfBytes + bx * rows * 128, &map_v, h * 64, kv_head, in_page,
                        page, &bar->full[st]);
          }
        }
      }
      // all copies this thread started must have landed before the CTA may exit
      for (int it = max(0, tiles - kDecodeStages); it < tiles; ++it)
        mbar_wait(&bar->full[it % kDecodeStages], (it / kDecodeStages) & 1, a.status, 31);
    }
  } else {
    // ---------------------------------------------------------------- consumer warps
    // A fragments of Q: rows = query heads of this KV head (rows >= group are zero).
    uint32_t qf[D / 16][4];
    {
      const int r0 = lane / 4, r1 = r0 + 8;
      const size_t head0 = static_cast<size_t>(b) * a.q_heads + static_cast<size_t>(kv_head) * group;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int col = ks * 16 + half * 8 + (lane % 4) * 2;
          float x0 = 0.f, x1 = 0.f, y0 = 0.f, y1 = 0.f;
          if (a.q_is_bf16) {
            const __nv_bfloat16* q = static_cast<const __nv_bfloat16*>(a.q);
            if (r0 < group) { x0 = __bfloat162float(q[(head0 + r0) * D + col]); x1 = __bfloat162float(q[(head0 + r0) * D + col + 1]); }
            if (r1 < group) { y0 = __bfloat162float(q[(head0 + r1) * D + col]); y1 = __bfloat162float(q[(head0 + r1) * D + col + 1]); }
          } else {
            const float* q = static_cast<const float*>(a.q);
            if (r0 < group) { x0 = q[(head0 + r0) * D + col]; x1 = q[(head0 + r0) * D + col + 1]; }
            if (r1 < group) { y0 = q[(head0 + r1) * D + col]; y1 = q[(head0 + r1) * D + col + 1]; }
          }
          qf[ks][half * 2 + 0] = pack_bf16(x0, x1);
          qf[ks][half * 2 + 1] = pack_bf16(y0, y1);
        }
      }
    }
#pragma unroll
    for (int nb = 0; nb < D / 8; ++nb)
#pragma unroll
      for (int i = 0; i < 4; ++i) o[nb][i] = 0.0f;
    const float scale_log2 = a.scale * 1.4426950408889634f;
    bool ok = true;
    for (int it = 0; it < tiles && ok; ++it) {
      const int st = it % kDecodeStages;
      ok = mbar_wait(&bar->full[st], (it / kDecodeStages) & 1, a.status, 32);
      if (!ok) break;
      const uint32_t k_tile = smem_u32(smem + st * kStageBytes);
      const uint32_t v_tile = k_tile + kTileBytes;
      const int live = end - (begin + it * kTile);  // live tokens in this tile (may exceed kTile)
      if (live < (warp + 1) * 16) {
        // Rows past the sequence end hold whatever the page (or an earlier stage) held; their
        // probabilities are zero, but 0 * NaN would poison P V, so this warp clears its own dead
        // V rows first.  Only the last tile of a sequence takes this path.
        for (int r = max(live, warp * 16); r < (warp + 1) * 16; ++r)
          for (int c = lane; c < kHalves * 8; c += 32)
            sts_b32x4(smem_u32(smem) + st * kStageBytes + kTileBytes + (c / 8) * kHalfBytes + r * 128 +
                          (c % 8) * 16, 0u, 0u, 0u, 0u);
        fence_proxy_async();
        __syncwarp();
      }
      // ---- S = Q K^T for this warp's 16 tokens: two n-blocks of 8 tokens
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
        for (int kp = 0; kp < D / 32; ++kp) {
          uint32_t kf[4];
          // element (row, col) of a tile sits in slab col/64 at row*128 + ((col%64)/8 ^ row%8)*16
          const int row = warp * 16 + nb * 8 + lane % 8;
          const int chunk = (kp * 4 + lane / 8) % 8;
          ldmatrix_x4(kf, k_tile + (kp / 2) * kHalfBytes + row * 128 + ((chunk ^ (row % 8)) * 16));
          mma_bf16(s[nb], qf[2 * kp], kf[0], kf[1]);
          mma_bf16(s[nb], qf[2 * kp + 1], kf[2], kf[3]);
        }
      }
      // ---- online softmax (rows lane/4 and lane/4+8; columns = tokens)
      const int token0 = begin + it * kTile + warp * 16 + (lane % 4) * 2;
      float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nb = 0; nb < 2; ++nb)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int token = token0 + nb * 8 + (i & 1);
          s[nb][i] = token < end ? s[nb][i] * scale_log2 : -INFINITY;
          tile_max[i >> 1] = fmaxf(tile_max[i >> 1], s[nb][i]);
        }
      // P is split into a bf16 high part and a bf16 remainder so that P V keeps ~16 mantissa
      // bits: the result then tracks the fp32 reference to ~1e-5 instead of a bf16 ulp, and the
      // extra MMAs are free in a bandwidth-bound kernel.
      uint32_t pf[4], pl[4];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
        const float m_new = fmaxf(m_run[r], tile_max[r]);
        const float m_safe = m_new == -INFINITY ? 0.0f : m_new;
        const float correction = fast_exp2(m_run[r] - m_safe);
        const float p00 = fast_exp2(s[0][2 * r] - m_safe), p01 = fast_exp2(s[0][2 * r + 1] - m_safe);
        const float p10 = fast_exp2(s[1][2 * r] - m_safe), p11 = fast_exp2(s[1][2 * r + 1] - m_safe);
        float sum = p00 + p01 + p10 + p11;
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        l_run[r] = l_run[r] * correction + sum;
        m_run[r] = m_new;
        pf[r] = pack_bf16(p00, p01);      // a0 / a1: tokens 0-7
        pf[2 + r] = pack_bf16(p10, p11);  // a2 / a3: tokens 8-15
        pl[r] = pack_bf16(p00 - bf16_lo(pf[r]), p01 - bf16_hi(pf[r]));
        pl[2 + r] = pack_bf16(p10 - bf16_lo(pf[2 + r]), p11 - bf16_hi(pf[2 + r]));
#pragma unroll
        for (int nb = 0; nb < D / 8; ++nb) {
          o[nb][2 * r] *= correction;
          o[nb][2 * r + 1] *= correction;
        }
      }
      // ---- O += P V
#pragma unroll
      for (int np = 0; np < D / 16; ++np) {
        uint32_t vf[4];
        const int row = warp * 16 + ((lane / 8) & 1) * 8 + lane % 8;
        const int chunk = (np * 2 + lane / 16) % 8;
        ldmatrix_x4_trans(vf, v_tile + (np / 4) * kHalfBytes + row * 128 + ((chunk ^ (row % 8)) * 16));
        mma_bf16(o[2 * np], pf, vf[0], vf[1]);
        mma_bf16(o[2 * np], pl, vf[0], vf[1]);
        mma_bf16(o[2 * np + 1], pf, vf[2], vf[3]);
        mma_bf16(o[2 * np + 1], pl, vf[2], vf[3]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->empty[st]);
    }
  }
  __syncthreads();  // every stage consumed, every copy landed: the ring can be reused as scratch

  // ---- merge the four warps' partial softmax states through shared memory (ld.shared / st.shared
  // by address: `smem` went through alignment arithmetic and is a generic pointer to the compiler)
  const uint32_t scratch = smem_u32(smem);                               // fp32 [warps][16][D]
  const uint32_t scratch_ml = scratch + kConsumerWarps * 16 * D * 4;     // fp32 [warps][16][2]
  if (warp < kConsumerWarps) {
    const int r0 = lane / 4;
#pragma unroll
    for (int nb = 0; nb < D / 8; ++nb) {
      const int col = nb * 8 + (lane % 4) * 2;
      sts_f32(scratch + ((warp * 16 + r0) * D + col) * 4, o[nb][0]);
      sts_f32(scratch + ((warp * 16 + r0) * D + col + 1) * 4, o[nb][1]);
      sts_f32(scratch + ((warp * 16 + r0 + 8) * D + col) * 4, o[nb][2]);
      sts_f32(scratch + ((warp * 16 + r0 + 8) * D + col + 1) * 4, o[nb][3]);
    }
    if (lane % 4 == 0) {
      sts_f32(scratch_ml + ((warp * 16 + r0) * 2) * 4, m_run[0]);
      sts_f32(scratch_ml + ((warp * 16 + r0) * 2 + 1) * 4, l_run[0]);
      sts_f32(scratch_ml + ((warp * 16 + r0 + 8) * 2) * 4, m_run[1]);
      sts_f32(scratch_ml + ((warp * 16 + r0 + 8) * 2 + 1) * 4, l_run[1]);
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < group * D; idx += kDecodeThreads) {
    const int r = idx / D, d = idx % D;
    float m_w[kConsumerWarps], m_tot = -INFINITY;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; ++w) {
      m_w[w] = lds_f32(scratch_ml + ((w * 16 + r) * 2) * 4);
      m_tot = fmaxf(m_tot, m_w[w]);
    }
    float acc = 0.0f, l_tot = 0.0f;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; ++w) {
      const float f = fast_exp2(m_w[w] - m_tot);
      acc += lds_f32(scratch + ((w * 16 + r) * D + d) * 4) * f;
      l_tot += lds_f32(scratch_ml + ((w * 16 + r) * 2 + 1) * 4) * f;
    }
    const size_t head = static_cast<size_t>(b) * a.q_heads + static_cast<size_t>(kv_head) * group + r;
    const size_t slot = head * a.splits + split;
    a.partial_acc[slot * D + d] = acc;
    if (d == 0) {
      a.partial_ml[slot * 2] = m_tot;
      a.partial_ml[slot * 2 + 1] = l_tot;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Exact fp32 kernel with the same split structure: grid (q_heads, batch, splits), one warp per
// token row in flight, each lane owning head_dim/32 (<= 8) channels.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) gqa_decode_generic(DecodeArgs a) {
  pdl_launch_dependents();
  const int split = gridDim.z - 1 - blockIdx.z, head = blockIdx.x, b = blockIdx.y;
  const int length = bounded_length(a, b, 37);
  const int begin = decode_chunk_begin(split, a.split_tokens);
  if (begin >= length) return;
  const int end = min(length, begin + decode_chunk_tokens(split, a.split_tokens));
  const int D = a.head_dim, kv_head = head / (a.q_heads / a.kv_heads);
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const size_t element = a.kv_is_bf16 ? 2 : 4;
  float q[8], acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int d = lane + 32 * i;
    const size_t idx = (static_cast<size_t>(b) * a.q_heads + head) * D + d;
    q[i] = d < D ? (a.q_is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(a.q)[idx])
                                : static_cast<const float*>(a.q)[idx])
                 : 0.0f;
    acc[i] = 0.0f;
  }
  float m = -INFINITY, l = 0.0f;
  for (int t = begin + warp; t < end; t += 4) {
    const char* kr = kv_row(a, false, b, t, kv_head, element);
    const char* vr = kv_row(a, true, b, t, kv_head, element);
    float dot = 0.0f, v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int d = lane + 32 * i;
      float kx = 0.0f;
      v[i] = 0.0f;
      if (d < D) {
        if (a.kv_is_bf16) {
          kx = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(kr)[d]);
          v[i] = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(vr)[d]);
        } else {
          kx = reinterpret_cast<const float*>(kr)[d];
          v[i] = reinterpret_cast<const float*>(vr)[d];
        }
      }
      dot = fmaf(kx, q[i], dot);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    const float s = dot * a.scale;
    const float m_new = fmaxf(m, s);
    const float correction = expf(m - m_new), p = expf(s - m_new);
    l = l * correction + p;
    m = m_new;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = fmaf(p, v[i], acc[i] * correction);
  }
  __shared__ float sh_acc[4][256];
  __shared__ float sh_ml[4][2];
#pragma unroll
  for (int i = 0; i < 8; ++i) sh_acc[warp][lane + 32 * i] = acc[i];
  if (lane == 0) { sh_ml[warp][0] = m; sh_ml[warp][1] = l; }
  __syncthreads();
  float m_tot = fmaxf(fmaxf(sh_ml[0][0], sh_ml[1][0]), fmaxf(sh_ml[2][0], sh_ml[3][0]));
  const size_t slot = (static_cast<size_t>(b) * a.q_heads + head) * a.splits + split;
  for (int d = threadIdx.x; d < D; d += 128) {
    float sum = 0.0f;
    for (int w = 0; w < 4; ++w) sum += sh_acc[w][d] * expf(sh_ml[w][0] - m_tot);
    a.partial_acc[slot * D + d] = sum;
  }
  if (threadIdx.x == 0) {
    float l_tot = 0.0f;
    for (int w = 0; w < 4; ++w) l_tot += sh_ml[w][1] * expf(sh_ml[w][0] - m_tot);
    // partial maxima are kept in log2 units so both producers feed one merge kernel
    a.partial_ml[slot * 2] = m_tot * 1.4426950408889634f;
    a.partial_ml[slot * 2 + 1] = l_tot;
  }
}

// Merge of the per-chunk partials in chunk order, then the reference's output stage
// (cached_attention_ops.cc:120-125): out = R(R(acc/l) * R(sigmoid(gate))).  grid (q_heads, batch),
// 128 threads.  The chunks' maxima are reduced in parallel and every chunk's weight
// 2^(m_s - m) is computed once, by one thread, into shared memory; the sums then run over the
// chunks in order (so the result does not depend on the thread count) with the loads of eight
// chunks in flight.
constexpr int kMergeThreads = 128;
constexpr int kMergeSplits = 1024;   // chunk weights held in shared memory per pass

__global__ void __launch_bounds__(kMergeThreads) gqa_decode_merge(DecodeArgs a) {
  pdl_wait();   // the chunk kernel's partials are complete and visible from here on
  const int head = blockIdx.x, b = blockIdx.y, D = a.head_dim;
  const int length = bounded_length(a, b, 38);
  const int splits = decode_chunk_count(length, a.split_tokens);   // <= a.splits
  if (length <= 0) {
    // nothing to attend to (a caller error: lengths are >= 1): zeros, not 0/0
    for (int d = threadIdx.x; d < D; d += kMergeThreads) {
      const size_t idx = (static_cast<size_t>(b) * a.q_heads + head) * D + d;
      if (a.out_is_bf16) static_cast<__nv_bfloat16*>(a.out)[idx] = __float2bfloat16_rn(0.0f);
      else static_cast<float*>(a.out)[idx] = 0.0f;
    }
    if (threadIdx.x == 0 && a.lse) a.lse[static_cast<size_t>(b) * a.q_heads + head] = -INFINITY;
    return;
  }
  const size_t slot0 = (static_cast<size_t>(b) * a.q_heads + head) * a.splits;
  __shared__ float weight[kMergeSplits];   // 2^(m_s - m_tot)
  __shared__ float scaled_l[kMergeSplits]; // l_s * weight_s
  __shared__ float warp_max[kMergeThreads / 32];
  const float2* ml = reinterpret_cast<const float2*>(a.partial_ml) + slot0;   // (m_s, l_s)

  float m_part = -INFINITY;
  for (int s = threadIdx.x; s < splits; s += kMergeThreads) m_part = fmaxf(m_part, ml[s].x);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m_part = fmaxf(m_part, __shfl_xor_sync(0xffffffffu, m_part, o));
  if (threadIdx.x % 32 == 0) warp_max[threadIdx.x / 32] = m_part;
  __syncthreads();
  float m_tot = warp_max[0];
#pragma unroll
  for (int w = 1; w < kMergeThreads / 32; ++w) m_tot = fmaxf(m_tot, warp_max[w]);

  float l_tot = 0.0f;
  float acc[2] = {0.0f, 0.0f};               // channels threadIdx.x and threadIdx.x + 128
  for (int s0 = 0; s0 < splits; s0 += kMergeSplits) {
    const int count = min(kMergeSplits, splits - s0);
    __syncthreads();                          // the previous pass is done with the arrays
    for (int s = threadIdx.x; s < count; s += kMergeThreads) {
      const float2 v = ml[s0 + s];
      const float w = exp2f(v.x - m_tot);
      weight[s] = w;
      scaled_l[s] = v.y * w;
    }
    __syncthreads();
    for (int s = 0; s < count; ++s) l_tot += scaled_l[s];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int d = threadIdx.x + c * kMergeThreads;
      if (d >= D) continue;
      const float* column = a.partial_acc + (slot0 + s0) * D + d;
      int s = 0;
      for (; s + 8 <= count; s += 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = column[static_cast<size_t>(s + u) * D];
#pragma unroll
        for (int u = 0; u < 8; ++u) acc[c] += v[u] * weight[s + u];
      }
      for (; s < count; ++s) acc[c] += column[static_cast<size_t>(s) * D] * weight[s];
    }
  }
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    const int d = threadIdx.x + c * kMergeThreads;
    if (d >= D) continue;
    float value = acc[c] / l_tot;
    if (a.round) value = bf16_round(value);
    if (a.gate) {
      const size_t g = static_cast<size_t>(b) * a.gate_token + static_cast<size_t>(head) * a.gate_head + d;
      const float x = a.gate_is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(a.gate)[g])
                                     : static_cast<const float*>(a.gate)[g];
      float sigmoid = 1.0f / (1.0f + expf(-x));
      if (a.round) sigmoid = bf16_round(sigmoid);
      value *= sigmoid;
      if (a.round) value = bf16_round(value);
    }
    const size_t idx = (static_cast<size_t>(b) * a.q_heads + head) * D + d;
    if (a.out_is_bf16) static_cast<__nv_bfloat16*>(a.out)[idx] = __float2bfloat16_rn(value);
    else static_cast<float*>(a.out)[idx] = value;
  }
  if (threadIdx.x == 0 && a.lse) {
    // natural-log sum-exp of the scaled scores
    a.lse[static_cast<size_t>(b) * a.q_heads + head] = m_tot * 0.6931471805599453f + logf(l_tot);
  }
}

// Two-pass softmax row per (head, sequence) for the inspection hook: row (b, h) of `length`
// entries starts at probs + b*batch_stride + h*head_stride.  grid (q_heads, batch), 256 threads.
__global__ void __launch_bounds__(256) gqa_decode_probs(DecodeArgs a, float* probs,
                                                        size_t batch_stride, size_t head_stride) {
  const int head = blockIdx.x, b = blockIdx.y, D = a.head_dim;
  const int length = a.seq_lens[b];
  const int kv_head = head / (a.q_heads / a.kv_heads);
  const size_t element = a.kv_is_bf16 ? 2 : 4;
  float* row = probs + static_cast<size_t>(b) * batch_stride + static_cast<size_t>(head) * head_stride;
  __shared__ float red[256];
  const size_t q0 = (static_cast<size_t>(b) * a.q_heads + head) * D;
  float local_max = -INFINITY;
  for (int t = threadIdx.x; t < length; t += 256) {
    const char* kr = kv_row(a, false, b, t, kv_head, element);
    float dot = 0.0f;
    for (int d = 0; d < D; ++d) {
      const float kx = a.kv_is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(kr)[d])
                                    : reinterpret_cast<const float*>(kr)[d];
      const float qx = a.q_is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(a.q)[q0 + d])
                                   : static_cast<const float*>(a.q)[q0 + d];
      dot = fmaf(kx, qx, dot);
    }
    row[t] = dot * a.scale;
    local_max = fmaxf(local_max, dot * a.scale);
  }
  red[threadIdx.x] = local_max;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) red[threadIdx.x] = fmaxf(red[threadIdx.x], red[threadIdx.x + o]);
    __syncthreads();
  }
  const float m = red[0];
  __syncthreads();
  float local_sum = 0.0f;
  for (int t = threadIdx.x; t < length; t += 256) local_sum += expf(row[t] - m);
  red[threadIdx.x] = local_sum;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  const float inv = 1.0f / red[0];
  for (int t = threadIdx.x; t < length; t += 256) row[t] = expf(row[t] - m) * inv;
}

template <int D>
constexpr size_t decode_smem() {
  return 1024 + kDecodeStages * 2 * kTile * D * 2 + sizeof(DecodeBarriers);
}

// 4-D map of a bf16 page pool: (column, kv head, token in page, page); box = 64 columns x
// box_rows tokens of one kv head, 128-byte swizzle, zero fill outside the pool.
bool make_pool_map(CUtensorMap* map, const void* base, const DecodeArgs& a, int pages) {
  using Encode = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                              const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                              const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static Encode encode = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &result) !=
            cudaSuccess || result != cudaDriverEntryPointSuccess)
      return static_cast<Encode>(nullptr);
    return reinterpret_cast<Encode>(sym);
  }();
  if (encode == nullptr) return false;
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(a.head_dim), static_cast<cuuint64_t>(a.kv_heads),
                              static_cast<cuuint64_t>(a.page_size), static_cast<cuuint64_t>(pages)};
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>(a.head_dim) * 2, a.token_stride * 2,
                                 a.page_stride * 2};
  const cuuint32_t box[4] = {64, 1, static_cast<cuuint32_t>(a.box_rows), 1};
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides,
                box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) ==
         CUDA_SUCCESS;
}

}  // namespace

bool gqa_decode_uses_tensor_cores(const DecodeArgs& a) {
  const int group = a.q_heads / a.kv_heads;
  const int pages = a.block_table ? a.num_pages : a.batch;
  return a.k_bases == nullptr && a.kv_is_bf16 && (a.head_dim == 64 || a.head_dim == 128) && group <= 16 &&
         (a.round || a.q_is_bf16) && a.token_stride % 8 == 0 && a.page_stride % 8 == 0 &&
         a.page_size % 16 == 0 && pages > 0 &&
         (reinterpret_cast<uintptr_t>(a.k_base) & 15u) == 0 &&
         (reinterpret_cast<uintptr_t>(a.v_base) & 15u) == 0;
}

cudaError_t gqa_decode(cudaStream_t stream, const DecodeArgs& args) {
  DecodeArgs a = args;
  if (gqa_decode_uses_tensor_cores(a)) {
    const dim3 grid(a.kv_heads, a.batch, a.splits);
    cudaError_t e;
    a.box_rows = a.page_size % kTile == 0 ? kTile : 16;
    const int pages = a.block_table ? a.num_pages : a.batch;
    CUtensorMap map_k, map_v;
    if (!make_pool_map(&map_k, a.k_base, a, pages) || !make_pool_map(&map_v, a.v_base, a, pages))
      return cudaErrorInvalidValue;
    if (a.head_dim == 128) {
      e = cudaFuncSetAttribute(gqa_decode_tc<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(decode_smem<128>()));
      if (e != cudaSuccess) return e;
      gqa_decode_tc<128><<<grid, kDecodeThreads, decode_smem<128>(), stream>>>(map_k, map_v, a);
    } else {
      e = cudaFuncSetAttribute(gqa_decode_tc<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(decode_smem<64>()));
      if (e != cudaSuccess) return e;
      gqa_decode_tc<64><<<grid, kDecodeThreads, decode_smem<64>(), stream>>>(map_k, map_v, a);
    }
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  } else {
    gqa_decode_generic<<<dim3(a.q_heads, a.batch, a.splits), 128, 0, stream>>>(a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  // The merge is launched with programmatic stream serialisation: its CTAs are placed while the
  // chunk kernel's last CTAs still run, and wait for that grid before they read a partial.
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(a.q_heads, a.batch);
  config.blockDim = dim3(kMergeThreads);
  config.stream = stream;
  config.attrs = &attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, gqa_decode_merge, a);
}

cudaError_t gqa_decode_probabilities(cudaStream_t stream, const DecodeArgs& a, float* probs,
                                     size_t batch_stride, size_t head_stride) {
  gqa_decode_probs<<<dim3(a.q_heads, a.batch), 256, 0, stream>>>(a, probs, batch_stride, head_stride);
  return cudaGetLastError();
}

}  // namespace pluto
