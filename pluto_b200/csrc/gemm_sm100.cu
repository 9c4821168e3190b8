// Dense projection GEMMs on the Blackwell tensor cores for the trainable form of
// FullyConnectedLayer (src/llm/layers/fully_connected.cc:97-232, 415-520):
//     forward          Y  = cast(X) cast(W) + b          [rows, out]   (activation dtype)
//     input gradient   dX = cast(dY) cast(W)^T           [rows, in]    fp32
//     weight gradient  dW = cast(X)^T cast(dY)           [in, out]     fp32 (overwritten)
//     bias gradient    db = column sums of dY            [out]         fp32 (overwritten)
// with fp32 master weights W [in, out], and `cast` = bf16 for bf16 activations, fp16 for the
// fp32-activation ("FP16") policy, fp32 accumulation -- the operand types of the reference's
// 64x64 tile MMAs.
//
// Here the operands are first cast once into zero-padded 2-byte copies (every extent rounded up to
// 128), so that all three products are the same kernel: C[M,N] = sum_k A(m,k) B(k,n) over
// 128 x 256 x 64 tiles (a 128 x 128 tile needs more shared-memory fill bandwidth per MMA cycle
// than an SM gets from L2), TMA-staged through a 4-stage shared-memory ring with 128-byte swizzle,
// tcgen05.mma with the accumulator in TMEM, and the two operand layouts the products need:
//   K-major   (k contiguous:  X for the forward, dY and W for dX)
//   MN-major  (m or n contiguous: W for the forward, X and dY for dW), read as 64-wide slabs.
// One persistent CTA per SM walks its output tiles: warp 0 issues the TMA loads, warp 1 the MMA
// schedule with one elected issuing lane into one of two TMEM accumulators, warps 4-7 move the
// other accumulator to global memory (one row per thread) adding the bias.  Products with at least
// one 256 x 256 tile per pair of SMs run the same schedule on clusters of two CTAs
// (gemm_sm100_pair, tcgen05.mma.cta_group::2).  All waits are bounded.
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "common.cuh"
#include "engine.h"

namespace pluto {
namespace {

constexpr int kTile = 128, kTileN = 256, kBK = 64, kGemmStages = 4, kGemmThreads = 256;
constexpr int kSlab = 64 * kBK * 2;              // one [64 x 64] 2-byte slab: 8 KB
constexpr int kABytes = kTile * kBK * 2;         // 16 KB per stage
constexpr int kBBytes = kTileN * kBK * 2;        // 32 KB per stage

struct GemmParams {
  int M, N;            // valid extent of C
  int k_tiles;         // K steps of 64 (over both halves of a split operand)
  int a_wrap, b_wrap;  // K steps per half: step kt reads A at (kt % a_wrap, half kt / a_wrap) and B at
                       // kt % b_wrap, so [hi | lo] * [B; B] needs neither B twice nor a wide A
  int c_accumulate;    // add to C instead of overwriting (single writer per element)
  uint32_t idesc;
  const float* bias;   // optional [N]
  void* c;             // row-major, ldc elements between rows
  size_t ldc;
  int c_kind;          // 0 fp32, 1 bf16
  uint32_t* status;
};

struct GemmBarriers {
  uint64_t full[kGemmStages], empty[kGemmStages], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
};

// kind::f16 instruction descriptor: D fp32; A/B format 0 = f16, 1 = bf16; major bits 15 (A) and
// 16 (B): 0 = K-major, 1 = MN-major; N >> 3 at [17,23), M >> 4 at [24,29).
constexpr uint32_t gemm_idesc(int format, bool a_mn, bool b_mn) {
  return (1u << 4) | (static_cast<uint32_t>(format) << 7) | (static_cast<uint32_t>(format) << 10) |
         (static_cast<uint32_t>(a_mn) << 15) | (static_cast<uint32_t>(b_mn) << 16) |
         (static_cast<uint32_t>(kTileN >> 3) << 17) | (static_cast<uint32_t>(kTile >> 4) << 24);
}

// Persistent: gridDim.x CTAs (one per SM) take the output tiles i = blockIdx.x, blockIdx.x +
// gridDim.x, ...  Tiles are numbered along M first inside bands of kBand tile columns, so the CTAs
// that run at the same time share B tiles (and neighbouring A tiles) in L2.  Two 256-column
// accumulators in TMEM alternate: the epilogue warps drain one while the MMA warp fills the other.
constexpr int kBand = 4;
__device__ __forceinline__ void tile_origin(int tile, int m_tiles, int n_tiles, int& m0, int& n0) {
  const int band = tile / (kBand * m_tiles);
  const int width = min(kBand, n_tiles - band * kBand);
  const int within = tile - band * kBand * m_tiles;
  m0 = (within / width) * kTile;
  n0 = (band * kBand + within % width) * kTileN;
}

// One epilogue warp's 32 rows x 256 columns of an accumulator to global memory, adding the bias.
// Each thread holds a row (that is how tcgen05.ld delivers it), and a thread writing its own row
// makes every store instruction of the warp touch 32 lines; so full, aligned 32-column blocks pass
// through a 4 KB per-warp staging tile (16-byte chunk c of row r at position c ^ (r & 7), or
// c ^ ((r >> 1) & 3) for 64-byte bf16 rows) and leave with 8 (fp32) or 4 (bf16) lanes per row.
// Ragged or unaligned blocks keep the row-per-thread stores.
constexpr int kDrainStageBytes = 4 * 32 * 32 * 4;   // four epilogue warps
__device__ __forceinline__ void drain_accumulator(uint32_t acc_tmem, int m0_warp, int lane, int n0,
                                                  const GemmParams& p, uint32_t stage) {
  const bool vec = (p.ldc % 4 == 0) && (reinterpret_cast<uintptr_t>(p.c) % 16 == 0);
  const bool vec16 = p.ldc % 8 == 0 && reinterpret_cast<uintptr_t>(p.c) % 16 == 0;
  const int m = m0_warp + lane;
#pragma unroll 2
  for (int c = 0; c < kTileN / 32; ++c) {
    uint32_t acc[32];
    tmem_ld32(acc_tmem + c * 32, acc);
    tmem_wait_ld();
    const int n_base = n0 + c * 32;
    if (m0_warp >= p.M || n_base >= p.N) continue;   // (uniform over the warp)
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      v[i] = __uint_as_float(acc[i]);
      if (p.bias != nullptr && n_base + i < p.N) v[i] += p.bias[n_base + i];
    }
    const bool full = n_base + 32 <= p.N;
    if (p.c_kind == 0 && vec && full) {
      float* block = static_cast<float*>(p.c) + static_cast<size_t>(m0_warp) * p.ldc + n_base;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        sts_b32x4(stage + lane * 128 + ((i ^ (lane & 7)) << 4), __float_as_uint(v[4 * i]),
                  __float_as_uint(v[4 * i + 1]), __float_as_uint(v[4 * i + 2]), __float_as_uint(v[4 * i + 3]));
      __syncwarp();
#pragma unroll
      for (int pass = 0; pass < 8; ++pass) {
        const int r = pass * 4 + lane / 8, piece = lane % 8;
        const uint4 raw = lds_b32x4(stage + r * 128 + ((piece ^ (r & 7)) << 4));
        if (m0_warp + r < p.M) {
          float4* dst = reinterpret_cast<float4*>(block + static_cast<size_t>(r) * p.ldc + piece * 4);
          float4 out = make_float4(__uint_as_float(raw.x), __uint_as_float(raw.y), __uint_as_float(raw.z),
                                   __uint_as_float(raw.w));
          if (p.c_accumulate) {
            const float4 old = *dst;
            out.x += old.x; out.y += old.y; out.z += old.z; out.w += old.w;
          }
          *dst = out;
        }
      }
      __syncwarp();
    } else if (p.c_kind == 1 && vec16 && full) {
      __nv_bfloat16* block = static_cast<__nv_bfloat16*>(p.c) + static_cast<size_t>(m0_warp) * p.ldc + n_base;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        sts_b32x4(stage + lane * 64 + ((i ^ ((lane >> 1) & 3)) << 4), pack_bf16(v[8 * i], v[8 * i + 1]),
                  pack_bf16(v[8 * i + 2], v[8 * i + 3]), pack_bf16(v[8 * i + 4], v[8 * i + 5]),
                  pack_bf16(v[8 * i + 6], v[8 * i + 7]));
      __syncwarp();
#pragma unroll
      for (int pass = 0; pass < 4; ++pass) {
        const int r = pass * 8 + lane / 4, piece = lane % 4;
        const uint4 raw = lds_b32x4(stage + r * 64 + ((piece ^ ((r >> 1) & 3)) << 4));
        if (m0_warp + r < p.M) *reinterpret_cast<uint4*>(block + static_cast<size_t>(r) * p.ldc + piece * 8) = raw;
      }
      __syncwarp();
    } else if (m < p.M) {
      if (p.c_kind == 0) {
        float* dst = static_cast<float*>(p.c) + static_cast<size_t>(m) * p.ldc + n_base;
        if (p.c_accumulate) {
          for (int i = 0; i < 32 && n_base + i < p.N; ++i) v[i] += dst[i];
        }
        for (int i = 0; i < 32 && n_base + i < p.N; ++i) dst[i] = v[i];
      } else {
        __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.c) + static_cast<size_t>(m) * p.ldc + n_base;
        for (int i = 0; i < 32 && n_base + i < p.N; ++i) dst[i] = __float2bfloat16_rn(v[i]);
      }
    }
  }
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_sm100(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
           GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* a_smem = smem;
  uint8_t* b_smem = smem + kGemmStages * kABytes;
  uint8_t* drain_stage = b_smem + kGemmStages * kBBytes;
  GemmBarriers* bar = reinterpret_cast<GemmBarriers*>(drain_stage + kDrainStageBytes);
  const int warp = uniform_warp_index(), lane = threadIdx.x % 32;
  const int m_tiles = (p.M + kTile - 1) / kTile, n_tiles = (p.N + kTileN - 1) / kTileN;
  const int tiles = m_tiles * n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kGemmStages; ++s) {
      mbar_init(&bar->full[s], 1);
      mbar_init(&bar->empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bar->acc_full[s], 1);
      mbar_init(&bar->acc_empty[s], 4);   // one arrival per epilogue warp
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&bar->tmem_base, 2 * kTileN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bar->tmem_base;
  // Launched with programmatic stream serialisation: everything above ran beside the kernel
  // before (an operand cast, or the previous product); its results are read only from here on.
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&map_a);
      tma_prefetch_desc(&map_b);
      bool ok = true;
      int it = 0;   // k-tile counter over all tiles of this CTA: the ring never restarts
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        int m0, n0;
        tile_origin(tile, m_tiles, n_tiles, m0, n0);
        for (int kt = 0; kt < p.k_tiles && ok; ++kt, ++it) {
          const int st = it % kGemmStages, use = it / kGemmStages;
          if (use > 0) ok = mbar_wait(&bar->empty[st], (use - 1) & 1, p.status, 70);
          if (!ok) break;
          mbar_expect_tx(&bar->full[st], kABytes + kBBytes);
          uint8_t* a_dst = a_smem + st * kABytes;
          uint8_t* b_dst = b_smem + st * kBBytes;
          const int ka = (kt % p.a_wrap) * kBK, half = kt / p.a_wrap, kb = (kt % p.b_wrap) * kBK;
          if (A_MN) {   // memory [k][m]: slabs of 64 m-columns x 64 k-rows
            for (int h = 0; h < kTile / 64; ++h)
              tma_load_3d(a_dst + h * kSlab, &map_a, m0 + 64 * h, ka, half, &bar->full[st]);
          } else {      // memory [m][k]: 64 k-columns x 128 m-rows
            tma_load_3d(a_dst, &map_a, ka, m0, half, &bar->full[st]);
          }
          if (B_MN) {
            for (int h = 0; h < kTileN / 64; ++h)
              tma_load_3d(b_dst + h * kSlab, &map_b, n0 + 64 * h, kb, 0, &bar->full[st]);
          } else {      // memory [n][k]: 64 k-columns x 256 n-rows
            tma_load_3d(b_dst, &map_b, kb, n0, 0, &bar->full[st]);
          }
        }
      }
      for (int back = max(0, it - kGemmStages); back < it; ++back)   // the last copies have landed
        mbar_wait(&bar->full[back % kGemmStages], (back / kGemmStages) & 1, p.status, 71);
    }
  } else if (warp == 1) {
    bool ok = true;
    int it = 0, local = 0;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++local) {
      const int buf = local & 1, use = local >> 1;
      if (use > 0)   // the epilogue has drained this accumulator's previous tile
        ok = __all_sync(0xffffffffu, mbar_wait(&bar->acc_empty[buf], (use - 1) & 1, p.status, 74));
      if (!ok) break;
      tc_fence_after();
      for (int kt = 0; kt < p.k_tiles && ok; ++kt, ++it) {
        const int st = it % kGemmStages;
        ok = __all_sync(0xffffffffu, mbar_wait(&bar->full[st], (it / kGemmStages) & 1, p.status, 72));
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
          const uint32_t a_addr = smem_u32(a_smem + st * kABytes);
          const uint32_t b_addr = smem_u32(b_smem + st * kBBytes);
          // K-major: rows of 128 bytes, a K step of 16 elements is 32 bytes along the row.
          // MN-major: [64 k-rows x 128 bytes] slabs, a K step is 16 rows (2048 bytes), the next
          // 64-wide slab sits kSlab bytes further (leading-dimension byte offset).
          const uint64_t a_desc = A_MN ? umma_desc_sw128(a_addr, kSlab, 1024)
                                       : umma_desc_sw128(a_addr, 16, 1024);
          const uint64_t b_desc = B_MN ? umma_desc_sw128(b_addr, kSlab, 1024)
                                       : umma_desc_sw128(b_addr, 16, 1024);
#pragma unroll
          for (int ks = 0; ks < kBK / 16; ++ks)
            umma_ss(tmem + buf * kTileN, a_desc + ks * ((A_MN ? 2048 : 32) >> 4),
                    b_desc + ks * ((B_MN ? 2048 : 32) >> 4), p.idesc, kt > 0 || ks > 0);
          tc_commit(&bar->empty[st]);
          if (kt + 1 == p.k_tiles) tc_commit(&bar->acc_full[buf]);
        }
        __syncwarp();
      }
    }
  } else if (warp >= 4) {
    const int quarter = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    int local = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      int m0, n0;
      tile_origin(tile, m_tiles, n_tiles, m0, n0);
      if (!mbar_wait(&bar->acc_full[buf], (local >> 1) & 1, p.status, 73)) break;
      tc_fence_after();
      drain_accumulator(tmem + lane_base + buf * kTileN, m0 + quarter * 32, lane, n0, p,
                        smem_u32(drain_stage) + quarter * (kDrainStageBytes / 4));
      // the accumulator has been read into registers by every lane of this warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->acc_empty[buf]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 2 * kTileN);
  }
}

// ------------------------------------------------------------------------------------------------
// The same product on pairs of SMs: a cluster of two CTAs owns a 256 x 256 output tile and issues
// tcgen05.mma.cta_group::2 (M 256, N 256, K 16).  Each CTA stages its own 128 rows of A and its own
// 128 columns of B (16 KB + 16 KB per K step of 64 instead of 16 KB + 32 KB), so a CTA pulls a third
// less through L2 and its shared memory per MMA cycle; every CTA keeps the 256 accumulator columns
// of its 128 rows in its own TMEM and drains them itself.  All loads are plain tiled TMA loads (no
// multicast); CTA 1's loads complete on CTA 0's `full` barrier, the MMA warp of CTA 0 issues for
// both and its commits arrive on both CTAs' barriers.
// ------------------------------------------------------------------------------------------------
constexpr int kPairTile = 256, kPairStages = 6;
constexpr int kPairABytes = kTile * kBK * 2;   // 16 KB: this CTA's 128 rows of A
constexpr int kPairBBytes = kTile * kBK * 2;   // 16 KB: this CTA's 128 columns of B
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu; // clears the CTA-of-the-pair bit of a shared::cluster address

struct PairGemmBarriers {
  uint64_t full[kPairStages], empty[kPairStages], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
};

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Tiled TMA load of the CTA's own operand part; the bytes are counted on the barrier at `mbar_addr`,
// a shared::cluster address (CTA 0's barrier for both CTAs of the pair).
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const CUtensorMap* map, int c0, int c1, int c2,
                                                 uint32_t mbar_addr) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(map), "r"(mbar_addr), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void umma_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(static_cast<uint32_t>(accumulate))
      : "memory");
}
// Arrives on the barrier at this shared-memory offset in both CTAs of the pair once every MMA
// issued so far has completed.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(static_cast<uint16_t>(3))
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t mbar_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(mbar_addr) : "memory");
}

constexpr uint32_t gemm_idesc_pair(int format, bool a_mn, bool b_mn) {
  return (1u << 4) | (static_cast<uint32_t>(format) << 7) | (static_cast<uint32_t>(format) << 10) |
         (static_cast<uint32_t>(a_mn) << 15) | (static_cast<uint32_t>(b_mn) << 16) |
         (static_cast<uint32_t>(kPairTile >> 3) << 17) | (static_cast<uint32_t>(kPairTile >> 4) << 24);
}

__device__ __forceinline__ void pair_tile_origin(int tile, int m_tiles, int n_tiles, int& m0, int& n0) {
  const int band = tile / (kBand * m_tiles);
  const int width = min(kBand, n_tiles - band * kBand);
  const int within = tile - band * kBand * m_tiles;
  m0 = (within / width) * kPairTile;
  n0 = (band * kBand + within % width) * kPairTile;
}

// map_b: for K-major B a box of 128 n-rows, for MN-major B the 64 x 64 slab box.  p.idesc is unused
// here (pair_idesc carries M = 256).
template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_sm100_pair(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                GemmParams p, uint32_t pair_idesc) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* a_smem = smem;
  uint8_t* b_smem = smem + kPairStages * kPairABytes;
  uint8_t* drain_stage = b_smem + kPairStages * kPairBBytes;
  PairGemmBarriers* bar = reinterpret_cast<PairGemmBarriers*>(drain_stage + kDrainStageBytes);
  const int warp = uniform_warp_index(), lane = threadIdx.x % 32;
  const int rank = static_cast<int>(cluster_cta_rank());   // 0 issues the MMAs
  const int cluster = blockIdx.x / 2, clusters = gridDim.x / 2;
  const int m_tiles = (p.M + kPairTile - 1) / kPairTile, n_tiles = (p.N + kPairTile - 1) / kPairTile;
  const int tiles = m_tiles * n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&bar->full[s], 1);
      mbar_init(&bar->empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bar->acc_full[s], 1);
      mbar_init(&bar->acc_empty[s], 8);   // one arrival per epilogue warp of both CTAs (used in CTA 0)
    }
    mbar_fence_init();
  }
  if (warp == 1) {   // the same warp of both CTAs, together
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bar->tmem_base)),
                 "r"(2 * kPairTile)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  cluster_sync_all();   // both CTAs' barriers exist before either touches the other's
  tc_fence_after();
  const uint32_t tmem = bar->tmem_base;
  pdl_wait();   // (as in the one-SM kernel: the set-up above ran beside the kernel before)
  pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&map_a);
      tma_prefetch_desc(&map_b);
      bool ok = true;
      int it = 0;
      for (int tile = cluster; tile < tiles && ok; tile += clusters) {
        int m0, n0;
        pair_tile_origin(tile, m_tiles, n_tiles, m0, n0);
        m0 += rank * kTile;   // this CTA's rows of A
        n0 += rank * kTile;   // this CTA's columns of B
        for (int kt = 0; kt < p.k_tiles && ok; ++kt, ++it) {
          const int st = it % kPairStages, use = it / kPairStages;
          if (use > 0) ok = mbar_wait(&bar->empty[st], (use - 1) & 1, p.status, 75);
          if (!ok) break;
          if (rank == 0) mbar_expect_tx(&bar->full[st], 2 * (kPairABytes + kPairBBytes));   // both CTAs' bytes
          const uint32_t full_addr = smem_u32(&bar->full[st]) & kPeerBitMask;
          uint8_t* a_dst = a_smem + st * kPairABytes;
          uint8_t* b_dst = b_smem + st * kPairBBytes;
          const int ka = (kt % p.a_wrap) * kBK, half = kt / p.a_wrap, kb = (kt % p.b_wrap) * kBK;
          if (A_MN) {
            for (int h = 0; h < kTile / 64; ++h)
              tma_load_3d_pair(a_dst + h * kSlab, &map_a, m0 + 64 * h, ka, half, full_addr);
          } else {
            tma_load_3d_pair(a_dst, &map_a, ka, m0, half, full_addr);
          }
          if (B_MN) {
            for (int h = 0; h < kTile / 64; ++h)
              tma_load_3d_pair(b_dst + h * kSlab, &map_b, n0 + 64 * h, kb, 0, full_addr);
          } else {
            tma_load_3d_pair(b_dst, &map_b, kb, n0, 0, full_addr);
          }
        }
      }
      // every stage this CTA filled has been consumed: its last `empty` phases have completed
      for (int back = max(0, it - kPairStages); back < it && ok; ++back)
        ok = mbar_wait(&bar->empty[back % kPairStages], (back / kPairStages) & 1, p.status, 76);
    }
  } else if (warp == 1 && rank == 0) {
    bool ok = true;
    int it = 0, local = 0;
    for (int tile = cluster; tile < tiles && ok; tile += clusters, ++local) {
      const int buf = local & 1, use = local >> 1;
      if (use > 0)   // both CTAs' epilogues have drained this accumulator's previous tile
        ok = __all_sync(0xffffffffu, mbar_wait(&bar->acc_empty[buf], (use - 1) & 1, p.status, 77));
      if (!ok) break;
      tc_fence_after();
      for (int kt = 0; kt < p.k_tiles && ok; ++kt, ++it) {
        const int st = it % kPairStages;
        ok = __all_sync(0xffffffffu, mbar_wait(&bar->full[st], (it / kPairStages) & 1, p.status, 78));
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
          const uint32_t a_addr = smem_u32(a_smem + st * kPairABytes);
          const uint32_t b_addr = smem_u32(b_smem + st * kPairBBytes);
          const uint64_t a_desc = A_MN ? umma_desc_sw128(a_addr, kSlab, 1024) : umma_desc_sw128(a_addr, 16, 1024);
          const uint64_t b_desc = B_MN ? umma_desc_sw128(b_addr, kSlab, 1024) : umma_desc_sw128(b_addr, 16, 1024);
#pragma unroll
          for (int ks = 0; ks < kBK / 16; ++ks)
            umma_ss_pair(tmem + buf * kPairTile, a_desc + ks * ((A_MN ? 2048 : 32) >> 4),
                         b_desc + ks * ((B_MN ? 2048 : 32) >> 4), pair_idesc, kt > 0 || ks > 0);
          tc_commit_pair(&bar->empty[st]);
          if (kt + 1 == p.k_tiles) tc_commit_pair(&bar->acc_full[buf]);
        }
        __syncwarp();
      }
    }
  } else if (warp >= 4) {
    const int quarter = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    int local = 0;
    for (int tile = cluster; tile < tiles; tile += clusters, ++local) {
      const int buf = local & 1;
      int m0, n0;
      pair_tile_origin(tile, m_tiles, n_tiles, m0, n0);
      if (!mbar_wait(&bar->acc_full[buf], (local >> 1) & 1, p.status, 79)) break;
      tc_fence_after();
      drain_accumulator(tmem + lane_base + buf * kPairTile, m0 + rank * kTile + quarter * 32, lane, n0, p,
                        smem_u32(drain_stage) + quarter * (kDrainStageBytes / 4));
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(smem_u32(&bar->acc_empty[buf]) & kPeerBitMask);   // CTA 0's barrier
    }
  }
  tc_fence_before();
  cluster_sync_all();   // neither CTA leaves while the other may still signal it or read its tiles
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(2 * kPairTile) : "memory");
  }
}

// src [rows, cols] (fp32 or bf16) -> dst [rows_p, cols_p] 2-byte (bf16 or fp16), zero padded.
// grid (cols_p / 8 / 256 rounded up, rows_p): a thread converts 8 consecutive columns.
template <typename In, bool kHalf>
__global__ void __launch_bounds__(256)
cast_pad_kernel(const In* __restrict__ src, uint16_t* __restrict__ dst, int rows, int cols, int cols_p) {
  pdl_launch_dependents();   // the product behind this cast may set itself up meanwhile
  const int r = blockIdx.y;
  const int c = (blockIdx.x * 256 + threadIdx.x) * 8;
  if (c >= cols_p) return;
  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = 0.0f;
  if (r < rows && c < cols) {
    const In* p = src + static_cast<size_t>(r) * cols + c;
    if (c + 8 <= cols && reinterpret_cast<uintptr_t>(p) % 16 == 0) {
      if constexpr (sizeof(In) == 4) {
        const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
      } else {
        const uint4 a = *reinterpret_cast<const uint4*>(p);
        v[0] = bf16_lo(a.x); v[1] = bf16_hi(a.x); v[2] = bf16_lo(a.y); v[3] = bf16_hi(a.y);
        v[4] = bf16_lo(a.z); v[5] = bf16_hi(a.z); v[6] = bf16_lo(a.w); v[7] = bf16_hi(a.w);
      }
    } else {
      for (int i = 0; i < 8 && c + i < cols; ++i) {
        if constexpr (sizeof(In) == 4) v[i] = p[i];
        else v[i] = __bfloat162float(p[i]);
      }
    }
  }
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (kHalf) {
      const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    } else {
      w[i] = pack_bf16(v[2 * i], v[2 * i + 1]);
    }
  }
  *reinterpret_cast<uint4*>(dst + static_cast<size_t>(r) * cols_p + c) = make_uint4(w[0], w[1], w[2], w[3]);
}

// Column sums of dy [rows, cols] in two fixed-order levels: CTA (x, y) sums rows y, y + gridDim.y,
// ... of its 128 columns (a lane owns 4, the 8 warps split the rows and are added in warp order)
// into partial[y][cols]; the second kernel adds the partial rows in order.
constexpr int kBiasChunks = 16;
__global__ void __launch_bounds__(256) bias_partial_kernel(const float* __restrict__ dy, int rows, int cols,
                                                           float* __restrict__ partial) {
  __shared__ float part[8][128];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int n = blockIdx.x * 128 + lane * 4;
  float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  const bool vec = cols % 4 == 0 && reinterpret_cast<uintptr_t>(dy) % 16 == 0 && n + 4 <= cols;
  for (int r = blockIdx.y * 8 + warp; r < rows; r += gridDim.y * 8) {
    const float* p = dy + static_cast<size_t>(r) * cols + n;
    if (vec) {
      const float4 v = *reinterpret_cast<const float4*>(p);
      sum[0] += v.x; sum[1] += v.y; sum[2] += v.z; sum[3] += v.w;
    } else {
      for (int i = 0; i < 4 && n + i < cols; ++i) sum[i] += p[i];
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) part[warp][lane * 4 + i] = sum[i];
  __syncthreads();
  if (threadIdx.x < 128 && blockIdx.x * 128 + threadIdx.x < cols) {
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += part[w][threadIdx.x];
    partial[static_cast<size_t>(blockIdx.y) * cols + blockIdx.x * 128 + threadIdx.x] = total;
  }
}
__global__ void bias_final_kernel(const float* __restrict__ partial, int chunks, int cols, float* __restrict__ db) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= cols) return;
  float total = 0.0f;
  for (int c = 0; c < chunks; ++c) total += partial[static_cast<size_t>(c) * cols + n];
  db[n] = total;
}

int pad128(int v) { return (v + 127) / 128 * 128; }

// b_pair: the B operand's map for the two-SM kernel (K-major B: boxes of 128 rows; MN-major B: the
// same slab map as `b`), or null to keep the call on the one-SM kernel.
template <bool A_MN, bool B_MN>
cudaError_t launch_gemm(cudaStream_t stream, const CUtensorMap& a, const CUtensorMap& b,
                        const GemmParams& p, const CUtensorMap* b_pair = nullptr) {
  int sms = 148, device = 0;
  if (cudaGetDevice(&device) == cudaSuccess)
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const int pair_tiles = ((p.N + kPairTile - 1) / kPairTile) * ((p.M + kPairTile - 1) / kPairTile);
  if (b_pair != nullptr && pair_tiles >= sms / 2) {   // enough 256 x 256 tiles to occupy every pair of SMs
    const size_t pair_smem =
        1024 + kPairStages * (kPairABytes + kPairBBytes) + kDrainStageBytes + sizeof(PairGemmBarriers);
    cudaError_t e = cudaFuncSetAttribute(gemm_sm100_pair<A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(pair_smem));
    if (e != cudaSuccess) return e;
    const uint32_t format = (p.idesc >> 7) & 7u;
    const int clusters = std::min(pair_tiles, sms / 2);
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2 * clusters);
    config.blockDim = dim3(kGemmThreads);
    config.dynamicSmemBytes = pair_smem;
    config.stream = stream;
    config.attrs = &attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, gemm_sm100_pair<A_MN, B_MN>, a, *b_pair, p,
                              gemm_idesc_pair(static_cast<int>(format), A_MN, B_MN));
  }
  const size_t smem = 1024 + kGemmStages * (kABytes + kBBytes) + kDrainStageBytes + sizeof(GemmBarriers);
  cudaError_t e = cudaFuncSetAttribute(gemm_sm100<A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  const int tiles = ((p.N + kTileN - 1) / kTileN) * ((p.M + kTile - 1) / kTile);
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(std::min(tiles, sms));
  config.blockDim = dim3(kGemmThreads);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  config.attrs = &attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, gemm_sm100<A_MN, B_MN>, a, b, p);
}

template <typename In>
cudaError_t cast_pad(cudaStream_t stream, const void* src, void* dst, int rows, int cols, bool half) {
  const int rows_p = pad128(rows), cols_p = pad128(cols);
  const dim3 grid((cols_p / 8 + 255) / 256, rows_p);
  if (half)
    cast_pad_kernel<In, true><<<grid, 256, 0, stream>>>(static_cast<const In*>(src),
                                                         static_cast<uint16_t*>(dst), rows, cols, cols_p);
  else
    cast_pad_kernel<In, false><<<grid, 256, 0, stream>>>(static_cast<const In*>(src),
                                                          static_cast<uint16_t*>(dst), rows, cols, cols_p);
  return cudaGetLastError();
}

// The bf16 activation can be read by TMA in place (rows and columns past its extent read as zero)
// when its rows are 16-byte aligned; otherwise, and for fp32 activations, a padded 2-byte copy is made.
struct Operand {
  const void* base;
  int cols, rows;        // extents the tensor map describes
  size_t pitch;          // elements between rows
};
cudaError_t activation_operand(cudaStream_t stream, const void* x, bool x_is_bf16, int rows, int cols,
                               void* copy, Operand* out) {
  if (x_is_bf16 && cols % 8 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0) {
    *out = Operand{x, cols, rows, static_cast<size_t>(cols)};
    return cudaSuccess;
  }
  *out = Operand{copy, pad128(cols), pad128(rows), static_cast<size_t>(pad128(cols))};
  return x_is_bf16 ? cast_pad<__nv_bfloat16>(stream, x, copy, rows, cols, false)
                   : cast_pad<float>(stream, x, copy, rows, cols, true);
}
bool operand_map(CUtensorMap* map, const Operand& t, int box_rows) {
  return make_token_map(map, t.base, t.cols, t.rows, 1, t.pitch, box_rows);
}

}  // namespace

size_t dense_workspace_bytes(int rows, int in, int out) {
  const size_t r = pad128(rows), i = pad128(in), o = pad128(out);
  return 2 * (r * i + i * o + r * o) + sizeof(float) * kBiasChunks * o;   // casts of X, W, dY; bias partials
}

// x: [rows, in] bf16 (x_is_bf16) or fp32; w fp32 [in, out]; bias fp32 [out]; y same dtype as x.
cudaError_t dense_fwd(cudaStream_t stream, const void* x, bool x_is_bf16, const float* w,
                      const float* bias, void* y, int rows, int in, int out, void* workspace,
                      uint32_t* status) {
  const int r = pad128(rows), i = pad128(in), o = pad128(out);
  auto* xc = static_cast<uint8_t*>(workspace);
  auto* wc = xc + 2 * static_cast<size_t>(r) * i;
  const bool half = !x_is_bf16;
  Operand xo;
  cudaError_t e = activation_operand(stream, x, x_is_bf16, rows, in, xc, &xo);
  if (e != cudaSuccess) return e;
  e = cast_pad<float>(stream, w, wc, in, out, half);
  if (e != cudaSuccess) return e;
  CUtensorMap ma, mb;
  if (!operand_map(&ma, xo, kTile) ||                      // A K-major: [rows][in]
      !make_token_map(&mb, wc, o, i, 1, o, kBK))           // B MN-major: [in][out]
    return cudaErrorInvalidValue;
  GemmParams p{rows, out, i / kBK, i / kBK, i / kBK, 0, gemm_idesc(half ? 0 : 1, false, true), bias, y,
               static_cast<size_t>(out), x_is_bf16 ? 1 : 0, status};
  return launch_gemm<false, true>(stream, ma, mb, p, &mb);
}

// dy fp32 [rows, out]; dx fp32 [rows, in]; dw fp32 [in, out]; db fp32 [out] (all overwritten)
cudaError_t dense_bwd(cudaStream_t stream, const void* x, bool x_is_bf16, const float* w,
                      const float* dy, float* dx, float* dw, float* db, int rows, int in, int out,
                      void* workspace, uint32_t* status) {
  const int r = pad128(rows), i = pad128(in), o = pad128(out);
  auto* xc = static_cast<uint8_t*>(workspace);
  auto* wc = xc + 2 * static_cast<size_t>(r) * i;
  auto* gc = wc + 2 * static_cast<size_t>(i) * o;
  const bool half = !x_is_bf16;
  Operand xo;
  cudaError_t e = activation_operand(stream, x, x_is_bf16, rows, in, xc, &xo);
  if (e == cudaSuccess) e = cast_pad<float>(stream, w, wc, in, out, half);
  if (e == cudaSuccess) e = cast_pad<float>(stream, dy, gc, rows, out, half);
  if (e != cudaSuccess) return e;
  const int format = half ? 0 : 1;
  CUtensorMap ma, mb;
  // dX[rows, in] = dY[rows][out] (K-major) * W^T: B(k, n) = W[n][k], memory [in][out] = K-major
  CUtensorMap mb_pair;
  if (!make_token_map(&ma, gc, o, r, 1, o, kTile) || !make_token_map(&mb, wc, o, i, 1, o, kTileN) ||
      !make_token_map(&mb_pair, wc, o, i, 1, o, kTile))
    return cudaErrorInvalidValue;
  GemmParams pdx{rows, in, o / kBK, o / kBK, o / kBK, 0, gemm_idesc(format, false, false), nullptr, dx,
                 static_cast<size_t>(in), 0, status};
  e = launch_gemm<false, false>(stream, ma, mb, pdx, &mb_pair);
  if (e != cudaSuccess) return e;
  // dW[in, out] = X^T dY: A(m, k) = X[k][m], memory [rows][in] = MN-major; B = dY [rows][out] MN-major
  if (!operand_map(&ma, xo, kBK) || !make_token_map(&mb, gc, o, r, 1, o, kBK))
    return cudaErrorInvalidValue;
  GemmParams pdw{in, out, r / kBK, r / kBK, r / kBK, 0, gemm_idesc(format, true, true), nullptr, dw,
                 static_cast<size_t>(out), 0, status};
  e = launch_gemm<true, true>(stream, ma, mb, pdw, &mb);
  if (e != cudaSuccess) return e;
  float* partial = reinterpret_cast<float*>(gc + 2 * static_cast<size_t>(r) * o);
  bias_partial_kernel<<<dim3((out + 127) / 128, kBiasChunks), 256, 0, stream>>>(dy, rows, out, partial);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  bias_final_kernel<<<(out + 255) / 256, 256, 0, stream>>>(partial, kBiasChunks, out, db);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// BlockLinearLayer (src/llm/layers/block_training.cc:38-98, 321-399): resident bf16 weight
// [out, in] (output-major, no bias), bf16 activations, fp32 arithmetic on the exact bf16 values.
//   forward          Y[t][r]  = sum_c X[t][c] W[r][c]                       bf16 or fp32 output
//   input gradient   dX[t][c] = sum_r dY[t][r] W[r][c]                      fp32
//   weight gradient  dW[r][c] += sum_t dY[t][r] X[t][c]                     fp32, accumulated
// bf16 x bf16 products are exact in fp32, so the forward is the tensor-core GEMM as it is.  The
// gradients multiply an fp32 dY: it is split into hi = bf16(dY) and lo = bf16(dY - hi) (relative
// error 2^-17 instead of bf16's 2^-9) and both halves are accumulated into the same TMEM tile:
// [hi | lo] x [W; W], with the second pass re-reading the same W / X tiles (b_wrap).
// ------------------------------------------------------------------------------------------------
namespace {

// dst[0] = bf16(src), dst[1] = bf16(src - dst[0]); both [rows_p][cols_p], zero padded
__global__ void __launch_bounds__(256)
split_pad_kernel(const float* __restrict__ src, uint16_t* __restrict__ dst, int rows, int cols,
                 int rows_p, int cols_p) {
  pdl_launch_dependents();   // the product behind this split may set itself up meanwhile
  const int r = blockIdx.y;
  const int c = (blockIdx.x * 256 + threadIdx.x) * 8;
  if (c >= cols_p) return;
  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = 0.0f;
  if (r < rows && c < cols) {
    const float* p = src + static_cast<size_t>(r) * cols + c;
    if (c + 8 <= cols && reinterpret_cast<uintptr_t>(p) % 16 == 0) {
      const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
      for (int i = 0; i < 8 && c + i < cols; ++i) v[i] = p[i];
    }
  }
  uint32_t hi[4], lo[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float h0 = bf16_round(v[2 * i]), h1 = bf16_round(v[2 * i + 1]);
    hi[i] = pack_bf16(h0, h1);
    lo[i] = pack_bf16(v[2 * i] - h0, v[2 * i + 1] - h1);
  }
  const size_t at = static_cast<size_t>(r) * cols_p + c;
  *reinterpret_cast<uint4*>(dst + at) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
  *reinterpret_cast<uint4*>(dst + static_cast<size_t>(rows_p) * cols_p + at) =
      make_uint4(lo[0], lo[1], lo[2], lo[3]);
}

// DequantizeKernel (block_training.cc:19-36): fp32 or FP8 E4M3 (x block scale) -> bf16
__global__ void dequantize_kernel(const void* __restrict__ input, int storage, const float* __restrict__ scales,
                                  long long rows, int cols, __nv_bfloat16* __restrict__ output) {
  const long long total = rows * cols;
  const int scale_cols = (cols + 127) / 128;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float v;
    if (storage == 1) {
      v = static_cast<const float*>(input)[i];
    } else {
      const long long r = i / cols;
      const int c = static_cast<int>(i % cols);
      const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<const uint8_t*>(input)[i], __NV_E4M3);
      v = __half2float(*reinterpret_cast<const __half*>(&h)) * scales[(r / 128) * scale_cols + c / 128];
    }
    output[i] = __float2bfloat16_rn(v);
  }
}

// A bf16 matrix [rows][cols] as a TMA operand: in place when its rows are 16-byte aligned, else
// through a padded copy.
cudaError_t bf16_operand(cudaStream_t stream, const void* x, int rows, int cols, void* copy, Operand* out) {
  return activation_operand(stream, x, true, rows, cols, copy, out);
}

}  // namespace

size_t block_linear_workspace_bytes(int tokens, int in, int out) {
  const size_t t = pad128(tokens), i = pad128(in), o = pad128(out);
  return 2 * (t * i + o * i + 2 * t * o);   // copies of X and W (only if unaligned), hi/lo split of dY
}

cudaError_t block_linear_fwd(cudaStream_t stream, const void* weight, const void* x, void* y,
                             bool y_is_fp32, int tokens, int in, int out, void* workspace,
                             uint32_t* status) {
  const size_t t = pad128(tokens), i = pad128(in), o = pad128(out);
  auto* xc = static_cast<uint8_t*>(workspace);
  auto* wc = xc + 2 * t * i;
  Operand xo, wo;
  cudaError_t e = bf16_operand(stream, x, tokens, in, xc, &xo);
  if (e == cudaSuccess) e = bf16_operand(stream, weight, out, in, wc, &wo);
  if (e != cudaSuccess) return e;
  CUtensorMap ma, mb, mb_pair;
  if (!operand_map(&ma, xo, kTile) || !operand_map(&mb, wo, kTileN) || !operand_map(&mb_pair, wo, kTile))
    return cudaErrorInvalidValue;
  const int k_tiles = static_cast<int>(i / kBK);
  GemmParams p{tokens, out, k_tiles, k_tiles, k_tiles, 0, gemm_idesc(1, false, false), nullptr, y,
               static_cast<size_t>(out), y_is_fp32 ? 0 : 1, status};
  return launch_gemm<false, false>(stream, ma, mb, p, &mb_pair);
}

cudaError_t block_linear_bwd(cudaStream_t stream, const void* weight, const void* x, const float* dy,
                             float* dx, float* d_weight, int tokens, int in, int out, void* workspace,
                             uint32_t* status) {
  const size_t t = pad128(tokens), i = pad128(in), o = pad128(out);
  auto* xc = static_cast<uint8_t*>(workspace);
  auto* wc = xc + 2 * t * i;
  auto* gc = wc + 2 * o * i;
  Operand xo, wo;
  cudaError_t e = bf16_operand(stream, weight, out, in, wc, &wo);
  if (e == cudaSuccess && d_weight != nullptr) e = bf16_operand(stream, x, tokens, in, xc, &xo);
  if (e != cudaSuccess) return e;
  split_pad_kernel<<<dim3((static_cast<unsigned>(o) / 8 + 255) / 256, static_cast<unsigned>(t)), 256, 0,
                     stream>>>(dy, reinterpret_cast<uint16_t*>(gc), tokens, out, static_cast<int>(t),
                               static_cast<int>(o));
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  // hi and lo of dY as the two "batches" of one 3-D tensor [2][tokens_p][out_p]
  CUtensorMap ma, mb;
  // dX[tokens, in]: A = dY halves, K-major over out; B(k = r, n = c) = W[r][c]: MN-major, wraps
  if (!make_token_map(&ma, gc, static_cast<int>(o), static_cast<int>(t), 2, o, kTile) ||
      !operand_map(&mb, wo, kBK))
    return cudaErrorInvalidValue;
  const int ko = static_cast<int>(o / kBK), kt = static_cast<int>(t / kBK);
  GemmParams pdx{tokens, in, 2 * ko, ko, ko, 0, gemm_idesc(1, false, true), nullptr, dx,
                 static_cast<size_t>(in), 0, status};
  e = launch_gemm<false, true>(stream, ma, mb, pdx, &mb);
  if (e != cudaSuccess || d_weight == nullptr) return e;
  // dW[out, in] += dY^T X: A(m = r, k = t) = dY[t][r]: MN-major halves over tokens; B = X MN-major
  if (!make_token_map(&ma, gc, static_cast<int>(o), static_cast<int>(t), 2, o, kBK) ||
      !operand_map(&mb, xo, kBK))
    return cudaErrorInvalidValue;
  GemmParams pdw{out, in, 2 * kt, kt, kt, 1, gemm_idesc(1, true, true), nullptr, d_weight,
                 static_cast<size_t>(in), 0, status};
  return launch_gemm<true, true>(stream, ma, mb, pdw, &mb);
}

cudaError_t dequantize_matrix(cudaStream_t stream, const void* input, int storage, const float* scales,
                              long long rows, int cols, void* output) {
  const long long total = rows * cols;
  const unsigned blocks = static_cast<unsigned>(std::min<long long>((total + 255) / 256, 148 * 32));
  dequantize_kernel<<<blocks, 256, 0, stream>>>(input, storage, scales, rows, cols,
                                                static_cast<__nv_bfloat16*>(output));
  return cudaGetLastError();
}

}  // namespace pluto
