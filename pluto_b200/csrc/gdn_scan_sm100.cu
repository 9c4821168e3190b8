// Chunked gated delta-net prefill on the 5th-generation tensor cores: the sequential part.
//
// Notation of gdn_chunked.cu (chunk of C = 64 tokens, chunk-start state S0 [dk x dv]):
//     D = U - W S0,      O = (c.Q) S0 + M D,      S_C = gamma S0 + Kt^T D          (Kt = K . c_C/c)
// Substituting D removes the dependent pair of products from the chain between chunks:
//     S_C = gamma S0 + Kt^T U - (Kt^T W) S0  =  gamma S0 + Kt^T U + Pn S0,     Pn = -(Kt^T W)
//     O   = (c.Q - M W) S0 + M U             =  Qt S0 + M U,                   Qt = c.Q - M W
// Pn [dk x dk], Qt [C x dk], M, Kt and U depend only on the chunk's own tokens, so a prepare
// kernel computes them for all chunks in parallel; what is left per chunk on the sequential path
// is ONE product with the state plus a rescale by gamma.
//
// gdn_scan_sm100: one CTA per (sequence, head, slice of 128 value columns) walks the chunks.
//   * The state lives in TMEM for the whole sequence, transposed: lane j = value column, 128 fp32
//     columns = keys.  Each chunk the eight arithmetic warps read it (tcgen05.ld), write back
//     gamma * S (tcgen05.st) and a bf16 copy of S that the tensor core reads as its A operand
//     straight from TMEM.
//   * One elected thread issues, per chunk, tcgen05.mma M128 N128:  acc += U^T Kt  (A = U from
//     shared memory, token-major as stored) and  acc += S_bf16^T Pn^T  (A from TMEM): 12
//     instructions on the chain; then, off the chain, M128 N64:  O^T = S_bf16^T Qt^T + U^T M^T  into
//     one of two TMEM output buffers.
//   * The arithmetic warps drain an output buffer while the next chunk's state product runs: O^T is
//     lane = value column, so it is turned through a shared-memory tile into [token][value
//     column] rows and leaves as 16-byte stores.
//   * A producer thread streams the chunk records (already in the 128-byte-swizzled operand
//     layout, so a record is two linear bulk copies) through a two-stage ring.
// Measured on the way here: with bf16 remainders of S and U in the state products (24
// instructions on the chain instead of 12) the state error against the fp32 token-recurrent
// kernel fell only from 1.8e-3 to 1.1e-3 (it is set by the bf16 rounding of Pn and W), so the
// remainders are not used; scattering O^T as 2-byte stores took 5000 cycles per chunk and made
// the stores, not the tensor pipe, the limit.
// TMEM columns: state 0-127 | S_bf16 buffers 128-191, 192-255 | O^T buffers 256-319, 320-383.
// Every wait is bounded (common.cuh); on a time-out the kernel falls through to its exit path,
// frees its TMEM and reports through the status word.
#include "common.cuh"
#include "engine.h"
#include "gdn_records.cuh"

namespace pluto {
namespace {

constexpr int kScanThreads = 320;     // warp 0 producer, warp 1 MMA issuer, warps 2-9 arithmetic
constexpr int kScanStages = 2;
constexpr uint32_t kStageBytes = GdnRecord::kCommon + GdnRecord::kSlice;   // 91136
constexpr uint32_t kOutTileBytes = kGdnChunk * kGdnSliceCols * 2;          // [64 tokens][128 columns] bf16
constexpr uint32_t kColState = 0, kColSbf = 128, kColOut = 256;

struct ScanBarriers {
  uint64_t full[kScanStages], empty[kScanStages];
  uint64_t sbf_ready;     // 8 warp arrivals: the chunk's scaled state and its bf16 copy are in TMEM
  uint64_t state_done;    // tcgen05.commit: the chunk's state products have landed
  uint64_t out_done[2];   // tcgen05.commit: O^T of a chunk is complete
  uint64_t out_free[2];   // 8 warp arrivals: the arithmetic warps hold that buffer in registers
  uint32_t tmem_base;
};

// Barrier among the 256 arithmetic threads only (the producer and the MMA warp never join it).
// Every arithmetic thread executes every one of these, whatever its waits returned, so the
// arrival counts always match.
__device__ __forceinline__ void arithmetic_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

__global__ void __launch_bounds__(kScanThreads, 1)
gdn_scan_sm100(GdnArgs a, const uint8_t* __restrict__ records, int first_chunk, int chunks, int all_chunks,
               float* __restrict__ state_dump, uint32_t* status) {
  // walks chunks first_chunk .. first_chunk + chunks - 1 of the sequence's all_chunks; the state is
  // read from and left in a.state, so consecutive launches continue one another.  state_dump (optional, for the backward pass): the
  // state at the START of every chunk, [sequence, head, chunk, key, value column]
  extern __shared__ uint8_t scan_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(scan_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* out_tile = smem + kScanStages * kStageBytes;
  ScanBarriers* bar = reinterpret_cast<ScanBarriers*>(out_tile + kOutTileBytes);
  const int slice = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = uniform_warp_index(), lane = threadIdx.x % 32;
  const int dv = a.value_dim;
  const size_t record_bytes = GdnRecord::bytes(dv);
  const uint8_t* rec0 = records + ((static_cast<size_t>(b) * a.value_heads + h) * all_chunks + first_chunk) * record_bytes;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kScanStages; ++s) {
      mbar_init(&bar->full[s], 1);
      mbar_init(&bar->empty[s], 1);
    }
    mbar_init(&bar->sbf_ready, 8);
    mbar_init(&bar->state_done, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bar->out_done[s], 1);
      mbar_init(&bar->out_free[s], 8);
    }
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

  if (warp == 0) {
    // ------------------------------------------------------------------ record producer
    if (lane == 0) {
      bool ok = true;
      for (int c = 0; c < chunks && ok; ++c) {
        const int st = c % kScanStages, use = c / kScanStages;
        if (use > 0) ok = mbar_wait(&bar->empty[st], (use - 1) & 1, status, 50);
        if (!ok) break;
        uint8_t* dst = smem + st * kStageBytes;
        const uint8_t* rec = rec0 + static_cast<size_t>(c) * record_bytes;
        mbar_expect_tx(&bar->full[st], kStageBytes);
        bulk_load(dst, rec, GdnRecord::kCommon, &bar->full[st]);
        bulk_load(dst + GdnRecord::kCommon, rec + GdnRecord::kCommon + static_cast<size_t>(slice) * GdnRecord::kSlice,
                  GdnRecord::kSlice, &bar->full[st]);
      }
      // nothing may still be writing this CTA's shared memory when it exits
      for (int c = max(0, chunks - kScanStages); c < chunks; ++c)
        mbar_wait(&bar->full[c % kScanStages], (c / kScanStages) & 1, status, 51);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t kIdescUpdU = umma_idesc_bf16_majors(128, 128, true, true);    // U^T Kt
    constexpr uint32_t kIdescUpdS = umma_idesc_bf16_majors(128, 128, false, false);  // S Pn^T
    constexpr uint32_t kIdescOutS = umma_idesc_bf16_majors(128, 64, false, false);   // S Qt^T
    constexpr uint32_t kIdescOutU = umma_idesc_bf16_majors(128, 64, true, false);    // U^T M^T
    bool ok = true;
    for (int c = 0; c < chunks && ok; ++c) {
      const int st = c % kScanStages, buf = c & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&bar->full[st], (c / kScanStages) & 1, status, 52));
      if (!ok) break;
      ok = __all_sync(0xffffffffu, mbar_wait(&bar->sbf_ready, c & 1, status, 53));
      if (!ok) break;
      tc_fence_after();
      const uint32_t base = smem_u32(smem + st * kStageBytes);
      const uint32_t sbf = tmem + kColSbf + buf * 64;
      // token-major tiles (MN-major operands): 64-column slabs 8192 bytes apart, 16 tokens = 2048 bytes
      const uint64_t u = umma_desc_sw128(base + GdnRecord::kCommon + GdnRecord::kUH, 8192, 1024);
      const uint64_t kt = umma_desc_sw128(base + GdnRecord::kKT, 8192, 1024);
      // K-major tiles: a K step of 16 elements is 32 bytes along the row, 64-element slabs apart
      const uint64_t pn = umma_desc_sw128(base + GdnRecord::kPN, 16, 1024);
      const uint64_t qt = umma_desc_sw128(base + GdnRecord::kQT, 16, 1024);
      const uint64_t mm = umma_desc_sw128(base + GdnRecord::kMM, 16, 1024);
      if (elect_one()) {
        // state: acc (= gamma S) += U^T Kt + S Pn^T
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_ss(tmem + kColState, u + ks * 128, kt + ks * 128, kIdescUpdU, true);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ts(tmem + kColState, sbf + ks * 8, pn + (((ks / 4) * 16384 + (ks % 4) * 32) >> 4),
                  kIdescUpdS, true);
        tc_commit(&bar->state_done);
      }
      __syncwarp();
      if (c >= 2) {   // the arithmetic warps have taken this output buffer's previous chunk
        ok = __all_sync(0xffffffffu, mbar_wait(&bar->out_free[buf], ((c >> 1) - 1) & 1, status, 54));
        if (!ok) break;
        tc_fence_after();
      }
      if (elect_one()) {
        const uint32_t out = tmem + kColOut + buf * 64;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ts(out, sbf + ks * 8, qt + (((ks / 4) * 8192 + (ks % 4) * 32) >> 4), kIdescOutS, ks > 0);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) umma_ss(out, u + ks * 128, mm + ks * 2, kIdescOutU, true);
        tc_commit(&bar->out_done[buf]);
        tc_commit(&bar->empty[st]);
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ arithmetic warps
    const int quarter = warp & 3;                 // the TMEM lanes this warp may touch
    const int half = (warp - 2) / 4;              // its half of the columns
    const int jl = quarter * 32 + lane;           // value column inside the slice == TMEM lane
    const int j = slice * kGdnSliceCols + jl;
    const int u256 = (warp - 2) * 32 + lane;      // index among the arithmetic threads
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    float* state = a.state + (static_cast<size_t>(b) * a.value_heads + h) * kGdnKeyDim * dv + j;
    // (uniform over the CTA) bf16 output rows that can leave as 16-byte pieces
    const bool wide_stores = a.out_is_bf16 && (reinterpret_cast<uintptr_t>(a.out) & 15u) == 0 && dv % 8 == 0;
    {
      // chunk-start state of the sequence: keys half*64 .. +63 of this value column
      uint32_t s0[2][32];
#pragma unroll
      for (int g = 0; g < 2; ++g)
#pragma unroll
        for (int i = 0; i < 32; ++i)
          s0[g][i] = __float_as_uint(state[static_cast<size_t>(half * 64 + g * 32 + i) * dv]);
      tmem_st32(tmem + lane_base + kColState + half * 64, s0[0]);
      tmem_st32(tmem + lane_base + kColState + half * 64 + 32, s0[1]);
      tmem_wait_st();
    }
    bool ok = true;
    // O^T of chunk e: this thread holds tokens half*32 .. +31 of value column jl.  Called by every
    // arithmetic thread for every chunk; the work inside is skipped once a wait has failed.
    auto drain_output = [&](int e) {
      const int buf = e & 1;
      ok = __all_sync(0xffffffffu, ok && mbar_wait(&bar->out_done[buf], (e >> 1) & 1, status, 55));
      uint32_t o[32];
      if (ok) {
        tc_fence_after();
        tmem_ld32(tmem + lane_base + kColOut + buf * 64 + half * 32, o);
        tmem_wait_ld();
        tc_fence_before();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->out_free[buf]);
      if (wide_stores) {
        arithmetic_sync();   // the previous chunk's rows have left the tile
        if (ok) {
#pragma unroll
          for (int i = 0; i < 32; ++i)   // (st.shared by address: `out_tile` is a generic pointer to the compiler)
            sts_b16(smem_u32(out_tile) + ((half * 32 + i) * kGdnSliceCols + jl) * 2,
                    __bfloat16_as_ushort(__float2bfloat16_rn(__uint_as_float(o[i]))));
        }
        arithmetic_sync();
        if (ok) {
          // 16 threads per token row of 256 bytes, four passes of 16 rows
#pragma unroll
          for (int pass = 0; pass < 4; ++pass) {
            const int row = pass * 16 + u256 / 16, piece = u256 % 16;
            const int t = (first_chunk + e) * kGdnChunk + row;
            if (t < a.tokens) {
              const size_t off = ((static_cast<size_t>(b) * a.tokens + t) * a.value_heads + h) * dv +
                                 slice * kGdnSliceCols + piece * 8;
              *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.out) + off) =
                  lds_b32x4(smem_u32(out_tile) + row * (kGdnSliceCols * 2) + piece * 16);
            }
          }
        }
      } else if (ok) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int t = (first_chunk + e) * kGdnChunk + half * 32 + i;
          if (t < a.tokens) {
            const size_t off = ((static_cast<size_t>(b) * a.tokens + t) * a.value_heads + h) * dv + j;
            const float value = a.round ? bf16_round(__uint_as_float(o[i])) : __uint_as_float(o[i]);
            if (a.out_is_bf16) static_cast<__nv_bfloat16*>(a.out)[off] = __float2bfloat16_rn(value);
            else static_cast<float*>(a.out)[off] = value;
          }
        }
      }
    };
    for (int c = 0; c < chunks; ++c) {
      const int st = c % kScanStages, buf = c & 1;
      if (c > 0) ok = ok && mbar_wait(&bar->state_done, (c - 1) & 1, status, 56);
      // (warp-uniform from here on: the tcgen05 loads and stores below are warp-wide instructions)
      ok = __all_sync(0xffffffffu, ok && mbar_wait(&bar->full[st], (c / kScanStages) & 1, status, 57));   // gamma is in the record
      if (ok) {
        tc_fence_after();
        const float gamma = lds_f32(smem_u32(smem) + st * kStageBytes + GdnRecord::kGM);
        uint32_t s[2][32], packed[32];
        tmem_ld32(tmem + lane_base + kColState + half * 64, s[0]);
        tmem_ld32(tmem + lane_base + kColState + half * 64 + 32, s[1]);
        tmem_wait_ld();
        if (state_dump != nullptr) {
          // (one key per store: the 32 lanes of a warp write 32 neighbouring value columns)
          float* dst = state_dump + (((static_cast<size_t>(b) * a.value_heads + h) * all_chunks + first_chunk + c) *
                                         kGdnKeyDim + half * 64) * dv + j;
#pragma unroll
          for (int g = 0; g < 2; ++g)
#pragma unroll
            for (int i = 0; i < 32; ++i) dst[static_cast<size_t>(g * 32 + i) * dv] = __uint_as_float(s[g][i]);
        }
#pragma unroll
        for (int g = 0; g < 2; ++g)
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float x = __uint_as_float(s[g][i]), y = __uint_as_float(s[g][i + 1]);
            packed[g * 16 + i / 2] = pack_bf16(x, y);
            s[g][i] = __float_as_uint(x * gamma);
            s[g][i + 1] = __float_as_uint(y * gamma);
          }
        // bf16 pairs: the 64 keys of this half are 32 packed columns
        tmem_st32(tmem + lane_base + kColSbf + buf * 64 + half * 32, packed);
        tmem_st32(tmem + lane_base + kColState + half * 64, s[0]);
        tmem_st32(tmem + lane_base + kColState + half * 64 + 32, s[1]);
        tmem_wait_st();
        tc_fence_before();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->sbf_ready);
      if (c > 0) drain_output(c - 1);
    }
    ok = __all_sync(0xffffffffu, ok && mbar_wait(&bar->state_done, (chunks - 1) & 1, status, 58));
    if (ok) {
      tc_fence_after();
      uint32_t s[2][32];
      tmem_ld32(tmem + lane_base + kColState + half * 64, s[0]);
      tmem_ld32(tmem + lane_base + kColState + half * 64 + 32, s[1]);
      tmem_wait_ld();
#pragma unroll
      for (int g = 0; g < 2; ++g)
#pragma unroll
        for (int i = 0; i < 32; ++i)
          state[static_cast<size_t>(half * 64 + g * 32 + i) * dv] = __uint_as_float(s[g][i]);
    }
    drain_output(chunks - 1);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}


// ---------------------------------------------------------------------------------------------
// Reverse scan of the backward pass.  With the chunk's records, the gradient of the state at the
// chunk's start follows from the one at its end by the transposed map of the forward step,
//     dS_0 = gamma dS_C + Pn^T dS_C + Qt^T dO,
// again ONE dependent product per chunk.  The state gradient lives in TMEM transposed like the
// state (lane = value column, columns = keys), so per chunk: acc (= gamma dS^T) += dO^T Qt
// (token-major operands, as U^T Kt forward) + dS^T_bf16 Pn (Pn now read as an MN-major operand:
// its 64-column slabs are 16384 bytes apart, 16 keys = 2048 bytes).  What the per-chunk part of
// the backward pass needs is the gradient at every chunk's END: dumped,
// [sequence, head, chunk, key, value column], before the chunk's step.  One CTA per (sequence, head,
// 128 value columns); warp roles as in the forward scan, no output products.
// ---------------------------------------------------------------------------------------------
constexpr int kRevStages = 3;
constexpr uint32_t kRevPn = 0, kRevQt = 32768, kRevDo = 49152, kRevGm = 65536, kRevStageBytes = 66560;

struct RevBarriers {
  uint64_t full[kRevStages], empty[kRevStages];
  uint64_t sbf_ready;     // 8 warp arrivals
  uint64_t state_done;    // tcgen05.commit
  uint32_t tmem_base;
};

__global__ void __launch_bounds__(kScanThreads, 1)
gdn_scan_bwd_sm100(const __grid_constant__ CUtensorMap map_do, int value_heads,
                   const uint8_t* __restrict__ records, int chunks, float* __restrict__ dstate_dump,
                   uint32_t* status) {
  extern __shared__ uint8_t scan_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(scan_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  RevBarriers* bar = reinterpret_cast<RevBarriers*>(smem + kRevStages * kRevStageBytes);
  const int h = blockIdx.y, b = blockIdx.z;
  const int warp = uniform_warp_index(), lane = threadIdx.x % 32;
  constexpr int dv = kGdnSliceCols;
  const size_t record_bytes = GdnRecord::bytes(dv);
  const size_t unit = static_cast<size_t>(b) * value_heads + h;
  const uint8_t* rec0 = records + unit * chunks * record_bytes;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kRevStages; ++s) {
      mbar_init(&bar->full[s], 1);
      mbar_init(&bar->empty[s], 1);
    }
    mbar_init(&bar->sbf_ready, 8);
    mbar_init(&bar->state_done, 1);
    mbar_fence_init();
    tma_prefetch_desc(&map_do);
  }
  if (warp == 1) {
    tmem_alloc(&bar->tmem_base, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bar->tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      for (int n = 0; n < chunks && ok; ++n) {
        const int chunk = chunks - 1 - n, st = n % kRevStages, use = n / kRevStages;
        if (use > 0) ok = mbar_wait(&bar->empty[st], (use - 1) & 1, status, 44);
        if (!ok) break;
        uint8_t* dst = smem + st * kRevStageBytes;
        const uint8_t* rec = rec0 + static_cast<size_t>(chunk) * record_bytes;
        mbar_expect_tx(&bar->full[st], 32768 + 16384 + 16 + 16384);
        bulk_load(dst + kRevPn, rec + GdnRecord::kPN, 32768, &bar->full[st]);
        bulk_load(dst + kRevQt, rec + GdnRecord::kQT, 16384, &bar->full[st]);
        bulk_load(dst + kRevGm, rec + GdnRecord::kGM, 16, &bar->full[st]);
        for (int s = 0; s < 2; ++s)
          tma_load_3d(dst + kRevDo + s * 8192, &map_do, h * dv + s * 64, chunk * kGdnChunk, b, &bar->full[st]);
      }
      for (int n = max(0, chunks - kRevStages); n < chunks; ++n)
        mbar_wait(&bar->full[n % kRevStages], (n / kRevStages) & 1, status, 45);
    }
  } else if (warp == 1) {
    constexpr uint32_t kIdescTokens = umma_idesc_bf16_majors(128, 128, true, true);    // dO^T Qt
    constexpr uint32_t kIdescPn = umma_idesc_bf16_majors(128, 128, false, true);       // dS^T Pn
    bool ok = true;
    for (int n = 0; n < chunks && ok; ++n) {
      const int st = n % kRevStages, buf = n & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&bar->full[st], (n / kRevStages) & 1, status, 46));
      if (!ok) break;
      ok = __all_sync(0xffffffffu, mbar_wait(&bar->sbf_ready, n & 1, status, 47));
      if (!ok) break;
      tc_fence_after();
      const uint32_t base = smem_u32(smem + st * kRevStageBytes);
      const uint32_t sbf = tmem + kColSbf + buf * 64;
      const uint64_t d_out = umma_desc_sw128(base + kRevDo, 8192, 1024);
      const uint64_t qt = umma_desc_sw128(base + kRevQt, 8192, 1024);
      const uint64_t pn = umma_desc_sw128(base + kRevPn, 16384, 1024);
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_ss(tmem + kColState, d_out + ks * 128, qt + ks * 128, kIdescTokens, true);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ts(tmem + kColState, sbf + ks * 8, pn + ks * 128, kIdescPn, true);
        tc_commit(&bar->state_done);
        tc_commit(&bar->empty[st]);
      }
      __syncwarp();
    }
  } else {
    const int quarter = warp & 3, half = (warp - 2) / 4;
    const int j = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    {
      uint32_t zero[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) zero[i] = 0u;
      tmem_st32(tmem + lane_base + kColState + half * 64, zero);
      tmem_st32(tmem + lane_base + kColState + half * 64 + 32, zero);
      tmem_wait_st();
    }
    bool ok = true;
    for (int n = 0; n < chunks; ++n) {
      const int chunk = chunks - 1 - n, st = n % kRevStages, buf = n & 1;
      if (n > 0) ok = ok && mbar_wait(&bar->state_done, (n - 1) & 1, status, 48);
      ok = __all_sync(0xffffffffu, ok && mbar_wait(&bar->full[st], (n / kRevStages) & 1, status, 49));
      if (ok) {
        tc_fence_after();
        const float gamma = lds_f32(smem_u32(smem) + st * kRevStageBytes + kRevGm);
        uint32_t s[2][32], packed[32];
        tmem_ld32(tmem + lane_base + kColState + half * 64, s[0]);
        tmem_ld32(tmem + lane_base + kColState + half * 64 + 32, s[1]);
        tmem_wait_ld();
        float* dst = dstate_dump + ((unit * chunks + chunk) * kGdnKeyDim + half * 64) * dv + j;
#pragma unroll
        for (int g = 0; g < 2; ++g)
#pragma unroll
          for (int i = 0; i < 32; ++i) dst[static_cast<size_t>(g * 32 + i) * dv] = __uint_as_float(s[g][i]);
#pragma unroll
        for (int g = 0; g < 2; ++g)
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float x = __uint_as_float(s[g][i]), y = __uint_as_float(s[g][i + 1]);
            packed[g * 16 + i / 2] = pack_bf16(x, y);
            s[g][i] = __float_as_uint(x * gamma);
            s[g][i + 1] = __float_as_uint(y * gamma);
          }
        tmem_st32(tmem + lane_base + kColSbf + buf * 64 + half * 32, packed);
        tmem_st32(tmem + lane_base + kColState + half * 64, s[0]);
        tmem_st32(tmem + lane_base + kColState + half * 64 + 32, s[1]);
        tmem_wait_st();
        tc_fence_before();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->sbf_ready);
    }
    // the last products must have landed before the tensor memory is given back
    ok = __all_sync(0xffffffffu, ok && mbar_wait(&bar->state_done, (chunks - 1) & 1, status, 43));
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

}  // namespace

size_t gdn_scan_smem_bytes() {
  return 1024 + kScanStages * kStageBytes + kOutTileBytes + sizeof(ScanBarriers);
}

cudaError_t gdn_scan_launch(cudaStream_t stream, const GdnArgs& a, const void* records, int first_chunk,
                            int chunks, int all_chunks, float* state_dump, uint32_t* status) {
  const size_t smem = gdn_scan_smem_bytes();
  if (first_chunk == 0) {   // (every call starts with the piece at chunk 0)
    cudaError_t e = cudaFuncSetAttribute(gdn_scan_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return e;
  }
  gdn_scan_sm100<<<dim3(a.value_dim / kGdnSliceCols, a.value_heads, a.batch), kScanThreads, smem, stream>>>(
      a, static_cast<const uint8_t*>(records), first_chunk, chunks, all_chunks, state_dump, status);
  return cudaGetLastError();
}

// dcore_bf16: the output gradient as bf16 [batch, tokens, value_heads * 128]; dstate_dump as above.
cudaError_t gdn_scan_bwd_launch(cudaStream_t stream, const void* dcore_bf16, const void* records, int batch,
                                int tokens, int value_heads, int chunks, float* dstate_dump, uint32_t* status) {
  CUtensorMap map_do;
  if (!make_token_map(&map_do, dcore_bf16, value_heads * kGdnSliceCols, tokens, batch,
                      static_cast<size_t>(value_heads) * kGdnSliceCols, 64))
    return cudaErrorInvalidValue;
  const size_t smem = 1024 + kRevStages * kRevStageBytes + sizeof(RevBarriers);
  cudaError_t e = cudaFuncSetAttribute(gdn_scan_bwd_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  gdn_scan_bwd_sm100<<<dim3(1, value_heads, batch), kScanThreads, smem, stream>>>(
      map_do, value_heads, static_cast<const uint8_t*>(records), chunks, dstate_dump, status);
  return cudaGetLastError();
}

}  // namespace pluto
