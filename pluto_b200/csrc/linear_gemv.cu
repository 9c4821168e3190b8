// Imported (frozen, output-major) projection for a few tokens: y[t][r] = bf16(sum_c W[r][c] x[t][c]).
//
// Stands in for FullyConnectedLayer::ImportedForward (src/llm/layers/fully_connected.cc:295-341):
// ImportedMatVecKernel (:40-71) over fp32, bf16 or FP8-E4M3 weights with 128x128 block scales, and
// QuantizeImportedInputKernel (:73-95), the dynamic per-128 FP8 quantisation of the activation that
// the FP8 path applies first.  All arithmetic is fp32, as in the reference; only the summation
// order differs (the reference test allows 5e-5 + 0.8 %).
//
// The reference launches one program per 8 output rows that walks the row in 128-column steps, and
// casts the bf16 activation to fp32 (and quantises it) in separate launches.  This is a weight
// stream bound by HBM, so here the activation is cast (and, for FP8, quantised) inside the same
// kernel and staged in shared memory, a small decode batch shares one pass over the weights, and
// there are three forms of the stream itself:
//  * linear_gemv_stream, linear_gemv_stream_e4m3: persistent CTAs fed by a ring of bulk-copied
//    weight slabs (TMA unit), launched so that consecutive calls overlap; FMA arithmetic for one
//    bf16 token, E4M3 tensor-core MMAs for FP8 weights;
//  * linear_gemv_mma: bf16/FP8 batches of up to 8 tokens on the tensor cores (mma.sync), loading
//    from global memory;
//  * linear_gemv_kernel: fp32 weights, unaligned or small shapes -- 16-byte loads from global
//    memory, FMA arithmetic.
#include <cuda_fp8.h>

#include "common.cuh"
#include "engine.h"

namespace pluto {
namespace {

constexpr int kWarps = 8, kThreads = kWarps * 32;
constexpr int kRows = 4;          // output rows per task
constexpr int kChunk = 8192;      // staged activation floats per CTA (all tokens together)

// The staged activation is read as 16-byte chunks at a lane stride of 1, 2 or 4 chunks (fp32,
// bf16, FP8 weights); XOR-ing the chunk index with two bits of its octet index spreads every
// quarter-warp over all eight 16-byte bank groups.
__device__ __forceinline__ int swizzled(int c) {
  const int j = c >> 2;
  return ((j ^ ((j >> 3) & 3)) << 2) | (c & 3);
}
__device__ __forceinline__ float4 staged4(const float* xs, int c) {   // c % 4 == 0
  return *reinterpret_cast<const float4*>(xs + swizzled(c));
}

__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}
__device__ __forceinline__ float quantize_e4m3(float v, float scale) {
  const uint8_t q = __nv_cvt_float_to_fp8(v / fmaxf(scale, 1e-12f), __NV_SATFINITE, __NV_E4M3);
  return e4m3_to_float(q) * scale;
}

// Elements per 16-byte load and their conversion to fp32.
template <int STORAGE> struct Weights;
template <> struct Weights<0> {
  static constexpr int kPer = 4;
  __device__ static uint4 raw(const void* w, size_t i) {
    return *reinterpret_cast<const uint4*>(static_cast<const float*>(w) + i);
  }
  __device__ static void convert(const uint4& r, float (&v)[4]) {
    v[0] = __uint_as_float(r.x); v[1] = __uint_as_float(r.y);
    v[2] = __uint_as_float(r.z); v[3] = __uint_as_float(r.w);
  }
  __device__ static float one(const void* w, size_t i) { return static_cast<const float*>(w)[i]; }
};
template <> struct Weights<1> {
  static constexpr int kPer = 8;
  __device__ static uint4 raw(const void* w, size_t i) {
    return *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(w) + i);
  }
  __device__ static void convert(const uint4& r, float (&v)[8]) {
    v[0] = bf16_lo(r.x); v[1] = bf16_hi(r.x); v[2] = bf16_lo(r.y); v[3] = bf16_hi(r.y);
    v[4] = bf16_lo(r.z); v[5] = bf16_hi(r.z); v[6] = bf16_lo(r.w); v[7] = bf16_hi(r.w);
  }
  __device__ static float one(const void* w, size_t i) {
    return __bfloat162float(static_cast<const __nv_bfloat16*>(w)[i]);
  }
};
template <> struct Weights<2> {
  static constexpr int kPer = 16;
  __device__ static uint4 raw(const void* w, size_t i) {
    return *reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(w) + i);
  }
  __device__ static void convert(const uint4& r, float (&v)[16]) {
    const uint32_t words[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
#pragma unroll
      for (int p = 0; p < 2; ++p) {
        const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(
            static_cast<__nv_fp8x2_storage_t>((words[k] >> (16 * p)) & 0xffffu), __NV_E4M3);
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
        v[k * 4 + p * 2] = f.x;
        v[k * 4 + p * 2 + 1] = f.y;
      }
    }
  }
  __device__ static float one(const void* w, size_t i) {
    return e4m3_to_float(static_cast<const uint8_t*>(w)[i]);
  }
};

// bf16 -> fp32 into xs[t * ld + swizzled(c)] for the columns [c0, c0 + count) of every token; FP8
// path: each group of 128 is quantised (one warp a group) as QuantizeImportedInputKernel does.
template <int STORAGE, int TOK>
__device__ __forceinline__ void stage_activation(const __nv_bfloat16* __restrict__ x, float* xs, int ld,
                                                 int cols, int c0, int count, int warp, int lane) {
  const int groups = (count + 127) / 128;
  constexpr int kBatch = 4;   // groups whose loads are in flight together (the latency is paid once)
  for (int first = warp; first < TOK * groups; first += kWarps * kBatch) {
    float v[kBatch][4];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int group = min(first + u * kWarps, TOK * groups - 1);
      const int t = group / groups, g = group % groups;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = g * 128 + lane + 32 * i;
        v[u][i] = c < count ? __bfloat162float(x[static_cast<size_t>(t) * cols + c0 + c]) : 0.0f;
      }
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      // no early exit: the batch's reductions are independent chains that interleave
      const int group = min(first + u * kWarps, TOK * groups - 1);   // past the end: repeats the last group
      const int t = group / groups, g = group % groups;
      if (STORAGE == 2) {
        float maximum = fmaxf(fmaxf(fabsf(v[u][0]), fabsf(v[u][1])), fmaxf(fabsf(v[u][2]), fabsf(v[u][3])));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, o));
        const float scale = maximum / 448.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) v[u][i] = quantize_e4m3(v[u][i], scale);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = g * 128 + lane + 32 * i;
        if (c < ld) xs[t * ld + swizzled(c)] = v[u][i];
      }
    }
  }
}

// One task = kRows consecutive output rows, done by one CTA: its 256 threads interleave over the
// columns (thread i takes the 16-byte chunks i, i + 256, ...), then the eight warps' partial sums
// are combined through shared memory in warp order.  When the whole activation fits the staging
// buffer (cols <= kCols) the grid is three CTAs per SM, the activation is staged once per CTA and
// task i goes to CTA i % gridDim.x, so every SM gets the same number of 4-row tasks to within one.
// Longer rows take one task per CTA and several staging passes.
// VECTOR: every weight row starts 16-byte aligned and cols is a multiple of the elements per load.
template <int STORAGE, int TOK, bool VECTOR>
__global__ void __launch_bounds__(kThreads)
linear_gemv_kernel(const void* __restrict__ weights, const float* __restrict__ scales,
                   const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, int cols,
                   int rows) {
  constexpr int kPer = Weights<STORAGE>::kPer;
  constexpr int kCols = kChunk / TOK / 128 * 128;     // staged columns per pass (multiple of 128)
  constexpr size_t kElem = STORAGE == 0 ? 4 : (STORAGE == 1 ? 2 : 1);
  __shared__ float xs[TOK][kCols];
  __shared__ float partial[kWarps][kRows][TOK];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int scale_cols = (cols + 127) / 128;
  const int n_tasks = (rows + kRows - 1) / kRows;
  const uint8_t* wbytes = static_cast<const uint8_t*>(weights);

  auto stage = [&](int c0, int count) {
    stage_activation<STORAGE, TOK>(x, &xs[0][0], kCols, cols, c0, count, warp, lane);
  };
  // acc[r][t] += sum over the staged columns [c0, c0 + count) of W[row0 + r][c] * x[t][c]
  auto accumulate = [&](float (&acc)[kRows][TOK], int row0, int c0, int count) {
    if (VECTOR) {
      // all rows of the task advance together: kRows * kUnroll 16-byte loads in flight per lane,
      // and each staged activation chunk is read once for the kRows rows
      constexpr int kUnroll = 2;
      size_t base[kRows];
      const float* srow[kRows];
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        const int row = min(row0 + r, rows - 1);          // rows past the end repeat the last one
        base[r] = (static_cast<size_t>(row) * cols + c0) * kElem;
        srow[r] = STORAGE == 2 ? scales + static_cast<size_t>(row / 128) * scale_cols : nullptr;
      }
      for (int c = threadIdx.x * kPer; c < count; c += kUnroll * kThreads * kPer) {
        uint4 raw[kRows][kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const int cu = min(c + u * kThreads * kPer, count - kPer);   // a tail step re-reads a valid chunk
#pragma unroll
          for (int r = 0; r < kRows; ++r)
            raw[r][u] = *reinterpret_cast<const uint4*>(wbytes + base[r] + static_cast<size_t>(cu) * kElem);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const int cu = c + u * kThreads * kPer;
          if (cu >= count) break;
          float4 xv[TOK][kPer / 4];
#pragma unroll
          for (int t = 0; t < TOK; ++t)
#pragma unroll
            for (int i = 0; i < kPer / 4; ++i) xv[t][i] = staged4(xs[t], cu + 4 * i);
#pragma unroll
          for (int r = 0; r < kRows; ++r) {
            float w[kPer];
            Weights<STORAGE>::convert(raw[r][u], w);
            const float s = STORAGE == 2 ? srow[r][(c0 + cu) / 128] : 1.0f;
#pragma unroll
            for (int t = 0; t < TOK; ++t) {
              float part = 0.0f;
#pragma unroll
              for (int i = 0; i < kPer / 4; ++i) {
                part = fmaf(w[4 * i], xv[t][i].x, part);
                part = fmaf(w[4 * i + 1], xv[t][i].y, part);
                part = fmaf(w[4 * i + 2], xv[t][i].z, part);
                part = fmaf(w[4 * i + 3], xv[t][i].w, part);
              }
              acc[r][t] = STORAGE == 2 ? fmaf(part, s, acc[r][t]) : acc[r][t] + part;
            }
          }
        }
      }
    } else {
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        const int row = row0 + r;
        if (row >= rows) continue;
        const size_t base = static_cast<size_t>(row) * cols + c0;
        const float* srow = STORAGE == 2 ? scales + static_cast<size_t>(row / 128) * scale_cols : nullptr;
        for (int c = threadIdx.x; c < count; c += kThreads) {
          float wv = Weights<STORAGE>::one(weights, base + c);
          if (STORAGE == 2) wv *= srow[(c0 + c) / 128];
#pragma unroll
          for (int t = 0; t < TOK; ++t) acc[r][t] = fmaf(wv, xs[t][swizzled(c)], acc[r][t]);
        }
      }
    }
  };
  auto finish = [&](float (&acc)[kRows][TOK], int row0) {
#pragma unroll
    for (int r = 0; r < kRows; ++r)
#pragma unroll
      for (int t = 0; t < TOK; ++t) {
        float v = acc[r][t];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) partial[warp][r][t] = v;
      }
    __syncthreads();
    if (threadIdx.x < kRows * TOK) {
      const int r = threadIdx.x / TOK, t = threadIdx.x % TOK;
      float v = 0.0f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) v += partial[w][r][t];
      if (row0 + r < rows) y[static_cast<size_t>(t) * rows + row0 + r] = __float2bfloat16_rn(v);
    }
    __syncthreads();   // partial is rewritten by the next task
  };

  if (cols <= kCols) {
    stage(0, cols);
    __syncthreads();
    for (int task = blockIdx.x; task < n_tasks; task += gridDim.x) {
      float acc[kRows][TOK] = {};
      accumulate(acc, task * kRows, 0, cols);
      finish(acc, task * kRows);
    }
  } else {
    const int task = blockIdx.x;
    float acc[kRows][TOK] = {};
    for (int c0 = 0; c0 < cols; c0 += kCols) {
      const int count = min(kCols, cols - c0);
      __syncthreads();   // the previous pass is done with xs
      stage(c0, count);
      __syncthreads();
      accumulate(acc, task * kRows, c0, count);
    }
    finish(acc, task * kRows);
  }
}

// ------------------------------------------------------------------------------------------------
// Streaming form for bf16 and FP8 weights whose rows are 16-byte multiples: two persistent CTAs
// per SM; a copy thread keeps a ring of weight slabs (1-4 rows, one contiguous bulk copy each)
// in flight through the TMA unit, starting before the activation is staged, and the compute
// warps take each slab from shared memory.  The loads no longer depend on what the compute warps
// are doing (staging, the cross-warp sum, the store).  Measured on [10240 x 5120] bf16: the stream
// itself runs at 7.0 TB/s (time per extra 105 MB of rows), and a call costs ~6 us on top of that;
// two CTAs per SM with a 108 KB budget each (21.2 us) beat one CTA with 220 KB (23.5 us) because
// the next launch's CTAs can move in, and start their copies, while this launch's last CTAs
// still compute.
// ------------------------------------------------------------------------------------------------
constexpr int kStreamBudget = 108 * 1024;   // dynamic shared memory per CTA: two CTAs fit an SM
constexpr int kStreamCtasPerSm = 2;
constexpr int kStreamMaxStages = 8;
// The compute warps work as independent groups, each on its own slab: a slab's chain of
// dependent steps (barrier wait, loads, multiply-adds, shuffle and cross-warp sums, store) is
// then overlapped with three other slabs' instead of being paid once per slab.
constexpr int kGroups = 4, kGroupWarps = kWarps / kGroups, kGroupThreads = kGroupWarps * 32;

struct StreamLayout {
  int stages, slab_rows;
  size_t slab_bytes, xs_floats, xs_offset, partial_offset, bar_offset, total;
};
// Ring first (1024-byte aligned slabs), then the staged activation, the two partial-sum buffers
// and the barriers.  A slab holds 4, 2 or 1 rows, the most that leaves room for a ring slot per
// group; the number of slots is a multiple of the groups, so that a slot's barriers are only ever
// used by one group (a second group waiting for the slot's next phase could not tell it from
// the previous one by parity).  stages == 0: does not fit.
inline StreamLayout stream_layout(int cols, int tokens_per_pass, size_t elem) {
  StreamLayout l;
  l.xs_floats = static_cast<size_t>(cols + 15) / 16 * 16;
  const size_t fixed = static_cast<size_t>(tokens_per_pass) * l.xs_floats * 4 +
                       2 * kWarps * kRows * tokens_per_pass * 4 + 2 * kStreamMaxStages * 8 + 4 * kGroups;
  l.stages = 0;
  for (l.slab_rows = kRows; l.slab_rows >= 1 && l.stages == 0; l.slab_rows /= 2) {
    l.slab_bytes = (static_cast<size_t>(l.slab_rows) * cols * elem + 1023) / 1024 * 1024;
    if (fixed < static_cast<size_t>(kStreamBudget))
      l.stages = static_cast<int>(std::min<size_t>(kStreamMaxStages, (kStreamBudget - fixed) / l.slab_bytes)) /
                 kGroups * kGroups;
    if (l.stages > 0) break;
  }
  if (l.stages == 0) l.slab_rows = kRows;
  l.xs_offset = l.stages * l.slab_bytes;
  l.partial_offset = l.xs_offset + static_cast<size_t>(tokens_per_pass) * l.xs_floats * 4;
  l.bar_offset = l.partial_offset + 2 * kWarps * kRows * tokens_per_pass * 4;
  l.total = l.bar_offset + 2 * kStreamMaxStages * 8 + 4 * kGroups;
  return l;
}

template <int STORAGE, int TOK>
__global__ void __launch_bounds__(kThreads + 32, 2)
linear_gemv_stream(const void* __restrict__ weights, const float* __restrict__ scales,
                   const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, int cols,
                   int rows, StreamLayout layout, uint32_t* status) {
  constexpr int kPer = Weights<STORAGE>::kPer;
  constexpr size_t kElem = STORAGE == 1 ? 2 : 1;
  extern __shared__ __align__(1024) uint8_t stream_smem[];
  uint8_t* ring = stream_smem;
  float* xs = reinterpret_cast<float*>(stream_smem + layout.xs_offset);
  float* partial = reinterpret_cast<float*>(stream_smem + layout.partial_offset);   // [2][warp][row][tok]
  uint64_t* full = reinterpret_cast<uint64_t*>(stream_smem + layout.bar_offset);
  uint64_t* empty = full + kStreamMaxStages;
  int* failed = reinterpret_cast<int*>(empty + kStreamMaxStages);
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int stages = layout.stages;
  const int ld = static_cast<int>(layout.xs_floats);
  const int slab_rows = layout.slab_rows;
  const int n_tasks = (rows + slab_rows - 1) / slab_rows;
  const size_t row_bytes = static_cast<size_t>(cols) * kElem;
  const uint8_t* wbytes = static_cast<const uint8_t*>(weights);

  // Launched with programmatic stream serialisation: the next launch in the stream may start as
  // soon as every CTA of this one has got here, and stream its (frozen) weights while this grid
  // finishes; it reads its activation and writes its output only after griddepcontrol.wait.
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kGroupWarps);
    }
    for (int g = 0; g < kGroups; ++g) failed[g] = 0;
    mbar_fence_init();
  }
  __syncthreads();

  // slab n of this CTA = task blockIdx.x + n * gridDim.x
  auto issue = [&](int n) {
    const int task = blockIdx.x + n * gridDim.x;
    const int st = n % stages;
    const uint32_t bytes = static_cast<uint32_t>(min(slab_rows, rows - task * slab_rows) * row_bytes);
    mbar_expect_tx(&full[st], bytes);
    bulk_load(ring + st * layout.slab_bytes, wbytes + static_cast<size_t>(task) * slab_rows * row_bytes, bytes,
              &full[st]);
  };
  const int my_tasks = blockIdx.x < n_tasks ? (n_tasks - 1 - blockIdx.x) / gridDim.x + 1 : 0;

  if (warp == kWarps) {
    // ---------------------------------------------------------------- copy thread
    if (lane == 0) {
      for (int n = 0; n < min(stages, my_tasks); ++n) issue(n);
      for (int n = stages; n < my_tasks; ++n) {
        if (!mbar_wait(&empty[n % stages], (n / stages - 1) & 1, status, 40)) break;
        issue(n);
      }
    }
    return;
  }

  // ------------------------------------------------------------------ compute warps
  pdl_wait();   // the previous kernel's output may be this activation
  stage_activation<STORAGE, TOK>(x, xs, ld, cols, 0, cols, warp, lane);
  asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory");
  const int scale_cols = (cols + 127) / 128;
  const int group = warp / kGroupWarps, gwarp = warp % kGroupWarps;
  const int gthread = threadIdx.x % kGroupThreads;
  // slab n of this CTA goes to group n % kGroups
  for (int n = group, turn = 0; n < my_tasks; n += kGroups, ++turn) {
    const int task = blockIdx.x + n * gridDim.x, row0 = task * slab_rows, st = n % stages;
    const int rows_here = min(slab_rows, rows - row0);
    const float* srow = STORAGE == 2 ? scales + static_cast<size_t>(row0 / 128) * scale_cols : nullptr;
    float acc[kRows][TOK] = {};
    const bool ok = mbar_wait(&full[st], (n / stages) & 1, status, 41);
    if (!ok) *reinterpret_cast<volatile int*>(failed + group) = 1;
    if (ok) {
      const uint8_t* slab = ring + st * layout.slab_bytes;
      for (int c = gthread * kPer; c < cols; c += kGroupThreads * kPer) {
        float4 xv[TOK][kPer / 4];
#pragma unroll
        for (int t = 0; t < TOK; ++t)
#pragma unroll
          for (int i = 0; i < kPer / 4; ++i) xv[t][i] = staged4(xs + t * ld, c + 4 * i);
        // the rows of a slab lie in one 128-row scale block (1, 2 and 4 divide 128)
        const float s = STORAGE == 2 ? srow[c / 128] : 1.0f;
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
          if (r >= rows_here) break;
          float w[kPer];
          Weights<STORAGE>::convert(*reinterpret_cast<const uint4*>(slab + r * row_bytes + c * kElem), w);
#pragma unroll
          for (int t = 0; t < TOK; ++t) {
            float part = 0.0f;
#pragma unroll
            for (int i = 0; i < kPer / 4; ++i) {
              part = fmaf(w[4 * i], xv[t][i].x, part);
              part = fmaf(w[4 * i + 1], xv[t][i].y, part);
              part = fmaf(w[4 * i + 2], xv[t][i].z, part);
              part = fmaf(w[4 * i + 3], xv[t][i].w, part);
            }
            acc[r][t] = STORAGE == 2 ? fmaf(part, s, acc[r][t]) : acc[r][t] + part;
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[st]);   // this warp has read its share of the slab
    }
    // [buffer][group][warp of the group][row][token]
    float* mine = partial + (((turn & 1) * kGroups + group) * kGroupWarps) * kRows * TOK;
#pragma unroll
    for (int r = 0; r < kRows; ++r)
#pragma unroll
      for (int t = 0; t < TOK; ++t) {
        float v = acc[r][t];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) mine[(gwarp * kRows + r) * TOK + t] = v;
      }
    // one barrier of the group per slab: the partial sums alternate between two buffers
    asm volatile("bar.sync %0, %1;" ::"r"(2 + group), "n"(kGroupThreads) : "memory");
    if (*reinterpret_cast<volatile int*>(failed + group)) break;   // same for the whole group: set before the barrier
    if (gthread < kRows * TOK) {
      const int r = gthread / TOK, t = gthread % TOK;
      float v = 0.0f;
#pragma unroll
      for (int w = 0; w < kGroupWarps; ++w) v += mine[(w * kRows + r) * TOK + t];
      if (r < rows_here) y[static_cast<size_t>(t) * rows + row0 + r] = __float2bfloat16_rn(v);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// bf16 and FP8 weights with cols % 128 == 0: the multiply-adds run on the tensor cores
// (mma.sync, fp32 accumulation of exact products), which leaves the issue slots to the loads -- the
// FMA form spends ~2 (bf16) to ~4 (FP8: cvt, scale, fma) instructions per weight and is
// instruction-bound for FP8.  One CTA per 16 output rows; its 8 warps interleave over the K
// blocks and are summed through shared memory in warp order.  A lane loads 16 consecutive bytes
// of rows g and g + 8 (g = lane / 4) at byte offset 16 * (lane % 4) of the block; the four words
// feed two MMAs, and the activation fragment is read from the same K positions, so the
// permutation of K inside a block is the same on both sides.  Up to 8 tokens are the N columns
// (absent tokens contribute zero fragments).  FP8: the activation is quantised to E4M3 codes in
// shared memory with its per-128 scale kept apart, and every 64-column block's partial sum is
// multiplied by (weight block scale x activation group scale) when it is added.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_e4m3(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int kMmaRows = 16, kMmaTokens = 8;

// dynamic shared memory: activation rows [tokens][cols] (bf16, or E4M3 codes), then for FP8 the
// activation scales [tokens][cols / 128]
template <int STORAGE>
__global__ void __launch_bounds__(kThreads)
linear_gemv_mma(const void* __restrict__ weights, const float* __restrict__ scales,
                const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, int cols, int rows,
                int tokens) {
  constexpr int kElem = STORAGE == 1 ? 2 : 1;            // bytes per weight
  constexpr int kBlock = 64 / kElem;                      // K elements per block: 32 bf16 or 64 fp8
  extern __shared__ __align__(16) uint8_t gemv_smem[];
  __shared__ float partial[kWarps][kMmaRows][kMmaTokens];
  uint8_t* xs = gemv_smem;
  float* xscale = reinterpret_cast<float*>(gemv_smem + static_cast<size_t>(tokens) * cols * kElem);
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int groups = cols / 128;

  if (STORAGE == 1) {
    const int chunks = tokens * cols / 8;                 // 16-byte chunks; x rows are contiguous
    for (int i = threadIdx.x; i < chunks; i += kThreads)
      reinterpret_cast<uint4*>(xs)[i] = reinterpret_cast<const uint4*>(x)[i];
  } else {
    for (int group = warp; group < tokens * groups; group += kWarps) {
      const int t = group / groups, g = group % groups;
      float v[4], maximum = 0.0f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[i] = __bfloat162float(x[static_cast<size_t>(t) * cols + g * 128 + lane * 4 + i]);
        maximum = fmaxf(maximum, fabsf(v[i]));
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, o));
      const float scale = maximum / 448.0f, divisor = fmaxf(scale, 1e-12f);
      uint32_t word = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        word |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(v[i] / divisor, __NV_SATFINITE, __NV_E4M3)) << (8 * i);
      reinterpret_cast<uint32_t*>(xs + static_cast<size_t>(t) * cols + g * 128)[lane] = word;
      if (lane == 0) xscale[t * groups + g] = scale;
    }
  }
  __syncthreads();

  const int g = lane / 4, q = lane % 4;
  const int r0 = blockIdx.x * kMmaRows;
  const int ra = min(r0 + g, rows - 1), rb = min(r0 + g + 8, rows - 1);   // rows past the end repeat
  const uint8_t* wa = static_cast<const uint8_t*>(weights) + static_cast<size_t>(ra) * cols * kElem + q * 16;
  const uint8_t* wb = static_cast<const uint8_t*>(weights) + static_cast<size_t>(rb) * cols * kElem + q * 16;
  const uint8_t* xg = xs + static_cast<size_t>(min(g, tokens - 1)) * cols * kElem + q * 16;
  const bool has_token = g < tokens;                      // N column g of the MMA is token g
  const float* sa = STORAGE == 2 ? scales + static_cast<size_t>(ra / 128) * groups : nullptr;
  const float* sb = STORAGE == 2 ? scales + static_cast<size_t>(rb / 128) * groups : nullptr;
  // accumulator element i: row (i < 2 ? g : g + 8), token 2 q + (i & 1)
  const int t0 = min(2 * q, tokens - 1), t1 = min(2 * q + 1, tokens - 1);
  float total[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  const int blocks = cols / kBlock;
  constexpr int kUnroll = 4;
  for (int kb = warp; kb < blocks; kb += kWarps * kUnroll) {
    uint4 a[kUnroll], b[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int k = min(kb + u * kWarps, blocks - 1);      // a tail step re-reads a valid block
      a[u] = *reinterpret_cast<const uint4*>(wa + static_cast<size_t>(k) * 64);
      b[u] = *reinterpret_cast<const uint4*>(wb + static_cast<size_t>(k) * 64);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int k = kb + u * kWarps;
      if (k >= blocks) break;
      uint4 xv = make_uint4(0u, 0u, 0u, 0u);
      if (has_token) xv = *reinterpret_cast<const uint4*>(xg + static_cast<size_t>(k) * 64);
      if (STORAGE == 1) {
        mma_bf16(total, a[u].x, b[u].x, a[u].y, b[u].y, xv.x, xv.y);
        mma_bf16(total, a[u].z, b[u].z, a[u].w, b[u].w, xv.z, xv.w);
      } else {
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        mma_e4m3(acc, a[u].x, b[u].x, a[u].y, b[u].y, xv.x, xv.y);
        mma_e4m3(acc, a[u].z, b[u].z, a[u].w, b[u].w, xv.z, xv.w);
        const int group = k / 2;
        const float wsa = sa[group], wsb = sb[group];
        const float x0 = xscale[t0 * groups + group], x1 = xscale[t1 * groups + group];
        total[0] = fmaf(acc[0], wsa * x0, total[0]);
        total[1] = fmaf(acc[1], wsa * x1, total[1]);
        total[2] = fmaf(acc[2], wsb * x0, total[2]);
        total[3] = fmaf(acc[3], wsb * x1, total[3]);
      }
    }
  }
  partial[warp][g][2 * q] = total[0];
  partial[warp][g][2 * q + 1] = total[1];
  partial[warp][g + 8][2 * q] = total[2];
  partial[warp][g + 8][2 * q + 1] = total[3];
  __syncthreads();
  if (threadIdx.x < kMmaRows * kMmaTokens) {
    const int r = threadIdx.x / kMmaTokens, t = threadIdx.x % kMmaTokens;
    float v = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) v += partial[w][r][t];
    if (r0 + r < rows && t < tokens) y[static_cast<size_t>(t) * rows + r0 + r] = __float2bfloat16_rn(v);
  }
}

// ------------------------------------------------------------------------------------------------
// FP8 weights, one to four tokens, cols % 256 == 0: the streaming ring feeding the tensor cores.
// The FMA form above spends its time converting E4M3 to fp32 (its slope is 4.1 TB/s); an
// m16n8k32 E4M3 MMA takes the codes as they are.  A slab is 4 (2, 1) weight rows in one contiguous
// piece of memory, so the MMA is laid out around that: every row is cut into two halves of
// cols / 2, the 8 columns of the B operand are the 8 (row, half) pieces, and the rows of the A
// operand are the (token, half) pieces of the quantised activation.  D[(t, h)][(r, h')] is the
// dot product of token t's half h with row r's half h'; only h == h' means anything, and
// y[t][r] = D[(t,0)][(r,0)] + D[(t,1)][(r,1)].  Half of the tensor work is thrown away, which
// costs nothing here.  Every piece sits in shared memory at a stride of its length + 64 bytes,
// which makes the fragments' 16-byte loads conflict-free, and a lane loads 16 consecutive bytes
// at 16 * (lane % 4) of a 64-byte block on both sides, so the K order inside a block is the same
// permutation for A and B.  Scales: each 128-column group's four MMAs go into a fresh
// accumulator that is added with (weight block scale x activation group scale).
// ------------------------------------------------------------------------------------------------
constexpr int kPiecePad = 64;

struct StreamMmaLayout {
  int stages, slab_rows, half;               // half = cols / 2
  size_t piece_stride, slab_bytes, xs_offset, xscale_offset, partial_offset, bar_offset, total;
};
inline StreamMmaLayout stream_mma_layout(int cols, int tokens) {
  StreamMmaLayout l;
  l.half = cols / 2;
  l.piece_stride = static_cast<size_t>(l.half) + kPiecePad;
  const size_t xs_bytes = 2 * static_cast<size_t>(tokens) * l.piece_stride;
  const size_t xscale_bytes = static_cast<size_t>(tokens) * (cols / 128) * 4;
  const size_t partial_bytes = 2 * kWarps * 4 * kRows * 4;   // [buffer][warp][token][row]
  const size_t tail = 2 * kStreamMaxStages * 8 + 4 * kGroups;
  const size_t fixed = xs_bytes + xscale_bytes + partial_bytes + tail;
  l.stages = 0;
  for (l.slab_rows = kRows; l.slab_rows >= 1; l.slab_rows /= 2) {
    l.slab_bytes = (2 * l.slab_rows * l.piece_stride + 1023) / 1024 * 1024;
    if (fixed < static_cast<size_t>(kStreamBudget))
      l.stages = static_cast<int>(std::min<size_t>(kStreamMaxStages, (kStreamBudget - fixed) / l.slab_bytes)) /
                 kGroups * kGroups;
    if (l.stages > 0) break;
  }
  if (l.stages == 0) l.slab_rows = kRows;
  l.xs_offset = l.stages * l.slab_bytes;
  l.xscale_offset = l.xs_offset + xs_bytes;
  l.partial_offset = l.xscale_offset + xscale_bytes;
  l.bar_offset = (l.partial_offset + partial_bytes + 7) / 8 * 8;
  l.total = l.bar_offset + tail;
  return l;
}

__global__ void __launch_bounds__(kThreads + 32, 2)
linear_gemv_stream_e4m3(const uint8_t* __restrict__ weights, const float* __restrict__ scales,
                        const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, int cols,
                        int rows, int tokens, StreamMmaLayout layout, uint32_t* status) {
  extern __shared__ __align__(1024) uint8_t stream_smem[];
  uint8_t* ring = stream_smem;
  uint8_t* xs = stream_smem + layout.xs_offset;                                   // [token][half][piece]
  float* xscale = reinterpret_cast<float*>(stream_smem + layout.xscale_offset);   // [token][cols / 128]
  float* partial = reinterpret_cast<float*>(stream_smem + layout.partial_offset);
  uint64_t* full = reinterpret_cast<uint64_t*>(stream_smem + layout.bar_offset);
  uint64_t* empty = full + kStreamMaxStages;
  int* failed = reinterpret_cast<int*>(empty + kStreamMaxStages);
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int stages = layout.stages, slab_rows = layout.slab_rows, half = layout.half;
  const size_t stride = layout.piece_stride;
  const int n_tasks = (rows + slab_rows - 1) / slab_rows;
  const int groups128 = cols / 128;

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kGroupWarps);
    }
    for (int g = 0; g < kGroups; ++g) failed[g] = 0;
    mbar_fence_init();
  }
  __syncthreads();

  // slab n of this CTA = task blockIdx.x + n * gridDim.x; piece 2 r + h = half h of its row r
  auto issue = [&](int n) {
    const int task = blockIdx.x + n * gridDim.x;
    const int st = n % stages;
    const int rows_here = min(slab_rows, rows - task * slab_rows);
    mbar_expect_tx(&full[st], static_cast<uint32_t>(rows_here) * cols);
    const uint8_t* src = weights + static_cast<size_t>(task) * slab_rows * cols;
    uint8_t* dst = ring + st * layout.slab_bytes;
    for (int piece = 0; piece < 2 * rows_here; ++piece)
      bulk_load(dst + piece * stride, src + static_cast<size_t>(piece) * half, half, &full[st]);
  };
  const int my_tasks = blockIdx.x < n_tasks ? (n_tasks - 1 - blockIdx.x) / gridDim.x + 1 : 0;

  if (warp == kWarps) {
    if (lane == 0) {
      for (int n = 0; n < min(stages, my_tasks); ++n) issue(n);
      for (int n = stages; n < my_tasks; ++n) {
        if (!mbar_wait(&empty[n % stages], (n / stages - 1) & 1, status, 42)) break;
        issue(n);
      }
    }
    return;
  }

  // activation -> E4M3 codes per (token, half) piece + one scale per group of 128 (one warp a group)
  pdl_wait();   // the previous kernel's output may be this activation
  {
    constexpr int kBatch = 5;   // groups whose 8-byte loads are in flight together
    const int total = tokens * groups128;
    for (int first = warp; first < total; first += kWarps * kBatch) {
      uint2 raw[kBatch];
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const int group = min(first + u * kWarps, total - 1);
        const int t = group / groups128, g = group % groups128;
        raw[u] = *reinterpret_cast<const uint2*>(x + static_cast<size_t>(t) * cols + g * 128 + lane * 4);
      }
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        // no early exit: the batch's reductions are independent chains that interleave
        const int group = min(first + u * kWarps, total - 1);   // past the end: repeats the last group
        const int t = group / groups128, g = group % groups128;
        const float v[4] = {bf16_lo(raw[u].x), bf16_hi(raw[u].x), bf16_lo(raw[u].y), bf16_hi(raw[u].y)};
        float maximum = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, o));
        const float scale = maximum / 448.0f, divisor = fmaxf(scale, 1e-12f);
        uint32_t word = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          word |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(v[i] / divisor, __NV_SATFINITE, __NV_E4M3)) << (8 * i);
        const int c = g * 128 + lane * 4, h = c / half;
        *reinterpret_cast<uint32_t*>(xs + (2 * t + h) * stride + (c - h * half)) = word;
        if (lane == 0) xscale[t * groups128 + g] = scale;
      }
    }
  }
  asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory");

  const int group = warp / kGroupWarps, gwarp = warp % kGroupWarps;
  const int gthread = threadIdx.x % kGroupThreads;
  const int g = lane / 4, q = lane % 4;
  // A row g = (token g / 2, half g % 2); B column g = piece g = (row g / 2, half g % 2);
  // accumulator element i < 2 of this lane: A row g, B column 2 q + i = (row q, half i)
  const int my_half = g & 1, my_token = g >> 1;
  const bool a_valid = my_token < tokens;
  const uint8_t* a_ptr = xs + g * stride + q * 16;
  const int half_groups = half / 128;
  const float* my_xscale = xscale + min(my_token, tokens - 1) * groups128 + my_half * half_groups;
  for (int n = group, turn = 0; n < my_tasks; n += kGroups, ++turn) {
    const int task = blockIdx.x + n * gridDim.x, row0 = task * slab_rows, st = n % stages;
    const int rows_here = min(slab_rows, rows - row0);
    // the rows of a slab lie in one 128-row scale block (1, 2 and 4 divide 128)
    const float* wscale = scales + static_cast<size_t>(row0 / 128) * groups128 + my_half * half_groups;
    float total = 0.0f;
    const bool ok = mbar_wait(&full[st], (n / stages) & 1, status, 43);
    if (!ok) *reinterpret_cast<volatile int*>(failed + group) = 1;
    if (ok) {
      // columns past the slab's pieces (slabs of fewer than 4 rows) re-read its last piece; their
      // results are never stored
      const uint8_t* b_ptr = ring + st * layout.slab_bytes + min(g, 2 * slab_rows - 1) * stride + q * 16;
      for (int kg = gwarp; kg < half_groups; kg += kGroupWarps) {
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int block = 0; block < 2; ++block) {
          const uint4 b = *reinterpret_cast<const uint4*>(b_ptr + kg * 128 + block * 64);
          uint4 a = make_uint4(0u, 0u, 0u, 0u);
          if (a_valid) a = *reinterpret_cast<const uint4*>(a_ptr + kg * 128 + block * 64);
          mma_e4m3(acc, a.x, 0u, a.y, 0u, b.x, b.y);
          mma_e4m3(acc, a.z, 0u, a.w, 0u, b.z, b.w);
        }
        // the element whose B half matches this lane's A half
        total = fmaf(my_half ? acc[1] : acc[0], wscale[kg] * my_xscale[kg], total);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[st]);
    }
    total += __shfl_xor_sync(0xffffffffu, total, 4);   // the two halves: lanes g and g ^ 1
    // [buffer][group][warp of the group][token][row]
    float* mine = partial + (((turn & 1) * kGroups + group) * kGroupWarps) * 4 * kRows;
    if (my_half == 0) mine[(gwarp * 4 + my_token) * kRows + q] = total;
    asm volatile("bar.sync %0, %1;" ::"r"(2 + group), "n"(kGroupThreads) : "memory");
    if (*reinterpret_cast<volatile int*>(failed + group)) break;   // same for the whole group
    if (gthread < 4 * kRows) {
      const int t = gthread / kRows, r = gthread % kRows;
      float v = 0.0f;
#pragma unroll
      for (int w = 0; w < kGroupWarps; ++w) v += mine[(w * 4 + t) * kRows + r];
      if (t < tokens && r < rows_here) y[static_cast<size_t>(t) * rows + row0 + r] = __float2bfloat16_rn(v);
    }
  }
}

// Rows so long that only slabs of fewer than 4 rows fit the ring leave B columns unused and were
// measured slower than the FMA form ([5120 x 8192]: 19.8 against 18.3 us), so they do not qualify.
inline bool stream_mma_ok(const void* weights, const void* x, int cols, int rows, int tokens, int sms) {
  if (tokens > 4 || cols % 256 != 0 || reinterpret_cast<uintptr_t>(weights) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(x) % 8 != 0 || rows < 2 * kRows * kStreamCtasPerSm * sms)
    return false;
  const StreamMmaLayout layout = stream_mma_layout(cols, tokens);
  return layout.stages > 0 && layout.slab_rows == kRows;
}

inline cudaError_t launch_stream_mma(cudaStream_t stream, const void* weights, const float* scales,
                                     const void* x, void* y, int cols, int rows, int tokens, int sms) {
  const StreamMmaLayout layout = stream_mma_layout(cols, tokens);
  const cudaError_t e = cudaFuncSetAttribute(linear_gemv_stream_e4m3, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(layout.total));
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(kStreamCtasPerSm * sms);
  config.blockDim = dim3(kThreads + 32);
  config.dynamicSmemBytes = layout.total;
  config.stream = stream;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, linear_gemv_stream_e4m3, static_cast<const uint8_t*>(weights), scales,
                            static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), cols, rows,
                            tokens, layout, kernel_status_word());
}

template <int STORAGE>
bool mma_path_ok(const void* weights, const void* x, int cols, int tokens) {
  const size_t smem = static_cast<size_t>(tokens) * cols * (STORAGE == 1 ? 2 : 1) +
                      (STORAGE == 2 ? static_cast<size_t>(tokens) * (cols / 128) * 4 : 0);
  return cols % 128 == 0 && reinterpret_cast<uintptr_t>(weights) % 16 == 0 &&
         reinterpret_cast<uintptr_t>(x) % 16 == 0 && smem <= 96 * 1024;
}

template <int STORAGE>
cudaError_t launch_mma(cudaStream_t stream, const void* weights, const float* scales, const void* x,
                       void* y, int cols, int rows, int tokens) {
  const size_t smem = static_cast<size_t>(tokens) * cols * (STORAGE == 1 ? 2 : 1) +
                      (STORAGE == 2 ? static_cast<size_t>(tokens) * (cols / 128) * 4 : 0);
  cudaError_t e = cudaFuncSetAttribute(linear_gemv_mma<STORAGE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  linear_gemv_mma<STORAGE><<<(rows + kMmaRows - 1) / kMmaRows, kThreads, smem, stream>>>(
      weights, scales, static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), cols, rows,
      tokens);
  return cudaGetLastError();
}

// The streaming form wants 16-byte rows, at least two ring slots and enough 4-row tasks to give
// every SM a few.
template <int STORAGE>
bool stream_path_ok(const void* weights, int cols, int rows, int tokens_per_pass, int sms) {
  const size_t elem = STORAGE == 1 ? 2 : 1;
  return reinterpret_cast<uintptr_t>(weights) % 16 == 0 && (static_cast<size_t>(cols) * elem) % 16 == 0 &&
         stream_layout(cols, tokens_per_pass, elem).stages > 0 && rows >= 2 * kRows * kStreamCtasPerSm * sms;
}

template <int STORAGE, int TOK>
cudaError_t launch(cudaStream_t stream, const void* weights, const float* scales, const void* x,
                   void* y, int cols, int rows) {
  constexpr int kCols = kChunk / TOK / 128 * 128;
  const int n_tasks = (rows + kRows - 1) / kRows;
  unsigned grid = n_tasks;
  int sms = 148, device = 0;
  if (cudaGetDevice(&device) == cudaSuccess)
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  if (cols <= kCols) grid = min(grid, static_cast<unsigned>(3 * sms));
  const size_t elem = STORAGE == 0 ? 4 : (STORAGE == 1 ? 2 : 1);
  const bool vector = reinterpret_cast<uintptr_t>(weights) % 16 == 0 &&
                      (static_cast<size_t>(cols) * elem) % 16 == 0;
  auto* xin = static_cast<const __nv_bfloat16*>(x);
  auto* yout = static_cast<__nv_bfloat16*>(y);
  if constexpr (STORAGE != 0) {
    const StreamLayout layout = stream_layout(cols, TOK, elem);
    if (stream_path_ok<STORAGE>(weights, cols, rows, TOK, sms)) {
      auto kernel = linear_gemv_stream<STORAGE, TOK>;
      const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 static_cast<int>(layout.total));
      if (e != cudaSuccess) return e;
      cudaLaunchConfig_t config = {};
      config.gridDim = dim3(kStreamCtasPerSm * sms);
      config.blockDim = dim3(kThreads + 32);
      config.dynamicSmemBytes = layout.total;
      config.stream = stream;
      cudaLaunchAttribute attribute;
      attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attribute.val.programmaticStreamSerializationAllowed = 1;
      config.attrs = &attribute;
      config.numAttrs = 1;
      return cudaLaunchKernelEx(&config, kernel, weights, scales, xin, yout, cols, rows, layout,
                                kernel_status_word());
    }
  }
  if (vector)
    linear_gemv_kernel<STORAGE, TOK, true><<<grid, kThreads, 0, stream>>>(weights, scales, xin, yout, cols, rows);
  else
    linear_gemv_kernel<STORAGE, TOK, false><<<grid, kThreads, 0, stream>>>(weights, scales, xin, yout, cols, rows);
  return cudaGetLastError();
}

template <int STORAGE>
cudaError_t dispatch(cudaStream_t stream, const void* weights, const float* scales, const void* x,
                     void* y, int tokens, int cols, int rows) {
  auto* xin = static_cast<const __nv_bfloat16*>(x);
  auto* yout = static_cast<__nv_bfloat16*>(y);
  if constexpr (STORAGE != 0) {
    // Measured on a [10240 x 5120] matrix, us per call with the weights coming from HBM:
    //   tokens                          1      2      3      4      8
    //   bf16 ring, FMA                 21.2   29.0    -     35.3    -
    //   bf16 tensor cores from global  24.7   24.7    -     35.4   38.2
    //   FP8 ring, tensor cores         14.8   17.0    -     21.5   41.2 (two passes)
    //   FP8 ring, FMA                  17.2   23.2   38.3   56.1    -
    //   FP8 tensor cores from global   26.9   33.0    -     45.1   69.0
    // (the FMA form without the ring: 25.7 and 23.3 for one token, 80-143 for FP8 batches whose
    // activation no longer fits its staging buffer).  So FP8 takes the ring with tensor cores in
    // passes of 4 tokens when the shape qualifies, else the FMA ring for up to three tokens; one
    // bf16 token takes the FMA ring; everything else that qualifies takes the tensor-core form
    // that loads from global memory, 8 tokens per pass.
    int sms = 148, device = 0;
    if (cudaGetDevice(&device) == cudaSuccess)
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (STORAGE == 2 && stream_mma_ok(weights, x, cols, rows, std::min(tokens, 4), sms)) {
      for (int t0 = 0; t0 < tokens; t0 += 4) {
        const cudaError_t e = launch_stream_mma(stream, weights, scales, xin + static_cast<size_t>(t0) * cols,
                                                yout + static_cast<size_t>(t0) * rows, cols, rows,
                                                std::min(4, tokens - t0), sms);
        if (e != cudaSuccess) return e;
      }
      return cudaSuccess;
    }
    const bool streamed = tokens <= (STORAGE == 1 ? 1 : 3) &&
                          stream_path_ok<STORAGE>(weights, cols, rows, tokens >= 2 ? 2 : 1, sms);
    if (!streamed && mma_path_ok<STORAGE>(weights, x, cols, std::min(tokens, kMmaTokens))) {
      for (int t0 = 0; t0 < tokens; t0 += kMmaTokens) {
        const cudaError_t e = launch_mma<STORAGE>(stream, weights, scales, xin + static_cast<size_t>(t0) * cols,
                                                  yout + static_cast<size_t>(t0) * rows, cols, rows,
                                                  std::min(kMmaTokens, tokens - t0));
        if (e != cudaSuccess) return e;
      }
      return cudaSuccess;
    }
  }
  // FMA form: tokens in passes of at most 4 (each pass streams the weights once)
  for (int t0 = 0; t0 < tokens;) {
    const int left = tokens - t0;
    cudaError_t e;
    const void* xp = xin + static_cast<size_t>(t0) * cols;
    void* yp = yout + static_cast<size_t>(t0) * rows;
    if (left >= 4) { e = launch<STORAGE, 4>(stream, weights, scales, xp, yp, cols, rows); t0 += 4; }
    else if (left >= 2) { e = launch<STORAGE, 2>(stream, weights, scales, xp, yp, cols, rows); t0 += 2; }
    else { e = launch<STORAGE, 1>(stream, weights, scales, xp, yp, cols, rows); t0 += 1; }
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

}  // namespace

cudaError_t linear_imported(cudaStream_t stream, const void* weights, int storage, const float* scales,
                            const void* x, void* y, int tokens, int cols, int rows) {
  if (storage == 0) return dispatch<0>(stream, weights, scales, x, y, tokens, cols, rows);
  if (storage == 1) return dispatch<1>(stream, weights, scales, x, y, tokens, cols, rows);
  return dispatch<2>(stream, weights, scales, x, y, tokens, cols, rows);
}

}  // namespace pluto
