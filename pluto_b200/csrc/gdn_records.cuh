// Per-chunk records that the chunked gated delta-net prepare kernel writes and the tcgen05 scan
// kernel (gdn_scan_sm100.cu) streams.  Every tile is stored in the byte order of a 128-byte
// swizzled shared-memory operand tile -- rows of 64 bf16 (128 bytes), the eight 16-byte pieces of
// row r permuted by (piece ^ (r & 7)), 64-column slabs one after the other -- so a record goes
// from global to a 1024-byte-aligned stage of shared memory as a linear bulk copy and is used by
// tcgen05.mma in place.
#pragma once

#include <stddef.h>
#include <stdint.h>

namespace pluto {

constexpr int kGdnChunk = 64;      // tokens per chunk
constexpr int kGdnKeyDim = 128;    // key width of the chunked path
constexpr int kGdnSliceCols = 128; // value columns per scan CTA

struct GdnRecord {
  // common to all value columns of a (sequence, head, chunk)
  static constexpr uint32_t kPN = 0;        // Pn = -(Kt^T W)   [128 key rows][128 keys], K-major: 2 slabs x 16384
  static constexpr uint32_t kKT = 32768;    // Kt = K . c_C/c   [64 tokens][128 keys], token-major: 2 slabs x 8192
  static constexpr uint32_t kQT = 49152;    // Qt = c.Q - M W   [64 tokens][128 keys], K-major: 2 slabs x 8192
  static constexpr uint32_t kMM = 65536;    // M                [64 tokens][64 tokens], K-major: 8192
  static constexpr uint32_t kGM = 73728;    // gamma (one float), padded to 1024
  static constexpr uint32_t kCommon = 74752;
  // per slice of 128 value columns
  static constexpr uint32_t kUH = 0;        // U (bf16)  [64 tokens][128 value columns], token-major
  static constexpr uint32_t kSlice = 16384;
  static __host__ __device__ size_t bytes(int value_dim) {
    return kCommon + static_cast<size_t>(value_dim / kGdnSliceCols) * kSlice;
  }
};

// Byte offset of element (row, col) inside a swizzled tile whose 64-column slabs hold
// `rows_per_slab` rows each.
__host__ __device__ inline uint32_t gdn_swizzled_offset(int rows_per_slab, int row, int col) {
  return static_cast<uint32_t>((col / 64) * rows_per_slab * 128 + row * 128 +
                               ((((col % 64) / 8) ^ (row & 7)) * 16) + (col % 8) * 2);
}

}  // namespace pluto
