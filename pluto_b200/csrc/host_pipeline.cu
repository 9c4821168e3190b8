// Prefill from host memory: the K/V heads are independent, so the sequence is cut into groups of
// key/value heads and each group's host->device copy, attention kernel and device->host copy run
// on three streams, two groups in flight.  PCIe then carries inputs and outputs at the same time
// and the kernel hides behind the copies; the call a host makes when activations live in pinned
// host memory (offloaded prefill, or a CPU-resident producer/consumer either side of the layer).
//
// The copies are strided (a group's columns of every token row): cudaMemcpy2DAsync, one per
// tensor and group.  Streams and events are created once per device and reused; the call itself
// allocates nothing and does not synchronise: everything is ordered behind `stream`, and `stream`
// is made to wait for the last output copy.
//
// kv_heads_per_group = 0 selects the other cut, by query tokens: a causal query only needs the
// keys before it, so chunk c of a sequence's tokens (queries, keys and values alike) is copied as
// three contiguous pieces, its queries run against all keys copied so far, and its output rows
// leave as one contiguous piece.  The device then holds the whole Q, K, V and output.  Measured
// on the 8192-token, 40/8-head prompt (117 MB in, 84 MB out; the link moves 84 MB one way in
// 1.52 ms): head groups 3.16-3.26 ms, token chunks of 1024 3.05 ms, 512 3.21 ms, 256 3.53 ms; the
// same copies with no kernels at all take 2.97-3.24 ms, because the two directions slow each
// other down, so both cuts sit at what the link delivers.
#include <mutex>

#include "../../include/pluto_b200.h"
#include "engine.h"

namespace {

constexpr int kSlots = 2;
constexpr int kMaxDevices = 64;
constexpr int kChunkTokens = 1024;  // token-chunk mode: smallest full-size chunk (8 query tiles; whole pairs)
constexpr size_t kChunkBytes = 4u << 20;   // ... grown until a chunk's input is at least this much
constexpr int kMaxChunkEvents = 64; // chunks in flight before the events are reused

struct Lanes {
  cudaStream_t h2d = nullptr, d2h = nullptr;
  cudaEvent_t start = nullptr, loaded[kSlots] = {}, computed[kSlots] = {}, stored[kSlots] = {};
  cudaEvent_t chunk_loaded[kMaxChunkEvents] = {}, chunk_computed[kMaxChunkEvents] = {}, last_stored = nullptr;
  bool ok = false;
};
Lanes g_lanes[kMaxDevices];
std::once_flag g_once[kMaxDevices];

Lanes* lanes_for_current_device() {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return nullptr;
  std::call_once(g_once[device], [device] {
    Lanes& l = g_lanes[device];
    bool ok = cudaStreamCreateWithFlags(&l.h2d, cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&l.d2h, cudaStreamNonBlocking) == cudaSuccess &&
              cudaEventCreateWithFlags(&l.start, cudaEventDisableTiming) == cudaSuccess;
    for (int s = 0; s < kSlots && ok; ++s)
      ok = cudaEventCreateWithFlags(&l.loaded[s], cudaEventDisableTiming) == cudaSuccess &&
           cudaEventCreateWithFlags(&l.computed[s], cudaEventDisableTiming) == cudaSuccess &&
           cudaEventCreateWithFlags(&l.stored[s], cudaEventDisableTiming) == cudaSuccess;
    for (int s = 0; s < kMaxChunkEvents && ok; ++s)
      ok = cudaEventCreateWithFlags(&l.chunk_loaded[s], cudaEventDisableTiming) == cudaSuccess &&
           cudaEventCreateWithFlags(&l.chunk_computed[s], cudaEventDisableTiming) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&l.last_stored, cudaEventDisableTiming) == cudaSuccess;
    l.ok = ok;
  });
  return g_lanes[device].ok ? &g_lanes[device] : nullptr;
}

size_t round256(size_t n) { return (n + 255) / 256 * 256; }

bool chunked_shape(int head_dim, int seq) { return (head_dim == 64 || head_dim == 128) && seq >= 1; }

// Token-chunk mode.  Device layout = host layout, so every copy is one contiguous piece.
int prefill_by_token_chunks(Lanes* l, cudaStream_t compute, const void* q_host, const void* k_host,
                            const void* v_host, void* out_host, void* workspace, int batch, int seq,
                            int q_heads, int kv_heads, int head_dim) {
  const size_t tokens = static_cast<size_t>(batch) * seq, D = head_dim;
  const size_t q_row = static_cast<size_t>(q_heads) * D * 2, kv_row = static_cast<size_t>(kv_heads) * D * 2;
  uint8_t* q_dev = static_cast<uint8_t*>(workspace);
  uint8_t* out_dev = q_dev + round256(tokens * q_row);
  uint8_t* k_dev = out_dev + round256(tokens * q_row);
  uint8_t* v_dev = k_dev + round256(tokens * kv_row);
  uint32_t* status = pluto::kernel_status_word();
  if (!status) return pluto::report(PLUTO_E_INTERNAL, "kernel status word unavailable");
  // With few heads per rank a 1024-token chunk is a fraction of a megabyte and the per-copy cost
  // would dominate: the full-size chunk grows (in steps of 1024 tokens) to at least kChunkBytes.
  const size_t token_bytes = q_row + 2 * kv_row;
  const int full = static_cast<int>(std::max<size_t>(1, (kChunkBytes / token_bytes + kChunkTokens - 1) / kChunkTokens)) *
                   kChunkTokens;
  cudaError_t e = cudaSuccess;
  int n = 0;   // chunks issued so far
  for (int b = 0; b < batch; ++b) {
    for (int t0 = 0, count = 0; t0 < seq; t0 += count, ++n) {
      // The last chunk's kernel and output copy have nothing to hide behind, so the chunks get
      // smaller towards the end of a sequence (all sizes are multiples of 256: whole tile pairs).
      const int left = seq - t0;
      count = std::min(left, left > 2 * full ? full : (left > full ? full / 2 : full / 4));
      const size_t first = static_cast<size_t>(b) * seq + t0;
      const int slot = n % kMaxChunkEvents;
      // the events of chunk n - kMaxChunkEvents are reused: its kernel must have taken them
      if (n >= kMaxChunkEvents) e = cudaStreamWaitEvent(l->h2d, l->chunk_computed[slot], 0);
      if (e == cudaSuccess)
        e = cudaMemcpyAsync(k_dev + first * kv_row, static_cast<const uint8_t*>(k_host) + first * kv_row,
                            count * kv_row, cudaMemcpyHostToDevice, l->h2d);
      if (e == cudaSuccess)
        e = cudaMemcpyAsync(v_dev + first * kv_row, static_cast<const uint8_t*>(v_host) + first * kv_row,
                            count * kv_row, cudaMemcpyHostToDevice, l->h2d);
      if (e == cudaSuccess)
        e = cudaMemcpyAsync(q_dev + first * q_row, static_cast<const uint8_t*>(q_host) + first * q_row,
                            count * q_row, cudaMemcpyHostToDevice, l->h2d);
      if (e == cudaSuccess) e = cudaEventRecord(l->chunk_loaded[slot], l->h2d);
      if (e == cudaSuccess) e = cudaStreamWaitEvent(compute, l->chunk_loaded[slot], 0);
      if (e != cudaSuccess) return pluto::report_cuda(e, "host prefill input copy");
      pluto::AttnFwdArgs a{};
      a.q = q_dev + static_cast<size_t>(b) * seq * q_row;
      a.k = k_dev + static_cast<size_t>(b) * seq * kv_row;
      a.v = v_dev + static_cast<size_t>(b) * seq * kv_row;
      a.q_cols = static_cast<int>(q_heads * D);
      a.kv_cols = static_cast<int>(kv_heads * D);
      a.q_token = q_heads * D; a.kv_token = kv_heads * D;
      a.q_head_cols = head_dim;
      a.batch = 1; a.seq = seq; a.heads = q_heads; a.group = q_heads / kv_heads; a.head_dim = head_dim;
      a.out = out_dev + static_cast<size_t>(b) * seq * q_row;
      a.out_token = q_heads * D; a.out_head = D;
      a.round_gate = 1;
      a.status = status;
      a.tile_begin = t0 / 128;
      a.tile_count = (count + 127) / 128;
      e = pluto::attn_fwd_tc(compute, a);
      if (e == cudaSuccess) e = cudaEventRecord(l->chunk_computed[slot], compute);
      if (e == cudaSuccess) e = cudaStreamWaitEvent(l->d2h, l->chunk_computed[slot], 0);
      if (e == cudaSuccess)
        e = cudaMemcpyAsync(static_cast<uint8_t*>(out_host) + first * q_row, out_dev + first * q_row,
                            count * q_row, cudaMemcpyDeviceToHost, l->d2h);
      if (e != cudaSuccess) return pluto::report_cuda(e, "host prefill kernel or output copy");
    }
  }
  e = cudaEventRecord(l->last_stored, l->d2h);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(compute, l->last_stored, 0);   // later work sees the whole output
  if (e != cudaSuccess) return pluto::report_cuda(e, "host prefill stream ordering");
  return PLUTO_OK;
}

}  // namespace

extern "C" {

size_t pluto_gqa_prefill_host_workspace_bytes(int batch, int seq, int q_heads, int kv_heads,
                                              int head_dim, int kv_heads_per_group) {
  if (batch <= 0 || seq <= 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 ||
      q_heads % kv_heads != 0 || kv_heads_per_group < 0)
    return 0;
  const size_t tokens = static_cast<size_t>(batch) * seq;
  if (kv_heads_per_group == 0) {   // token chunks: whole Q, out, K, V on the device
    if (!chunked_shape(head_dim, seq)) return 0;
    return 2 * round256(tokens * q_heads * head_dim * 2) + 2 * round256(tokens * kv_heads * head_dim * 2);
  }
  const size_t g = q_heads / kv_heads, hc = kv_heads_per_group;
  const size_t q_bytes = round256(tokens * hc * g * head_dim * 2);
  const size_t kv_bytes = round256(tokens * hc * head_dim * 2);
  return kSlots * (2 * q_bytes + 2 * kv_bytes);   // q, out, k, v per slot
}

int pluto_gqa_prefill_fwd_host(pluto_stream_t stream, const void* q_host, const void* k_host,
                               const void* v_host, void* out_host, void* workspace,
                               size_t workspace_bytes, int batch, int seq, int q_heads, int kv_heads,
                               int head_dim, int kv_heads_per_group) {
  const size_t need = pluto_gqa_prefill_host_workspace_bytes(batch, seq, q_heads, kv_heads, head_dim,
                                                             kv_heads_per_group);
  if (need == 0) return pluto::report(PLUTO_E_INVALID, "invalid full-attention dimensions or parameters");
  if (!q_host || !k_host || !v_host || !out_host)
    return pluto::report(PLUTO_E_INVALID, "attention requires non-null host pointers");
  if (!workspace || workspace_bytes < need || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
    return pluto::report(PLUTO_E_INVALID, "host prefill workspace is missing, misaligned or too small");
  if (!pluto::stream_on_current_device(static_cast<cudaStream_t>(stream)))
    return pluto::report(PLUTO_E_INVALID, "the stream belongs to another device than the current one; "
                                          "the copy streams are per device");
  Lanes* l = lanes_for_current_device();
  if (l == nullptr) return pluto::report(PLUTO_E_INTERNAL, "copy streams could not be created");
  if (kv_heads_per_group == 0) {
    cudaStream_t compute = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaEventRecord(l->start, compute);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(l->h2d, l->start, 0);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(l->d2h, l->start, 0);
    if (e != cudaSuccess) return pluto::report_cuda(e, "host prefill stream ordering");
    return prefill_by_token_chunks(l, compute, q_host, k_host, v_host, out_host, workspace, batch, seq,
                                   q_heads, kv_heads, head_dim);
  }
  const size_t tokens = static_cast<size_t>(batch) * seq;
  const size_t g = q_heads / kv_heads, D = head_dim;
  const size_t hc_max = kv_heads_per_group;
  const size_t q_bytes = round256(tokens * hc_max * g * D * 2);
  const size_t kv_bytes = round256(tokens * hc_max * D * 2);
  const size_t slot_bytes = 2 * q_bytes + 2 * kv_bytes;
  const size_t q_pitch = static_cast<size_t>(q_heads) * D * 2, kv_pitch = static_cast<size_t>(kv_heads) * D * 2;
  cudaStream_t compute = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaEventRecord(l->start, compute);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(l->h2d, l->start, 0);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(l->d2h, l->start, 0);
  if (e != cudaSuccess) return pluto::report_cuda(e, "host prefill stream ordering");
  const int groups = (kv_heads + kv_heads_per_group - 1) / kv_heads_per_group;
  for (int c = 0; c < groups; ++c) {
    const int slot = c % kSlots;
    const size_t h0 = static_cast<size_t>(c) * hc_max;
    const size_t hc = (h0 + hc_max <= static_cast<size_t>(kv_heads)) ? hc_max : kv_heads - h0;
    uint8_t* base = static_cast<uint8_t*>(workspace) + slot * slot_bytes;
    uint8_t *q_dev = base, *out_dev = base + q_bytes, *k_dev = base + 2 * q_bytes,
            *v_dev = base + 2 * q_bytes + kv_bytes;
    const size_t q_width = hc * g * D * 2, kv_width = hc * D * 2;
    // inputs of this group; the slot's buffers are free once the kernel of group c-2 is done
    if (c >= kSlots) e = cudaStreamWaitEvent(l->h2d, l->computed[slot], 0);
    if (e == cudaSuccess)
      e = cudaMemcpy2DAsync(q_dev, q_width, static_cast<const uint8_t*>(q_host) + h0 * g * D * 2, q_pitch,
                            q_width, tokens, cudaMemcpyHostToDevice, l->h2d);
    if (e == cudaSuccess)
      e = cudaMemcpy2DAsync(k_dev, kv_width, static_cast<const uint8_t*>(k_host) + h0 * D * 2, kv_pitch,
                            kv_width, tokens, cudaMemcpyHostToDevice, l->h2d);
    if (e == cudaSuccess)
      e = cudaMemcpy2DAsync(v_dev, kv_width, static_cast<const uint8_t*>(v_host) + h0 * D * 2, kv_pitch,
                            kv_width, tokens, cudaMemcpyHostToDevice, l->h2d);
    if (e == cudaSuccess) e = cudaEventRecord(l->loaded[slot], l->h2d);
    // kernel: after its inputs landed and after the output buffer's previous content left
    if (e == cudaSuccess) e = cudaStreamWaitEvent(compute, l->loaded[slot], 0);
    if (e == cudaSuccess && c >= kSlots) e = cudaStreamWaitEvent(compute, l->stored[slot], 0);
    if (e != cudaSuccess) return pluto::report_cuda(e, "host prefill input copy");
    const int rc = pluto_gqa_prefill_fwd(stream, q_dev, nullptr, k_dev, v_dev, out_dev, nullptr, nullptr,
                                         nullptr, batch, seq, static_cast<int>(hc * g),
                                         static_cast<int>(hc), head_dim, hc * g * D, D, 0, 0, 1, nullptr, 0);
    if (rc != PLUTO_OK) return rc;
    e = cudaEventRecord(l->computed[slot], compute);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(l->d2h, l->computed[slot], 0);
    if (e == cudaSuccess)
      e = cudaMemcpy2DAsync(static_cast<uint8_t*>(out_host) + h0 * g * D * 2, q_pitch, out_dev, q_width,
                            q_width, tokens, cudaMemcpyDeviceToHost, l->d2h);
    if (e == cudaSuccess) e = cudaEventRecord(l->stored[slot], l->d2h);
    if (e != cudaSuccess) return pluto::report_cuda(e, "host prefill output copy");
  }
  // later work on the caller's stream sees the whole output
  for (int s = 0; s < kSlots && s < groups; ++s) {
    e = cudaStreamWaitEvent(compute, l->stored[s], 0);
    if (e != cudaSuccess) return pluto::report_cuda(e, "host prefill stream ordering");
  }
  // (the last copy on each slot's event covers earlier ones: events are re-recorded per group)
  return PLUTO_OK;
}

}  // extern "C"
