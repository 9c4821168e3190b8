/*
 * TEST INFRASTRUCTURE -- not part of the shipped engine.
 *
 * CPU restatement, in plain C, of the reference project's arithmetic for every layer on the
 * attention hot path.  Only the test-suite, the smoke check and the benchmark's CPU-baseline leg
 * may load this library; the CUDA engine never links or calls it.
 *
 * Pinning status (how each function is anchored to the reference):
 *   oracle_attention_fwd / _bwd   restate AttentionLayerReference (src/llm/layers/
 *       attention_reference.cc:36-114 and :116-230) with the same scalar operation order; the
 *       tests require BIT equality with the reference's own compiled code (oracle/_ref) on the
 *       reference test-suite's shapes and inputs (attention_reference_test.cc:35-44,148-197) and
 *       reproduce its hand-computable answer (attention_test.cc:282-360).
 *   oracle_qk_prepare, oracle_gqa_decode, oracle_gqa_probabilities   restate PrepareAttentionKernel,
 *       FullAttentionKernel, AttentionProbabilitiesKernel (src/llm/layers/util/
 *       cached_attention_ops.cc:30-79, :83-126, :131-178).  The GPU kernels themselves cannot be
 *       compiled without cuTile, but the scalar specification the reference tests them against can:
 *       class AttentionReference (cached_attention_ops_test.cc:43-131) is compiled from the
 *       reference tree into oracle/_ref/libpluto_ref_specs.so, its outputs on that test's own 35
 *       steps, shapes and inputs are committed (tests/golden/reference_specs.npz), and these
 *       functions must match them at the test's tolerance (3e-5 + 1e-4|x| unrounded, 2e-4 + 0.8 %
 *       rounded); plus the tests' known answers (:364-398 exact gate products, :472-503 uniform
 *       1/length rows, cached_attention_test.cc:108-156).
 *   oracle_gqa_prefill   restates the attention core of ForwardKernel
 *       (src/llm/layers/qwen_attention.cc:68-119); pinned by equality with oracle_gqa_decode run
 *       token by token (the reference's own cross-path check, qwen_attention_test.cc:155-228), and
 *       the sequence layer as a whole by the compiled Reference of qwen_attention_test.cc:26-95 on
 *       that test's shapes.
 *   oracle_gdn_*   restate ConvolutionKernel/ConvForward, DeltaRecurrenceKernel/RecurrenceForward,
 *       DeltaOutputKernel/OutputForward (cached_attention_ops.cc:180-272,
 *       sequence_delta_net.cc:31-121); pinned by the compiled class DeltaReference
 *       (cached_attention_ops_test.cc:133-220; six steps incl. the a=+-100 softplus extremes) and
 *       the compiled Reference of sequence_delta_net_test.cc:66-159 on the three shapes of
 *       :241-297, at those tests' tolerances, through the same committed records.
 *   oracle_gqa_sequence_bwd, oracle_gdn_sequence_bwd   restate the backward kernels
 *       (qwen_attention.cc:124-239, sequence_delta_net.cc:126-339); pinned by the central
 *       differences the reference's gradient tests take of those compiled specifications
 *       (qwen_attention_test.cc:230-301, 3e-5; sequence_delta_net_test.cc:299-373, 2e-5 + 0.2 %),
 *       recorded in the same file.
 *   Where oracle/_ref/libpluto_ref_specs.so is present the comparisons also run live on random
 *   inputs (tests/test_oracle_specs.py).
 *
 * All tensors are caller-owned; nothing here allocates except scratch rows on the stack/heap.
 */
#include <math.h>
#include <pthread.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ---- bf16 helpers: round-to-nearest-even, as reference_internal.h:109-119 ---------------- */
static inline uint16_t f2bf(float v) {
  uint32_t b;
  memcpy(&b, &v, 4);
  if ((b & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((b >> 16) | 0x40u); /* quiet NaN */
  b += 0x7fffu + ((b >> 16) & 1u);
  return (uint16_t)(b >> 16);
}
static inline float bf2f(uint16_t h) {
  uint32_t b = (uint32_t)h << 16;
  float v;
  memcpy(&v, &b, 4);
  return v;
}
static inline float rnd(float v, int round) { return round ? bf2f(f2bf(v)) : v; }
static inline float load_act(const void* p, size_t i, int bf16) {
  return bf16 ? bf2f(((const uint16_t*)p)[i]) : ((const float*)p)[i];
}
static inline void store_act(void* p, size_t i, int bf16, float v) {
  if (bf16) ((uint16_t*)p)[i] = f2bf(v);
  else ((float*)p)[i] = v;
}
uint16_t oracle_float_to_bf16(float v) { return f2bf(v); }
float oracle_bf16_to_float(uint16_t h) { return bf2f(h); }

/* ---- tiny pthread parallel-for over independent units ------------------------------------ */
typedef void (*unit_fn)(int unit, void* ctx);
typedef struct { unit_fn fn; void* ctx; int begin, end; } span_t;
static void* run_span(void* arg) {
  span_t* s = (span_t*)arg;
  for (int u = s->begin; u < s->end; ++u) s->fn(u, s->ctx);
  return NULL;
}
static void parallel_units(int units, int threads, unit_fn fn, void* ctx) {
  if (threads > units) threads = units;
  if (threads <= 1) { for (int u = 0; u < units; ++u) fn(u, ctx); return; }
  pthread_t* ids = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)threads);
  span_t* spans = (span_t*)malloc(sizeof(span_t) * (size_t)threads);
  for (int t = 0; t < threads; ++t) {
    spans[t].fn = fn; spans[t].ctx = ctx;
    spans[t].begin = (int)((long long)units * t / threads);
    spans[t].end = (int)((long long)units * (t + 1) / threads);
    pthread_create(&ids[t], NULL, run_span, &spans[t]);
  }
  for (int t = 0; t < threads; ++t) pthread_join(ids[t], NULL);
  free(ids); free(spans);
}

/* ========================================================================================== *
 * Causal multi-head attention over packed [rows, 3E]   (AttentionLayerReference)
 * ========================================================================================== */
typedef struct {
  const void* qkv; const void* out_in; const float* d_out; void* out; float* maxima;
  float* normalizers; float* d_qkv; float* probs; int rows, context, heads, embed, bf16;
} mha_t;

/* attention_reference.cc:61-110, one sequence per unit.  Also emits the statistics the GPU layer
 * saves (row maximum of the scaled scores and the sum of exp(score - max), attention.cc:128-131,
 * 160-169) in its [(b*H+h)*S + s] layout, and optionally the full causal probabilities
 * [B,H,S,S] with zeros above the diagonal (attention.cc:176-230). */
static void mha_fwd_sequence(int sequence, void* ctx) {
  const mha_t* a = (const mha_t*)ctx;
  const int S = a->context, H = a->heads, E = a->embed, D = E / H;
  const float scale = 1.0f / sqrtf((float)D);
  float* scores = (float*)malloc(sizeof(float) * (size_t)S);
  for (int pos = 0; pos < S; ++pos) {
    const size_t row = (size_t)sequence * S + pos;
    for (int h = 0; h < H; ++h) {
      const int c0 = h * D;
      float maximum = -INFINITY;
      for (int kp = 0; kp <= pos; ++kp) {
        const size_t krow = (size_t)sequence * S + kp;
        float score = 0.0f;
        for (int d = 0; d < D; ++d)
          score += load_act(a->qkv, row * 3 * E + c0 + d, a->bf16) *
                   load_act(a->qkv, krow * 3 * E + E + c0 + d, a->bf16);
        scores[kp] = score * scale;
        maximum = fmaxf(maximum, scores[kp]);
      }
      float denominator = 0.0f;
      for (int kp = 0; kp <= pos; ++kp) {
        scores[kp] = expf(scores[kp] - maximum);
        denominator += scores[kp];
      }
      if (a->maxima) a->maxima[((size_t)sequence * H + h) * S + pos] = maximum;
      if (a->normalizers) a->normalizers[((size_t)sequence * H + h) * S + pos] = denominator;
      if (a->probs) {
        float* p = a->probs + (((size_t)sequence * H + h) * S + pos) * S;
        for (int kp = 0; kp < S; ++kp) p[kp] = kp <= pos ? scores[kp] / denominator : 0.0f;
      }
      if (a->out) {
        for (int d = 0; d < D; ++d) {
          float value = 0.0f;
          for (int kp = 0; kp <= pos; ++kp) {
            const size_t krow = (size_t)sequence * S + kp;
            value += (scores[kp] / denominator) *
                     load_act(a->qkv, krow * 3 * E + 2 * E + c0 + d, a->bf16);
          }
          store_act(a->out, row * E + c0 + d, a->bf16, value);
        }
      }
    }
  }
  free(scores);
}

int oracle_attention_fwd(const void* qkv, int rows, int context, int heads, int embed, int is_bf16,
                         int threads, void* out, float* maxima, float* normalizers, float* probs) {
  if (context <= 0 || heads <= 0 || embed <= 0 || embed % heads || rows <= 0 || rows % context)
    return 3;
  mha_t a = {qkv, NULL, NULL, out, maxima, normalizers, NULL, probs, rows, context, heads, embed,
             is_bf16};
  parallel_units(rows / context, threads, mha_fwd_sequence, &a);
  return 0;
}

/* attention_reference.cc:151-228, one sequence per unit; d_qkv must be zero-filled by the caller
 * (the reference clears it, :138-140) because keys/values accumulate across later queries. */
static void mha_bwd_sequence(int sequence, void* ctx) {
  const mha_t* a = (const mha_t*)ctx;
  const int S = a->context, H = a->heads, E = a->embed, D = E / H;
  const float scale = 1.0f / sqrtf((float)D);
  float* p = (float*)malloc(sizeof(float) * (size_t)S);
  for (int pos = 0; pos < S; ++pos) {
    const size_t row = (size_t)sequence * S + pos;
    for (int h = 0; h < H; ++h) {
      const int c0 = h * D;
      float maximum = -INFINITY;
      for (int kp = 0; kp <= pos; ++kp) {
        const size_t krow = (size_t)sequence * S + kp;
        float score = 0.0f;
        for (int d = 0; d < D; ++d)
          score += load_act(a->qkv, row * 3 * E + c0 + d, a->bf16) *
                   load_act(a->qkv, krow * 3 * E + E + c0 + d, a->bf16);
        p[kp] = score * scale;
        maximum = fmaxf(maximum, p[kp]);
      }
      float denominator = 0.0f;
      for (int kp = 0; kp <= pos; ++kp) { p[kp] = expf(p[kp] - maximum); denominator += p[kp]; }
      for (int kp = 0; kp <= pos; ++kp) p[kp] /= denominator;
      float delta = 0.0f;
      for (int d = 0; d < D; ++d)
        delta += a->d_out[row * E + c0 + d] * load_act(a->out_in, row * E + c0 + d, a->bf16);
      for (int kp = 0; kp <= pos; ++kp) {
        const size_t krow = (size_t)sequence * S + kp;
        float dp = 0.0f;
        for (int d = 0; d < D; ++d)
          dp += a->d_out[row * E + c0 + d] *
                load_act(a->qkv, krow * 3 * E + 2 * E + c0 + d, a->bf16);
        const float ds = p[kp] * (dp - delta);
        for (int d = 0; d < D; ++d) {
          const size_t q = row * 3 * E + c0 + d;
          const size_t k = krow * 3 * E + E + c0 + d;
          const size_t v = krow * 3 * E + 2 * E + c0 + d;
          a->d_qkv[q] += ds * load_act(a->qkv, k, a->bf16) * scale;
          a->d_qkv[k] += ds * load_act(a->qkv, q, a->bf16) * scale;
          a->d_qkv[v] += p[kp] * a->d_out[row * E + c0 + d];
        }
      }
    }
  }
  free(p);
}

int oracle_attention_bwd(const void* qkv, const void* out, const float* d_out, int rows,
                         int context, int heads, int embed, int is_bf16, int threads,
                         float* d_qkv) {
  if (context <= 0 || heads <= 0 || embed <= 0 || embed % heads || rows <= 0 || rows % context)
    return 3;
  memset(d_qkv, 0, sizeof(float) * (size_t)rows * 3 * embed);
  mha_t a = {qkv, out, d_out, NULL, NULL, NULL, d_qkv, NULL, rows, context, heads, embed, is_bf16};
  parallel_units(rows / context, threads, mha_bwd_sequence, &a);
  return 0;
}

/* ========================================================================================== *
 * Qwen GQA attention: prepare (RMSNorm + partial RoPE), decode over a cache, sequence core
 * ========================================================================================== */

/* PrepareAttentionKernel, cached_attention_ops.cc:30-79 (sequence form: qwen_attention.cc:30-63).
 * One head vector: x[dim] -> out[dim].  weight is zero-centred (multiplier 1+w). */
void oracle_qk_prepare_head(const float* x, const float* weight, int dim, int rotary, int position,
                            float epsilon, float theta, int round, float* out) {
  float square = 0.0f;
  for (int c = 0; c < dim; ++c) square += x[c] * x[c];
  const float inverse = 1.0f / sqrtf(square / (float)dim + epsilon);
  const float log_theta = logf(theta);
  const int half = rotary / 2;
  for (int c = 0; c < dim; ++c) {
    const float n = rnd(x[c] * inverse * (1.0f + weight[c]), round);
    if (c >= rotary) { out[c] = n; continue; }
    const int partner = c < half ? c + half : c - half;
    float rotated = rnd(x[partner] * inverse * (1.0f + weight[partner]), round);
    if (c < half) rotated = -rotated;
    const int f = c < half ? c : c - half;
    const float angle = (float)position * expf((float)f * (-2.0f * log_theta / (float)rotary));
    const float cosine = rnd(cosf(angle), round), sine = rnd(sinf(angle), round);
    out[c] = rnd(rnd(n * cosine, round) + rnd(rotated * sine, round), round);
  }
}

/* Whole-token prepare: q_gate [Hq,2,D] (query at h*2D), k,v [Hkv,D] -> queries [Hq,D] and the
 * cache row at `position` of keys/values [capacity,Hkv,D] (fp32 cache as key_value_cache.h:25-57). */
void oracle_qk_prepare(const float* q_gate, const float* k, const float* v, const float* q_norm,
                       const float* k_norm, int q_heads, int kv_heads, int dim, int rotary,
                       int position, float epsilon, float theta, int round, float* queries,
                       float* keys, float* values) {
  for (int h = 0; h < q_heads; ++h)
    oracle_qk_prepare_head(q_gate + (size_t)h * 2 * dim, q_norm, dim, rotary, position, epsilon,
                           theta, round, queries + (size_t)h * dim);
  for (int h = 0; h < kv_heads; ++h) {
    const size_t off = ((size_t)position * kv_heads + h) * dim;
    oracle_qk_prepare_head(k + (size_t)h * dim, k_norm, dim, rotary, position, epsilon, theta,
                           round, keys + off);
    for (int c = 0; c < dim; ++c) values[off + c] = rnd(v[(size_t)h * dim + c], round);
  }
}

/* FullAttentionKernel, cached_attention_ops.cc:83-126: one query head, online softmax over the
 * cached rows 32 at a time in fp32, then the optional sigmoid gate with the reference's rounding
 * sequence R(R(acc/l) * R(sigmoid(gate))).  K/V rows are `kv_is_bf16 ? bf16 : fp32`, laid out
 * [length, kv_heads, dim] with `kv_row_stride` elements between rows.  gate may be NULL
 * (then out = R(acc/l) when round, acc/l otherwise).  stats (optional) receives {max, sum}. */
static void decode_head(const float* query, const float* gate, const void* keys, const void* values,
                        int kv_is_bf16, size_t kv_row_stride, int kv_head, int dim, int length,
                        float scale, int round, float* out, float* stats) {
  float maximum = -3.402823466e+38f, denominator = 0.0f;
  float result[256];
  float score[32], prob[32];
  for (int c = 0; c < dim; ++c) result[c] = 0.0f;
  for (int start = 0; start < length; start += 32) {
    const int n = length - start < 32 ? length - start : 32;
    float tile_max = -3.402823466e+38f;
    for (int r = 0; r < n; ++r) {
      const size_t off = (size_t)(start + r) * kv_row_stride + (size_t)kv_head * dim;
      float s = 0.0f;
      for (int c = 0; c < dim; ++c) s += load_act(keys, off + c, kv_is_bf16) * query[c];
      score[r] = s * scale;
      tile_max = fmaxf(tile_max, score[r]);
    }
    const float next = fmaxf(maximum, tile_max);
    const float correction = expf(maximum - next);
    float psum = 0.0f;
    for (int r = 0; r < n; ++r) { prob[r] = expf(score[r] - next); psum += prob[r]; }
    for (int c = 0; c < dim; ++c) {
      float acc = 0.0f;
      for (int r = 0; r < n; ++r)
        acc += prob[r] * load_act(values, (size_t)(start + r) * kv_row_stride +
                                              (size_t)kv_head * dim + c, kv_is_bf16);
      result[c] = result[c] * correction + acc;
    }
    denominator = denominator * correction + psum;
    maximum = next;
  }
  if (stats) { stats[0] = maximum; stats[1] = denominator; }
  for (int c = 0; c < dim; ++c) {
    const float core = result[c] / denominator;
    if (gate) {
      const float sigmoid = rnd(1.0f / (1.0f + expf(-gate[c])), round);
      out[c] = rnd(rnd(core, round) * sigmoid, round);
    } else {
      out[c] = rnd(core, round);
    }
  }
}

/* One token of one sequence: queries [Hq,D] fp32 (already prepared), gate pointer q_gate
 * [Hq,2,D] or NULL, output [Hq,D] fp32. */
void oracle_gqa_decode(const float* queries, const float* q_gate, const void* keys,
                       const void* values, int kv_is_bf16, int q_heads, int kv_heads, int dim,
                       int length, int round, float* output) {
  const float scale = 1.0f / sqrtf((float)dim);
  for (int h = 0; h < q_heads; ++h)
    decode_head(queries + (size_t)h * dim, q_gate ? q_gate + ((size_t)h * 2 + 1) * dim : NULL,
                keys, values, kv_is_bf16, (size_t)kv_heads * dim, h / (q_heads / kv_heads), dim,
                length, scale, round, output + (size_t)h * dim, NULL);
}

/* Batched form used for the decode benchmark shape: sequence b has its own cache base pointers
 * and length; q [B,Hq,D] and out [B,Hq,D] are bf16 bit patterns (q_is_bf16) or fp32. */
typedef struct {
  const void* q; const void* const* keys; const void* const* values; const int* lengths;
  void* out; int q_bf16, kv_bf16, q_heads, kv_heads, dim, round;
} decode_batch_t;
static void decode_batch_unit(int unit, void* ctx) {
  const decode_batch_t* a = (const decode_batch_t*)ctx;
  const int b = unit / a->q_heads, h = unit % a->q_heads;
  float query[256], out[256];
  for (int c = 0; c < a->dim; ++c)
    query[c] = load_act(a->q, ((size_t)b * a->q_heads + h) * a->dim + c, a->q_bf16);
  decode_head(query, NULL, a->keys[b], a->values[b], a->kv_bf16, (size_t)a->kv_heads * a->dim,
              h / (a->q_heads / a->kv_heads), a->dim, a->lengths[b],
              1.0f / sqrtf((float)a->dim), a->round, out, NULL);
  for (int c = 0; c < a->dim; ++c)
    store_act(a->out, ((size_t)b * a->q_heads + h) * a->dim + c, a->q_bf16, out[c]);
}
void oracle_gqa_decode_batch(const void* q, const void* const* keys, const void* const* values,
                             const int* lengths, int batch, int q_is_bf16, int kv_is_bf16,
                             int q_heads, int kv_heads, int dim, int round, int threads,
                             void* out) {
  decode_batch_t a = {q, keys, values, lengths, out, q_is_bf16, kv_is_bf16, q_heads, kv_heads,
                      dim, round};
  parallel_units(batch * q_heads, threads, decode_batch_unit, &a);
}

/* AttentionProbabilitiesKernel, cached_attention_ops.cc:131-178: softmax row [Hq, length]. */
void oracle_gqa_probabilities(const float* queries, const void* keys, int kv_is_bf16, int q_heads,
                              int kv_heads, int dim, int length, float* probabilities) {
  const float scale = 1.0f / sqrtf((float)dim);
  for (int h = 0; h < q_heads; ++h) {
    const int kv = h / (q_heads / kv_heads);
    float* p = probabilities + (size_t)h * length;
    float maximum = -3.402823466e+38f;
    for (int t = 0; t < length; ++t) {
      float s = 0.0f;
      for (int c = 0; c < dim; ++c)
        s += load_act(keys, ((size_t)t * kv_heads + kv) * dim + c, kv_is_bf16) *
             queries[(size_t)h * dim + c];
      p[t] = s * scale;
      maximum = fmaxf(maximum, p[t]);
    }
    float denominator = 0.0f;
    for (int t = 0; t < length; ++t) denominator += expf(p[t] - maximum);
    for (int t = 0; t < length; ++t) p[t] = expf(p[t] - maximum) / denominator;
  }
}

/* Attention core of ForwardKernel, qwen_attention.cc:68-119, for a whole sequence:
 * q [T,Hq,D] with q_token_stride elements between tokens and q_head_stride between heads (so the
 * stride-2D view into [T,Hq,2,D] works), k,v [T,Hkv,D]; causal; 32-key online tiles.  Storage is
 * bf16 bit patterns when is_bf16.  gate (same indexing as q, or NULL).  out [T,Hq,D] (same
 * storage type); core (optional fp32 [T,Hq,D]) receives the unrounded acc/l; lse (optional
 * [Hq,T]) receives max + log(sum). */
typedef struct {
  const void* q; const void* gate; const void* k; const void* v; void* out; float* core;
  float* lse; int bf16, T, q_heads, kv_heads, dim, round; size_t q_token_stride, q_head_stride;
  int unit_base;
} prefill_t;
static void prefill_unit(int unit, void* ctx) {
  const prefill_t* a = (const prefill_t*)ctx;
  const int row = (unit + a->unit_base) / a->q_heads, h = (unit + a->unit_base) % a->q_heads;
  const int D = a->dim;
  float query[256], gate[256], out[256], stats[2];
  const size_t qoff = (size_t)row * a->q_token_stride + (size_t)h * a->q_head_stride;
  for (int c = 0; c < D; ++c) query[c] = load_act(a->q, qoff + c, a->bf16);
  if (a->gate)
    for (int c = 0; c < D; ++c) gate[c] = load_act(a->gate, qoff + c, a->bf16);
  /* unrounded core first (round = 0, no gate), then the output rounding sequence */
  decode_head(query, NULL, a->k, a->v, a->bf16, (size_t)a->kv_heads * D,
              h / (a->q_heads / a->kv_heads), D, row + 1, 1.0f / sqrtf((float)D), 0, out, stats);
  const size_t ooff = ((size_t)row * a->q_heads + h) * D;
  if (a->core) for (int c = 0; c < D; ++c) a->core[ooff + c] = out[c];
  if (a->lse) a->lse[(size_t)h * a->T + row] = stats[0] + logf(stats[1]);
  for (int c = 0; c < D; ++c) {
    float y;
    if (a->gate) {
      const float sigmoid = rnd(1.0f / (1.0f + expf(-gate[c])), a->round);
      y = rnd(rnd(out[c], a->round) * sigmoid, a->round);
    } else {
      y = rnd(out[c], a->round);
    }
    store_act(a->out, ooff + c, a->bf16, y);
  }
}
void oracle_gqa_prefill(const void* q, const void* gate, const void* k, const void* v, int is_bf16,
                        int T, int q_heads, int kv_heads, int dim, size_t q_token_stride,
                        size_t q_head_stride, int round, int threads, int row_begin, int row_end,
                        void* out, float* core, float* lse) {
  /* units are (row, head); a row range lets a caller check a sample of a long sequence */
  if (row_begin < 0) row_begin = 0;
  if (row_end > T) row_end = T;
  if (row_end <= row_begin) return;
  prefill_t a = {q, gate, k, v, out, core, lse, is_bf16, T, q_heads, kv_heads, dim, round,
                 q_token_stride, q_head_stride, row_begin * q_heads};
  parallel_units((row_end - row_begin) * q_heads, threads, prefill_unit, &a);
}

/* SequenceBackward of QwenAttentionLayer, qwen_attention.cc:124-239 (kernels) and :450-499 (host
 * order), for one sequence.  All tensors fp32 (values of bf16 inputs are bf16-exact):
 *   qg [T,Hq,2,D] (query at h*2D, gate at (2h+1)*D), k_in,v [T,Hkv,D], q_norm,k_norm [D]
 *   (zero-centred), dy [T,Hq,D].
 * Runs the forward first (PrepareKernel :30-63, ForwardKernel :68-119: prepared q/k, unrounded
 * core, probabilities P = exp(s - max)/denominator) and then, in the reference's order:
 *   GateBackwardKernel      dc = dy * R(sigmoid(gate)); d_gate = dy * R(core) * sig * (1 - sig)
 *   QueryBackwardKernel     delta = dc.core; dS = P * (dc.v - delta); dq_rope = scale * sum dS k
 *   KeyValueBackwardKernel  dk_rope = scale * sum_{h in group, t >= row} dS q; dv = sum P dc
 *   NormBackwardKernel      RoPE^-1 with the rounded cos/sin, then RMSNorm backward; per-row
 *                           weight-gradient parts normalized_grad * x * inv
 *   ReduceNormKernel        dw += sum of parts in row order
 * Outputs: dqg [T,Hq,2,D], dk [T,Hkv,D], dv [T,Hkv,D]; dqw/dkw [D] are ACCUMULATED into (NULL =
 * frozen norm); out_y (optional) [T,Hq,D] receives the forward output.  Returns 0, or -1 when a
 * scratch allocation fails. */
static void norm_backward_row(const float* x, const float* w, const float* grad, int d, int rotary,
                              int row, float epsilon, float log_theta, int round, float* dx,
                              float* dw_part) {
  const int half = rotary / 2;
  float square = 0.0f;
  for (int c = 0; c < d; ++c) square += x[c] * x[c];
  const float inv = 1.0f / sqrtf(square / (float)d + epsilon);
  float ng[256], dot = 0.0f;
  for (int c = 0; c < d; ++c) {
    float g = grad[c];
    if (c < rotary) {
      const int partner = c < half ? c + half : c - half;
      const int f = c < half ? c : c - half;
      const float angle = (float)row * expf((float)f * (-2.0f * log_theta / (float)rotary));
      const float co = rnd(cosf(angle), round), si = rnd(sinf(angle), round);
      const float gp = grad[partner];
      g = g * co + (c < half ? gp * si : -gp * si);
    }
    ng[c] = g;
    dot += g * (1.0f + w[c]) * x[c];
  }
  for (int c = 0; c < d; ++c) {
    const float weighted = ng[c] * (1.0f + w[c]);
    dx[c] = inv * weighted - x[c] * (inv * inv * inv / (float)d) * dot;
    if (dw_part) dw_part[c] = ng[c] * x[c] * inv;
  }
}

int oracle_gqa_sequence_bwd(const float* qg, const float* k_in, const float* v, const float* q_norm,
                            const float* k_norm, const float* dy, int T, int q_heads, int kv_heads,
                            int d, int rotary, float epsilon, float theta, int round, float* dqg,
                            float* dk, float* dv, float* dqw, float* dkw, float* out_y) {
  const size_t qn = (size_t)T * q_heads * d, kn = (size_t)T * kv_heads * d;
  const size_t pn = (size_t)q_heads * T * T;
  float* q = (float*)malloc(qn * sizeof(float));
  float* k = (float*)malloc(kn * sizeof(float));
  float* core = (float*)malloc(qn * sizeof(float));
  float* dc = (float*)malloc(qn * sizeof(float));
  float* dq_rope = (float*)malloc(qn * sizeof(float));
  float* dk_rope = (float*)malloc(kn * sizeof(float));
  float* p = (float*)calloc(pn, sizeof(float));
  float* ds = (float*)calloc(pn, sizeof(float));
  float* parts = (float*)malloc((qn > kn ? qn : kn) * sizeof(float));
  if (!q || !k || !core || !dc || !dq_rope || !dk_rope || !p || !ds || !parts) {
    free(q); free(k); free(core); free(dc); free(dq_rope); free(dk_rope); free(p); free(ds);
    free(parts);
    return -1;
  }
  const int group = q_heads / kv_heads;
  const float scale = 1.0f / sqrtf((float)d), log_theta = logf(theta);
  /* forward: prepare */
  for (int row = 0; row < T; ++row) {
    for (int h = 0; h < q_heads; ++h)
      oracle_qk_prepare_head(qg + ((size_t)row * q_heads + h) * 2 * d, q_norm, d, rotary, row,
                             epsilon, theta, round, q + ((size_t)row * q_heads + h) * d);
    for (int h = 0; h < kv_heads; ++h)
      oracle_qk_prepare_head(k_in + ((size_t)row * kv_heads + h) * d, k_norm, d, rotary, row,
                             epsilon, theta, round, k + ((size_t)row * kv_heads + h) * d);
  }
  /* forward: online softmax in 32-key tiles, core, probabilities, gated output */
  for (int row = 0; row < T; ++row)
    for (int h = 0; h < q_heads; ++h) {
      const int kv = h / group;
      const float* query = q + ((size_t)row * q_heads + h) * d;
      float maximum = -3.402823466e38f, denominator = 0.0f, sum[256];
      for (int c = 0; c < d; ++c) sum[c] = 0.0f;
      for (int start = 0; start <= row; start += 32) {
        float score[32], next_max = maximum;
        const int count = row + 1 - start < 32 ? row + 1 - start : 32;
        for (int r = 0; r < count; ++r) {
          const float* key = k + ((size_t)(start + r) * kv_heads + kv) * d;
          float dot = 0.0f;
          for (int c = 0; c < d; ++c) dot += key[c] * query[c];
          score[r] = dot * scale;
          if (score[r] > next_max) next_max = score[r];
        }
        const float correction = expf(maximum - next_max);
        float tile_sum = 0.0f;
        for (int c = 0; c < d; ++c) sum[c] *= correction;
        for (int r = 0; r < count; ++r) {
          const float pr = expf(score[r] - next_max);
          const float* value = v + ((size_t)(start + r) * kv_heads + kv) * d;
          for (int c = 0; c < d; ++c) sum[c] += pr * value[c];
          tile_sum += pr;
        }
        denominator = denominator * correction + tile_sum;
        maximum = next_max;
      }
      float* crow = core + ((size_t)row * q_heads + h) * d;
      for (int c = 0; c < d; ++c) crow[c] = sum[c] / denominator;
      if (out_y)
        for (int c = 0; c < d; ++c) {
          const float gate = qg[(((size_t)row * q_heads + h) * 2 + 1) * d + c];
          const float sigmoid = rnd(1.0f / (1.0f + expf(-gate)), round);
          out_y[((size_t)row * q_heads + h) * d + c] = rnd(rnd(crow[c], round) * sigmoid, round);
        }
      for (int t = 0; t <= row; ++t) {
        const float* key = k + ((size_t)t * kv_heads + kv) * d;
        float dot = 0.0f;
        for (int c = 0; c < d; ++c) dot += key[c] * query[c];
        p[((size_t)h * T + row) * T + t] = expf(dot * scale - maximum) / denominator;
      }
    }
  /* GateBackwardKernel */
  for (size_t i = 0; i < (size_t)T * q_heads; ++i)
    for (int c = 0; c < d; ++c) {
      const float gate = qg[(i * 2 + 1) * d + c];
      const float sigmoid = 1.0f / (1.0f + expf(-gate));
      const float grad = dy[i * d + c];
      dc[i * d + c] = grad * rnd(sigmoid, round);
      dqg[(i * 2 + 1) * d + c] = grad * rnd(core[i * d + c], round) * sigmoid * (1.0f - sigmoid);
    }
  /* QueryBackwardKernel */
  for (int row = 0; row < T; ++row)
    for (int h = 0; h < q_heads; ++h) {
      const int kv = h / group;
      const float* grad = dc + ((size_t)row * q_heads + h) * d;
      const float* value = core + ((size_t)row * q_heads + h) * d;
      float delta = 0.0f, sum[256];
      for (int c = 0; c < d; ++c) { delta += grad[c] * value[c]; sum[c] = 0.0f; }
      for (int t = 0; t <= row; ++t) {
        const float* values = v + ((size_t)t * kv_heads + kv) * d;
        const float* keys = k + ((size_t)t * kv_heads + kv) * d;
        float dot = 0.0f;
        for (int c = 0; c < d; ++c) dot += grad[c] * values[c];
        const float score_grad = p[((size_t)h * T + row) * T + t] * (dot - delta);
        ds[((size_t)h * T + row) * T + t] = score_grad;
        for (int c = 0; c < d; ++c) sum[c] += score_grad * keys[c] * scale;
      }
      for (int c = 0; c < d; ++c) dq_rope[((size_t)row * q_heads + h) * d + c] = sum[c];
    }
  /* KeyValueBackwardKernel: fixed order over the group's heads, then over later rows */
  for (int row = 0; row < T; ++row)
    for (int kv = 0; kv < kv_heads; ++kv) {
      float kg[256], vg[256];
      for (int c = 0; c < d; ++c) kg[c] = vg[c] = 0.0f;
      for (int h = kv * group; h < (kv + 1) * group; ++h)
        for (int t = row; t < T; ++t) {
          const float prob = p[((size_t)h * T + t) * T + row];
          const float score_grad = ds[((size_t)h * T + t) * T + row];
          const float* query = q + ((size_t)t * q_heads + h) * d;
          const float* grad = dc + ((size_t)t * q_heads + h) * d;
          for (int c = 0; c < d; ++c) {
            kg[c] += score_grad * query[c] * scale;
            vg[c] += prob * grad[c];
          }
        }
      for (int c = 0; c < d; ++c) {
        dk_rope[((size_t)row * kv_heads + kv) * d + c] = kg[c];
        dv[((size_t)row * kv_heads + kv) * d + c] = vg[c];
      }
    }
  /* NormBackwardKernel + ReduceNormKernel, queries then keys */
  for (size_t i = 0; i < (size_t)T * q_heads; ++i)
    norm_backward_row(qg + i * 2 * d, q_norm, dq_rope + i * d, d, rotary, (int)(i / q_heads),
                      epsilon, log_theta, round, dqg + i * 2 * d, dqw ? parts + i * d : NULL);
  if (dqw)
    for (int c = 0; c < d; ++c) {
      float sum = 0.0f;
      for (size_t i = 0; i < (size_t)T * q_heads; ++i) sum += parts[i * d + c];
      dqw[c] += sum;
    }
  for (size_t i = 0; i < (size_t)T * kv_heads; ++i)
    norm_backward_row(k_in + i * d, k_norm, dk_rope + i * d, d, rotary, (int)(i / kv_heads),
                      epsilon, log_theta, round, dk + i * d, dkw ? parts + i * d : NULL);
  if (dkw)
    for (int c = 0; c < d; ++c) {
      float sum = 0.0f;
      for (size_t i = 0; i < (size_t)T * kv_heads; ++i) sum += parts[i * d + c];
      dkw[c] += sum;
    }
  free(q); free(k); free(core); free(dc); free(dq_rope); free(dk_rope); free(p); free(ds);
  free(parts);
  return 0;
}

/* ========================================================================================== *
 * Gated delta-net
 * ========================================================================================== */

/* decay gate of DeltaRecurrenceKernel, cached_attention_ops.cc:231-236:
 * g = exp(-exp(A_log) * softplus(a + dt_bias)), softplus in its overflow-safe form. */
float oracle_gdn_decay(float a, float dt_bias, float a_log) {
  const float alpha = a + dt_bias;
  const float softplus = fmaxf(alpha, 0.0f) + logf(1.0f + expf(-fabsf(alpha)));
  return expf(-expf(a_log) * softplus);
}
float oracle_gdn_beta(float b, int round) { return rnd(1.0f / (1.0f + expf(-b)), round); }

/* The recurrence of RecurrenceForward (sequence_delta_net.cc:55-102) / DeltaRecurrenceKernel
 * (cached_attention_ops.cc:205-251) for one (batch, value head) over T tokens:
 *     q^ = q * rsqrt(sum q^2 + 1e-6) / sqrt(dk),  k^ = k * rsqrt(sum k^2 + 1e-6)   [normalize_qk]
 *     S <- g_t S ;  delta = (v_t - S^T k^) * beta_t ;  S <- S + k^ (x) delta ;  o_t = R(S^T q^)
 * q,k: [B,T,Hk,dk]; v,out: [B,T,Hv,dv]; g,beta: fp32 [B,T,Hv]; state fp32 [B,Hv,dk,dv], updated
 * in place (zero it for a prefill from scratch).  q,k,v,out are bf16 bit patterns when is_bf16.
 * When normalize_qk == 0 the vectors are used as given and q is multiplied by q_scale. */
typedef struct {
  const void* q; const void* k; const void* v; const float* g; const float* beta; float* state;
  void* out; int bf16, B, T, Hk, Hv, dk, dv, normalize, round; float q_scale;
} gdn_t;
static void gdn_unit(int unit, void* ctx) {
  const gdn_t* a = (const gdn_t*)ctx;
  const int b = unit / a->Hv, h = unit % a->Hv, kh = h / (a->Hv / a->Hk);
  const int dk = a->dk, dv = a->dv;
  float* S = a->state + ((size_t)b * a->Hv + h) * dk * dv;
  float q[128], k[128];
  for (int t = 0; t < a->T; ++t) {
    const size_t qk = (((size_t)b * a->T + t) * a->Hk + kh) * dk;
    const size_t vo = (((size_t)b * a->T + t) * a->Hv + h) * dv;
    float qs = 0.0f, ks = 0.0f;
    for (int i = 0; i < dk; ++i) {
      q[i] = load_act(a->q, qk + i, a->bf16);
      k[i] = load_act(a->k, qk + i, a->bf16);
      qs += q[i] * q[i];
      ks += k[i] * k[i];
    }
    if (a->normalize) {
      const float qn = (1.0f / sqrtf(qs + 1e-6f)) / sqrtf((float)dk);
      const float kn = 1.0f / sqrtf(ks + 1e-6f);
      for (int i = 0; i < dk; ++i) { q[i] *= qn; k[i] *= kn; }
    } else {
      for (int i = 0; i < dk; ++i) q[i] *= a->q_scale;
    }
    const float decay = a->g[((size_t)b * a->T + t) * a->Hv + h];
    const float beta = a->beta[((size_t)b * a->T + t) * a->Hv + h];
    for (int j = 0; j < dv; ++j) {
      float prediction = 0.0f;
      for (int i = 0; i < dk; ++i) {
        S[(size_t)i * dv + j] *= decay;
        prediction += S[(size_t)i * dv + j] * k[i];
      }
      const float delta = (load_act(a->v, vo + j, a->bf16) - prediction) * beta;
      float core = 0.0f;
      for (int i = 0; i < dk; ++i) {
        S[(size_t)i * dv + j] += k[i] * delta;
        core += S[(size_t)i * dv + j] * q[i];
      }
      store_act(a->out, vo + j, a->bf16, rnd(core, a->round));
    }
  }
}
int oracle_gdn_recurrence(const void* q, const void* k, const void* v, const float* g,
                          const float* beta, int is_bf16, int B, int T, int Hk, int Hv, int dk,
                          int dv, int normalize_qk, float q_scale, int round, int threads,
                          float* state, void* out) {
  if (dk > 128 || dv > 256 || Hk <= 0 || Hv % Hk) return 3;
  gdn_t a = {q, k, v, g, beta, state, out, is_bf16, B, T, Hk, Hv, dk, dv, normalize_qk, round,
             q_scale};
  parallel_units(B * Hv, threads, gdn_unit, &a);
  return 0;
}

/* ConvolutionKernel (cached_attention_ops.cc:180-203): single-token causal depthwise conv over a
 * shift-register state [channels, width] followed by SiLU.  ConvForward
 * (sequence_delta_net.cc:31-51) is the same arithmetic with an explicit zero history. */
void oracle_gdn_conv_step(const float* input, const float* weight, int channels, int width,
                          int round, float* state, float* output) {
  for (int c = 0; c < channels; ++c) {
    float sum = 0.0f;
    for (int tap = 0; tap < width - 1; ++tap) {
      const float previous = state[(size_t)c * width + tap + 1];
      sum += previous * weight[(size_t)c * width + tap];
      state[(size_t)c * width + tap] = previous;
    }
    const float current = rnd(input[c], round);
    state[(size_t)c * width + width - 1] = current;
    sum = rnd(sum + current * weight[(size_t)c * width + width - 1], round);
    output[c] = rnd(sum / (1.0f + expf(-sum)), round);
  }
}

/* DeltaOutputKernel (cached_attention_ops.cc:253-272): per head RMSNorm * weight * SiLU(z) with
 * a rounding after each product.  final_round = 0 reproduces OutputForward
 * (sequence_delta_net.cc:104-121), which leaves the last product unrounded before its bf16 store. */
void oracle_gdn_output(const float* core, const float* z, const float* norm_weight, int heads,
                       int dim, float epsilon, int round, int final_round, float* output) {
  for (int h = 0; h < heads; ++h) {
    float square = 0.0f;
    for (int c = 0; c < dim; ++c) square += core[(size_t)h * dim + c] * core[(size_t)h * dim + c];
    const float inverse = 1.0f / sqrtf(square / (float)dim + epsilon);
    for (int c = 0; c < dim; ++c) {
      const float normalized = rnd(core[(size_t)h * dim + c] * inverse, round);
      const float affine = rnd(normalized * norm_weight[c], round);
      const float gate = z[(size_t)h * dim + c];
      const float silu = gate / (1.0f + expf(-gate));
      output[(size_t)h * dim + c] = rnd(affine * silu, round && final_round);
    }
  }
}

/* SequenceDeltaNetLayer forward + backward for one sequence, sequence_delta_net.cc:31-121
 * (ConvForward, RecurrenceForward, OutputForward) and :126-339 with the host order of :482-561
 * (OutputBackward, SumNormGradient, RecurrenceBackward, GatherQkGradient, GatherScalarGradient,
 * ConvSiluBackward, ConvInputBackward, ConvWeightBackward).  All arrays fp32 (bf16 inputs hold
 * bf16-exact values): qkv [T,channels] with channels = 2*kh*kd + vh*vd laid out all-Q, all-K,
 * all-V; z [T,vh*vd]; a, b [T,vh]; conv_w [channels,kernel] oldest tap first; a_log, dt_bias
 * [vh]; norm [vd]; dy [T,vh*vd].  Outputs dqkv, dz, da, db; the four parameter gradients are
 * ACCUMULATED into (NULL = frozen).  y_out (optional) receives the forward output (the final
 * product is left unrounded, as OutputForward's bf16 store is the only rounding there).
 * Stores every intermediate state like the reference, so it is for short sequences. */
int oracle_gdn_sequence_bwd(const float* qkv, const float* z, const float* a, const float* b,
                            const float* conv_w, const float* a_log, const float* dt_bias,
                            const float* norm, const float* dy, int T, int kh, int vh, int kd,
                            int vd, int kernel, float epsilon, int round, float* dqkv, float* dz,
                            float* da, float* db, float* d_conv, float* d_a_log, float* d_dt_bias,
                            float* d_norm, float* y_out) {
  const int channels = 2 * kh * kd + vh * vd, width = vh * vd, tiles = (vd + 31) / 32;
  const size_t stride = (size_t)vh * kd * vd;
  float* pre = (float*)malloc((size_t)T * channels * sizeof(float));
  float* post = (float*)malloc((size_t)T * channels * sizeof(float));
  float* core = (float*)malloc((size_t)T * width * sizeof(float));
  float* states = (float*)calloc((size_t)(T + 1) * stride, sizeof(float));
  float* dcore = (float*)malloc((size_t)T * width * sizeof(float));
  float* dpost = (float*)calloc((size_t)T * channels, sizeof(float));
  float* dpre = (float*)malloc((size_t)T * channels * sizeof(float));
  float* qk = (float*)calloc((size_t)T * vh * tiles * 2 * kd, sizeof(float));
  float* scalars = (float*)calloc((size_t)T * vh * tiles * 3, sizeof(float));
  float* parts = (float*)malloc((size_t)T * width * sizeof(float));
  if (!pre || !post || !core || !states || !dcore || !dpost || !dpre || !qk || !scalars || !parts) {
    free(pre); free(post); free(core); free(states); free(dcore); free(dpost); free(dpre);
    free(qk); free(scalars); free(parts);
    return -1;
  }
  const float norm_scale = sqrtf((float)kd);
  /* ConvForward */
  for (int t = 0; t < T; ++t)
    for (int c = 0; c < channels; ++c) {
      float sum = 0.0f;
      for (int tap = 0; tap < kernel; ++tap) {
        const int source = t + tap - kernel + 1;
        if (source >= 0) sum += qkv[(size_t)source * channels + c] * conv_w[(size_t)c * kernel + tap];
      }
      sum = rnd(sum, round);
      pre[(size_t)t * channels + c] = sum;
      post[(size_t)t * channels + c] = rnd(sum / (1.0f + expf(-sum)), round);
    }
  /* RecurrenceForward: per (head, 32-column tile), every S_t saved */
  for (int head = 0; head < vh; ++head)
    for (int tile = 0; tile < tiles; ++tile) {
      const int key_head = head / (vh / kh);
      const int c0 = tile * 32, c1 = c0 + 32 < vd ? c0 + 32 : vd;
      for (int t = 0; t < T; ++t) {
        const float* row = post + (size_t)t * channels;
        float q[128], k[128], sq = 0.0f, sk = 0.0f;
        for (int i = 0; i < kd; ++i) {
          q[i] = row[key_head * kd + i];
          k[i] = row[(kh + key_head) * kd + i];
          sq += q[i] * q[i];
          sk += k[i] * k[i];
        }
        const float iq = 1.0f / sqrtf(sq + 1e-6f), ik = 1.0f / sqrtf(sk + 1e-6f);
        for (int i = 0; i < kd; ++i) { q[i] = q[i] * iq / norm_scale; k[i] = k[i] * ik; }
        const float decay = oracle_gdn_decay(a[(size_t)t * vh + head], dt_bias[head], a_log[head]);
        const float beta = oracle_gdn_beta(b[(size_t)t * vh + head], round);
        const float* prev = states + (size_t)t * stride + (size_t)head * kd * vd;
        float* next = states + (size_t)(t + 1) * stride + (size_t)head * kd * vd;
        for (int c = c0; c < c1; ++c) {
          float prediction = 0.0f;
          for (int i = 0; i < kd; ++i) {
            next[(size_t)i * vd + c] = prev[(size_t)i * vd + c] * decay;
            prediction += next[(size_t)i * vd + c] * k[i];
          }
          const float delta = (row[2 * kh * kd + head * vd + c] - prediction) * beta;
          float out = 0.0f;
          for (int i = 0; i < kd; ++i) {
            next[(size_t)i * vd + c] += k[i] * delta;
            out += next[(size_t)i * vd + c] * q[i];
          }
          core[((size_t)t * vh + head) * vd + c] = rnd(out, round);
        }
      }
    }
  /* OutputForward (optional) and OutputBackward */
  for (int r = 0; r < T * vh; ++r) {
    const float* x = core + (size_t)r * vd;
    float square = 0.0f;
    for (int c = 0; c < vd; ++c) square += x[c] * x[c];
    const float inverse = 1.0f / sqrtf(square / (float)vd + epsilon);
    float dot = 0.0f;
    for (int c = 0; c < vd; ++c) {
      const float gate = z[(size_t)r * vd + c], sigmoid = 1.0f / (1.0f + expf(-gate));
      dot += dy[(size_t)r * vd + c] * gate * sigmoid * norm[c] * x[c];
    }
    for (int c = 0; c < vd; ++c) {
      const size_t i = (size_t)r * vd + c;
      const float normalized = rnd(x[c] * inverse, round);
      const float affine = rnd(normalized * norm[c], round);
      const float gate = z[i], sigmoid = 1.0f / (1.0f + expf(-gate));
      if (y_out) y_out[i] = affine * gate / (1.0f + expf(-gate));
      const float dn = dy[i] * gate * sigmoid * norm[c];
      dcore[i] = inverse * dn - x[c] * inverse * inverse * inverse / (float)vd * dot;
      dz[i] = dy[i] * affine * sigmoid * (1.0f + gate * (1.0f - sigmoid));
      parts[i] = dy[i] * gate * sigmoid * normalized;
    }
  }
  if (d_norm)   /* SumNormGradient */
    for (int c = 0; c < vd; ++c) {
      float sum = 0.0f;
      for (int r = 0; r < T * vh; ++r) sum += parts[(size_t)r * vd + c];
      d_norm[c] += sum;
    }
  /* RecurrenceBackward */
  float* dm = (float*)malloc((size_t)kd * 32 * sizeof(float));
  if (!dm) return -1;
  for (int head = 0; head < vh; ++head)
    for (int tile = 0; tile < tiles; ++tile) {
      const int key_head = head / (vh / kh);
      const int c0 = tile * 32, c1 = c0 + 32 < vd ? c0 + 32 : vd, nc = c1 - c0;
      for (int i = 0; i < kd * 32; ++i) dm[i] = 0.0f;
      for (int t = T - 1; t >= 0; --t) {
        const float* row = post + (size_t)t * channels;
        float raw_q[128], raw_k[128], q[128], k[128], sq = 0.0f, sk = 0.0f;
        for (int i = 0; i < kd; ++i) {
          raw_q[i] = row[key_head * kd + i];
          raw_k[i] = row[(kh + key_head) * kd + i];
          sq += raw_q[i] * raw_q[i];
          sk += raw_k[i] * raw_k[i];
        }
        const float iq = 1.0f / sqrtf(sq + 1e-6f), ik = 1.0f / sqrtf(sk + 1e-6f);
        for (int i = 0; i < kd; ++i) { q[i] = raw_q[i] * iq / norm_scale; k[i] = raw_k[i] * ik; }
        const float alpha = a[(size_t)t * vh + head] + dt_bias[head];
        const float softplus = fmaxf(alpha, 0.0f) + logf(1.0f + expf(-fabsf(alpha)));
        const float rate = expf(a_log[head]);
        const float decay = expf(-rate * softplus);
        const float sigmoid = 1.0f / (1.0f + expf(-b[(size_t)t * vh + head]));
        const float beta = rnd(sigmoid, round);
        const float* prev = states + (size_t)t * stride + (size_t)head * kd * vd;
        const float* matrix = states + (size_t)(t + 1) * stride + (size_t)head * kd * vd;
        float dq[128], dk[128], difference[32], delta[32], ddelta[32], dv[32];
        for (int j = 0; j < nc; ++j) {
          float prediction = 0.0f;
          for (int i = 0; i < kd; ++i) prediction += prev[(size_t)i * vd + c0 + j] * decay * k[i];
          difference[j] = row[2 * kh * kd + head * vd + c0 + j] - prediction;
          delta[j] = difference[j] * beta;
        }
        for (int i = 0; i < kd; ++i) {
          float s = 0.0f;
          for (int j = 0; j < nc; ++j)
            s += matrix[(size_t)i * vd + c0 + j] * dcore[((size_t)t * vh + head) * vd + c0 + j];
          dq[i] = s;
          for (int j = 0; j < nc; ++j)
            dm[i * 32 + j] += q[i] * dcore[((size_t)t * vh + head) * vd + c0 + j];
        }
        float dbeta_sum = 0.0f;
        for (int j = 0; j < nc; ++j) {
          float s = 0.0f;
          for (int i = 0; i < kd; ++i) s += dm[i * 32 + j] * k[i];
          ddelta[j] = s;
          dv[j] = s * beta;
          dbeta_sum += s * difference[j];
        }
        float dg = 0.0f;
        for (int i = 0; i < kd; ++i) {
          float s = 0.0f;
          for (int j = 0; j < nc; ++j) {
            const float decayed = prev[(size_t)i * vd + c0 + j] * decay;
            s += dm[i * 32 + j] * delta[j] - decayed * dv[j];
          }
          dk[i] = s;
        }
        /* ddecayed = dm - k dv; dg = sum(ddecayed * previous); dm <- ddecayed * decay */
        float dg_cols[32];
        for (int j = 0; j < nc; ++j) dg_cols[j] = 0.0f;
        for (int i = 0; i < kd; ++i)
          for (int j = 0; j < nc; ++j) {
            const float ddecayed = dm[i * 32 + j] - k[i] * dv[j];
            dg_cols[j] += ddecayed * prev[(size_t)i * vd + c0 + j];
            dm[i * 32 + j] = ddecayed * decay;
          }
        for (int j = 0; j < nc; ++j) dg += dg_cols[j];
        const size_t partial = ((size_t)t * vh + head) * tiles + tile;
        scalars[partial * 3 + 0] = -dg * decay * rate / (1.0f + expf(-alpha));
        scalars[partial * 3 + 1] = dbeta_sum * sigmoid * (1.0f - sigmoid);
        scalars[partial * 3 + 2] = -dg * decay * rate * softplus;
        float dot_q = 0.0f, dot_k = 0.0f;
        for (int i = 0; i < kd; ++i) { dot_q += dq[i] * raw_q[i]; dot_k += dk[i] * raw_k[i]; }
        for (int i = 0; i < kd; ++i) {
          qk[partial * 2 * kd + i] = (dq[i] * iq - raw_q[i] * iq * iq * iq * dot_q) / norm_scale;
          qk[partial * 2 * kd + kd + i] = dk[i] * ik - raw_k[i] * ik * ik * ik * dot_k;
        }
        for (int j = 0; j < nc; ++j)
          dpost[(size_t)t * channels + 2 * kh * kd + head * vd + c0 + j] = dv[j];
      }
    }
  free(dm);
  /* GatherQkGradient */
  for (int t = 0; t < T; ++t)
    for (int key_head = 0; key_head < kh; ++key_head) {
      const int group = vh / kh;
      for (int i = 0; i < kd; ++i) {
        float sq = 0.0f, sk = 0.0f;
        for (int h = key_head * group; h < (key_head + 1) * group; ++h)
          for (int tile = 0; tile < tiles; ++tile) {
            const size_t partial = (((size_t)t * vh + h) * tiles + tile) * 2 * kd;
            sq += qk[partial + i];
            sk += qk[partial + kd + i];
          }
        dpost[(size_t)t * channels + key_head * kd + i] = sq;
        dpost[(size_t)t * channels + (kh + key_head) * kd + i] = sk;
      }
    }
  /* GatherScalarGradient */
  for (int head = 0; head < vh; ++head) {
    float sum_log = 0.0f, sum_a = 0.0f;
    for (int t = 0; t < T; ++t) {
      float ga = 0.0f, gb = 0.0f, gl = 0.0f;
      for (int tile = 0; tile < tiles; ++tile) {
        const size_t index = (((size_t)t * vh + head) * tiles + tile) * 3;
        ga += scalars[index]; gb += scalars[index + 1]; gl += scalars[index + 2];
      }
      da[(size_t)t * vh + head] = ga;
      db[(size_t)t * vh + head] = gb;
      sum_log += gl;
      sum_a += ga;
    }
    if (d_a_log) d_a_log[head] += sum_log;
    if (d_dt_bias) d_dt_bias[head] += sum_a;
  }
  /* ConvSiluBackward, ConvInputBackward, ConvWeightBackward */
  for (size_t i = 0; i < (size_t)T * channels; ++i) {
    const float x = pre[i], sigmoid = 1.0f / (1.0f + expf(-x));
    dpre[i] = dpost[i] * sigmoid * (1.0f + x * (1.0f - sigmoid));
  }
  for (int t = 0; t < T; ++t)
    for (int c = 0; c < channels; ++c) {
      float sum = 0.0f;
      for (int tap = 0; tap < kernel; ++tap) {
        const int future = t + kernel - 1 - tap;
        if (future < T) sum += dpre[(size_t)future * channels + c] * conv_w[(size_t)c * kernel + tap];
      }
      dqkv[(size_t)t * channels + c] = sum;
    }
  if (d_conv)
    for (int c = 0; c < channels; ++c)
      for (int tap = 0; tap < kernel; ++tap) {
        float sum = 0.0f;
        for (int t = kernel - 1 - tap; t < T; ++t)
          sum += dpre[(size_t)t * channels + c] * qkv[(size_t)(t + tap - kernel + 1) * channels + c];
        d_conv[(size_t)c * kernel + tap] += sum;
      }
  free(pre); free(post); free(core); free(states); free(dcore); free(dpost); free(dpre);
  free(qk); free(scalars); free(parts);
  return 0;
}

/* ========================================================================================== *
 * Imported (frozen, output-major) projections: FullyConnectedLayer::ImportedForward,
 * src/llm/layers/fully_connected.cc:40-95, 295-341
 * ========================================================================================== */

/* FP8 E4M3 (4 exponent bits, bias 7, 3 mantissa bits, no infinities, 0x7f/0xff = NaN, largest
 * finite 448), the format of __nv_fp8_e4m3: round to nearest even, saturating to +-448. */
float oracle_e4m3_to_float(uint8_t b) {
  const int sign = b >> 7, e = (b >> 3) & 15, m = b & 7;
  float v;
  if (e == 15 && m == 7) return NAN;
  if (e == 0) v = ldexpf((float)m, -9);
  else v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
  return sign ? -v : v;
}
uint8_t oracle_float_to_e4m3(float x) {
  if (x != x) return 0x7f;
  const uint8_t sign = signbit(x) ? 0x80 : 0;
  const float a = fabsf(x);
  if (a >= 448.0f) return sign | 0x7e;
  if (a < ldexpf(1.0f, -6)) {                    /* subnormal range: multiples of 2^-9 */
    const int q = (int)nearbyintf(ldexpf(a, 9));  /* ties to even; q = 8 is the smallest normal */
    return sign | (uint8_t)q;
  }
  int e;
  const float mant = frexpf(a, &e) * 2.0f;       /* in [1, 2) */
  e -= 1;
  int q = (int)nearbyintf((mant - 1.0f) * 8.0f);
  if (q == 8) { q = 0; e += 1; }
  return sign | (uint8_t)(((e + 7) << 3) | q);
}

/* QuantizeImportedInputKernel (:73-95): per group of 128 inputs scale = max|x| / 448,
 * x <- e4m3(x / max(scale, 1e-12)) * scale. */
void oracle_quantize_imported_input(const float* input, int n, float* output) {
  for (int start = 0; start < n; start += 128) {
    const int end = start + 128 < n ? start + 128 : n;
    float maximum = 0.0f;
    for (int i = start; i < end; ++i) maximum = fmaxf(maximum, fabsf(input[i]));
    const float scale = maximum / 448.0f;
    for (int i = start; i < end; ++i)
      output[i] = oracle_e4m3_to_float(oracle_float_to_e4m3(input[i] / fmaxf(scale, 1e-12f))) * scale;
  }
}

/* ImportedMatVecKernel (:40-71): y[r] = bf16(sum_c w[r][c] * x[c]) with all arithmetic in fp32;
 * weights [rows, cols] output-major in fp32 (storage 0), bf16 bits (1) or e4m3 bytes (2, each
 * multiplied by scales[(r/128) * ceil(cols/128) + c/128]); for e4m3 weights the input is first
 * quantized in groups of 128.  The reference accumulates 128 column lanes per output row and
 * reduces them at the end; the same here.  input: fp32 values of the bf16 activation. */
void oracle_linear_imported(const void* weights, int storage, const float* scales,
                            const float* input, int cols, int rows, uint16_t* output) {
  float* x = (float*)malloc((size_t)cols * sizeof(float));
  if (storage == 2) oracle_quantize_imported_input(input, cols, x);
  else memcpy(x, input, (size_t)cols * sizeof(float));
  const int scale_cols = (cols + 127) / 128;
  for (int r = 0; r < rows; ++r) {
    float lanes[128];
    for (int l = 0; l < 128; ++l) lanes[l] = 0.0f;
    for (int c = 0; c < cols; ++c) {
      const size_t i = (size_t)r * cols + c;
      float w;
      if (storage == 0) w = ((const float*)weights)[i];
      else if (storage == 1) w = bf2f(((const uint16_t*)weights)[i]);
      else w = oracle_e4m3_to_float(((const uint8_t*)weights)[i]) * scales[(size_t)(r / 128) * scale_cols + c / 128];
      lanes[c % 128] += w * x[c];
    }
    float sum = 0.0f;
    for (int l = 0; l < 128; ++l) sum += lanes[l];
    output[r] = f2bf(sum);
  }
  free(x);
}
