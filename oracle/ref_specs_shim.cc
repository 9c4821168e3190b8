// TEST INFRASTRUCTURE -- not part of the shipped engine.
//
// C entry points over the scalar specifications the reference project keeps inside its own GPU
// layer tests.  Those specifications are the reference's statement of what its decode, delta-net
// and Qwen sequence layers must compute (its GPU kernels are tested against them), and unlike the
// kernels they are plain host C++:
//   PLUTO_SPEC == 1  src/llm/layers/util/cached_attention_ops_test.cc
//                    class AttentionReference (:43-131), class DeltaReference (:133-220)
//   PLUTO_SPEC == 2  src/llm/layers/sequence_delta_net_test.cc
//                    MakeExample (:31-62), Reference (:66-159), Loss (:161-165)
//   PLUTO_SPEC == 3  src/llm/layers/qwen_attention_test.cc
//                    Reference (:26-95), Values (:97-102)
// oracle/Makefile compiles this file three times, once per value, each time including the test
// file where it lies in the reference tree (never copied) against the Abseil and GoogleTest
// stand-ins beside this file; the tests' bodies compile but nothing registers or runs them.  The
// three test files define the same helper names in anonymous namespaces, hence one translation
// unit each.  Everything below the include only adapts the specifications to plain pointers.
#include <cstddef>
#include <vector>

#if PLUTO_SPEC == 1
#include "src/llm/layers/util/cached_attention_ops_test.cc"

namespace ops = pluto::llm::cached_attention_ops;

// `steps` consecutive CachedAttentionStep calls from an empty cache.
//   q_gate [steps][Hq*2*D], key/value [steps][Hkv*D], q_norm/k_norm [D]
//   out [steps][Hq*D]; probabilities (optional) packed step after step, step t holding
//   [Hq][t+1] values (offset Hq * t(t+1)/2).
extern "C" int ref_spec_attention_steps(int query_heads, int key_value_heads, int head_dim,
                                        int rotary_dim, int capacity, float rms_norm_epsilon,
                                        float rope_theta, int round_to_bfloat16, int steps,
                                        const float* q_gate, const float* key, const float* value,
                                        const float* q_norm, const float* k_norm, float* out,
                                        float* probabilities) {
  ops::FullAttentionParameters p;
  p.query_heads = query_heads;
  p.key_value_heads = key_value_heads;
  p.head_dim = head_dim;
  p.rotary_dim = rotary_dim;
  p.capacity = capacity;
  p.rms_norm_epsilon = rms_norm_epsilon;
  p.rope_theta = rope_theta;
  p.round_to_bfloat16 = round_to_bfloat16 != 0;
  ops::AttentionReference reference(p);
  const size_t qg = static_cast<size_t>(query_heads) * 2 * head_dim;
  const size_t kv = static_cast<size_t>(key_value_heads) * head_dim;
  const size_t width = static_cast<size_t>(query_heads) * head_dim;
  const std::vector<float> qn(q_norm, q_norm + head_dim), kn(k_norm, k_norm + head_dim);
  size_t probability_offset = 0;
  for (int t = 0; t < steps; ++t) {
    const std::vector<float> q(q_gate + t * qg, q_gate + (t + 1) * qg);
    const std::vector<float> k(key + t * kv, key + (t + 1) * kv);
    const std::vector<float> v(value + t * kv, value + (t + 1) * kv);
    const std::vector<float> result = reference.Step(q, k, v, qn, kn);
    for (size_t i = 0; i < width; ++i) out[t * width + i] = result[i];
    if (probabilities != nullptr) {
      const std::vector<float>& row = reference.probabilities();
      for (size_t i = 0; i < row.size(); ++i) probabilities[probability_offset + i] = row[i];
      probability_offset += row.size();
    }
  }
  return 0;
}

// `steps` consecutive DeltaNetState::Step calls from a fresh (Reset) state.
//   qkv [steps][channels], z [steps][Hv*dv], a/b [steps][Hv], weights [channels*kernel],
//   a_log/dt_bias [Hv], norm [dv]; out [steps][Hv*dv].
extern "C" int ref_spec_delta_steps(int key_heads, int value_heads, int key_head_dim,
                                    int value_head_dim, int conv_kernel_dim,
                                    float rms_norm_epsilon, int round_to_bfloat16, int steps,
                                    const float* qkv, const float* z, const float* a,
                                    const float* b, const float* weights, const float* a_log,
                                    const float* dt_bias, const float* norm, float* out) {
  ops::DeltaNetParameters p;
  p.key_heads = key_heads;
  p.value_heads = value_heads;
  p.key_head_dim = key_head_dim;
  p.value_head_dim = value_head_dim;
  p.conv_kernel_dim = conv_kernel_dim;
  p.rms_norm_epsilon = rms_norm_epsilon;
  p.round_to_bfloat16 = round_to_bfloat16 != 0;
  const size_t channels = 2 * static_cast<size_t>(key_heads) * key_head_dim +
                          static_cast<size_t>(value_heads) * value_head_dim;
  const size_t width = static_cast<size_t>(value_heads) * value_head_dim;
  ops::DeltaReference reference(p);
  const std::vector<float> w(weights, weights + channels * conv_kernel_dim);
  const std::vector<float> al(a_log, a_log + value_heads), dt(dt_bias, dt_bias + value_heads);
  const std::vector<float> nm(norm, norm + value_head_dim);
  for (int t = 0; t < steps; ++t) {
    const std::vector<float> x(qkv + t * channels, qkv + (t + 1) * channels);
    const std::vector<float> zz(z + t * width, z + (t + 1) * width);
    const std::vector<float> aa(a + t * value_heads, a + (t + 1) * value_heads);
    const std::vector<float> bb(b + t * value_heads, b + (t + 1) * value_heads);
    const std::vector<float> result = reference.Step(x, zz, aa, bb, w, al, dt, nm);
    for (size_t i = 0; i < width; ++i) out[t * width + i] = result[i];
  }
  return 0;
}

#elif PLUTO_SPEC == 2
#include "src/llm/layers/sequence_delta_net_test.cc"

namespace {
// Sizes of the eight tensors of an Example (QKV, Z, A, B, convolution, A_log, dt_bias, norm).
void ExampleSizes(int length, int kh, int vh, int kd, int vd, int kernel, long long sizes[8]) {
  const long long channels = 2LL * kh * kd + 1LL * vh * vd;
  sizes[0] = length * channels;
  sizes[1] = 1LL * length * vh * vd;
  sizes[2] = sizes[3] = 1LL * length * vh;
  sizes[4] = channels * kernel;
  sizes[5] = sizes[6] = vh;
  sizes[7] = vd;
}

pluto::llm::Example FromArrays(int length, int kh, int vh, int kd, int vd, int kernel, float epsilon,
                               int round, const double* const tensors[8], const float* upstream) {
  pluto::llm::Example e;
  e.p = {kh, vh, kd, vd, kernel, epsilon, round != 0};
  e.length = length;
  long long sizes[8];
  ExampleSizes(length, kh, vh, kd, vd, kernel, sizes);
  for (int t = 0; t < 8; ++t) e.values[t].assign(tensors[t], tensors[t] + sizes[t]);
  e.upstream.assign(static_cast<size_t>(sizes[1]), 0.0f);
  if (upstream != nullptr) e.upstream.assign(upstream, upstream + sizes[1]);
  return e;
}
}  // namespace

// The reference's own example generator (kernel 3, epsilon 0.03): fills the eight tensors
// (caller-sized, see ExampleSizes: [T*channels], [T*Hv*dv], [T*Hv], [T*Hv], [channels*3], [Hv],
// [Hv], [dv]) and the upstream gradient [T*Hv*dv].
extern "C" int ref_spec_sequence_delta_example(int length, int kh, int vh, int kd, int vd, int round,
                                               double* const tensors[8], float* upstream) {
  const pluto::llm::Example e = pluto::llm::MakeExample(length, kh, vh, kd, vd, round != 0);
  for (int t = 0; t < 8; ++t)
    for (size_t i = 0; i < e.values[t].size(); ++i) tensors[t][i] = e.values[t][i];
  for (size_t i = 0; i < e.upstream.size(); ++i) upstream[i] = e.upstream[i];
  return 0;
}

// SequenceDeltaNetLayer forward as the specification states it: out [T*Hv*dv] doubles.
extern "C" int ref_spec_sequence_delta_forward(int length, int kh, int vh, int kd, int vd, int kernel,
                                               float epsilon, int round,
                                               const double* const tensors[8], double* out) {
  const pluto::llm::Example e = FromArrays(length, kh, vh, kd, vd, kernel, epsilon, round, tensors, nullptr);
  const std::vector<double> result = pluto::llm::Reference(e);
  for (size_t i = 0; i < result.size(); ++i) out[i] = result[i];
  return 0;
}

// Numerical BPTT exactly as the reference's gradient test does it
// (sequence_delta_net_test.cc:299-373): rounding offsets recorded at the base point and held
// constant, central differences of Loss with step `epsilon` in every coordinate of the eight
// tensors.  gradients[t] has the size of tensor t.
extern "C" int ref_spec_sequence_delta_gradients(int length, int kh, int vh, int kd, int vd, int kernel,
                                                 float rms_epsilon, int round,
                                                 const double* const tensors[8], const float* upstream,
                                                 double epsilon, double* const gradients[8]) {
  pluto::llm::Example e = FromArrays(length, kh, vh, kd, vd, kernel, rms_epsilon, round, tensors, upstream);
  std::vector<double> offsets;
  pluto::llm::Reference(e, &offsets);
  for (int t = 0; t < 8; ++t)
    for (size_t i = 0; i < e.values[t].size(); ++i) {
      const double original = e.values[t][i];
      e.values[t][i] = original + epsilon;
      const double plus = pluto::llm::Loss(e, offsets);
      e.values[t][i] = original - epsilon;
      const double minus = pluto::llm::Loss(e, offsets);
      e.values[t][i] = original;
      gradients[t][i] = (plus - minus) / (2 * epsilon);
    }
  return 0;
}

#elif PLUTO_SPEC == 3
#include "src/llm/layers/qwen_attention_test.cc"

namespace {
pluto::llm::FullAttentionParameters QwenParameters(int query_heads, int key_value_heads, int head_dim,
                                                   int rotary_dim, float rms_norm_epsilon,
                                                   float rope_theta, int round) {
  pluto::llm::FullAttentionParameters p;
  p.query_heads = query_heads;
  p.key_value_heads = key_value_heads;
  p.head_dim = head_dim;
  p.rotary_dim = rotary_dim;
  p.rms_norm_epsilon = rms_norm_epsilon;
  p.rope_theta = rope_theta;
  p.round_to_bfloat16 = round != 0;
  return p;
}
}  // namespace

// QwenAttentionLayer sequence forward as the specification states it.
//   qg [T][Hq][2][D], k/v [T][Hkv][D], qw/kw [D] (zero-centred norm weights); out [T][Hq][D].
extern "C" int ref_spec_qwen_sequence_forward(int query_heads, int key_value_heads, int head_dim,
                                              int rotary_dim, float rms_norm_epsilon, float rope_theta,
                                              int round, int length, const double* qg, const double* k,
                                              const double* v, const double* qw, const double* kw,
                                              double* out) {
  const auto p = QwenParameters(query_heads, key_value_heads, head_dim, rotary_dim, rms_norm_epsilon,
                                rope_theta, round);
  const size_t d = head_dim;
  const std::vector<double> a(qg, qg + length * query_heads * 2 * d), b(k, k + length * key_value_heads * d),
      c(v, v + length * key_value_heads * d), e(qw, qw + d), f(kw, kw + d);
  std::vector<double> rounding;
  const std::vector<double> result = pluto::llm::Reference(p, length, a, b, c, e, f, rounding, true);
  for (size_t i = 0; i < result.size(); ++i) out[i] = result[i];
  return 0;
}

// Central differences of sum(output * upstream) exactly as the reference's gradient test
// (qwen_attention_test.cc:230-301): rounding errors recorded at the base point and held.
// gradients: d_qg, d_k, d_v, d_qw, d_kw with the inputs' sizes.
extern "C" int ref_spec_qwen_sequence_gradients(int query_heads, int key_value_heads, int head_dim,
                                                int rotary_dim, float rms_norm_epsilon, float rope_theta,
                                                int round, int length, const double* qg, const double* k,
                                                const double* v, const double* qw, const double* kw,
                                                const double* upstream, double epsilon,
                                                double* const gradients[5]) {
  const auto p = QwenParameters(query_heads, key_value_heads, head_dim, rotary_dim, rms_norm_epsilon,
                                rope_theta, round);
  const size_t d = head_dim;
  std::vector<std::vector<double>> values = {
      std::vector<double>(qg, qg + length * query_heads * 2 * d),
      std::vector<double>(k, k + length * key_value_heads * d),
      std::vector<double>(v, v + length * key_value_heads * d), std::vector<double>(qw, qw + d),
      std::vector<double>(kw, kw + d)};
  std::vector<double> rounding;
  pluto::llm::Reference(p, length, values[0], values[1], values[2], values[3], values[4], rounding, true);
  const auto loss = [&] {
    const auto output =
        pluto::llm::Reference(p, length, values[0], values[1], values[2], values[3], values[4], rounding);
    double sum = 0;
    for (size_t i = 0; i < output.size(); ++i) sum += output[i] * upstream[i];
    return sum;
  };
  for (size_t input = 0; input < values.size(); ++input)
    for (size_t i = 0; i < values[input].size(); ++i) {
      const double original = values[input][i];
      values[input][i] = original + epsilon;
      const double plus = loss();
      values[input][i] = original - epsilon;
      const double minus = loss();
      values[input][i] = original;
      gradients[input][i] = (plus - minus) / (2 * epsilon);
    }
  return 0;
}

#else
#error "compile with -DPLUTO_SPEC=1, 2 or 3"
#endif
