// GPU test of the C++ host adapter (pluto_b200/host): the reference-shaped layer classes driven
// the way the reference's own tests drive them (attention_reference_test.cc,
// cached_attention_ops_test.cc), checked against the CPU oracle library.  Prints one line per
// check and exits non-zero on the first failure.  Test infrastructure: links oracle/.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../../pluto_b200/host/layers.h"
#include "../../pluto_b200/host/qwen_layers.h"

extern "C" {
int oracle_attention_fwd(const void*, int, int, int, int, int, int, void*, float*, float*, float*);
int oracle_attention_bwd(const void*, const void*, const float*, int, int, int, int, int, int, float*);
uint16_t oracle_float_to_bf16(float);
float oracle_bf16_to_float(uint16_t);
void oracle_qk_prepare(const float*, const float*, const float*, const float*, const float*, int, int,
                       int, int, int, float, float, int, float*, float*, float*);
void oracle_gqa_decode(const float*, const float*, const void*, const void*, int, int, int, int, int,
                       int, float*);
void oracle_gqa_probabilities(const float*, const void*, int, int, int, int, int, float*);
float oracle_gdn_decay(float, float, float);
float oracle_gdn_beta(float, int);
int oracle_gdn_recurrence(const void*, const void*, const void*, const float*, const float*, int, int,
                          int, int, int, int, int, int, float, int, int, float*, void*);
void oracle_gdn_conv_step(const float*, const float*, int, int, int, float*, float*);
void oracle_gdn_output(const float*, const float*, const float*, int, int, float, int, int, float*);
int oracle_gqa_sequence_bwd(const float*, const float*, const float*, const float*, const float*, const float*,
                            int, int, int, int, int, float, float, int, float*, float*, float*, float*, float*,
                            float*);
int oracle_gdn_sequence_bwd(const float*, const float*, const float*, const float*, const float*, const float*,
                            const float*, const float*, const float*, int, int, int, int, int, int, float, int,
                            float*, float*, float*, float*, float*, float*, float*, float*, float*);
}

using namespace pluto;
using namespace pluto::llm;
namespace ops = pluto::llm::cached_attention_ops;

static int g_checks = 0;
#define CHECK(cond)                                                        \
  do {                                                                     \
    ++g_checks;                                                            \
    if (!(cond)) {                                                         \
      std::printf("FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond);          \
      std::exit(1);                                                        \
    }                                                                      \
  } while (false)
#define CHECK_OK(expr)                                                     \
  do {                                                                     \
    ++g_checks;                                                            \
    const ::pluto::Status s_ = (expr);                                     \
    if (!s_.ok()) {                                                        \
      std::printf("FAIL %s:%d: %s -> %s\n", __FILE__, __LINE__, #expr, s_.message().c_str()); \
      std::exit(1);                                                        \
    }                                                                      \
  } while (false)

static cuda::Buffer Upload(cuda::Executor& ex, const void* data, size_t bytes) {
  auto b = cuda::Buffer::Allocate(ex, bytes);
  CHECK(b.ok());
  CHECK(cudaMemcpyAsync(b->data(), data, bytes, cudaMemcpyHostToDevice, ex.stream()) == cudaSuccess);
  CHECK_OK(ex.Synchronize());
  return *b;
}
template <class T>
static std::vector<T> Download(cuda::Executor& ex, const void* device, size_t count) {
  std::vector<T> host(count);
  CHECK(cudaMemcpyAsync(host.data(), device, count * sizeof(T), cudaMemcpyDeviceToHost, ex.stream()) == cudaSuccess);
  CHECK_OK(ex.Synchronize());
  return host;
}
static std::vector<float> Values(int count, float phase, float scale = 1.0f) {
  std::vector<float> r(count);
  for (int i = 0; i < count; ++i) r[i] = scale * std::sin(phase + i * 0.29f);
  return r;
}
static float MaxAbsDiff(const std::vector<float>& a, const std::vector<float>& b) {
  float m = 0;
  for (size_t i = 0; i < a.size(); ++i) m = std::fmax(m, std::fabs(a[i] - b[i]));
  return m;
}

static void TestAttentionLayer(cuda::Executor& ex, bool bf16) {
  const int S = 65, H = 2, E = 128, B = 2, rows = S * B;
  std::vector<float> qkv(static_cast<size_t>(rows) * 3 * E), dout(static_cast<size_t>(rows) * E);
  for (size_t i = 0; i < qkv.size(); ++i)
    qkv[i] = 0.35f * std::sin(static_cast<float>(i) * 0.071f) + 0.05f * std::cos(static_cast<float>(i) * 0.19f);
  for (size_t i = 0; i < dout.size(); ++i) dout[i] = 0.2f * std::cos(static_cast<float>(i) * 0.13f);
  std::vector<uint16_t> bits(qkv.size());
  for (size_t i = 0; i < qkv.size(); ++i) bits[i] = oracle_float_to_bf16(qkv[i]);
  const void* host_in = bf16 ? static_cast<const void*>(bits.data()) : qkv.data();
  const size_t element = bf16 ? 2 : 4;
  const DataType type = bf16 ? DataType::BF16 : DataType::FP16;

  auto layer = AttentionLayer::Create(ex, S, H, E, type);
  CHECK(layer.ok());
  CHECK((*layer)->input_types()[0] == (ActivationType{bf16 ? DataType::BF16 : DataType::FP32, {-2, S, 3 * E}}));
  BufferVec inputs = {Upload(ex, host_in, qkv.size() * element)};
  int hook_calls = 0;
  LayerHooks hooks;
  hooks.attention_probabilities_hook = [&](cuda::Executor&, const std::string& name,
                                           const ActivationType& shape, const Buffer& buffer) {
    ++hook_calls;
    CHECK(name == "AttentionLayer");
    CHECK(shape == (ActivationType{DataType::FP32, {B, H, S, S}}));
    CHECK(buffer.size_bytes() == static_cast<size_t>(B) * H * S * S * 4);
    return OkStatus();
  };
  auto fwd = (*layer)->fwd(ex, inputs, &hooks);
  CHECK(fwd.ok());
  CHECK(hook_calls == 1 && fwd->state.intermediates.size() == 4);
  BufferVec grads = {Upload(ex, dout.data(), dout.size() * 4)};
  auto bwd = (*layer)->bwd(ex, grads, fwd->state);
  CHECK(bwd.ok());

  std::vector<uint8_t> ref_out(static_cast<size_t>(rows) * E * element);
  std::vector<float> ref_grad(qkv.size());
  CHECK(oracle_attention_fwd(host_in, rows, S, H, E, bf16, 4, ref_out.data(), nullptr, nullptr, nullptr) == 0);
  CHECK(oracle_attention_bwd(host_in, ref_out.data(), dout.data(), rows, S, H, E, bf16, 4, ref_grad.data()) == 0);
  std::vector<float> got_out(static_cast<size_t>(rows) * E), want_out(got_out.size());
  if (bf16) {
    auto raw = Download<uint16_t>(ex, fwd->outputs[0].data(), got_out.size());
    for (size_t i = 0; i < raw.size(); ++i) {
      got_out[i] = oracle_bf16_to_float(raw[i]);
      want_out[i] = oracle_bf16_to_float(reinterpret_cast<uint16_t*>(ref_out.data())[i]);
    }
  } else {
    got_out = Download<float>(ex, fwd->outputs[0].data(), got_out.size());
    std::memcpy(want_out.data(), ref_out.data(), ref_out.size());
  }
  const float tol = bf16 ? 2e-2f : 1e-4f;
  CHECK(MaxAbsDiff(got_out, want_out) <= tol);
  CHECK(MaxAbsDiff(Download<float>(ex, (*bwd)[0].data(), ref_grad.size()), ref_grad) <= tol);

  // validation (attention_test.cc:549-626) and hook failure (attention_test.cc:246-280)
  auto other = AttentionLayer::Create(ex, S, H, E, type);
  auto foreign = (*other)->bwd(ex, grads, fwd->state);
  CHECK(!foreign.ok() && foreign.status().code() == StatusCode::kInvalidArgument);
  auto odd = (*layer)->fwd(ex, {Upload(ex, host_in, static_cast<size_t>(S + 1) * 3 * E * element)});
  CHECK(!odd.ok() && odd.status().message().find("divisible by context_length") != std::string::npos);
  hooks.attention_probabilities_hook = [](cuda::Executor&, const std::string&, const ActivationType&,
                                          const Buffer&) { return Status(StatusCode::kCancelled, "stop"); };
  auto cancelled = (*layer)->fwd(ex, inputs, &hooks);
  CHECK(!cancelled.ok() && cancelled.status().code() == StatusCode::kCancelled);
  CHECK(!AttentionLayer::Create(ex, 8, 3, 32, DataType::BF16).ok());
  CHECK(AttentionLayer::Create(ex, 8, 2, 32, DataType::FP8).status().code() == StatusCode::kUnimplemented);
  std::printf("ok AttentionLayer %s\n", bf16 ? "bf16" : "fp32");
}

static void TestCachedAttention(cuda::Executor& ex, int dim, bool round) {
  ops::FullAttentionParameters p;
  p.query_heads = dim == 6 ? 4 : 24;
  p.key_value_heads = dim == 6 ? 2 : 4;
  p.head_dim = dim;
  p.rotary_dim = dim == 6 ? 4 : 64;
  p.capacity = 35;
  p.rope_theta = dim == 6 ? 73.0f : 10000000.0f;
  p.round_to_bfloat16 = round;
  auto cache = KeyValueCache::Create(ex, p.capacity, p.key_value_heads, p.head_dim);
  CHECK(cache.ok());
  CHECK_OK(ops::ValidateCachedAttention(ex, p, **cache));
  const auto qn = Values(dim, 0.2f, 0.3f), kn = Values(dim, 0.8f, 0.4f);
  auto dqn = Upload(ex, qn.data(), qn.size() * 4), dkn = Upload(ex, kn.data(), kn.size() * 4);
  auto out = cuda::Buffer::Allocate(ex, static_cast<size_t>(p.query_heads) * dim * 4);
  CHECK(out.ok());
  std::vector<float> okeys(static_cast<size_t>(p.capacity) * p.key_value_heads * dim, 0.f), ovals(okeys);
  std::vector<float> first, last;
  for (int t = 0; t < p.capacity; ++t) {
    auto q = Values(p.query_heads * 2 * dim, 0.15f + t * 0.21f);
    auto k = Values(p.key_value_heads * dim, 0.78f + t * 0.13f);
    auto v = Values(p.key_value_heads * dim, -0.31f + t * 0.37f);
    auto dq = Upload(ex, q.data(), q.size() * 4), dk = Upload(ex, k.data(), k.size() * 4),
         dv = Upload(ex, v.data(), v.size() * 4);
    auto probs = cuda::Buffer::Allocate(ex, static_cast<size_t>(p.query_heads) * (t + 1) * 4);
    CHECK(probs.ok());
    CHECK_OK(ops::CachedAttentionStep(ex, p, **cache, static_cast<float*>(dq.data()),
                                      static_cast<float*>(dk.data()), static_cast<float*>(dv.data()),
                                      static_cast<float*>(dqn.data()), static_cast<float*>(dkn.data()),
                                      static_cast<float*>(out->data()), static_cast<float*>(probs->data())));
    CHECK((*cache)->position() == t + 1);
    std::vector<float> queries(static_cast<size_t>(p.query_heads) * dim), want(queries.size()),
        want_p(static_cast<size_t>(p.query_heads) * (t + 1));
    oracle_qk_prepare(q.data(), k.data(), v.data(), qn.data(), kn.data(), p.query_heads,
                      p.key_value_heads, dim, p.rotary_dim, t, p.rms_norm_epsilon, p.rope_theta,
                      round, queries.data(), okeys.data(), ovals.data());
    oracle_gqa_decode(queries.data(), q.data(), okeys.data(), ovals.data(), 0, p.query_heads,
                      p.key_value_heads, dim, t + 1, round, want.data());
    oracle_gqa_probabilities(queries.data(), okeys.data(), 0, p.query_heads, p.key_value_heads, dim,
                             t + 1, want_p.data());
    last = Download<float>(ex, out->data(), want.size());
    auto got_p = Download<float>(ex, probs->data(), want_p.size());
    for (size_t i = 0; i < want.size(); ++i)
      CHECK(std::fabs(last[i] - want[i]) <= (round ? 2e-4f + 8e-3f * std::fabs(want[i]) : 3e-5f + 1e-4f * std::fabs(want[i])));
    for (size_t i = 0; i < want_p.size(); ++i)
      CHECK(std::fabs(got_p[i] - want_p[i]) <= (round ? 2e-4f + 8e-3f * want_p[i] : 3e-5f + 1e-4f * want_p[i]));
    if (t == 0) first = last;
    if (t + 1 == p.capacity) {
      auto full = ops::CachedAttentionStep(ex, p, **cache, static_cast<float*>(dq.data()),
                                           static_cast<float*>(dk.data()), static_cast<float*>(dv.data()),
                                           static_cast<float*>(dqn.data()), static_cast<float*>(dkn.data()),
                                           static_cast<float*>(out->data()));
      CHECK(full.code() == StatusCode::kResourceExhausted && (*cache)->position() == p.capacity);
      CHECK(Download<float>(ex, out->data(), want.size()) == last);
    }
  }
  (*cache)->Reset();
  auto q = Values(p.query_heads * 2 * dim, 0.15f), k = Values(p.key_value_heads * dim, 0.78f),
       v = Values(p.key_value_heads * dim, -0.31f);
  auto dq = Upload(ex, q.data(), q.size() * 4), dk = Upload(ex, k.data(), k.size() * 4),
       dv = Upload(ex, v.data(), v.size() * 4);
  CHECK_OK(ops::CachedAttentionStep(ex, p, **cache, static_cast<float*>(dq.data()),
                                    static_cast<float*>(dk.data()), static_cast<float*>(dv.data()),
                                    static_cast<float*>(dqn.data()), static_cast<float*>(dkn.data()),
                                    static_cast<float*>(out->data())));
  CHECK(Download<float>(ex, out->data(), first.size()) == first);
  ops::FullAttentionParameters bad = p;
  bad.rotary_dim = 3;
  CHECK(ops::ValidateCachedAttention(ex, bad, **cache).code() == StatusCode::kInvalidArgument);
  CHECK(ops::CachedAttentionStep(ex, p, **cache, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr).code() ==
        StatusCode::kInvalidArgument);
  std::printf("ok CachedAttentionStep dim %d round %d\n", dim, round);
}

static void TestDeltaNetState(cuda::Executor& ex, int dim, bool round) {
  ops::DeltaNetParameters p;
  p.key_heads = 2;
  p.value_heads = 6;
  p.key_head_dim = dim;
  p.value_head_dim = dim == 5 ? 7 : 128;
  p.conv_kernel_dim = 4;
  p.round_to_bfloat16 = round;
  const int channels = 2 * p.key_heads * p.key_head_dim + p.value_heads * p.value_head_dim;
  auto state = ops::DeltaNetState::Create(ex, p);
  CHECK(state.ok());
  auto w = Values(channels * 4, 0.73f, 0.6f), alog = Values(6, 0.18f, 0.5f), dt = Values(6, -0.7f, 0.3f),
       norm = Values(p.value_head_dim, 0.5f, 0.6f);
  auto dw = Upload(ex, w.data(), w.size() * 4), dalog = Upload(ex, alog.data(), 24), ddt = Upload(ex, dt.data(), 24),
       dn = Upload(ex, norm.data(), norm.size() * 4);
  auto out = cuda::Buffer::Allocate(ex, static_cast<size_t>(6) * p.value_head_dim * 4);
  CHECK(out.ok());
  std::vector<float> conv_state(static_cast<size_t>(channels) * 4, 0.f),
      rec_state(static_cast<size_t>(6) * dim * p.value_head_dim, 0.f), first;
  for (int step = 0; step < 7; ++step) {
    const int t = step == 6 ? 0 : step;
    if (step == 6) CHECK_OK((*state)->Reset());
    auto qkv = Values(channels, 0.3f + t * 0.71f), z = Values(6 * p.value_head_dim, -0.6f + t * 0.27f),
         a = Values(6, 0.1f + t * 0.1f), b = Values(6, -0.7f + t * 0.3f);
    a[0] = 100.0f;
    a[1] = -100.0f;
    auto dqkv = Upload(ex, qkv.data(), qkv.size() * 4), dz = Upload(ex, z.data(), z.size() * 4),
         da = Upload(ex, a.data(), 24), db = Upload(ex, b.data(), 24);
    CHECK_OK((*state)->Step(static_cast<float*>(dqkv.data()), static_cast<float*>(dz.data()),
                            static_cast<float*>(da.data()), static_cast<float*>(db.data()),
                            static_cast<float*>(dw.data()), static_cast<float*>(dalog.data()),
                            static_cast<float*>(ddt.data()), static_cast<float*>(dn.data()),
                            static_cast<float*>(out->data())));
    auto got = Download<float>(ex, out->data(), static_cast<size_t>(6) * p.value_head_dim);
    if (step < 6) {
      std::vector<float> conv(channels), g(6), beta(6), core(got.size()), want(got.size());
      oracle_gdn_conv_step(qkv.data(), w.data(), channels, 4, round, conv_state.data(), conv.data());
      for (int h = 0; h < 6; ++h) {
        g[h] = oracle_gdn_decay(a[h], dt[h], alog[h]);
        beta[h] = oracle_gdn_beta(b[h], round);
      }
      const int kq = p.key_heads * dim;
      CHECK(oracle_gdn_recurrence(conv.data(), conv.data() + kq, conv.data() + 2 * kq, g.data(), beta.data(),
                                  0, 1, 1, 2, 6, dim, p.value_head_dim, 1, 1.0f, round, 1,
                                  rec_state.data(), core.data()) == 0);
      oracle_gdn_output(core.data(), z.data(), norm.data(), 6, p.value_head_dim, p.rms_norm_epsilon,
                        round, 1, want.data());
      for (size_t i = 0; i < want.size(); ++i)
        CHECK(std::fabs(got[i] - want[i]) <= (round ? 2e-4f + 8e-3f * std::fabs(want[i]) : 3e-5f + 1e-4f * std::fabs(want[i])));
    }
    if (step == 0) first = got;
    if (step == 6) CHECK(got == first);
  }
  ops::DeltaNetParameters bad = p;
  bad.key_head_dim = 129;
  CHECK(!ops::DeltaNetState::Create(ex, bad).ok());
  std::printf("ok DeltaNetState dim %d round %d\n", dim, round);
}

// ---- the three Qwen decoder layer classes -------------------------------------------------------
static std::vector<float> Bf16Values(int count, float phase) {   // qwen_attention_test.cc:97-102
  std::vector<float> r(count);
  for (int i = 0; i < count; ++i)
    r[i] = oracle_bf16_to_float(oracle_float_to_bf16(static_cast<float>(0.8 * std::sin(phase + 0.29 * i))));
  return r;
}
static cuda::Buffer UploadBf16(cuda::Executor& ex, const std::vector<float>& values) {
  std::vector<uint16_t> bits(values.size());
  for (size_t i = 0; i < values.size(); ++i) bits[i] = oracle_float_to_bf16(values[i]);
  return Upload(ex, bits.data(), bits.size() * 2);
}
static std::vector<float> DownloadBf16(cuda::Executor& ex, const cuda::Buffer& buffer) {
  auto raw = Download<uint16_t>(ex, buffer.data(), buffer.size_bytes() / 2);
  std::vector<float> r(raw.size());
  for (size_t i = 0; i < raw.size(); ++i) r[i] = oracle_bf16_to_float(raw[i]);
  return r;
}
static std::shared_ptr<BlockParameter> Parameter(cuda::Executor& ex, const std::vector<float>& values, bool active) {
  auto parameter = BlockParameter::Create(ex, Upload(ex, values.data(), values.size() * 4), DataType::FP32);
  CHECK(parameter.ok());
  if (active) CHECK_OK((*parameter)->Activate());
  return *parameter;
}

// qwen_attention_test.cc:155-228: sequence forward against the oracle, the causal hook, and the
// cached layer fed token by token.
static void TestQwenAttentionForward(cuda::Executor& ex, int d) {
  FullAttentionParameters p;
  p.query_heads = 2;
  p.key_value_heads = 1;
  p.head_dim = d;
  p.rotary_dim = d == 3 ? 2 : 64;
  p.capacity = 40;
  const int length = d == 3 ? 33 : 3;
  auto qg = Bf16Values(length * 2 * p.query_heads * d, .1f), k = Bf16Values(length * d, 1.2f),
       v = Bf16Values(length * d, 2.3f), qw = Bf16Values(d, .2f), kw = Bf16Values(d, .4f);
  auto layer = QwenAttentionLayer::Create(ex, p, Parameter(ex, qw, false), Parameter(ex, kw, false), length);
  CHECK(layer.ok());
  CHECK((*layer)->input_types()[0] == (ActivationType{DataType::BF16, {-2, length, 4 * d}}));
  BufferVec inputs = {UploadBf16(ex, qg), UploadBf16(ex, k), UploadBf16(ex, v)};
  int hook_calls = 0;
  LayerHooks hooks;
  hooks.attention_probabilities_hook = [&](cuda::Executor& e, const std::string&, const ActivationType& type,
                                           const Buffer& buffer) {
    CHECK(type == (ActivationType{DataType::FP32, {1, 2, length, length}}));
    auto probs = Download<float>(e, buffer.data(), static_cast<size_t>(2) * length * length);
    for (int h = 0; h < 2; ++h)
      for (int row = 0; row < length; ++row) {
        double sum = 0;
        for (int t = 0; t < length; ++t) {
          const float value = probs[(static_cast<size_t>(h) * length + row) * length + t];
          if (t > row) CHECK(value == 0);
          sum += value;
        }
        CHECK(std::fabs(sum - 1) <= 2e-6);
      }
    ++hook_calls;
    return OkStatus();
  };
  auto fwd = (*layer)->fwd(ex, inputs, &hooks);
  CHECK(fwd.ok());
  CHECK(hook_calls == 1 && fwd->state.intermediates.size() == QwenAttentionLayer::kSavedBuffers);
  const auto actual = DownloadBf16(ex, fwd->outputs[0]);
  std::vector<float> want(actual.size()), zero(actual.size(), 0.f), dqg(qg.size()), dk(k.size()), dv(v.size());
  CHECK(oracle_gqa_sequence_bwd(qg.data(), k.data(), v.data(), qw.data(), kw.data(), zero.data(), length, 2, 1, d,
                                p.rotary_dim, p.rms_norm_epsilon, p.rope_theta, 1, dqg.data(), dk.data(), dv.data(),
                                nullptr, nullptr, want.data()) == 0);
  for (size_t i = 0; i < want.size(); ++i) CHECK(std::fabs(actual[i] - want[i]) <= 2e-4f + 8e-3f * std::fabs(want[i]));
  // the cached layer, one token at a time, must reproduce the sequence layer's rows
  auto cache = KeyValueCache::Create(ex, p.capacity, p.key_value_heads, p.head_dim);
  CHECK(cache.ok());
  auto cached = QwenAttentionLayer::Create(ex, p, Upload(ex, qw.data(), qw.size() * 4),
                                           Upload(ex, kw.data(), kw.size() * 4), 1, cache->get());
  CHECK(cached.ok());
  for (int row = 0; row < length; ++row) {
    BufferVec token = {UploadBf16(ex, {qg.begin() + row * 4 * d, qg.begin() + (row + 1) * 4 * d}),
                       UploadBf16(ex, {k.begin() + row * d, k.begin() + (row + 1) * d}),
                       UploadBf16(ex, {v.begin() + row * d, v.begin() + (row + 1) * d})};
    auto output = (*cached)->fwd(ex, token);
    CHECK(output.ok());
    CHECK((*cache)->position() == row + 1);
    const auto expected = DownloadBf16(ex, output->outputs[0]);
    // (the reference pins bit equality here; the two kernels of this engine agree within bf16
    // rounding of the same fp32 result)
    for (int c = 0; c < 2 * d; ++c)
      CHECK(std::fabs(actual[static_cast<size_t>(row) * 2 * d + c] - expected[c]) <=
            2e-4f + 1.6e-2f * std::fabs(expected[c]));
  }
  auto no_backward = (*cached)->bwd(ex, {fwd->outputs[0]}, BackwardState{cached->get(), {}, {}});
  CHECK(!no_backward.ok() && no_backward.status().code() == StatusCode::kUnimplemented);
  CHECK(!QwenAttentionLayer::Create(ex, p, Parameter(ex, qw, false), Parameter(ex, kw, false), 2, cache->get()).ok());
  FullAttentionParameters bad = p;
  bad.rotary_dim = 3;
  CHECK(!QwenAttentionLayer::Create(ex, bad, Parameter(ex, qw, false), Parameter(ex, kw, false), 3).ok());
  std::printf("ok QwenAttentionLayer forward d %d\n", d);
}

// qwen_attention_test.cc:230-301: every gradient against the oracle's backward (itself pinned by
// the reference's finite differences), and accumulation of the shared norm gradients.
static void TestQwenAttentionBackward(cuda::Executor& ex) {
  FullAttentionParameters p;
  p.query_heads = 2;
  p.key_value_heads = 1;
  p.head_dim = 3;
  p.rotary_dim = 2;
  const int t = 3;
  auto qg = Bf16Values(t * 12, .1f), k = Bf16Values(t * 3, 1.2f), v = Bf16Values(t * 3, 2.3f),
       qw = Bf16Values(3, .2f), kw = Bf16Values(3, .4f), upstream = Bf16Values(t * 6, .7f);
  auto qp = Parameter(ex, qw, true), kp = Parameter(ex, kw, true);
  auto layer = QwenAttentionLayer::Create(ex, p, qp, kp, t);
  CHECK(layer.ok());
  BufferVec inputs = {UploadBf16(ex, qg), UploadBf16(ex, k), UploadBf16(ex, v)};
  BufferVec dy = {Upload(ex, upstream.data(), upstream.size() * 4)};
  auto fwd = (*layer)->fwd(ex, inputs);
  CHECK(fwd.ok());
  auto backward = (*layer)->bwd(ex, dy, fwd->state);
  CHECK(backward.ok() && backward->size() == 3);
  std::vector<float> dqg(qg.size()), dk(k.size()), dv(v.size()), dqw(3, 0.f), dkw(3, 0.f), y(t * 6);
  CHECK(oracle_gqa_sequence_bwd(qg.data(), k.data(), v.data(), qw.data(), kw.data(), upstream.data(), t, 2, 1, 3, 2,
                                p.rms_norm_epsilon, p.rope_theta, 1, dqg.data(), dk.data(), dv.data(), dqw.data(),
                                dkw.data(), y.data()) == 0);
  const std::vector<float>* wants[] = {&dqg, &dk, &dv};
  std::vector<std::vector<float>> first;
  for (int i = 0; i < 3; ++i) {
    first.push_back(Download<float>(ex, (*backward)[i].data(), wants[i]->size()));
    CHECK(MaxAbsDiff(first.back(), *wants[i]) <= 3e-5f);
  }
  auto got_qw = Download<float>(ex, qp->gradient().data(), 3), got_kw = Download<float>(ex, kp->gradient().data(), 3);
  CHECK(MaxAbsDiff(got_qw, dqw) <= 3e-5f && MaxAbsDiff(got_kw, dkw) <= 3e-5f);
  auto second = (*layer)->fwd(ex, inputs);
  CHECK(second.ok());
  auto repeated = (*layer)->bwd(ex, dy, second->state);
  CHECK(repeated.ok());
  for (int i = 0; i < 3; ++i) CHECK(Download<float>(ex, (*repeated)[i].data(), first[i].size()) == first[i]);
  auto summed = Download<float>(ex, qp->gradient().data(), 3);
  for (int i = 0; i < 3; ++i) CHECK(std::fabs(summed[i] - 2 * got_qw[i]) <= 1e-6f);
  auto wrong = (*layer)->bwd(ex, {inputs[1]}, second->state);   // a buffer of the wrong size
  CHECK(!wrong.ok() && wrong.status().code() == StatusCode::kInvalidArgument);
  std::printf("ok QwenAttentionLayer backward\n");
}

// The reference's closed-form example (sequence_delta_net_test.cc:31-62).
struct DeltaExample {
  DeltaNetParameters p;
  int length, channels;
  std::vector<float> values[8], upstream;
};
static DeltaExample MakeDeltaExample(int length, int kh, int vh, int kd, int vd) {
  DeltaExample e;
  e.p = {kh, vh, kd, vd, 3, 0.03f, true};
  e.length = length;
  e.channels = 2 * kh * kd + vh * vd;
  const int sizes[] = {length * e.channels, length * vh * vd, length * vh, length * vh, e.channels * 3, vh, vh, vd};
  for (int tensor = 0; tensor < 8; ++tensor)
    for (int i = 0; i < sizes[tensor]; ++i) {
      float value = 0.15f + 0.4f * std::sin(0.37f * i + 0.41f * tensor);
      if (tensor == 5) value -= 0.7f;
      if (tensor == 7) value += 1.f;
      e.values[tensor].push_back(tensor < 4 ? oracle_bf16_to_float(oracle_float_to_bf16(value)) : value);
    }
  e.upstream.assign(static_cast<size_t>(length) * vh * vd, 0.f);
  for (int i = (length - 1) * vh * vd; i < length * vh * vd; ++i) e.upstream[i] = 0.4f * std::cos(0.2f * i);
  return e;
}

// sequence_delta_net_test.cc:241-297 (forward, cached-token equivalence) and :299-373 (gradients).
static void TestSequenceDeltaNet(cuda::Executor& ex, int length, int kh, int vh, int kd, int vd, bool gradients) {
  const DeltaExample e = MakeDeltaExample(length, kh, vh, kd, vd);
  std::shared_ptr<BlockParameter> parameters[4];
  for (int i = 0; i < 4; ++i) parameters[i] = Parameter(ex, e.values[4 + i], gradients);
  auto layer = SequenceDeltaNetLayer::Create(ex, e.p, parameters[0], parameters[1], parameters[2], parameters[3], length);
  CHECK(layer.ok());
  BufferVec inputs;
  for (int i = 0; i < 4; ++i) inputs.push_back(UploadBf16(ex, e.values[i]));
  auto result = (*layer)->fwd(ex, inputs);
  CHECK(result.ok());
  CHECK(result->state.intermediates.size() == SequenceDeltaNetLayer::kSavedBuffers);
  const auto actual = DownloadBf16(ex, result->outputs[0]);
  const int width = vh * vd;
  std::vector<float> y(actual.size()), dqkv(e.values[0].size()), dz(e.values[1].size()), da(e.values[2].size()),
      db(e.values[3].size()), dparam[4];
  for (int i = 0; i < 4; ++i) dparam[i].assign(e.values[4 + i].size(), 0.f);
  CHECK(oracle_gdn_sequence_bwd(e.values[0].data(), e.values[1].data(), e.values[2].data(), e.values[3].data(),
                                e.values[4].data(), e.values[5].data(), e.values[6].data(), e.values[7].data(),
                                e.upstream.data(), length, kh, vh, kd, vd, 3, 0.03f, 1, dqkv.data(), dz.data(),
                                da.data(), db.data(), dparam[0].data(), dparam[1].data(), dparam[2].data(),
                                dparam[3].data(), y.data()) == 0);
  for (size_t i = 0; i < actual.size(); ++i) {
    const float want = oracle_bf16_to_float(oracle_float_to_bf16(y[i]));
    CHECK(std::fabs(actual[i] - want) <= 1.5e-4f + 0.015f * std::fabs(want) + 2e-3f * std::fabs(want));
  }
  // the single-token layer, fed the same tokens, agrees with the sequence layer
  auto cached = DeltaNetLayer::Create(ex, e.p, parameters[0]->value(), parameters[1]->value(),
                                      parameters[2]->value(), parameters[3]->value());
  CHECK(cached.ok());
  const int counts[] = {e.channels, width, vh, vh};
  for (int t = 0; t < length; ++t) {
    BufferVec token;
    for (int i = 0; i < 4; ++i)
      token.push_back(UploadBf16(ex, {e.values[i].begin() + t * counts[i], e.values[i].begin() + (t + 1) * counts[i]}));
    auto step = (*cached)->fwd(ex, token);
    CHECK(step.ok());
    const auto one = DownloadBf16(ex, step->outputs[0]);
    for (int i = 0; i < width; ++i)
      CHECK(std::fabs(actual[static_cast<size_t>(t) * width + i] - one[i]) <= 1.5e-4f + 0.015f * std::fabs(one[i]));
  }
  CHECK_OK((*cached)->Reset());
  CHECK((*cached)->bwd(ex, {}, BackwardState{cached->get(), {}, {}}).status().code() == StatusCode::kUnimplemented);
  // a second sequence must not inherit state from the first
  auto repeat = (*layer)->fwd(ex, inputs);
  CHECK(repeat.ok() && DownloadBf16(ex, repeat->outputs[0]) == actual);
  if (gradients) {
    BufferVec dy = {Upload(ex, e.upstream.data(), e.upstream.size() * 4)};
    auto backward = (*layer)->bwd(ex, dy, result->state);
    CHECK(backward.ok() && backward->size() == 4);
    const std::vector<float>* wants[] = {&dqkv, &dz, &da, &db};
    auto close = [](const std::vector<float>& got, const std::vector<float>& want) {
      for (size_t i = 0; i < want.size(); ++i)
        if (std::fabs(got[i] - want[i]) > 3e-5f + 0.003f * std::fabs(want[i])) return false;
      return true;
    };
    for (int i = 0; i < 4; ++i) CHECK(close(Download<float>(ex, (*backward)[i].data(), wants[i]->size()), *wants[i]));
    for (int i = 0; i < 4; ++i)
      CHECK(close(Download<float>(ex, parameters[i]->gradient().data(), dparam[i].size()), dparam[i]));
  }
  DeltaNetParameters bad = e.p;
  bad.value_heads = vh + 1;   // not a multiple of the key heads (or a parameter size mismatch)
  CHECK(!SequenceDeltaNetLayer::Create(ex, bad, parameters[0], parameters[1], parameters[2], parameters[3], length).ok());
  std::printf("ok SequenceDeltaNetLayer + DeltaNetLayer (%d,%d,%d,%d,%d)%s\n", length, kh, vh, kd, vd,
              gradients ? " with gradients" : "");
}

int main() {
  auto executor = cuda::Executor::Create();
  CHECK(executor.ok());
  cuda::Executor& ex = **executor;
  auto other = cuda::Executor::Create();
  CHECK(other.ok());
  TestAttentionLayer(ex, false);
  TestAttentionLayer(ex, true);
  {  // a layer bound to one Executor rejects work submitted through another
    auto layer = AttentionLayer::Create(ex, 4, 2, 32, DataType::FP16);
    auto input = cuda::Buffer::Allocate(**other, 4 * 96 * 4);
    CHECK(layer.ok() && input.ok());
    CHECK(!(*layer)->fwd(**other, {*input}).ok());
    CHECK(!(*layer)->fwd(ex, {*input}).ok());
  }
  for (int dim : {6, 128, 256})
    for (bool round : {false, true}) TestCachedAttention(ex, dim, round);
  for (int dim : {5, 128})
    for (bool round : {false, true}) TestDeltaNetState(ex, dim, round);
  for (int d : {3, 256}) TestQwenAttentionForward(ex, d);
  TestQwenAttentionBackward(ex);
  TestSequenceDeltaNet(ex, 3, 1, 2, 3, 5, false);
  TestSequenceDeltaNet(ex, 3, 2, 4, 5, 35, false);
  TestSequenceDeltaNet(ex, 3, 16, 48, 128, 128, false);
  TestSequenceDeltaNet(ex, 5, 1, 2, 3, 5, true);
  TestSequenceDeltaNet(ex, 3, 2, 4, 5, 35, true);
  CHECK_OK(ex.Synchronize());
  std::printf("PASS %d checks\n", g_checks);
  return 0;
}
