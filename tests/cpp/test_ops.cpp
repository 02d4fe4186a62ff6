// C++ parity test through the header-only class layer (include/vkllama/vkllama.h), written
// the way the reference's own tests are (tests/test_rmsnorm.cpp, test_feedforward.cpp,
// test_embedding.cpp): build GPUDevice + Command, upload, run the op, download, compare —
// here against the CPU oracle (liboracle.so) instead of Eigen expressions.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "vkllama/vkllama.h"

extern "C" {
void orc_synth_normal_f32(uint64_t, uint64_t, uint64_t, uint64_t, float, float, float *);
void orc_synth_normal_f16(uint64_t, uint64_t, uint64_t, uint64_t, float, float, uint16_t *);
void orc_synth_q8_0(uint64_t, uint64_t, uint64_t, uint64_t, float, float, uint8_t *);
void orc_rms_norm_f16(const uint16_t *, const float *, uint16_t *, uint32_t, uint32_t, float);
void orc_feed_forward_q8_0(const uint16_t *, const uint8_t *, const uint8_t *, const uint8_t *, uint16_t *, uint32_t, uint32_t, uint32_t);
void *orc_model_create(uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, float, float);
void orc_model_synth(void *, uint64_t, float, float);
const void *orc_model_weight(void *, uint32_t, uint32_t, uint64_t *);
void orc_model_forward(void *, const uint32_t *, uint32_t, uint32_t, float *, uint16_t *);
void orc_model_destroy(void *);
}

using namespace vkllama;

static float h2f(uint16_t u) {
  _Float16 h;
  memcpy(&h, &u, 2);
  return (float)h;
}
static double max_rel(const std::vector<uint16_t> &a, const std::vector<uint16_t> &b) {
  double err = 0, ref = 1e-30;
  for (size_t i = 0; i < a.size(); ++i) {
    err = std::max(err, (double)std::fabs(h2f(a[i]) - h2f(b[i])));
    ref = std::max(ref, (double)std::fabs(h2f(b[i])));
  }
  return err / ref;
}
#define CHECK_OK(expr)                                                  \
  do {                                                                  \
    auto s__ = (expr);                                                  \
    if (!s__.ok()) {                                                    \
      fprintf(stderr, "%s failed: %s\n", #expr, s__.ToString().c_str()); \
      return 1;                                                         \
    }                                                                   \
  } while (0)

int main() {
  GPUDevice gpu(0);
  CHECK_OK(gpu.init());
  Command cmd(&gpu);
  CHECK_OK(cmd.init());
  int failures = 0;

  {  // RMSNorm, tests/test_rmsnorm.cpp shape [1,1,128] and a 7B row
    for (uint32_t W : {128u, 4096u}) {
      std::vector<uint16_t> x(W), want(W), got(W);
      std::vector<float> w(W);
      orc_synth_normal_f16(1, 1, 0, W, 0.f, 1.f, x.data());
      orc_synth_normal_f32(1, 2, 0, W, 1.f, 0.01f, w.data());
      orc_rms_norm_f16(x.data(), w.data(), want.data(), 1, W, 1e-3f);
      CHECK_OK(cmd.begin());
      Tensor tx(1, 1, W, &gpu, FP16), tw(1, 1, W, &gpu, FP32);
      CHECK_OK(tx.create());
      CHECK_OK(cmd.upload(x.data(), x.size(), tx));
      CHECK_OK(cmd.upload(w.data(), w.size(), tw));
      RMSNorm op(&gpu, &cmd, tw, 1e-3f, FP16);
      CHECK_OK(op.init());
      auto out = op(tx);
      CHECK_OK(out.status().ok() ? absl::OkStatus() : out.status());
      CHECK_OK(cmd.download(*out, got.data(), got.size()));
      CHECK_OK(cmd.end());
      CHECK_OK(cmd.submit_and_wait());
      const double r = max_rel(got, want);
      printf("rms_norm W=%u max-rel %.2e\n", W, r);
      failures += r > 2e-3;
      RMSNorm bad(&gpu, &cmd, tx, 1e-3f, FP16);  // weight must be FP32 (rms_norm.cpp:33)
      failures += bad.init().ok();
    }
  }
  {  // FeedForward Q8_0, tests/test_feedforward.cpp:143-148 shapes and the 7B shape
    struct S { uint32_t M, dim, hidden; };
    for (S s : {S{64, 32, 256}, S{1, 4096, 11008}}) {
      const size_t qg = (size_t)s.hidden * (s.dim / 32) * 34, qd = (size_t)s.dim * (s.hidden / 32) * 34;
      std::vector<uint8_t> gate(qg), up(qg), down(qd);
      std::vector<uint16_t> x((size_t)s.M * s.dim), want((size_t)s.M * s.dim), got((size_t)s.M * s.dim);
      orc_synth_q8_0(2, 1, s.hidden, s.dim, 0.f, 0.02f, gate.data());
      orc_synth_q8_0(2, 2, s.dim, s.hidden, 0.f, 0.02f, down.data());
      orc_synth_q8_0(2, 3, s.hidden, s.dim, 0.f, 0.02f, up.data());
      orc_synth_normal_f16(2, 4, 0, x.size(), 0.f, 1.f, x.data());
      orc_feed_forward_q8_0(x.data(), gate.data(), down.data(), up.data(), want.data(), s.M, s.dim, s.hidden);
      CHECK_OK(cmd.begin());
      Tensor w1(1, s.hidden, s.dim, &gpu, Q8_0), w2(1, s.dim, s.hidden, &gpu, Q8_0), w3(1, s.hidden, s.dim, &gpu, Q8_0), tx(1, s.M, s.dim, &gpu, FP16);
      CHECK_OK(cmd.upload(gate.data(), gate.size(), w1));
      CHECK_OK(cmd.upload(down.data(), down.size(), w2));
      CHECK_OK(cmd.upload(up.data(), up.size(), w3));
      CHECK_OK(cmd.upload(x.data(), x.size(), tx));
      FeedForward op(&gpu, &cmd, w1, w2, w3, true, Q8_0);
      CHECK_OK(op.init());
      auto out = op(tx);
      CHECK_OK(out.status().ok() ? absl::OkStatus() : out.status());
      CHECK_OK(cmd.download(*out, got.data(), got.size()));
      CHECK_OK(cmd.end());
      CHECK_OK(cmd.submit_and_wait());
      const double r = max_rel(got, want);
      printf("feed_forward M=%u dim=%u hidden=%u max-rel %.2e, op time %llu us\n", s.M, s.dim, s.hidden, r, (unsigned long long)op.time());
      failures += r > 1e-2;
    }
  }
  {  // Model::init by tensor name + Model::operator() (models/llama2.h:348-843)
    const uint32_t dim = 256, heads = 4, ffn = 512, vocab = 1000, layers = 2, maxlen = 64;
    void *om = orc_model_create(dim, heads, ffn, vocab, layers, maxlen, 1e-5f, 1e-6f);
    orc_model_synth(om, 21, 0.02f, 0.01f);
    Model model(0);
    ModelConfig c;
    c.dim = dim; c.head_count = heads; c.ffn = ffn; c.vocab = vocab; c.block_count = layers; c.context_length = maxlen;
    CHECK_OK(model.init(c));
    const char *names[9] = {"attn_norm", "attn_q", "attn_k", "attn_v", "attn_output", "ffn_norm", "ffn_gate", "ffn_up", "ffn_down"};
    for (uint32_t l = 0; l < layers; ++l)
      for (uint32_t s = 0; s < 9; ++s) {
        uint64_t n = 0;
        const void *p = orc_model_weight(om, l, s, &n);
        char nm[64];
        snprintf(nm, sizeof(nm), "blk.%u.%s.weight", l, names[s]);
        CHECK_OK(model.load_tensor(nm, (s == 0 || s == 5) ? 0 : 8, p, n));
      }
    const char *gn[3] = {"token_embd.weight", "output_norm.weight", "output.weight"};
    for (uint32_t s = 0; s < 3; ++s) {
      uint64_t n = 0;
      const void *p = orc_model_weight(om, layers, s, &n);
      CHECK_OK(model.load_tensor(gn[s], s == 1 ? 0 : 8, p, n));
    }
    std::vector<uint32_t> toks = {5, 17, 900, 3, 42};
    std::vector<float> want(vocab);
    orc_model_forward(om, toks.data(), (uint32_t)toks.size(), 0, want.data(), nullptr);
    auto got = model(toks, 0);
    CHECK_OK(got.status().ok() ? absl::OkStatus() : got.status());
    double err = 0;
    for (uint32_t i = 0; i < vocab; ++i) err = std::max(err, (double)std::fabs((*got)[i] - want[i]));
    printf("model prefill logits max-abs %.2e\n", err);
    failures += err > 5e-2;
    std::vector<uint32_t> one = {7};
    orc_model_forward(om, one.data(), 1, 5, want.data(), nullptr);
    got = model(one, 5);
    err = 0;
    for (uint32_t i = 0; i < vocab; ++i) err = std::max(err, (double)std::fabs((*got)[i] - want[i]));
    printf("model decode logits max-abs %.2e\n", err);
    failures += err > 5e-2;
    orc_model_destroy(om);
  }
  printf(failures ? "FAIL (%d)\n" : "PASS\n", failures);
  return failures ? 1 : 0;
}
