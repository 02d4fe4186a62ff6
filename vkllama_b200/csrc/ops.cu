// Operator layer behind the C ABI: argument and dtype checks, output
// allocation and kernel selection. Mirrors src/ops of the reference op by op
// (same constructor arguments, same checks and status categories); the bodies
// launch CUDA kernels on the command's stream instead of recording Vulkan
// dispatches.
#include <math.h>

#include <algorithm>
#include <cmath>

#include "runtime.h"

using namespace vkl;

struct vkl_op {
  vkl_device *dev;
  vkl_command *cmd;
  bool inited = false;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  bool timed = false;
  vkl_op(vkl_device *d, vkl_command *c) : dev(d), cmd(c) {}
  virtual int init() = 0;
  virtual ~vkl_op() {
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
  }
  int base_init() {
    if (!dev || !cmd) return fail(VKL_INVALID_ARGUMENT, "op: null device or command");
    VKL_CUDA(cudaEventCreate(&e0));
    VKL_CUDA(cudaEventCreate(&e1));
    inited = true;
    return VKL_OK;
  }
  int enter(const char *who) {
    if (!inited) return fail(VKL_FAILED_PRECONDITION, "%s: init() was not called", who);
    VKL_OKAY(recording(cmd, who));
    VKL_CUDA(cudaEventRecord(e0, cmd->stream));
    return VKL_OK;
  }
  int leave() {
    VKL_CUDA(cudaEventRecord(e1, cmd->stream));
    timed = true;
    return VKL_OK;
  }
};

namespace {

int need_dense(const vkl_tensor *t, const char *who) {
  if (!t) return fail(VKL_INVALID_ARGUMENT, "%s: null tensor", who);
  if (!t->dense()) return fail(VKL_UNIMPLEMENTED, "%s: strided views are not supported by this op", who);
  return VKL_OK;
}

// -------------------------------------------------------------------- MatMul
struct MatMulOp : vkl_op {
  vkl_tensor *weight;
  float scale, bias;
  int act, broadcast_type, transpose_b, a_dtype, b_dtype;
  vkl_tensor *out = nullptr;
  MatMulOp(vkl_device *d, vkl_command *c, vkl_tensor *w, float s, float b, int act_, int bt, int tb, int ad, int bd)
      : vkl_op(d, c), weight(w), scale(s), bias(b), act(act_), broadcast_type(bt), transpose_b(tb), a_dtype(ad), b_dtype(bd) {
    if (weight) vkl_tensor_retain(weight);
  }
  ~MatMulOp() override {
    vkl_tensor_release(weight);
    vkl_tensor_release(out);
  }
  // src/ops/mat_mul.cpp:34-151
  int init() override {
    if (weight && weight->size() > 0 && weight->dtype != b_dtype)
      return fail(VKL_INVALID_ARGUMENT, "matmul operator defined as %d b_dtype but dtype of weight tensor is %d", b_dtype, weight->dtype);
    if (broadcast_type < 0 || broadcast_type > 2)
      return fail(VKL_INVALID_ARGUMENT, "broadcast_type %d is unsupported.", broadcast_type);
    const bool ok = (a_dtype == VKL_FP16 && b_dtype == VKL_FP16) || (a_dtype == VKL_FP16 && b_dtype == VKL_Q8_0 && transpose_b);
    if (!ok) return fail(VKL_INVALID_ARGUMENT, "%d a_dtype and %d b_dtype is unsupported", a_dtype, b_dtype);
    return base_init();
  }
  // src/ops/mat_mul.cpp:160-228 (weight form)
  int run_weight(vkl_tensor *a, vkl_tensor **o) {
    if (!weight || weight->size() == 0 || !a || a->dtype != a_dtype)
      return fail(VKL_INVALID_ARGUMENT, "matmul op defined with %d a dtype but %d given.", a_dtype, a ? a->dtype : -1);
    // src/ops/mat_mul.cpp:117-124, 246-254: 0 = operands pair up channel by channel, 1 = one B for every channel of A,
    // 2 = one A for every channel of B
    if ((broadcast_type == 0 && weight->c != a->c) || (broadcast_type == 1 && weight->c != 1) || (broadcast_type == 2 && a->c != 1))
      return fail(VKL_INVALID_ARGUMENT, "matmul op defined with broadcast_type = %d but weight channels = %zu != a.channels = %zu", broadcast_type, weight->c, a->c);
    VKL_OKAY(need_dense(a, "matmul"));
    if (broadcast_type != 0 && (weight->c != 1 || a->c != 1)) {
      if (b_dtype != VKL_FP16) return fail(VKL_UNIMPLEMENTED, "matmul: batched Q8_0 weights are not supported");
      const size_t Kb = transpose_b ? weight->w : weight->h, Nb = transpose_b ? weight->h : weight->w, Cb = std::max(a->c, weight->c);
      if (a->w != Kb) return fail(VKL_INVALID_ARGUMENT, "matmul: a.width = %zu but the weight expects %zu", a->w, Kb);
      VKL_OKAY(enter("matmul"));
      VKL_OKAY(ensure_tensor(dev, &out, Cb, a->h, Nb, VKL_FP16));
      VKL_LAUNCH(1, launch_bmm_f16((const __half *)a->data(), (const __half *)weight->data(), (__half *)out->data(), (uint32_t)Cb, (uint32_t)a->h,
                                   (uint32_t)Nb, (uint32_t)Kb, a->c == 1 ? 0 : a->cs / 2, a->hs / 2, weight->c == 1 ? 0 : weight->cs / 2,
                                   weight->hs / 2, out->cs / 2, out->hs / 2, transpose_b, scale, bias, act, cmd->stream));
      *o = out;
      return leave();
    }
    const size_t K = transpose_b ? weight->w : weight->h, N = transpose_b ? weight->h : weight->w;
    if (a->w != K) return fail(VKL_INVALID_ARGUMENT, "matmul: a.width = %zu but the weight expects %zu", a->w, K);
    VKL_OKAY(enter("matmul"));
    VKL_OKAY(ensure_tensor(dev, &out, a->c, a->h, N, VKL_FP16));
    if (transpose_b && a->c == 1) {
      MvParams p = {};
      p.codes[0] = weight->data();
      p.scales[0] = b_dtype == VKL_Q8_0 ? weight->scales() : nullptr;
      p.out[0] = (__half *)out->data();
      p.x = (const __half *)a->data();
      p.nmat = 1;
      p.N = (uint32_t)N; p.K = (uint32_t)K; p.M = (uint32_t)a->h;
      p.x_ld = (uint32_t)K; p.out_ld = (uint32_t)N;
      p.scale = scale; p.bias = bias; p.act = act;
      p.fp16_weights = b_dtype == VKL_FP16;
      if (a->h >= gemm_min_rows(!p.fp16_weights) && gemm_tcgen05_supported((uint32_t)a->h, (uint32_t)N, (uint32_t)K)) {
        // many rows: one pass over the weights on the tcgen05 tensor cores (Q8_0 dequantised on the way in)
        GemmParams g = {};
        g.a = (const __half *)a->data(); g.c = (__half *)out->data();
        if (p.fp16_weights) {
          g.w = (const __half *)weight->data();
        } else {
          g.w_codes = weight->codes();
          g.w_scales = weight->scales();
        }
        g.M = (uint32_t)a->h; g.N = (uint32_t)N; g.K = (uint32_t)K;
        g.scale = scale; g.bias = bias; g.act = act;
        VKL_OKAY(command_error_word(cmd, &g.error));
        VKL_LAUNCH(1, launch_gemm_tcgen05(g, cmd->stream));
      } else if (p.fp16_weights && (K & 7)) {
        VKL_LAUNCH(1, launch_bmm_f16((const __half *)a->data(), (const __half *)weight->data(), (__half *)out->data(), 1,
                                     (uint32_t)a->h, (uint32_t)N, (uint32_t)K, 0, K, 0, K, 0, N, 1, scale, bias, act, cmd->stream));
      } else {
        VKL_LAUNCH((a->h + 63) / 64, launch_matvec(p, EPI_PLAIN, false, cmd->stream));
      }
    } else {
      if (b_dtype != VKL_FP16) return fail(VKL_UNIMPLEMENTED, "matmul: batched Q8_0 weights are not supported");
      VKL_LAUNCH(1, launch_bmm_f16((const __half *)a->data(), (const __half *)weight->data(), (__half *)out->data(), (uint32_t)a->c,
                                   (uint32_t)a->h, (uint32_t)N, (uint32_t)K, a->cs / 2, a->hs / 2, weight->cs / 2, weight->hs / 2,
                                   out->cs / 2, out->hs / 2, transpose_b, scale, bias, act, cmd->stream));
    }
    *o = out;
    return leave();
  }
  // src/ops/mat_mul.cpp:230-291 (two-operand form; operands may be strided views)
  int run_pair(vkl_tensor *a, vkl_tensor *b, vkl_tensor **o) {
    if (!a || !b || b->size() == 0 || a->dtype != a_dtype || b->dtype != b_dtype)
      return fail(VKL_INVALID_ARGUMENT, "matmul op defined with %d a_dtype and %d b_dtype but inputs a.dtype() = %d, b.dtype() = %d", a_dtype,
                  b_dtype, a ? a->dtype : -1, b ? b->dtype : -1);
    if ((broadcast_type == 0 && b->c != a->c) || (broadcast_type == 1 && b->c != 1) || (broadcast_type == 2 && a->c != 1))
      return fail(VKL_INVALID_ARGUMENT, "matmul defined with %d broadcast_type but a.channels() = %zu, b.channels() = %zu", broadcast_type, a->c, b->c);
    if (b_dtype != VKL_FP16) return fail(VKL_UNIMPLEMENTED, "matmul: the two-operand form takes FP16 operands");
    const size_t K = a->w, N = transpose_b ? b->h : b->w, C = std::max(a->c, b->c);
    if ((transpose_b ? b->w : b->h) != K) return fail(VKL_INVALID_ARGUMENT, "matmul: inner extents differ (%zu vs %zu)", K, transpose_b ? b->w : b->h);
    VKL_OKAY(enter("matmul"));
    VKL_OKAY(ensure_tensor(dev, &out, C, a->h, N, VKL_FP16));
    // a broadcast operand (src/shaders/matmul_broadcast1_fp16_v2.comp, matmul_broadcast2_fp16_v2.comp) is a channel stride of 0
    VKL_LAUNCH(1, launch_bmm_f16((const __half *)a->data(), (const __half *)b->data(), (__half *)out->data(), (uint32_t)C, (uint32_t)a->h,
                                 (uint32_t)N, (uint32_t)K, broadcast_type == 2 ? 0 : a->cs / 2, a->hs / 2, broadcast_type == 1 ? 0 : b->cs / 2,
                                 b->hs / 2, out->cs / 2, out->hs / 2, transpose_b, scale, bias, act, cmd->stream));
    *o = out;
    return leave();
  }
};

// --------------------------------------------------------------- FeedForward
struct FeedForwardOp : vkl_op {
  vkl_tensor *w1, *w2, *w3;  // gate, down, up
  int transposed_weight, dtype;
  vkl_tensor *t0 = nullptr, *out = nullptr, *gu32 = nullptr;
  FeedForwardOp(vkl_device *d, vkl_command *c, vkl_tensor *a, vkl_tensor *b, vkl_tensor *e, int tw, int dt)
      : vkl_op(d, c), w1(a), w2(b), w3(e), transposed_weight(tw), dtype(dt) {
    vkl_tensor_retain(w1); vkl_tensor_retain(w2); vkl_tensor_retain(w3);
  }
  ~FeedForwardOp() override {
    vkl_tensor_release(w1); vkl_tensor_release(w2); vkl_tensor_release(w3);
    vkl_tensor_release(t0); vkl_tensor_release(out); vkl_tensor_release(gu32);
  }
  // src/ops/feed_forward.cpp:24-68
  int init() override {
    if (dtype != VKL_FP16 && dtype != VKL_Q8_0) return fail(VKL_INVALID_ARGUMENT, "FeedForward op: only fp16 and q8_0 are supported.");
    if (!w1 || !w2 || !w3) return fail(VKL_INVALID_ARGUMENT, "FeedForward op: null weight");
    if (w1->dtype != w2->dtype || w2->dtype != w3->dtype || dtype != w1->dtype)
      return fail(VKL_INVALID_ARGUMENT, "feed_forward op defined with %d dtype but w1.dtype = %d, w2.dtype = %d, w3.dtype = %d", dtype, w1->dtype, w2->dtype, w3->dtype);
    // The up/gate kernel reads weights as [N,K] whatever transposed_weight says
    // (ffn_up_and_gate_q8_0.comp:49-52); the down MatMul honours it.
    if (!transposed_weight) return fail(VKL_UNIMPLEMENTED, "FeedForward op: weights must be [out,in] (transposed_weight = true), as the model driver passes them");
    if (w1->h != w3->h || w1->w != w3->w || w2->w != w1->h || w1->c != 1 || w2->c != 1 || w3->c != 1)
      return fail(VKL_INVALID_ARGUMENT, "FeedForward op: weight shapes do not chain");
    if (dtype == VKL_FP16 && ((w1->w & 7) || (w2->w & 7))) return fail(VKL_UNIMPLEMENTED, "FeedForward op: FP16 widths must be multiples of 8");
    return base_init();
  }
  // src/ops/feed_forward.cpp:88-133
  int run(vkl_tensor *x, vkl_tensor **o) {
    if (!x || x->dtype != VKL_FP16)
      return fail(VKL_INVALID_ARGUMENT, "feed_forward op defined with FP16 input but input X.dtype() = %d", x ? x->dtype : -1);
    VKL_OKAY(need_dense(x, "feed_forward"));
    if (x->c != 1 || x->w != w1->w) return fail(VKL_INVALID_ARGUMENT, "feed_forward: input shape (%zu, %zu, %zu) does not match the weights", x->c, x->h, x->w);
    VKL_OKAY(enter("feed_forward"));
    VKL_OKAY(ensure_tensor(dev, &t0, x->c, x->h, w1->h, VKL_FP16));
    VKL_OKAY(ensure_tensor(dev, &out, x->c, x->h, w2->h, VKL_FP16));
    const bool q8 = dtype == VKL_Q8_0;
    if (x->h >= gemm_min_rows(q8) && gemm_tcgen05_supported((uint32_t)x->h, (uint32_t)w1->h, (uint32_t)w1->w) &&
        gemm_tcgen05_supported((uint32_t)x->h, (uint32_t)w2->h, (uint32_t)w2->w)) {
      // many rows: gate and up as tensor-core GEMMs with raw fp32 results, SwiGLU on those
      // (the rounding points of ffn_up_and_gate_fp16.comp), then the down GEMM
      VKL_OKAY(ensure_tensor(dev, &gu32, 2, x->h, w1->h, VKL_FP32));
      auto weight_of = [q8](GemmParams &gp, const vkl_tensor *w) {
        gp.w = q8 ? nullptr : (const __half *)w->data();
        gp.w_codes = q8 ? w->codes() : nullptr;
        gp.w_scales = q8 ? w->scales() : nullptr;
      };
      GemmParams g = {};
      g.a = (const __half *)x->data(); g.c_f32 = (float *)gu32->data();
      weight_of(g, w1);
      g.M = (uint32_t)x->h; g.N = (uint32_t)w1->h; g.K = (uint32_t)w1->w;
      g.scale = 1.f;
      VKL_OKAY(command_error_word(cmd, &g.error));
      VKL_LAUNCH(1, launch_gemm_tcgen05(g, cmd->stream));
      weight_of(g, w3);
      g.c_f32 += (size_t)x->h * w1->h;
      VKL_LAUNCH(1, launch_gemm_tcgen05(g, cmd->stream));
      VKL_LAUNCH(1, launch_swiglu_f32((const float *)gu32->data(), (const float *)gu32->data() + (size_t)x->h * w1->h, (__half *)t0->data(),
                                      (size_t)x->h * w1->h, cmd->stream));
      GemmParams d = {};
      d.a = (const __half *)t0->data(); d.c = (__half *)out->data();
      weight_of(d, w2);
      d.M = (uint32_t)x->h; d.N = (uint32_t)w2->h; d.K = (uint32_t)w2->w;
      d.scale = 1.f; d.error = g.error;
      VKL_LAUNCH(1, launch_gemm_tcgen05(d, cmd->stream));
      *o = out;
      return leave();
    }
    MvParams p = {};
    p.codes[0] = w1->data(); p.codes[1] = w3->data();
    p.scales[0] = q8 ? w1->scales() : nullptr; p.scales[1] = q8 ? w3->scales() : nullptr;
    p.out[0] = (__half *)t0->data();
    p.x = (const __half *)x->data();
    p.nmat = 1;
    p.N = (uint32_t)w1->h; p.K = (uint32_t)w1->w; p.M = (uint32_t)x->h;
    p.x_ld = p.K; p.out_ld = p.N;
    p.scale = 1.f; p.fp16_weights = !q8;
    VKL_LAUNCH((x->h + 63) / 64, launch_matvec(p, EPI_SWIGLU, false, cmd->stream));
    MvParams d = {};
    d.codes[0] = w2->data(); d.scales[0] = q8 ? w2->scales() : nullptr;
    d.out[0] = (__half *)out->data();
    d.x = (const __half *)t0->data();
    d.nmat = 1;
    d.N = (uint32_t)w2->h; d.K = (uint32_t)w2->w; d.M = (uint32_t)x->h;
    d.x_ld = d.K; d.out_ld = d.N;
    d.scale = 1.f; d.fp16_weights = !q8;
    VKL_LAUNCH((x->h + 63) / 64, launch_matvec(d, EPI_PLAIN, false, cmd->stream));
    *o = out;
    return leave();
  }
};

// ------------------------------------------------------------- rope tables
// src/ops/rope.cpp:19-47: freq_k = 1/pow(10000, 2k/dim) in fp32, angle =
// freq_k*float(pos), std::cos/std::sin on float. Computed on the host exactly
// like the reference and uploaded.
int make_rope_tables(vkl_device *dev, cudaStream_t s, int dim, int rows, vkl_tensor **fc, vkl_tensor **fs) {
  std::vector<float> freq(dim / 2), c((size_t)rows * dim / 2), si((size_t)rows * dim / 2);
  float n = .0f;
  for (int k = 0; k < dim / 2; ++k) {
    freq[k] = 1.0f / std::pow(10000.0f, n / dim);
    n += 2.0;
  }
  for (int i = 0; i < rows; ++i)
    for (int k = 0; k < dim / 2; ++k) {
      const float f = freq[k] * static_cast<float>(i);
      c[(size_t)i * (dim / 2) + k] = std::cos(f);
      si[(size_t)i * (dim / 2) + k] = std::sin(f);
    }
  VKL_OKAY(tensor_new(dev, 1, rows, dim / 2, VKL_FP32, fc));
  VKL_OKAY(tensor_new(dev, 1, rows, dim / 2, VKL_FP32, fs));
  VKL_CUDA(cudaMemcpyAsync((*fc)->data(), c.data(), c.size() * 4, cudaMemcpyHostToDevice, s));
  VKL_CUDA(cudaMemcpyAsync((*fs)->data(), si.data(), si.size() * 4, cudaMemcpyHostToDevice, s));
  VKL_CUDA(cudaStreamSynchronize(s));
  return VKL_OK;
}

__global__ void set_u32_kernel(uint32_t *p, uint32_t v) { *p = v; }

// ---------------------------------------------------------------------- MHA
struct MhaOp : vkl_op {
  vkl_tensor *wk, *wq, *wv, *wo;
  int maxlen, dim, transposed_weight, dtype, use_kvcache, clip_output;
  vkl_tensor *k = nullptr, *q = nullptr, *v = nullptr, *heads_out = nullptr, *out = nullptr;
  vkl_tensor *kcache = nullptr, *vcache = nullptr, *fc = nullptr, *fs = nullptr;
  vkl_tensor *scratch = nullptr, *counters = nullptr, *pos = nullptr;
  uint32_t splits = 1;
  MhaOp(vkl_device *d, vkl_command *c, vkl_tensor *a, vkl_tensor *b, vkl_tensor *e, vkl_tensor *f, int ml, int dm, int tw, int dt, int kv, int clip)
      : vkl_op(d, c), wk(a), wq(b), wv(e), wo(f), maxlen(ml), dim(dm), transposed_weight(tw), dtype(dt), use_kvcache(kv), clip_output(clip) {
    vkl_tensor_retain(wk); vkl_tensor_retain(wq); vkl_tensor_retain(wv); vkl_tensor_retain(wo);
  }
  ~MhaOp() override {
    for (vkl_tensor *t : {wk, wq, wv, wo, k, q, v, heads_out, out, kcache, vcache, fc, fs, scratch, counters, pos}) vkl_tensor_release(t);
  }
  // src/ops/multiheadattention_v2.cpp:33-136
  int init() override {
    if (dtype != VKL_FP16) return fail(VKL_INVALID_ARGUMENT, "MultiHeadAttentionV2: only fp16 dtype is supported.");
    if (!wk || !wq || !wv || !wo) return fail(VKL_INVALID_ARGUMENT, "MultiHeadAttentionV2: null weight");
    if (wk->c != wq->c || wk->h != wq->h || wk->w != wq->w || wq->c != wv->c || wq->w != wv->w || wq->h != wv->h)
      return fail(VKL_INVALID_ARGUMENT, "shape of weights error wk.shape = (%zu, %zu, %zu), wq.shape = (%zu, %zu, %zu), wv.shape = (%zu, %zu, %zu), wo.shape = (%zu, %zu, %zu)",
                  wk->c, wk->h, wk->w, wq->c, wq->h, wq->w, wv->c, wv->h, wv->w, wo->c, wo->h, wo->w);
    // The KQV kernel of the reference is hard-wired to Q8_0 [out,in] weights
    // (multiheadattention_v2.cpp:55-61); FP16 weights are accepted here too.
    if (!transposed_weight) return fail(VKL_UNIMPLEMENTED, "MultiHeadAttentionV2: weights must be [out,in] (transposed_weight = true)");
    if (wk->dtype != wq->dtype || wq->dtype != wv->dtype || wv->dtype != wo->dtype || (wk->dtype != VKL_Q8_0 && wk->dtype != VKL_FP16))
      return fail(VKL_INVALID_ARGUMENT, "MultiHeadAttentionV2: weights must all be Q8_0 or all FP16");
    if (dim <= 0 || dim > 128 || (dim & 7) || wk->h % dim) return fail(VKL_INVALID_ARGUMENT, "MultiHeadAttentionV2: head dim %d is unsupported for width %zu", dim, wk->h);
    if (!use_kvcache) return fail(VKL_UNIMPLEMENTED, "MultiHeadAttentionV2: use_kvcache = false has no caller on the Llama-2 path and is not built");
    if (maxlen <= 0) return fail(VKL_INVALID_ARGUMENT, "MultiHeadAttentionV2: maxlen must be positive");
    VKL_OKAY(base_init());
    const size_t heads = wk->h / dim;
    VKL_OKAY(tensor_new(dev, heads, maxlen, dim, VKL_FP16, &kcache));
    VKL_OKAY(tensor_new(dev, heads, maxlen, dim, VKL_FP16, &vcache));
    VKL_CUDA(cudaMemsetAsync(kcache->data(), 0, kcache->device_bytes(), cmd->stream));
    VKL_CUDA(cudaMemsetAsync(vcache->data(), 0, vcache->device_bytes(), cmd->stream));
    VKL_OKAY(make_rope_tables(dev, cmd->stream, dim, 2 * maxlen, &fc, &fs));
    splits = 4;
    VKL_OKAY(tensor_new(dev, 1, 1, heads * 4, VKL_UINT32, &counters));
    VKL_CUDA(cudaMemsetAsync(counters->data(), 0, counters->device_bytes(), cmd->stream));
    VKL_OKAY(tensor_new(dev, 1, 1, 1, VKL_UINT32, &pos));
    return VKL_OK;
  }
  // src/ops/multiheadattention_v2.cpp:140-325
  int run(vkl_tensor *X, size_t offset, vkl_tensor **o) {
    if (!X || X->dtype != dtype)
      return fail(VKL_INVALID_ARGUMENT, "multiheadattention op defined with %d dtype but input0's dtype = %d", dtype, X ? X->dtype : -1);
    if (wv->w != X->w)
      return fail(VKL_INVALID_ARGUMENT, "shape error. wv.shape = (%zu, %zu, %zu), input0.shape = (%zu, %zu, %zu)", wv->c, wv->h, wv->w, X->c, X->h, X->w);
    VKL_OKAY(need_dense(X, "multiheadattention"));
    if (X->c != 1) return fail(VKL_INVALID_ARGUMENT, "multiheadattention: input channels must be 1");
    const size_t T = X->h, Wd = wk->h, heads = Wd / dim;
    if (T == 0) return fail(VKL_INVALID_ARGUMENT, "multiheadattention: empty input");
    if (offset + T > (size_t)2 * maxlen) return fail(VKL_OUT_OF_RANGE, "multiheadattention: position %zu is beyond the RoPE table (2*maxlen = %d)", offset + T, 2 * maxlen);
    if (T > (size_t)maxlen) return fail(VKL_OUT_OF_RANGE, "multiheadattention: %zu rows exceed maxlen %d", T, maxlen);
    VKL_OKAY(enter("multiheadattention"));
    VKL_OKAY(ensure_tensor(dev, &k, 1, T, Wd, VKL_FP16));
    VKL_OKAY(ensure_tensor(dev, &q, 1, T, Wd, VKL_FP16));
    VKL_OKAY(ensure_tensor(dev, &v, 1, T, Wd, VKL_FP16));
    const size_t To = clip_output ? 1 : T;
    VKL_OKAY(ensure_tensor(dev, &heads_out, 1, To, Wd, VKL_FP16));
    VKL_OKAY(ensure_tensor(dev, &out, 1, To, wo->h, VKL_FP16));
    const bool q8 = wk->dtype == VKL_Q8_0;
    MvParams p = {};
    p.codes[0] = wk->data(); p.codes[1] = wq->data(); p.codes[2] = wv->data();
    if (q8) { p.scales[0] = wk->scales(); p.scales[1] = wq->scales(); p.scales[2] = wv->scales(); }
    p.out[0] = (__half *)k->data(); p.out[1] = (__half *)q->data(); p.out[2] = (__half *)v->data();
    p.x = (const __half *)X->data();
    p.nmat = 3;
    p.N = (uint32_t)Wd; p.K = (uint32_t)wk->w; p.M = (uint32_t)T;
    p.x_ld = p.K; p.out_ld = p.N; p.scale = 1.f; p.fp16_weights = !q8;
    VKL_LAUNCH((T + 63) / 64, launch_matvec(p, EPI_PLAIN, false, cmd->stream));

    const uint32_t sp = T == 1 ? splits : 1;
    const size_t need = attention_scratch_bytes((uint32_t)To, (uint32_t)heads, dim, sp);
    if (!scratch || scratch->device_bytes() < need) {
      vkl_tensor_release(scratch);
      scratch = nullptr;
      VKL_OKAY(tensor_new(dev, 1, 1, need / 4, VKL_FP32, &scratch));
    }
    set_u32_kernel<<<1, 1, 0, cmd->stream>>>((uint32_t *)pos->data(), (uint32_t)offset);
    VKL_LAUNCH(1, cudaGetLastError());
    AttnParams a = {};
    a.q = (__half *)q->data(); a.k = (const __half *)k->data(); a.v = (const __half *)v->data();
    a.kcache = (__half *)kcache->data(); a.vcache = (__half *)vcache->data();
    a.out = (__half *)heads_out->data();
    a.freqc = (const float *)fc->data(); a.freqs = (const float *)fs->data();
    a.pos_dev = (const uint32_t *)pos->data();
    a.scratch = (float *)scratch->data(); a.counters = (uint32_t *)counters->data();
    a.T = (uint32_t)T; a.heads = (uint32_t)heads; a.dim = dim; a.maxlen = maxlen; a.splits = sp;
    a.clip = clip_output ? 1 : 0;
    VKL_LAUNCH(T > 1 ? 2 : 1, launch_attention(a, cmd->stream));

    MvParams w = {};
    w.codes[0] = wo->data(); w.scales[0] = q8 ? wo->scales() : nullptr;
    w.out[0] = (__half *)out->data();
    w.x = (const __half *)heads_out->data();
    w.nmat = 1;
    w.N = (uint32_t)wo->h; w.K = (uint32_t)wo->w; w.M = (uint32_t)To;
    w.x_ld = w.K; w.out_ld = w.N; w.scale = 1.f; w.fp16_weights = !q8;
    VKL_LAUNCH((To + 63) / 64, launch_matvec(w, EPI_PLAIN, false, cmd->stream));
    *o = out;
    return leave();
  }
};

// ------------------------------------------------------------ UpdateKVCache
struct UpdateKVCacheOp : vkl_op {
  int dtype;
  UpdateKVCacheOp(vkl_device *d, vkl_command *c, int dt) : vkl_op(d, c), dtype(dt) {}
  int init() override {
    if (dtype != VKL_FP16) return fail(VKL_INVALID_ARGUMENT, "UpdateKVCache op: only fp16 dtype is supported.");
    return base_init();
  }
  // src/ops/update_kv_cache.cpp:36-76
  int run(vkl_tensor *cache, vkl_tensor *kv, uint32_t offset) {
    if (!cache || !kv) return fail(VKL_INVALID_ARGUMENT, "update_kvcache: null tensor");
    if (cache->dtype != dtype || kv->dtype != dtype) return fail(VKL_INVALID_ARGUMENT, "update_kvcache: tensors must be FP16");
    if (cache->h < kv->h || cache->c < kv->c || cache->w != kv->w)
      return fail(VKL_OUT_OF_RANGE, "size of value is larger than cache. value.shape = (%zu, %zu, %zu), cache.shape = (%zu, %zu, %zu)", kv->c, kv->h, kv->w, cache->c, cache->h, cache->w);
    VKL_OKAY(need_dense(cache, "update_kvcache"));
    VKL_OKAY(need_dense(kv, "update_kvcache"));
    VKL_OKAY(enter("update_kvcache"));
    VKL_LAUNCH(1, launch_update_kvcache((__half *)cache->data(), (const __half *)kv->data(), (uint32_t)kv->c, (uint32_t)kv->h, (uint32_t)kv->w,
                                        (uint32_t)cache->h, (uint32_t)cache->w, offset, cmd->stream));
    return leave();
  }
};

// ------------------------------------------------------------------ RMSNorm
struct RmsNormOp : vkl_op {
  vkl_tensor *weight;
  float eps;
  int dtype;
  vkl_tensor *out = nullptr;
  RmsNormOp(vkl_device *d, vkl_command *c, vkl_tensor *w, float e, int dt) : vkl_op(d, c), weight(w), eps(e), dtype(dt) { vkl_tensor_retain(weight); }
  ~RmsNormOp() override { vkl_tensor_release(weight); vkl_tensor_release(out); }
  // src/ops/rms_norm.cpp:24-53
  int init() override {
    if (dtype != VKL_FP16) return fail(VKL_INVALID_ARGUMENT, "RMSNorm op: only fp16 dtype is supported.");
    if (!weight) return fail(VKL_INVALID_ARGUMENT, "RMSNorm op: null weight");
    if (weight->dtype != VKL_FP32) return fail(VKL_INVALID_ARGUMENT, "rms_norm op defined with %d dtype but the dtype of weight is %d", dtype, weight->dtype);
    return base_init();
  }
  // src/ops/rms_norm.cpp:61-91
  int run(vkl_tensor *x, vkl_tensor **o) {
    if (!x || x->dtype != dtype) return fail(VKL_INVALID_ARGUMENT, "rms_norm op defined with %d dtype but the dtype of input0 is %d", dtype, x ? x->dtype : -1);
    VKL_OKAY(need_dense(x, "rms_norm"));
    if (weight->size() < x->w) return fail(VKL_INVALID_ARGUMENT, "rms_norm: weight has %zu elements, rows have %zu", weight->size(), x->w);
    VKL_OKAY(enter("rms_norm"));
    VKL_OKAY(ensure_tensor(dev, &out, x->c, x->h, x->w, dtype));
    VKL_LAUNCH(1, launch_rms_norm((const __half *)x->data(), (const float *)weight->data(), (__half *)out->data(), (uint32_t)x->rows(), (uint32_t)x->w, eps, cmd->stream));
    *o = out;
    return leave();
  }
};

// --------------------------------------------------------------------- Rope
struct RopeOp : vkl_op {
  int maxlen, dim, dtype;
  vkl_tensor *fc = nullptr, *fs = nullptr;
  RopeOp(vkl_device *d, vkl_command *c, int ml, int dm, int dt) : vkl_op(d, c), maxlen(ml), dim(dm), dtype(dt) {}
  ~RopeOp() override { vkl_tensor_release(fc); vkl_tensor_release(fs); }
  // src/ops/rope.cpp:49-105. The reference sizes its tables for 2*maxlen rows
  // but uploads only the first half of the bytes (rope.cpp:73-96); all 2*maxlen
  // rows are valid here.
  int init() override {
    if (dtype != VKL_FP16) return fail(VKL_INVALID_ARGUMENT, "Rope op: only fp16 dtype is supported.");
    if (maxlen <= 0 || dim <= 0 || (dim & 1)) return fail(VKL_INVALID_ARGUMENT, "Rope op: bad maxlen %d or dim %d", maxlen, dim);
    VKL_OKAY(base_init());
    return make_rope_tables(dev, cmd->stream, dim, 2 * maxlen, &fc, &fs);
  }
  // src/ops/rope.cpp:113-150
  int run(vkl_tensor *q, size_t offset, vkl_tensor **o) {
    if (!q) return fail(VKL_INVALID_ARGUMENT, "rope: null tensor");
    if (q->w != (size_t)dim || q->h > (size_t)maxlen)
      return fail(VKL_INVALID_ARGUMENT, "rope shape error. input0.shape = (%zu, %zu, %zu) dim = %d, maxlen = %d", q->c, q->h, q->w, dim, maxlen);
    if (q->dtype != dtype) return fail(VKL_INVALID_ARGUMENT, "rope defined with dtype %d. but query.dtype = %d", dtype, q->dtype);
    if (offset + q->h > (size_t)2 * maxlen) return fail(VKL_OUT_OF_RANGE, "rope: position %zu is beyond the table (2*maxlen = %d)", offset + q->h, 2 * maxlen);
    VKL_OKAY(enter("rope"));
    VKL_LAUNCH(1, launch_rope((__half *)q->data(), (uint32_t)q->c, (uint32_t)q->h, (uint32_t)q->w, q->cs / 2, q->hs / 2, nullptr, (uint32_t)offset,
                              (const float *)fc->data(), (const float *)fs->data(), cmd->stream));
    *o = q;
    return leave();
  }
};

// ------------------------------------------------------------------ Softmax
struct SoftmaxOp : vkl_op {
  int seq_mask, dtype;
  float temp;
  vkl_tensor *out = nullptr;
  SoftmaxOp(vkl_device *d, vkl_command *c, int sm, float t, int dt) : vkl_op(d, c), seq_mask(sm), dtype(dt), temp(t) {}
  ~SoftmaxOp() override { vkl_tensor_release(out); }
  int init() override {
    if (dtype != VKL_FP16) return fail(VKL_INVALID_ARGUMENT, "Softmax op: only fp16 dtype is supported.");
    return base_init();
  }
  // src/ops/softmax.cpp:53-92
  int run(vkl_tensor *a, size_t offset, vkl_tensor **o) {
    if (!a || a->dtype != dtype) return fail(VKL_INVALID_ARGUMENT, "softmax op defined with %d dtype but input0's dtype = %d", dtype, a ? a->dtype : -1);
    VKL_OKAY(need_dense(a, "softmax"));
    VKL_OKAY(enter("softmax"));
    VKL_OKAY(ensure_tensor(dev, &out, a->c, a->h, a->w, dtype));
    VKL_LAUNCH(1, launch_softmax((const __half *)a->data(), (__half *)out->data(), (uint32_t)a->c, (uint32_t)a->h, (uint32_t)a->w, seq_mask, (uint32_t)offset, cmd->stream));
    *o = out;
    return leave();
  }
};

// -------------------------------------------------------------------- ArgOp
struct ArgOpOp : vkl_op {
  int op_type, dtype;
  vkl_tensor *out = nullptr, *stage0 = nullptr;
  ArgOpOp(vkl_device *d, vkl_command *c, int t, int dt) : vkl_op(d, c), op_type(t), dtype(dt) {}
  ~ArgOpOp() override { vkl_tensor_release(out); vkl_tensor_release(stage0); }
  int init() override {
    if (dtype != VKL_FP16) return fail(VKL_INVALID_ARGUMENT, "ArgOp: only fp16 dtype is supported.");
    if (op_type != 0 && op_type != 1) return fail(VKL_INVALID_ARGUMENT, "ArgOp: op_type %d is unknown", op_type);
    return base_init();
  }
  // src/ops/argop.h:72-140
  int run(vkl_tensor *in, vkl_tensor **o) {
    if (!in || in->dtype != dtype) return fail(VKL_INVALID_ARGUMENT, "operator defined as %d dtype but %d given.", dtype, in ? in->dtype : -1);
    VKL_OKAY(need_dense(in, "argop"));
    if (in->w == 0) return fail(VKL_INVALID_ARGUMENT, "argop: empty rows");
    VKL_OKAY(enter("argop"));
    VKL_OKAY(ensure_tensor(dev, &out, in->c, in->h, 1, VKL_UINT32));
    VKL_OKAY(ensure_tensor(dev, &stage0, in->c, in->h, ((in->w + 1023) / 1024) * 2, VKL_FP32));
    VKL_LAUNCH(2, launch_argop((const __half *)in->data(), (uint32_t *)out->data(), stage0->data(), (uint32_t)in->rows(), (uint32_t)in->w, op_type, cmd->stream));
    *o = out;
    return leave();
  }
};

// ---------------------------------------------------------------- Embedding
struct EmbeddingOp : vkl_op {
  vkl_tensor *vocab;
  uint32_t unk;
  int dtype;
  vkl_tensor *out = nullptr;
  EmbeddingOp(vkl_device *d, vkl_command *c, vkl_tensor *v, uint32_t u, int dt) : vkl_op(d, c), vocab(v), unk(u), dtype(dt) { vkl_tensor_retain(vocab); }
  ~EmbeddingOp() override { vkl_tensor_release(vocab); vkl_tensor_release(out); }
  // src/ops/embedding.cpp:20-56
  int init() override {
    if (!vocab) return fail(VKL_INVALID_ARGUMENT, "Embedding op: null vocab");
    if (dtype != VKL_FP16 && dtype != VKL_Q8_0) return fail(VKL_INVALID_ARGUMENT, "Embedding op: only fp16 and q8_0 vocab is supported.");
    return base_init();
  }
  // src/ops/embedding.cpp:58-114
  int run(vkl_tensor *idx, vkl_tensor **o) {
    if (!idx) return fail(VKL_INVALID_ARGUMENT, "embedding: null indices");
    if (vocab->c != 1 || idx->c != 1)
      return fail(VKL_INVALID_ARGUMENT, "only channels = 1 is supported. vocab channels = %zu, indices channels = %zu\n", vocab->c, idx->c);
    if (idx->dtype != VKL_UINT32 || vocab->dtype != dtype) return fail(VKL_INVALID_ARGUMENT, "only indices.dtype = UINT32 is supported");
    VKL_OKAY(need_dense(idx, "embedding"));
    VKL_OKAY(enter("embedding"));
    VKL_OKAY(ensure_tensor(dev, &out, idx->h, idx->w, vocab->w, VKL_FP16));
    VKL_LAUNCH(1, launch_embedding(vocab->data(), dtype == VKL_Q8_0, (const uint32_t *)idx->data(), (__half *)out->data(), (uint32_t)(idx->h * idx->w),
                                   (uint32_t)vocab->h, (uint32_t)vocab->w, unk, cmd->stream));
    *o = out;
    return leave();
  }
};

// -------------------------------------------------------------- ElementWise
struct ElementWiseOp : vkl_op {
  int type, dtype;
  ElementWiseOp(vkl_device *d, vkl_command *c, int t, int dt) : vkl_op(d, c), type(t), dtype(dt) {}
  int init() override {
    if (dtype != VKL_FP16) return fail(VKL_INVALID_ARGUMENT, "ElementWise op: only fp16 dtype is supported.");
    if (type < 0 || type > 3) return fail(VKL_INVALID_ARGUMENT, "ElementWise op: type %d is unknown", type);
    return base_init();
  }
  // src/ops/elementwise.cpp:68-102: the result is written into y.
  int run(vkl_tensor *x, vkl_tensor *y, vkl_tensor **o) {
    if (!x || !y || x->dtype != dtype || y->dtype != dtype)
      return fail(VKL_INVALID_ARGUMENT, "elementwise op defined with %d dtype but inputs have %d and %d", dtype, x ? x->dtype : -1, y ? y->dtype : -1);
    if (x->c != y->c || x->h != y->h || x->w != y->w)
      return fail(VKL_INVALID_ARGUMENT, "elementwise: shapes differ (%zu, %zu, %zu) vs (%zu, %zu, %zu)", x->c, x->h, x->w, y->c, y->h, y->w);
    VKL_OKAY(need_dense(x, "elementwise"));
    VKL_OKAY(need_dense(y, "elementwise"));
    VKL_OKAY(enter("elementwise"));
    VKL_LAUNCH(1, launch_add((const __half *)x->data(), (__half *)y->data(), x->size(), type, cmd->stream));
    *o = y;
    return leave();
  }
  // src/ops/elementwise.cpp:104-133: x <- x op y for a scalar y, in place. The reference hands the scalar over as
  // fp32 or, on devices with fp16 arithmetic, truncated to fp16; this is the fp32 form.
  int run_scalar(vkl_tensor *x, float y, vkl_tensor **o) {
    if (!x) return fail(VKL_INVALID_ARGUMENT, "elementwise: null tensor");
    if (x->dtype != dtype) return fail(VKL_INVALID_ARGUMENT, "elementwise op defined with %d dtype but the input has %d", dtype, x->dtype);
    VKL_OKAY(need_dense(x, "elementwise"));
    VKL_OKAY(enter("elementwise"));
    VKL_LAUNCH(1, launch_scalar_op((__half *)x->data(), x->size(), type, y, cmd->stream));
    *o = x;
    return leave();
  }
};

// ------------------------------------------------------------------- Concat
struct ConcatOp : vkl_op {
  int num, axis, dtype;
  vkl_tensor *out = nullptr;
  ConcatOp(vkl_device *d, vkl_command *c, int n, int ax, int dt) : vkl_op(d, c), num(n), axis(ax), dtype(dt) {}
  ~ConcatOp() override { vkl_tensor_release(out); }
  // src/ops/concat.cpp:20-65
  int init() override {
    if (dtype != VKL_FP16) return fail(VKL_INVALID_ARGUMENT, "Concat op: only fp16 dtype is supported.");
    if (num < 1) return fail(VKL_INVALID_ARGUMENT, "Concat op: %d inputs", num);
    return base_init();
  }
  // src/ops/concat.cpp:67-184
  int run(vkl_tensor *const *in, size_t n, vkl_tensor **o) {
    if (!in || n != (size_t)num) return fail(VKL_INVALID_ARGUMENT, "operator has %zu inputs but %zu are given", (size_t)num, n);
    for (size_t i = 0; i < n; ++i) {
      if (!in[i] || in[i]->dtype != dtype) return fail(VKL_INVALID_ARGUMENT, "dtype of inputs are unsupported.");
      VKL_OKAY(need_dense(in[i], "concat"));
    }
    if (axis < 0 || axis > 2) return fail(VKL_INVALID_ARGUMENT, "axis %d is unsupported.", axis);
    const vkl_tensor *r = in[0];
    size_t c = r->c, h = r->h, w = r->w;
    for (size_t i = 1; i < n; ++i) {
      const vkl_tensor *t = in[i];
      if (axis == 0 && (t->h != r->h || t->w != r->w)) return fail(VKL_INVALID_ARGUMENT, "inputs shape error on axis 0");
      if (axis == 1 && (t->c != r->c || t->w != r->w)) return fail(VKL_INVALID_ARGUMENT, "inputs shape error on axis 1");
      if (axis == 2 && (t->c != r->c || t->h != r->h)) return fail(VKL_INVALID_ARGUMENT, "inputs shape error on axis 2");
      if (axis == 0) c += t->c;
      if (axis == 1) h += t->h;
      if (axis == 2) w += t->w;
    }
    VKL_OKAY(enter("concat"));
    VKL_OKAY(ensure_tensor(dev, &out, c, h, w, dtype));
    size_t offset = 0;  // in elements of the output: whole inputs (axis 0), rows (axis 1) or columns (axis 2)
    for (size_t i = 0; i < n; ++i) {
      const vkl_tensor *t = in[i];
      VKL_LAUNCH(1, launch_concat_copy((const __half *)t->data(), (__half *)out->data(), (uint32_t)t->c, (uint32_t)t->h, (uint32_t)t->w, out->cs / 2,
                                       out->hs / 2, offset, cmd->stream));
      offset += axis == 0 ? t->size() : axis == 1 ? t->w * t->h : t->w;
    }
    *o = out;
    return leave();
  }
};

// ------------------------------------------------------------------- Reduce
struct ReduceOp : vkl_op {
  int op_type, dtype;  // 0 sum, 1 max, 2 min, 3 mean (src/ops/reduce.h:18)
  vkl_tensor *out = nullptr;
  ReduceOp(vkl_device *d, vkl_command *c, int t, int dt) : vkl_op(d, c), op_type(t), dtype(dt) {}
  ~ReduceOp() override { vkl_tensor_release(out); }
  int init() override {
    if (dtype != VKL_FP16) return fail(VKL_INVALID_ARGUMENT, "Reduce op: only fp16 dtype is supported");
    if (op_type < 0 || op_type > 3) return fail(VKL_INVALID_ARGUMENT, "Reduce op: type %d is unknown", op_type);
    return base_init();
  }
  // src/ops/reduce.h:67-112: [c, h, w] -> [c, h, 1]
  int run(vkl_tensor *a, vkl_tensor **o) {
    if (!a || a->dtype != dtype) return fail(VKL_INTERNAL, "reduce op defined with %d dtype but the dtype of input0 is %d", dtype, a ? a->dtype : -1);
    if (a->w == 0) return fail(VKL_INVALID_ARGUMENT, "reduce: empty rows");
    VKL_OKAY(need_dense(a, "reduce"));
    VKL_OKAY(enter("reduce"));
    VKL_OKAY(ensure_tensor(dev, &out, a->c, a->h, 1, dtype));
    VKL_LAUNCH(1, launch_reduce((const __half *)a->data(), (__half *)out->data(), (uint32_t)a->rows(), (uint32_t)a->w, op_type == 3 ? 0 : op_type,
                                op_type == 3 ? 1.0f / (float)a->w : 1.0f, cmd->stream));
    *o = out;
    return leave();
  }
};

// -------------------------------------------------------------- ReadKVCache
struct ReadKVCacheOp : vkl_op {
  vkl_tensor *out = nullptr;
  ReadKVCacheOp(vkl_device *d, vkl_command *c) : vkl_op(d, c) {}
  ~ReadKVCacheOp() override { vkl_tensor_release(out); }
  int init() override { return base_init(); }
  // src/ops/read_kvcache_op.cpp:31-71: rows (offset + y) % maxlen of every head, y < len
  int run(vkl_tensor *cache, uint32_t offset, uint32_t len, vkl_tensor **o) {
    if (!cache || cache->dtype != VKL_FP16) return fail(VKL_INVALID_ARGUMENT, "read_kvcache: the cache must be an fp16 tensor");
    if (len > cache->h) return fail(VKL_OUT_OF_RANGE, "read %d len but size of cache is %zu", (int)len, cache->h);
    VKL_OKAY(need_dense(cache, "read_kvcache"));
    VKL_OKAY(enter("read_kvcache"));
    VKL_OKAY(ensure_tensor(dev, &out, cache->c, len, cache->w, VKL_FP16));
    VKL_LAUNCH(1, launch_read_kvcache((const __half *)cache->data(), (__half *)out->data(), (uint32_t)cache->c, (uint32_t)cache->h, (uint32_t)cache->w,
                                      offset, len, cmd->stream));
    *o = out;
    return leave();
  }
};

// ---------------------------------------------------------------- Transpose
struct TransposeOp : vkl_op {
  int type, dtype;
  vkl_tensor *out = nullptr;
  TransposeOp(vkl_device *d, vkl_command *c, int t, int dt) : vkl_op(d, c), type(t), dtype(dt) {}
  ~TransposeOp() override { vkl_tensor_release(out); }
  int init() override {
    if (dtype != VKL_FP16) return fail(VKL_INVALID_ARGUMENT, "Transpose op: only fp16 dtype is supported.");
    if (type != 0) return fail(VKL_INVALID_ARGUMENT, "Transpose op: unsupported type %d", type);
    return base_init();
  }
  // src/ops/transpose.cpp:33-79
  int run(vkl_tensor *in, vkl_tensor **o) {
    if (!in || in->dtype != dtype) return fail(VKL_INVALID_ARGUMENT, "transpose op defined with %d dtype but input has %d", dtype, in ? in->dtype : -1);
    VKL_OKAY(need_dense(in, "transpose"));
    VKL_OKAY(enter("transpose"));
    VKL_OKAY(ensure_tensor(dev, &out, in->h, in->c, in->w, dtype));
    VKL_LAUNCH(1, launch_transpose((const __half *)in->data(), (__half *)out->data(), (uint32_t)in->c, (uint32_t)in->h, (uint32_t)in->w, cmd->stream));
    *o = out;
    return leave();
  }
};

// -------------------------------------------------------------------- Slice
struct SliceOp : vkl_op {
  int dtype;
  vkl_tensor *out = nullptr;
  SliceOp(vkl_device *d, vkl_command *c, int dt) : vkl_op(d, c), dtype(dt) {}
  ~SliceOp() override { vkl_tensor_release(out); }
  int init() override {
    if (dtype != VKL_FP16) return fail(VKL_INVALID_ARGUMENT, "Slice op: only fp16 dtype is supported.");
    return base_init();
  }
  // src/ops/slice.cpp:33-76
  int run(vkl_tensor *in, const uint32_t st[3], const uint32_t ex[3], vkl_tensor **o) {
    if (!in || !st || !ex) return fail(VKL_INVALID_ARGUMENT, "slice: null argument");
    if (in->dtype != dtype) return fail(VKL_INVALID_ARGUMENT, "slice op defined with %d dtype but input has %d", dtype, in->dtype);
    if (st[0] + ex[0] > in->c || st[1] + ex[1] > in->h || st[2] + ex[2] > in->w)
      return fail(VKL_OUT_OF_RANGE, "slice (%u+%u, %u+%u, %u+%u) exceeds (%zu, %zu, %zu)", st[0], ex[0], st[1], ex[1], st[2], ex[2], in->c, in->h, in->w);
    VKL_OKAY(need_dense(in, "slice"));
    VKL_OKAY(enter("slice"));
    VKL_OKAY(ensure_tensor(dev, &out, ex[0], ex[1], ex[2], dtype));
    VKL_LAUNCH(1, launch_slice((const __half *)in->data(), (__half *)out->data(), (uint32_t)in->c, (uint32_t)in->h, (uint32_t)in->w, st[0], st[1], st[2], ex[0], ex[1], ex[2], cmd->stream));
    *o = out;
    return leave();
  }
};

// --------------------------------------------------------------------- Cast
struct CastOp : vkl_op {
  int from, to;
  vkl_tensor *out = nullptr;
  CastOp(vkl_device *d, vkl_command *c, int f, int t) : vkl_op(d, c), from(f), to(t) {}
  ~CastOp() override { vkl_tensor_release(out); }
  // src/ops/cast.cpp:14-45
  int init() override {
    if (!((from == VKL_FP16 && to == VKL_FP32) || (from == VKL_FP32 && to == VKL_FP16)))
      return fail(VKL_INVALID_ARGUMENT, "cast op: only fp16 <-> fp32 is supported (from %d to %d)", from, to);
    return base_init();
  }
  // src/ops/cast.cpp:47-76
  int run(vkl_tensor *in, vkl_tensor **o) {
    if (!in || in->dtype != from) return fail(VKL_INVALID_ARGUMENT, "cast op defined from %d dtype but input has %d", from, in ? in->dtype : -1);
    VKL_OKAY(need_dense(in, "cast"));
    VKL_OKAY(enter("cast"));
    VKL_OKAY(ensure_tensor(dev, &out, in->c, in->h, in->w, to));
    if (from == VKL_FP16)
      VKL_LAUNCH(1, launch_cast_f16_f32((const __half *)in->data(), (float *)out->data(), in->size(), cmd->stream));
    else
      VKL_LAUNCH(1, launch_cast_f32_f16((const float *)in->data(), (__half *)out->data(), in->size(), cmd->stream));
    *o = out;
    return leave();
  }
};

template <class T>
int as(vkl_op *op, T **out, const char *who) {
  if (!op) return fail(VKL_INVALID_ARGUMENT, "%s: null op", who);
  T *t = dynamic_cast<T *>(op);
  if (!t) return fail(VKL_INVALID_ARGUMENT, "%s: handle is another kind of op", who);
  *out = t;
  return VKL_OK;
}

}  // namespace

namespace vkl {
int rope_tables(vkl_device *dev, cudaStream_t s, int dim, int rows, vkl_tensor **fc, vkl_tensor **fs) {
  return make_rope_tables(dev, s, dim, rows, fc, fs);
}
}  // namespace vkl

extern "C" {

int vkl_op_init(vkl_op *op) {
  if (!op) return fail(VKL_INVALID_ARGUMENT, "op_init: null op");
  VKL_CUDA(cudaSetDevice(op->dev ? op->dev->ordinal : 0));
  return op->init();
}
int vkl_op_time(vkl_op *op, uint64_t *usec) {
  if (!op || !usec) return fail(VKL_INVALID_ARGUMENT, "op_time: null argument");
  *usec = 0;
  if (!op->timed) return VKL_OK;
  float ms = 0.f;
  cudaError_t e = cudaEventElapsedTime(&ms, op->e0, op->e1);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(VKL_FAILED_PRECONDITION, "op_time: the op's last run has not finished (wait on its command first)");
  }
  *usec = (uint64_t)llroundf(ms * 1000.f);
  return VKL_OK;
}
int vkl_op_destroy(vkl_op *op) {
  delete op;
  return VKL_OK;
}

#define MAKE(Type, ...)                                                        \
  if (!out) return fail(VKL_INVALID_ARGUMENT, "op create: null output");       \
  if (!dev || !cmd) return fail(VKL_INVALID_ARGUMENT, "op create: null device or command"); \
  *out = new Type(dev, cmd, __VA_ARGS__);                                      \
  return VKL_OK;

int vkl_matmul_create(vkl_device *dev, vkl_command *cmd, vkl_tensor *weight, float scale, float bias, int act, int broadcast_type,
                      int transpose_b, int a_dtype, int b_dtype, vkl_op **out) {
  MAKE(MatMulOp, weight, scale, bias, act, broadcast_type, transpose_b, a_dtype, b_dtype)
}
int vkl_matmul_run(vkl_op *op, vkl_tensor *a, vkl_tensor *b, vkl_tensor **out) {
  MatMulOp *m;
  VKL_OKAY(as(op, &m, "matmul_run"));
  if (!out) return fail(VKL_INVALID_ARGUMENT, "matmul_run: null output");
  return b ? m->run_pair(a, b, out) : m->run_weight(a, out);
}
int vkl_matmul_run_many(vkl_op *const *ops, size_t n_ops, vkl_tensor *a, size_t reps, float *us_per_launch) {
  if (!ops || !n_ops || !a || !reps) return fail(VKL_INVALID_ARGUMENT, "matmul_run_many: null argument");
  MatMulOp *first;
  VKL_OKAY(as(ops[0], &first, "matmul_run_many"));
  cudaStream_t st = first->cmd->stream;
  auto record_all = [&]() -> int {
    for (size_t i = 0; i < reps; ++i) {
      MatMulOp *m;
      VKL_OKAY(as(ops[i % n_ops], &m, "matmul_run_many"));
      vkl_tensor *out = nullptr;
      VKL_OKAY(m->run_weight(a, &out));
    }
    return VKL_OK;
  };
  if (!us_per_launch) return record_all();
  // Timed form: the launches are captured into a CUDA graph (outputs were allocated by an earlier
  // untimed call), so the device runs them back to back with no host work in between.
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  VKL_CUDA(cudaEventCreate(&e0));
  VKL_CUDA(cudaEventCreate(&e1));
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  int status = VKL_OK;
  cudaError_t e = cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal);
  if (e == cudaSuccess) {
    status = record_all();
    e = cudaStreamEndCapture(st, &graph);
  }
  if (status == VKL_OK && e == cudaSuccess && graph) e = cudaGraphInstantiate(&exec, graph, 0);
  if (status == VKL_OK && e == cudaSuccess && exec) {
    cudaGraphLaunch(exec, st);  // warm
    cudaEventRecord(e0, st);
    cudaGraphLaunch(exec, st);
    cudaEventRecord(e1, st);
    e = cudaStreamSynchronize(st);
    float ms = 0.f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
    *us_per_launch = ms * 1000.f / (float)reps;
  }
  if (exec) cudaGraphExecDestroy(exec);
  if (graph) cudaGraphDestroy(graph);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (status != VKL_OK) return status;
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(VKL_INTERNAL, "matmul_run_many: %s", cudaGetErrorString(e));
  }
  return VKL_OK;
}
int vkl_feed_forward_create(vkl_device *dev, vkl_command *cmd, vkl_tensor *w1, vkl_tensor *w2, vkl_tensor *w3, int transposed_weight,
                            int dtype, vkl_op **out) {
  if (!w1 || !w2 || !w3) return fail(VKL_INVALID_ARGUMENT, "feed_forward_create: null weight");
  MAKE(FeedForwardOp, w1, w2, w3, transposed_weight, dtype)
}
int vkl_feed_forward_run(vkl_op *op, vkl_tensor *x, vkl_tensor **out) {
  FeedForwardOp *m;
  VKL_OKAY(as(op, &m, "feed_forward_run"));
  if (!out) return fail(VKL_INVALID_ARGUMENT, "feed_forward_run: null output");
  return m->run(x, out);
}
int vkl_mha_create(vkl_device *dev, vkl_command *cmd, vkl_tensor *wk, vkl_tensor *wq, vkl_tensor *wv, vkl_tensor *wo, int maxlen, int dim,
                   int transposed_weight, int dtype, int use_kvcache, int clip_output, vkl_op **out) {
  if (!wk || !wq || !wv || !wo) return fail(VKL_INVALID_ARGUMENT, "mha_create: null weight");
  MAKE(MhaOp, wk, wq, wv, wo, maxlen, dim, transposed_weight, dtype, use_kvcache, clip_output)
}
int vkl_mha_run(vkl_op *op, vkl_tensor *x, size_t offset, vkl_tensor **out) {
  MhaOp *m;
  VKL_OKAY(as(op, &m, "mha_run"));
  if (!out) return fail(VKL_INVALID_ARGUMENT, "mha_run: null output");
  return m->run(x, offset, out);
}
int vkl_mha_caches(vkl_op *op, vkl_tensor **kcache, vkl_tensor **vcache) {
  MhaOp *m;
  VKL_OKAY(as(op, &m, "mha_caches"));
  if (kcache) *kcache = m->kcache;
  if (vcache) *vcache = m->vcache;
  return VKL_OK;
}
int vkl_update_kvcache_create(vkl_device *dev, vkl_command *cmd, int dtype, vkl_op **out) { MAKE(UpdateKVCacheOp, dtype) }
int vkl_update_kvcache_run(vkl_op *op, vkl_tensor *cache, vkl_tensor *kv, uint32_t offset) {
  UpdateKVCacheOp *m;
  VKL_OKAY(as(op, &m, "update_kvcache_run"));
  return m->run(cache, kv, offset);
}
int vkl_rms_norm_create(vkl_device *dev, vkl_command *cmd, vkl_tensor *weight, float eps, int dtype, vkl_op **out) {
  if (!weight) return fail(VKL_INVALID_ARGUMENT, "rms_norm_create: null weight");
  MAKE(RmsNormOp, weight, eps, dtype)
}
int vkl_rms_norm_run(vkl_op *op, vkl_tensor *x, vkl_tensor **out) {
  RmsNormOp *m;
  VKL_OKAY(as(op, &m, "rms_norm_run"));
  if (!out) return fail(VKL_INVALID_ARGUMENT, "rms_norm_run: null output");
  return m->run(x, out);
}
int vkl_rope_create(vkl_device *dev, vkl_command *cmd, int maxlen, int dim, int dtype, vkl_op **out) { MAKE(RopeOp, maxlen, dim, dtype) }
int vkl_rope_run(vkl_op *op, vkl_tensor *q, size_t offset, vkl_tensor **out) {
  RopeOp *m;
  VKL_OKAY(as(op, &m, "rope_run"));
  if (!out) return fail(VKL_INVALID_ARGUMENT, "rope_run: null output");
  return m->run(q, offset, out);
}
int vkl_softmax_create(vkl_device *dev, vkl_command *cmd, int seq_mask, float temp, int dtype, vkl_op **out) { MAKE(SoftmaxOp, seq_mask, temp, dtype) }
int vkl_softmax_run(vkl_op *op, vkl_tensor *a, size_t offset, vkl_tensor **out) {
  SoftmaxOp *m;
  VKL_OKAY(as(op, &m, "softmax_run"));
  if (!out) return fail(VKL_INVALID_ARGUMENT, "softmax_run: null output");
  return m->run(a, offset, out);
}
int vkl_argop_create(vkl_device *dev, vkl_command *cmd, int op_type, int dtype, vkl_op **out) { MAKE(ArgOpOp, op_type, dtype) }
int vkl_argop_run(vkl_op *op, vkl_tensor *in, vkl_tensor **out) {
  ArgOpOp *m;
  VKL_OKAY(as(op, &m, "argop_run"));
  if (!out) return fail(VKL_INVALID_ARGUMENT, "argop_run: null output");
  return m->run(in, out);
}
int vkl_embedding_create(vkl_device *dev, vkl_command *cmd, vkl_tensor *vocab, uint32_t unk, int dtype, vkl_op **out) {
  if (!vocab) return fail(VKL_INVALID_ARGUMENT, "embedding_create: null vocab");
  MAKE(EmbeddingOp, vocab, unk, dtype)
}
int vkl_embedding_run(vkl_op *op, vkl_tensor *indices, vkl_tensor **out) {
  EmbeddingOp *m;
  VKL_OKAY(as(op, &m, "embedding_run"));
  if (!out) return fail(VKL_INVALID_ARGUMENT, "embedding_run: null output");
  return m->run(indices, out);
}
int vkl_elementwise_create(vkl_device *dev, vkl_command *cmd, int type, int dtype, vkl_op **out) { MAKE(ElementWiseOp, type, dtype) }
int vkl_elementwise_run(vkl_op *op, vkl_tensor *x, vkl_tensor *y, vkl_tensor **out) {
  ElementWiseOp *m;
  VKL_OKAY(as(op, &m, "elementwise_run"));
  if (!out) return fail(VKL_INVALID_ARGUMENT, "elementwise_run: null output");
  return m->run(x, y, out);
}
int vkl_elementwise_run_scalar(vkl_op *op, vkl_tensor *x, float y, vkl_tensor **out) {
  ElementWiseOp *m;
  VKL_OKAY(as(op, &m, "elementwise_run_scalar"));
  if (!out) return fail(VKL_INVALID_ARGUMENT, "elementwise_run_scalar: null output");
  return m->run_scalar(x, y, out);
}
int vkl_concat_create(vkl_device *dev, vkl_command *cmd, int num, int axis, int dtype, vkl_op **out) { MAKE(ConcatOp, num, axis, dtype) }
int vkl_concat_run(vkl_op *op, vkl_tensor *const *inputs, size_t n, vkl_tensor **out) {
  ConcatOp *m;
  VKL_OKAY(as(op, &m, "concat_run"));
  if (!out) return fail(VKL_INVALID_ARGUMENT, "concat_run: null output");
  return m->run(inputs, n, out);
}
int vkl_reduce_create(vkl_device *dev, vkl_command *cmd, int op_type, int dtype, vkl_op **out) { MAKE(ReduceOp, op_type, dtype) }
int vkl_reduce_run(vkl_op *op, vkl_tensor *a, vkl_tensor **out) {
  ReduceOp *m;
  VKL_OKAY(as(op, &m, "reduce_run"));
  if (!out) return fail(VKL_INVALID_ARGUMENT, "reduce_run: null output");
  return m->run(a, out);
}
int vkl_read_kvcache_create(vkl_device *dev, vkl_command *cmd, vkl_op **out) {
  if (!out) return fail(VKL_INVALID_ARGUMENT, "op create: null output");
  if (!dev || !cmd) return fail(VKL_INVALID_ARGUMENT, "op create: null device or command");
  *out = new ReadKVCacheOp(dev, cmd);
  return VKL_OK;
}
int vkl_read_kvcache_run(vkl_op *op, vkl_tensor *cache, uint32_t offset, uint32_t len, vkl_tensor **out) {
  ReadKVCacheOp *m;
  VKL_OKAY(as(op, &m, "read_kvcache_run"));
  if (!out) return fail(VKL_INVALID_ARGUMENT, "read_kvcache_run: null output");
  return m->run(cache, offset, len, out);
}
int vkl_transpose_create(vkl_device *dev, vkl_command *cmd, int type, int dtype, vkl_op **out) { MAKE(TransposeOp, type, dtype) }
int vkl_transpose_run(vkl_op *op, vkl_tensor *in, vkl_tensor **out) {
  TransposeOp *m;
  VKL_OKAY(as(op, &m, "transpose_run"));
  if (!out) return fail(VKL_INVALID_ARGUMENT, "transpose_run: null output");
  return m->run(in, out);
}
int vkl_slice_create(vkl_device *dev, vkl_command *cmd, int dtype, vkl_op **out) { MAKE(SliceOp, dtype) }
int vkl_slice_run(vkl_op *op, vkl_tensor *in, const uint32_t starts[3], const uint32_t extents[3], vkl_tensor **out) {
  SliceOp *m;
  VKL_OKAY(as(op, &m, "slice_run"));
  if (!out) return fail(VKL_INVALID_ARGUMENT, "slice_run: null output");
  return m->run(in, starts, extents, out);
}
int vkl_cast_create(vkl_device *dev, vkl_command *cmd, int from, int to, vkl_op **out) { MAKE(CastOp, from, to) }
int vkl_cast_run(vkl_op *op, vkl_tensor *in, vkl_tensor **out) {
  CastOp *m;
  VKL_OKAY(as(op, &m, "cast_run"));
  if (!out) return fail(VKL_INVALID_ARGUMENT, "cast_run: null output");
  return m->run(in, out);
}

}  // extern "C"
