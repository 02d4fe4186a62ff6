// Llama-2 driver behind the C ABI: weight table, KV caches, the multi-token
// (prefill) pass and the one-token decode step, which is captured once into a
// CUDA graph and replayed per token with the position, the current token and
// the output cursor living in device memory.
//
// Mirrors models/llama2.h of the reference: Model::init (348-681) becomes
// vkl_model_set_weight per GGUF tensor, Model::operator() (683-843) becomes
// vkl_model_forward, and the loop of app/llama2_infer.cpp:141-210 becomes
// vkl_model_generate. Per layer the reference records 19 dispatches
// (llama2.h:160-213, multiheadattention_v2.cpp:190-319); the decode step here
// is 5 kernels per layer:
//   RMSNorm+QKV mat-vec | RoPE+append+attention | o_proj+residual |
//   RMSNorm+gate/up+SwiGLU | down+residual
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>

#include <string>

#include "runtime.h"

namespace vkl {
int rope_tables(vkl_device *dev, cudaStream_t s, int dim, int rows, vkl_tensor **fc, vkl_tensor **fs);
}
using namespace vkl;

namespace {
struct Layer {
  vkl_tensor *attn_norm = nullptr, *ffn_norm = nullptr;
  vkl_tensor *wq = nullptr, *wk = nullptr, *wv = nullptr, *wo = nullptr;
  vkl_tensor *gate = nullptr, *up = nullptr, *down = nullptr;
  vkl_tensor *kcache = nullptr, *vcache = nullptr;
};

__global__ void set_u32(uint32_t *p, uint32_t v) { *p = v; }
// After the arg-max: publish the picked id, feed it back, advance the position.
__global__ void advance_kernel(const uint32_t *next, uint32_t *tok, uint32_t *pos, uint32_t *step,
                               uint32_t *out_ids, uint32_t cap, uint32_t pos_inc) {
  const uint32_t id = *next, s = *step;
  if (s < cap) out_ids[s] = id;
  *tok = id;
  *pos += pos_inc;
  *step = s + 1;
}
}  // namespace

struct vkl_model {
  vkl_device *dev = nullptr;
  vkl_model_config cfg;
  cudaStream_t stream = nullptr;
  uint32_t head_dim = 0, heads_l = 0, dim_l = 0, ffn_l = 0, vocab_l = 0;
  std::vector<Layer> L;
  vkl_tensor *tok_embd = nullptr, *output_norm = nullptr, *output = nullptr;
  vkl_tensor *fc = nullptr, *fs = nullptr;
  // activations, sized for `cap_T` rows
  uint32_t cap_T = 0;
  vkl_tensor *x = nullptr, *xn = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *ao = nullptr, *t = nullptr;
  vkl_tensor *gu32 = nullptr;  // [2, cap_T, ffn] fp32 gate and up results of the FP16 prefill GEMMs
  bool gemm_used = false;      // a tensor-core GEMM ran since the last check of state[6]
  vkl_tensor *logits16 = nullptr, *logits32 = nullptr;
  vkl_tensor *toks = nullptr;  // [cap_T] device token ids; toks[0] is the decode token
  vkl_tensor *state = nullptr; // uint32[8]: [0] pos, [1] step, [2] next id, [3] all-reduces, [4] arg exchanges, [5] forced tokens, [6] GEMM wait error
  vkl_tensor *forced = nullptr;  // prompt ids for token-by-token prefill
  // tensor parallelism: this rank's exchange buffer (plain cudaMalloc so that it can be
  // exported over CUDA IPC) and every rank's mapping of it
  void *tp_buf = nullptr;
  size_t tp_bytes = 0;
  uint32_t tp_flag_off = 0;
  void *tp_peer[8] = {};
  bool tp_connected = false;
  // many-token passes of a sharded model: two alternating regions of fp32 partial sums [tp_pf_rows, dim]
  // and the ranks' flag words behind the one-token exchange area, and the count of all-reduces so far
  size_t tp_pf_off = 0, tp_pf_flag_off = 0;
  uint32_t tp_pf_rows = 0, tp_pf_seq = 0;
  vkl_tensor *out_ids = nullptr;
  vkl_tensor *argpart = nullptr, *attn_scratch = nullptr, *attn_counters = nullptr;
  uint32_t splits = 8, out_cap = 0;
  cudaGraphExec_t decode_graph = nullptr;
  bool use_pdl = true;
  // persistent single-kernel decode step (decode_mega.cu)
  bool mega_ready = false, mega_tried = false;
  int mega_grid = 0;
  vkl_tensor *mega_ops = nullptr, *mega_sync = nullptr, *mega_arg = nullptr, *mega_attn = nullptr, *mega_stages = nullptr, *mega_counts = nullptr, *mega_ll = nullptr;
  std::vector<vkl_tensor *> mega_packed;  // the ops' weight streams in the persistent kernel's layout
  MegaParams mp;
  uint32_t mega_launches_per_token = 1;
  uint32_t sm_mhz = 0;  // measured SM clock, for the profiled launches' cycle counts
  uint32_t wait_limit = 0;  // polls a wait of the decode kernel may spin (0: the default of build_mega)
  bool tp_failed = false;   // a wait on another rank ran out: the ranks' sequence counters are out of step until they reconnect
  unsigned char *pin = nullptr;  // pinned host staging of the one-token call: this rank's fp32 logits, then the decode kernel's error word
  cudaEvent_t ev0 = nullptr, ev1 = nullptr, ev2 = nullptr;
  uint32_t *pos_dev() { return (uint32_t *)state->data(); }
  uint32_t *step_dev() { return (uint32_t *)state->data() + 1; }
  uint32_t *next_dev() { return (uint32_t *)state->data() + 2; }
  ~vkl_model() {
    if (decode_graph) cudaGraphExecDestroy(decode_graph);
    if (tp_buf) cudaFree(tp_buf);
    if (pin) cudaFreeHost(pin);
    for (auto &l : L)
      for (vkl_tensor *p : {l.attn_norm, l.ffn_norm, l.wq, l.wk, l.wv, l.wo, l.gate, l.up, l.down, l.kcache, l.vcache}) vkl_tensor_release(p);
    for (vkl_tensor *p : mega_packed) vkl_tensor_release(p);
    for (vkl_tensor *p : {tok_embd, output_norm, output, fc, fs, x, xn, q, k, v, ao, t, gu32, logits16, logits32, toks, state, out_ids, forced, argpart, attn_scratch, attn_counters, mega_ops, mega_sync, mega_arg, mega_attn, mega_stages, mega_counts, mega_ll})
      vkl_tensor_release(p);
    if (ev0) cudaEventDestroy(ev0);
    if (ev1) cudaEventDestroy(ev1);
    if (ev2) cudaEventDestroy(ev2);
    if (stream) {
      dev->remove_stream(stream);
      cudaStreamDestroy(stream);
    }
  }
};

namespace {

bool q8(const vkl_model *m) { return m->cfg.weight_dtype == VKL_Q8_0; }

int ensure_rows(vkl_model *m, uint32_t T) {
  if (T <= m->cap_T) return VKL_OK;
  if (m->decode_graph) {  // the graph holds the old buffers
    cudaGraphExecDestroy(m->decode_graph);
    m->decode_graph = nullptr;
  }
  VKL_CUDA(cudaStreamSynchronize(m->stream));
  if (m->mega_tried) {  // the op table of the persistent kernel holds the old buffers too
    for (vkl_tensor **t : {&m->mega_ops, &m->mega_sync, &m->mega_arg, &m->mega_attn, &m->mega_stages, &m->mega_counts, &m->mega_ll}) {
      vkl_tensor_release(*t);
      *t = nullptr;
    }
    m->mega_ready = m->mega_tried = false;  // the packed weight streams (mega_packed) do not depend on the row count: kept
  }
  const size_t D = m->cfg.dim;
  VKL_OKAY(ensure_tensor(m->dev, &m->x, 1, T, D, VKL_FP16));
  VKL_OKAY(ensure_tensor(m->dev, &m->xn, 1, T, D, VKL_FP16));
  VKL_OKAY(ensure_tensor(m->dev, &m->q, 1, T, m->dim_l, VKL_FP16));
  VKL_OKAY(ensure_tensor(m->dev, &m->k, 1, T, m->dim_l, VKL_FP16));
  VKL_OKAY(ensure_tensor(m->dev, &m->v, 1, T, m->dim_l, VKL_FP16));
  VKL_OKAY(ensure_tensor(m->dev, &m->ao, 1, T, m->dim_l, VKL_FP16));
  VKL_OKAY(ensure_tensor(m->dev, &m->t, 1, T, m->ffn_l, VKL_FP16));
  if (T >= gemm_min_rows(q8(m))) VKL_OKAY(ensure_tensor(m->dev, &m->gu32, 2, T, m->ffn_l, VKL_FP32));
  VKL_OKAY(ensure_tensor(m->dev, &m->toks, 1, 1, T, VKL_UINT32));
  const size_t sc = attention_scratch_bytes(1, m->heads_l, m->head_dim, m->splits);
  VKL_OKAY(ensure_tensor(m->dev, &m->attn_scratch, 1, 1, sc / 4, VKL_FP32));
  m->cap_T = T;
  return VKL_OK;
}

MvParams mv(const vkl_model *m, const vkl_tensor *w, const __half *x, __half *out, uint32_t M) {
  MvParams p = {};
  p.codes[0] = w->data();
  p.scales[0] = q8(m) ? w->scales() : nullptr;
  p.out[0] = out;
  p.x = x;
  p.nmat = 1;
  p.N = (uint32_t)w->h;
  p.K = (uint32_t)w->w;
  p.M = M;
  p.x_ld = p.K;
  p.out_ld = p.N;
  p.scale = 1.f;
  p.fp16_weights = !q8(m);
  p.use_pdl = 0;
  return p;
}

// Many-row projection on the tcgen05 tensor cores (Q8_0 weights are dequantised into the shared-memory tiles).
GemmParams gemm(vkl_model *m, const vkl_tensor *w, const __half *a, __half *out, uint32_t M) {
  GemmParams g = {};
  g.a = a;
  if (q8(m)) {
    g.w_codes = w->codes();
    g.w_scales = w->scales();
  } else {
    g.w = (const __half *)w->data();
  }
  g.c = out;
  g.M = M;
  g.N = (uint32_t)w->h;
  g.K = (uint32_t)w->w;
  g.scale = 1.f;
  g.error = (uint32_t *)m->state->data() + 6;
  m->gemm_used = true;
  return g;
}
bool use_gemm(const vkl_model *m, uint32_t rows) {
  static const bool off = [] { const char *e = getenv("VKLLAMA_PREFILL_GEMM"); return e && !strcmp(e, "0"); }();
  return !off && rows >= gemm_min_rows(q8(m)) && gemm_tcgen05_supported(rows, m->dim_l, m->cfg.dim) &&
         gemm_tcgen05_supported(rows, m->cfg.dim, m->dim_l) && gemm_tcgen05_supported(rows, m->ffn_l, m->cfg.dim) &&
         gemm_tcgen05_supported(rows, m->cfg.dim, m->ffn_l);
}

// Optional per-kernel timing of a pass: an event after every launch, tagged with
// the kernel's class (0 embedding, 1 norm+QKV, 2 attention, 3 o_proj, 4 gate/up,
// 5 down, 6 lm head, 7 arg-max).
struct Marker {
  std::vector<cudaEvent_t> ev;
  std::vector<int> cls;
  cudaStream_t s;
  void mark(int c) {
    cudaEvent_t e;
    cudaEventCreate(&e);
    cudaEventRecord(e, s);
    ev.push_back(e);
    cls.push_back(c);
  }
};
#define MARK(c) do { if (mk) mk->mark(c); } while (0)

// One pass over T tokens already in m->toks, first position in state[0].
// Leaves the last token's fp16/fp32 logits and its arg-max in state[2].
// `fill_only`: the pass only has to leave the T tokens' keys and values in the caches (it stops after the
// last block's attention and clips nothing); the one form tensor-parallel models run with T > 1, their
// K-split projections summed over the ranks by launch_tp_reduce_rows. `tok_off`: first token in m->toks.
int run_tokens(vkl_model *m, uint32_t T, bool pdl, Marker *mk = nullptr, bool fill_only = false, uint32_t tok_off = 0) {
  cudaStream_t s = m->stream;
  MARK(-1);
  const uint32_t D = m->cfg.dim, nl = m->cfg.layers;
  const bool dec = T == 1;
  __half *x = (__half *)m->x->data(), *xn = (__half *)m->xn->data();
  __half *qb = (__half *)m->q->data(), *kb = (__half *)m->k->data(), *vb = (__half *)m->v->data();
  __half *ao = (__half *)m->ao->data(), *tb = (__half *)m->t->data();
  const bool sharded = m->cfg.tp_size > 1;
  if (sharded && !(fill_only && T > 1 && T <= m->tp_pf_rows && use_gemm(m, T))) return fail(VKL_INTERNAL, "run_tokens: no sharded form of this pass");
  // K-split projection of a sharded model: fp32 partial sums into this rank's exchange region, then the sum over ranks
  auto reduce_rows = [&](GemmParams g, __half *xio, uint32_t nrows) -> int {
    const uint32_t seq = ++m->tp_pf_seq;
    const size_t region = m->tp_pf_off + (size_t)(seq & 1u) * m->tp_pf_rows * D * 4;
    g.c = nullptr;
    g.residual = nullptr;
    g.c_f32 = (float *)((char *)m->tp_buf + region);
    VKL_LAUNCH(1, launch_gemm_tcgen05(g, s));
    TpRowsParams r = {};
    for (uint32_t i = 0; i < m->cfg.tp_size; ++i) {
      r.part[i] = (const float *)((const char *)m->tp_peer[i] + region);
      r.flags[i] = (uint32_t *)((char *)m->tp_peer[i] + m->tp_pf_flag_off);
    }
    r.x = xio;
    r.n = (size_t)nrows * D;
    r.rank = m->cfg.tp_rank;
    r.tp = m->cfg.tp_size;
    r.seq = seq;
    r.wait_limit = m->wait_limit ? m->wait_limit : (1u << 24);
    r.error = (uint32_t *)m->state->data() + 6;
    VKL_LAUNCH(2, launch_tp_reduce_rows(r, m->dev->prop.multiProcessorCount, s));
    return VKL_OK;
  };
  VKL_LAUNCH(1, launch_embedding(m->tok_embd->data(), m->tok_embd->dtype == VKL_Q8_0, (const uint32_t *)m->toks->data() + tok_off, x, T,
                                 (uint32_t)m->tok_embd->h, D, 0, s));
  MARK(0);
  uint32_t rows = T;      // rows still alive (the last block keeps one: llama2.h:181-191)
  __half *xr = x;         // first live row of the residual stream
  for (uint32_t l = 0; l < nl; ++l) {
    Layer &y = m->L[l];
    const bool clip = (l == nl - 1) && T > 1 && !fill_only;
    // --- attention ---------------------------------------------------------
    MvParams p = mv(m, y.wk, dec ? x : xn, kb, T);
    p.codes[1] = y.wq->data(); p.codes[2] = y.wv->data();
    if (q8(m)) { p.scales[1] = y.wq->scales(); p.scales[2] = y.wv->scales(); }
    p.out[1] = qb; p.out[2] = vb;
    p.nmat = 3;
    if (dec) {
      p.norm_w = (const float *)y.attn_norm->data();
      p.eps = m->cfg.eps;
      p.use_pdl = pdl;
      VKL_LAUNCH(1, launch_matvec(p, EPI_PLAIN, true, s));
    } else if (use_gemm(m, T)) {
      VKL_LAUNCH(1, launch_rms_norm(x, (const float *)y.attn_norm->data(), xn, T, D, m->cfg.eps, s));
      VKL_LAUNCH(1, launch_gemm_tcgen05(gemm(m, y.wk, xn, kb, T), s));
      VKL_LAUNCH(1, launch_gemm_tcgen05(gemm(m, y.wq, xn, qb, T), s));
      VKL_LAUNCH(1, launch_gemm_tcgen05(gemm(m, y.wv, xn, vb, T), s));
    } else {
      VKL_LAUNCH(1, launch_rms_norm(x, (const float *)y.attn_norm->data(), xn, T, D, m->cfg.eps, s));
      VKL_LAUNCH((T + 63) / 64, launch_matvec(p, EPI_PLAIN, false, s));
    }
    MARK(1);
    AttnParams a = {};
    a.q = qb; a.k = kb; a.v = vb;
    a.kcache = (__half *)y.kcache->data(); a.vcache = (__half *)y.vcache->data();
    a.out = ao;
    a.freqc = (const float *)m->fc->data(); a.freqs = (const float *)m->fs->data();
    a.pos_dev = m->pos_dev();
    a.scratch = (float *)m->attn_scratch->data(); a.counters = (uint32_t *)m->attn_counters->data();
    a.T = T; a.heads = m->heads_l; a.dim = m->head_dim; a.maxlen = m->cfg.maxlen;
    a.splits = dec ? m->splits : 1;
    a.clip = clip;
    a.use_pdl = dec && pdl;
    VKL_LAUNCH(dec ? 1 : 2, launch_attention(a, s));
    MARK(2);
    if (fill_only && l == nl - 1) break;  // the caches are complete
    if (clip) {
      xr = x + (size_t)(T - 1) * D;
      rows = 1;
    }
    // --- o_proj + residual (add_op_(attn, in): llama2.h:193-196) -------------
    if (sharded) {
      VKL_OKAY(reduce_rows(gemm(m, y.wo, ao, xr, rows), xr, rows));
    } else if (use_gemm(m, rows)) {
      GemmParams g = gemm(m, y.wo, ao, xr, rows);
      g.residual = xr;
      VKL_LAUNCH(1, launch_gemm_tcgen05(g, s));
    } else {
      MvParams o = mv(m, y.wo, ao, xr, rows);
      o.residual = xr;
      o.use_pdl = dec && pdl;
      VKL_LAUNCH((rows + 63) / 64, launch_matvec(o, EPI_ADD, false, s));
    }
    MARK(3);
    // --- feed forward --------------------------------------------------------
    MvParams f = mv(m, y.gate, dec || rows == 1 ? xr : xn, tb, rows);
    f.codes[1] = y.up->data();
    if (q8(m)) f.scales[1] = y.up->scales();
    if (rows == 1) {
      f.norm_w = (const float *)y.ffn_norm->data();
      f.eps = m->cfg.eps;
      f.use_pdl = dec && pdl;
      VKL_LAUNCH(1, launch_matvec(f, EPI_SWIGLU, true, s));
    } else if (use_gemm(m, rows)) {
      VKL_LAUNCH(1, launch_rms_norm(xr, (const float *)y.ffn_norm->data(), xn, rows, D, m->cfg.eps, s));
      float *g32 = (float *)m->gu32->data(), *u32 = g32 + (size_t)rows * m->ffn_l;
      GemmParams g = gemm(m, y.gate, xn, nullptr, rows);
      g.c_f32 = g32;
      VKL_LAUNCH(1, launch_gemm_tcgen05(g, s));
      if (q8(m)) {
        g.w_codes = y.up->codes();
        g.w_scales = y.up->scales();
      } else {
        g.w = (const __half *)y.up->data();
      }
      g.c_f32 = u32;
      VKL_LAUNCH(1, launch_gemm_tcgen05(g, s));
      VKL_LAUNCH(1, launch_swiglu_f32(g32, u32, tb, (size_t)rows * m->ffn_l, s));
    } else {
      VKL_LAUNCH(1, launch_rms_norm(xr, (const float *)y.ffn_norm->data(), xn, rows, D, m->cfg.eps, s));
      VKL_LAUNCH((rows + 63) / 64, launch_matvec(f, EPI_SWIGLU, false, s));
    }
    MARK(4);
    if (sharded) {
      VKL_OKAY(reduce_rows(gemm(m, y.down, tb, xr, rows), xr, rows));
    } else if (use_gemm(m, rows)) {
      GemmParams g = gemm(m, y.down, tb, xr, rows);
      g.residual = xr;
      VKL_LAUNCH(1, launch_gemm_tcgen05(g, s));
    } else {
      MvParams d = mv(m, y.down, tb, xr, rows);
      d.residual = xr;
      d.use_pdl = dec && pdl;
      VKL_LAUNCH((rows + 63) / 64, launch_matvec(d, EPI_ADD, false, s));
    }
    MARK(5);
  }
  if (fill_only) return VKL_OK;
  // --- output layer: RMSNorm(1e-6) -> lm head -> fp32 cast (llama2.h:283-298) --
  if (T > 1 && nl == 0) xr = x + (size_t)(T - 1) * D;
  MvParams h = mv(m, m->output, xr, (__half *)m->logits16->data(), 1);
  h.norm_w = (const float *)m->output_norm->data();
  h.eps = m->cfg.final_eps;
  h.out_f32 = (float *)m->logits32->data();
  h.use_pdl = dec && pdl;
  VKL_LAUNCH(1, launch_matvec(h, EPI_PLAIN, true, s));
  MARK(6);
  VKL_LAUNCH(2, launch_argop((const __half *)m->logits16->data(), m->next_dev(), m->argpart->data(), 1, m->vocab_l, 0, s));
  MARK(7);
  return VKL_OK;
}

int launch_advance(vkl_model *m, uint32_t pos_inc) {
  advance_kernel<<<1, 1, 0, m->stream>>>(m->next_dev(), (uint32_t *)m->toks->data(), m->pos_dev(), m->step_dev(),
                                         (uint32_t *)m->out_ids->data(), m->out_cap, pos_inc);
  VKL_LAUNCH(1, cudaGetLastError());
  return VKL_OK;
}

// Builds the op table of the persistent decode kernel. Q8_0 weights, one GPU.
// VKLLAMA_DECODE=graph keeps the multi-kernel CUDA-graph step instead.
int build_mega(vkl_model *m) {
  if (m->mega_tried) return VKL_OK;
  m->mega_tried = true;
  const char *env = getenv("VKLLAMA_DECODE");
  if (env && !strcmp(env, "graph")) return VKL_OK;
  if (!q8(m) || m->tok_embd->dtype != VKL_Q8_0) return VKL_OK;
  const uint32_t tp = m->cfg.tp_size;
  if (tp > 1 && !m->tp_connected) return fail(VKL_FAILED_PRECONDITION, "model: tensor-parallel ranks are not connected (vkl_model_tp_connect)");
  const vkl_model_config &c = m->cfg;
  if ((int)c.dim > decode_mega_max_k() || (int)c.ffn > decode_mega_max_k() || (c.dim % 32) || (c.ffn % 32) || (m->head_dim & 1)) return VKL_OK;
  int coop = 0;
  VKL_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, m->dev->ordinal));
  if (!coop) return VKL_OK;
  const int G = m->dev->prop.multiProcessorCount;
  uint32_t splits = (uint32_t)G / m->heads_l;
  if (splits < 1) return VKL_OK;  // more heads than SMs: keep the graph path
  // One GPU: at most 8 splits per head. Tensor-parallel ranks have few heads each: there the
  // splits spread a head's cache rows over (nearly) all SMs, the attention op's time would not
  // shrink with the rank count otherwise.
  {
    const char *se = getenv("VKLLAMA_ATTN_SPLITS");
    const uint32_t cap = se ? std::max(1u, (uint32_t)atoi(se)) : (tp > 1 ? 32u : 8u);
    if (splits > cap) splits = cap;
  }
  const uint32_t max_blocks = std::max({c.dim, m->dim_l, m->ffn_l}) / 32;
  // Rows per attention split (VKLLAMA_SPLIT_ROWS; 0 = always all splits). Short contexts run one CTA
  // per head and skip the merge between CTAs; the default keeps a split's K rows within three ring stages.
  const char *sr_env = getenv("VKLLAMA_SPLIT_ROWS");
  const uint32_t split_rows = sr_env ? (uint32_t)atoi(sr_env) : 384u;
  const size_t xs_bytes = decode_mega_xs_bytes(max_blocks, m->head_dim, c.maxlen, splits, split_rows);
  // every tile a CTA gets of an op needs a reduction slot: QKV = 3 matrices of 32-row tiles, gate/up = one
  // tile per 16 outputs, the others one tile per 32 rows
  auto slots = [&](uint32_t tiles) { return (tiles + G - 1) / G; };
  const uint32_t red_slots = std::max({slots(3 * ((m->dim_l + 31) / 32)), slots((c.dim + 31) / 32), slots((m->ffn_l + 15) / 16), slots((m->vocab_l + 31) / 32)});
  uint32_t nst = (uint32_t)decode_mega_max_stages();  // as many ring stages as fit
  if (const char *rs = getenv("VKLLAMA_RING_STAGES")) nst = std::min(nst, std::max(2u, (uint32_t)atoi(rs)));  // experiments: a shallower ring
  while (nst >= 2 && decode_mega_smem(xs_bytes, nst, red_slots) > (size_t)m->dev->prop.sharedMemPerBlockOptin) --nst;
  if (nst < 2) return VKL_OK;
  int occ = 0;
  VKL_CUDA(decode_mega_occupancy(decode_mega_smem(xs_bytes, nst, red_slots), &occ));
  if (occ < 1) return VKL_OK;
  VKL_OKAY(ensure_rows(m, 1));

  std::vector<MegaOp> ops;
  uint32_t rot = 0;
  // Tagged activation buffers of the kernel (one 32-bit word per element): x [dim], k, q, v and the
  // attention output [dim_l each], the SwiGLU output [ffn_l].
  const size_t ll_words = (size_t)c.dim + 4 * (size_t)m->dim_l + m->ffn_l;
  VKL_OKAY(tensor_new(m->dev, 1, 1, ll_words, VKL_UINT32, &m->mega_ll));
  VKL_CUDA(cudaMemsetAsync(m->mega_ll->data(), 0, ll_words * 4, m->stream));
  {  // no op of the first launches may expect tag 0, the tag of the zeroed words
    const uint32_t one = 1;
    VKL_CUDA(cudaMemcpyAsync((uint32_t *)m->state->data() + 7, &one, 4, cudaMemcpyHostToDevice, m->stream));
  }
  uint32_t *x = (uint32_t *)m->mega_ll->data(), *kb = x + c.dim, *qb = kb + m->dim_l, *vb = qb + m->dim_l, *ao = vb + m->dim_l, *tb = ao + m->dim_l;
  uint32_t x_writer = 0;  // index of the op that last wrote the residual stream x
  int pack_status = VKL_OK;
  size_t pack_index = 0;
  auto matvec = [&](std::initializer_list<const vkl_tensor *> ws, const float *norm, float eps, const uint32_t *in, uint32_t src_op,
                    std::initializer_list<uint32_t *> outs, int epi) {
    MegaOp o = {};
    o.kind = MK_MATVEC;
    o.epi = epi;
    const vkl_tensor *w0 = *ws.begin();
    o.N = (uint32_t)w0->h;
    o.K = (uint32_t)w0->w;
    o.blocks = o.K / 32;
    o.nmat = (uint32_t)ws.size();
    const bool swiglu = epi == EPI_SWIGLU;
    o.tiles = swiglu ? (o.N + 15) / 16 : o.nmat * ((o.N + 31) / 32);
    // the op's weights in the kernel's stream layout (a second copy: the tiled planes stay for the
    // multi-token passes and the per-op API)
    {
      const uint8_t *planes[3] = {nullptr, nullptr, nullptr};
      int j = 0;
      for (const vkl_tensor *w : ws) planes[j++] = w->data();
      const size_t units = (size_t)o.tiles * o.blocks;
      const bool packed = pack_index < m->mega_packed.size();  // an earlier build of the tables packed it already
      vkl_tensor *pk = packed ? m->mega_packed[pack_index] : nullptr;
      if (!packed) {
        if (int st = tensor_new(m->dev, 1, 1, units * (MEGA_UNIT_CODES + MEGA_UNIT_SCALES) / 4, VKL_UINT32, &pk)) {
          pack_status = st;
          return 0u;
        }
        m->mega_packed.push_back(pk);
      }
      ++pack_index;
      uint8_t *codes = pk->data();
      if (!packed) {
        cudaError_t pe = launch_mega_pack(planes, o.nmat, swiglu ? 1 : 0, o.N, o.K, o.tiles, (uint32_t)G, codes, m->stream);
        count_launches(1);
        if (pe != cudaSuccess && pack_status == VKL_OK) pack_status = fail(VKL_INTERNAL, "decode kernel: packing the weights failed: %s", cudaGetErrorString(pe));
      }
      o.codes = codes;
    }
    int i = 0;
    for (uint32_t *p : outs) o.out_ll[i++] = p;
    o.norm_w = norm;
    o.eps = eps;
    o.in = in;
    o.src_op = src_op;
    o.res_op = x_writer;  // (read by the residual epilogues only: x is what they add to)
    o.tag_op = (uint32_t)ops.size();
    o.barrier_after = 0;
    o.rot = rot;
    rot = (rot + o.tiles) % (uint32_t)G;
    ops.push_back(o);
    return (uint32_t)ops.size() - 1;
  };
  // How the split partials of a head are merged (VKLLAMA_DECODE_COMBINE): "last" (default) = by the
  // split CTA that finishes last, inside the attention op; "separate" = a combine op after a grid barrier.
  const char *cenv = getenv("VKLLAMA_DECODE_COMBINE");
  const bool last_combine = !(cenv && !strcmp(cenv, "separate"));
  // Tensor parallelism: the all-reduce after o_proj and down runs inside their epilogues (EPI_REDUCE);
  // VKLLAMA_TP_ALLREDUCE=separate keeps it as an op of its own behind them (MK_ALLREDUCE).
  const char *arenv = getenv("VKLLAMA_TP_ALLREDUCE");
  const bool reduce_in_place = !(arenv && !strcmp(arenv, "separate"));
  MegaOp e = {};
  e.kind = MK_EMBED;
  ops.push_back(e);  // op 0 writes x
  for (uint32_t l = 0; l < c.layers; ++l) {
    Layer &y = m->L[l];
    const uint32_t qkv = matvec({y.wk, y.wq, y.wv}, (const float *)y.attn_norm->data(), c.eps, x, x_writer, {kb, qb, vb}, EPI_PLAIN);
    MegaOp a = {};
    a.kind = MK_ATTN_PART;
    a.kcache = (__half *)y.kcache->data();
    a.vcache = (__half *)y.vcache->data();
    a.src_op = qkv;
    // with one split per head the attention op writes the output itself, under the tag the reader expects
    a.tag_op = (uint32_t)ops.size() + (last_combine ? 0u : 1u);
    a.barrier_after = last_combine ? 0u : 1u;
    ops.push_back(a);
    uint32_t ao_writer = (uint32_t)ops.size() - 1;
    if (!last_combine) {
      MegaOp cb = {};
      cb.kind = MK_ATTN_COMBINE;
      cb.tag_op = (uint32_t)ops.size();
      ops.push_back(cb);
      ao_writer = (uint32_t)ops.size() - 1;
    }
    auto allreduce = [&](uint32_t res_writer) {
      MegaOp r = {};
      r.kind = MK_ALLREDUCE;
      r.N = c.dim;
      r.out_ll[0] = x;
      r.res_op = res_writer;
      r.tag_op = (uint32_t)ops.size();
      ops.push_back(r);
      return (uint32_t)ops.size() - 1;
    };
    uint32_t before = x_writer;
    x_writer = matvec({y.wo}, nullptr, 0.f, ao, ao_writer, {x}, tp > 1 ? (reduce_in_place ? EPI_REDUCE : EPI_PARTIAL) : EPI_ADD);
    if (tp > 1 && !reduce_in_place) x_writer = allreduce(before);
    const uint32_t gu = matvec({y.gate, y.up}, (const float *)y.ffn_norm->data(), c.eps, x, x_writer, {tb}, EPI_SWIGLU);
    before = x_writer;
    x_writer = matvec({y.down}, nullptr, 0.f, tb, gu, {x}, tp > 1 ? (reduce_in_place ? EPI_REDUCE : EPI_PARTIAL) : EPI_ADD);
    if (tp > 1 && !reduce_in_place) x_writer = allreduce(before);
  }
  matvec({m->output}, (const float *)m->output_norm->data(), c.final_eps, x, x_writer, {}, EPI_PLAIN);
  ops.back().out[0] = (__half *)m->logits16->data();  // plain fp16 + fp32 logits and arg-max candidates: a grid barrier follows
  ops.back().out_f32 = (float *)m->logits32->data();
  ops.back().track_argmax = 1;
  ops.back().barrier_after = 1;
  MegaOp am = {};
  am.kind = MK_ARGMAX;
  ops.push_back(am);

  if (pack_status != VKL_OK) return pack_status;
  // Stage tables: every CTA's ring stages for one token, in the order its consumers walk them
  // (the same cutting rule as the kernel: mega_stage_cut / mega_stage_advance).
  std::vector<std::vector<MegaStage>> per_cta(G);
  std::vector<uint32_t> op_stages;  // [mat-vec op][cta]
  std::vector<size_t> op_index;     // index into `ops` of every mat-vec op
  for (size_t oi = 0; oi < ops.size(); ++oi) {
    const MegaOp &o = ops[oi];
    if (o.kind == MK_ATTN_PART) {
      // the cached K and V rows of every (head, split) CTA go through the ring too: one marker
      // entry, which the kernel turns into as many stages as the token's KV length needs
      for (uint32_t cta = 0; cta < m->heads_l * splits; ++cta) {
        MegaStage e = {};
        e.n0 = MEGA_KV_MARK;
        e.src = (const uint8_t *)o.kcache;
        e.src2 = (const uint8_t *)o.vcache;
        per_cta[cta].push_back(e);
      }
      continue;
    }
    if (o.kind != MK_MATVEC) continue;
    op_index.push_back(oi);
    for (int cta = 0; cta < G; ++cta) {
      const size_t before = per_cta[cta].size();
      const uint32_t tile0 = ((uint32_t)cta + G - (o.rot % G)) % G;
      const uint32_t tl = tile0 < o.tiles ? (o.tiles - tile0 + G - 1) / G : 0u;
      // the CTA's units of the op are consecutive in the packed stream (mega_stream_tile): a stage is one range
      auto run = [&](uint32_t lt, uint32_t kg) {
        const size_t unit = (size_t)mega_stream_tile(tile0 + lt * (uint32_t)G, o.tiles, (uint32_t)G) * o.blocks + kg;
        return o.codes + unit * (MEGA_UNIT_CODES + MEGA_UNIT_SCALES);
      };
      uint32_t tm = 0, kg = 0;
      while (tm < tl) {
        const MegaCut cut = mega_stage_cut(kg, o.blocks, tm + 1 < tl);
        MegaStage e = {};
        e.n0 = cut.n0;
        e.n1 = cut.n1;
        e.tm = tm;
        e.kg = kg;
        e.src = run(tm, kg);
        if (cut.n1 && run(tm + 1, 0) != e.src + (size_t)cut.n0 * (MEGA_UNIT_CODES + MEGA_UNIT_SCALES))
          return fail(VKL_INTERNAL, "decode kernel: a stage's two runs are not consecutive");
        per_cta[cta].push_back(e);
        mega_stage_advance(cut, o.blocks, tm, kg);
      }
      op_stages.push_back((uint32_t)(per_cta[cta].size() - before));
    }
  }
  size_t stride = 0;
  for (auto &v : per_cta) stride = std::max(stride, v.size());
  std::vector<MegaStage> flat((size_t)G * stride);
  std::vector<uint32_t> counts(G);
  for (int cta = 0; cta < G; ++cta) {
    counts[cta] = (uint32_t)per_cta[cta].size();
    std::copy(per_cta[cta].begin(), per_cta[cta].end(), flat.begin() + (size_t)cta * stride);
  }
  VKL_OKAY(tensor_new(m->dev, 1, 1, flat.size() * sizeof(MegaStage) / 4, VKL_UINT32, &m->mega_stages));
  VKL_OKAY(tensor_new(m->dev, 1, 1, (size_t)G + op_stages.size(), VKL_UINT32, &m->mega_counts));  // totals, then per op
  VKL_CUDA(cudaMemcpyAsync(m->mega_stages->data(), flat.data(), flat.size() * sizeof(MegaStage), cudaMemcpyHostToDevice, m->stream));
  VKL_CUDA(cudaMemcpyAsync(m->mega_counts->data(), counts.data(), (size_t)G * 4, cudaMemcpyHostToDevice, m->stream));
  VKL_CUDA(cudaMemcpyAsync((uint32_t *)m->mega_counts->data() + G, op_stages.data(), op_stages.size() * 4, cudaMemcpyHostToDevice, m->stream));
  for (size_t k = 0; k < op_index.size(); ++k) ops[op_index[k]].stages_per_cta = (const uint32_t *)m->mega_counts->data() + G + k * (size_t)G;
  VKL_CUDA(cudaStreamSynchronize(m->stream));

  const size_t ob = ops.size() * sizeof(MegaOp);
  VKL_OKAY(tensor_new(m->dev, 1, 1, (ob + 3) / 4, VKL_UINT32, &m->mega_ops));
  VKL_OKAY(tensor_new(m->dev, 1, 1, 16, VKL_UINT32, &m->mega_sync));  // [0..3] barrier words, [4] error
  VKL_OKAY(tensor_new(m->dev, 1, 1, (size_t)G * 2, VKL_FP32, &m->mega_arg));
  VKL_OKAY(tensor_new(m->dev, 1, 1, 2 * (size_t)m->heads_l * splits * (m->head_dim + 4) + m->heads_l, VKL_FP32, &m->mega_attn));
  VKL_CUDA(cudaMemcpyAsync(m->mega_ops->data(), ops.data(), ob, cudaMemcpyHostToDevice, m->stream));
  VKL_CUDA(cudaMemsetAsync(m->mega_sync->data(), 0, 64, m->stream));
  VKL_CUDA(cudaStreamSynchronize(m->stream));
  MegaParams &p = m->mp;
  p = MegaParams{};
  p.ops = (const MegaOp *)m->mega_ops->data();
  p.stages = (const MegaStage *)m->mega_stages->data();
  p.stage_count = (const uint32_t *)m->mega_counts->data();
  p.stage_stride = (uint32_t)stride;
  p.nops = (uint32_t)ops.size();
  p.nbarriers = p.nops - 1;
  p.state = (uint32_t *)m->state->data();
  p.forced = (const uint32_t *)m->forced->data();
  p.tp_rank = (uint32_t)c.tp_rank;
  p.tp_size = tp;
  p.tp_flag_off = m->tp_flag_off;
  for (int i = 0; i < 8; ++i) p.tp_peer[i] = m->tp_peer[i];
  p.tok = (uint32_t *)m->toks->data();
  p.out_ids = (uint32_t *)m->out_ids->data();
  p.out_cap = m->out_cap;
  p.embd = m->tok_embd->data();
  p.embd_rows = (uint32_t)m->tok_embd->h;
  p.x = x; p.q = qb; p.k = kb; p.v = vb; p.ao = ao;  // tagged words
  p.freqc = (const float *)m->fc->data();
  p.freqs = (const float *)m->fs->data();
  p.attn_scratch = (float *)m->mega_attn->data();
  {
    const char *cenv = getenv("VKLLAMA_DECODE_COMBINE");
    p.attn_merge = cenv && !strcmp(cenv, "separate") ? 0u : 1u;
    uint32_t *counters = (uint32_t *)(p.attn_scratch + 2 * (size_t)m->heads_l * splits * (m->head_dim + 4));
    p.attn_counters = p.attn_merge == 1 ? counters : nullptr;
    VKL_CUDA(cudaMemsetAsync(m->mega_attn->data(), 0, (2 * (size_t)m->heads_l * splits * (m->head_dim + 4) + m->heads_l) * 4, m->stream));
  }
  p.arg_scratch = (float *)m->mega_arg->data();
  p.bar = (unsigned long long *)m->mega_sync->data();
  p.error = (uint32_t *)m->mega_sync->data() + 4;
  p.dim = c.dim; p.heads = m->heads_l; p.head_dim = m->head_dim; p.maxlen = c.maxlen; p.splits = splits; p.vocab = m->vocab_l;
  p.xs_bytes = (uint32_t)xs_bytes;
  p.xmax_blocks = max_blocks;
  {
    p.nst = nst;
    p.red_slots = red_slots;
    p.timing_mode = (getenv("VKLLAMA_DEBUG_NOCOPY") ? 2 : 0) | (getenv("VKLLAMA_DEBUG_NOMATH") ? 4 : 0) | (getenv("VKLLAMA_DEBUG_INSTANCE") ? 16 : 0) |
                    (getenv("VKLLAMA_DEBUG_NOBODY") ? 64 : 0) | (getenv("VKLLAMA_DEBUG_NOHANDSHAKE") ? 128 : 0);  // diagnostics
    const char *bp = getenv("VKLLAMA_BARRIER_POLLERS");
    p.barrier_pollers = bp ? std::min(std::max((uint32_t)atoi(bp), 1u), 8u) : 1u;
    p.split_rows = split_rows;
  }
  // One bound for every wait of the kernel (about half a microsecond per poll: 2^21 polls are a second or
  // two; tensor-parallel ranks get eight times that, for a rank that starts its launch late).
  p.wait_limit = m->wait_limit ? m->wait_limit : (tp > 1 ? (1u << 24) : (1u << 21));
  m->mega_grid = G;
  m->mega_ready = true;
  return VKL_OK;
}

__global__ void bump_sequence_kernel(uint32_t *seq, uint32_t by) { *seq += by; }

// Start of a one-token call: position, step counter, no forced tokens, the token itself (one launch instead of
// three small copies).
__global__ void begin_token_kernel(uint32_t *state, uint32_t *tok, uint32_t pos, uint32_t id) {
  state[0] = pos;
  state[1] = 0;
  state[5] = 0;
  tok[0] = id;
}

// SM cycles and nanoseconds of one thread spinning for about 50 us: the SM clock a profiled
// launch converts its cycle counts with.
__global__ void clock_probe_kernel(unsigned long long *out) {
  unsigned long long t0, t1, c0 = clock64();
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  do {
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
  } while (t1 - t0 < 50000ull);
  out[0] = clock64() - c0;
  out[1] = t1 - t0;
}

// After a batch of decode launches: a wait that timed out inside the kernel is
// reported as an error and the barrier words are reset.
int check_mega(vkl_model *m) {
  if (!m->mega_ready) return VKL_OK;
  uint32_t err = 0;
  VKL_CUDA(cudaMemcpyAsync(&err, m->mp.error, 4, cudaMemcpyDeviceToHost, m->stream));
  VKL_CUDA(cudaStreamSynchronize(m->stream));
  if (err) {
    cudaMemsetAsync(m->mega_sync->data(), 0, 64, m->stream);
    if (m->mp.attn_counters) cudaMemsetAsync(m->mp.attn_counters, 0, (size_t)m->heads_l * 4, m->stream);
    // the aborted launch did not advance the ops' sequence base: words it tagged must not look current
    bump_sequence_kernel<<<1, 1, 0, m->stream>>>((uint32_t *)m->state->data() + 7, m->mp.nops);
    cudaStreamSynchronize(m->stream);
    // Under tensor parallelism the aborted launch leaves the ranks out of step (all-reduce and arg-max
    // sequence numbers, words already pushed under the number a retry would expect): the model refuses
    // further steps until every rank has called vkl_model_tp_connect again, between two host barriers.
    if (m->cfg.tp_size > 1) m->tp_failed = true;
    return fail(VKL_INTERNAL, "decode kernel: a bounded wait ran out (code %u: 1 weight stage, 2 ring slot, 3 grid barrier, 4 all-reduce, 5 arg-max exchange, 6 tagged input)", err);
  }
  return VKL_OK;
}

// After a pass that ran tensor-core GEMMs (stream already synchronised): report a wait that ran out.
int check_gemm(vkl_model *m) {
  if (!m->gemm_used) return VKL_OK;
  m->gemm_used = false;
  uint32_t err = 0;
  VKL_CUDA(cudaMemcpy(&err, (uint32_t *)m->state->data() + 6, 4, cudaMemcpyDeviceToHost));
  if (err) {
    cudaMemset((uint32_t *)m->state->data() + 6, 0, 4);
    if (err == 16u) {  // the ranks' all-reduce counters are out of step from here on
      m->tp_failed = true;
      return fail(VKL_INTERNAL, "prefill: the wait for another tensor-parallel rank's partial sums ran out");
    }
    return fail(VKL_INTERNAL, "prefill GEMM: a bounded mbarrier wait ran out");
  }
  return VKL_OK;
}

int build_decode_graph(vkl_model *m);

// Enqueue one decode step: the persistent kernel when available, else the graph.
int decode_step(vkl_model *m) {
  if (m->tp_failed)
    return fail(VKL_FAILED_PRECONDITION, "model: a wait on another tensor-parallel rank ran out earlier; reconnect the ranks (vkl_model_tp_connect on every rank, between host barriers) before the next step");
  if (m->mega_ready) {
    VKL_LAUNCH(1, launch_decode_mega(m->mp, m->mega_grid, m->stream));
    return VKL_OK;
  }
  VKL_CUDA(cudaGraphLaunch(m->decode_graph, m->stream));
  count_launches(5 * m->cfg.layers + 5);
  return VKL_OK;
}

int prepare_decode(vkl_model *m) {
  VKL_OKAY(ensure_rows(m, 1));
  VKL_OKAY(build_mega(m));
  if (!m->mega_ready) VKL_OKAY(build_decode_graph(m));
  return VKL_OK;
}

int build_decode_graph(vkl_model *m) {
  if (m->decode_graph) return VKL_OK;
  VKL_OKAY(ensure_rows(m, 1));
  cudaGraph_t g = nullptr;
  VKL_CUDA(cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeRelaxed));
  int st = run_tokens(m, 1, m->use_pdl);
  if (st == VKL_OK) st = launch_advance(m, 1);
  cudaError_t e = cudaStreamEndCapture(m->stream, &g);
  if (st != VKL_OK) {
    if (g) cudaGraphDestroy(g);
    return st;
  }
  if (e != cudaSuccess) return fail(VKL_INTERNAL, "decode graph capture failed: %s", cudaGetErrorString(e));
  e = cudaGraphInstantiate(&m->decode_graph, g, 0);
  cudaGraphDestroy(g);
  if (e != cudaSuccess) {
    m->decode_graph = nullptr;
    return fail(VKL_INTERNAL, "decode graph instantiation failed: %s", cudaGetErrorString(e));
  }
  return VKL_OK;
}

int check_ready(vkl_model *m) {
  if (!m) return fail(VKL_INVALID_ARGUMENT, "model: null handle");
  if (!m->tok_embd || !m->output || !m->output_norm) return fail(VKL_FAILED_PRECONDITION, "model: token_embd/output/output_norm weights are not set");
  for (uint32_t l = 0; l < m->cfg.layers; ++l) {
    Layer &y = m->L[l];
    if (!y.attn_norm || !y.ffn_norm || !y.wq || !y.wk || !y.wv || !y.wo || !y.gate || !y.up || !y.down)
      return fail(VKL_FAILED_PRECONDITION, "model: weights of block %u are incomplete", l);
  }
  return VKL_OK;
}

// Destination slot and shard geometry of a GGUF tensor name.
struct Slot {
  vkl_tensor **dst;
  uint32_t rows, cols;        // full shape
  uint32_t r0, nr, c0, nc;    // this rank's window
  bool norm;
  uint64_t synth_id;
};

int find_slot(vkl_model *m, const char *name, Slot *s) {
  const vkl_model_config &c = m->cfg;
  const uint32_t tp = c.tp_size, rk = c.tp_rank;
  auto full = [&](vkl_tensor **d, uint32_t r, uint32_t k, uint64_t id) { *s = Slot{d, r, k, 0, r, 0, k, false, id}; };
  auto rowsplit = [&](vkl_tensor **d, uint32_t r, uint32_t k, uint64_t id) { *s = Slot{d, r, k, rk * (r / tp), r / tp, 0, k, false, id}; };
  auto colsplit = [&](vkl_tensor **d, uint32_t r, uint32_t k, uint64_t id) { *s = Slot{d, r, k, 0, r, rk * (k / tp), k / tp, false, id}; };
  auto norm = [&](vkl_tensor **d, uint64_t id) { *s = Slot{d, 1, c.dim, 0, 1, 0, c.dim, true, id}; };
  const uint64_t g = (uint64_t)c.layers * 16;
  if (!strcmp(name, "token_embd.weight")) { full(&m->tok_embd, c.vocab, c.dim, g + 0); return VKL_OK; }
  if (!strcmp(name, "output_norm.weight")) { norm(&m->output_norm, g + 1); return VKL_OK; }
  if (!strcmp(name, "output.weight")) { rowsplit(&m->output, c.vocab, c.dim, g + 2); return VKL_OK; }
  unsigned b = 0;
  char kind[64];
  if (sscanf(name, "blk.%u.%63s", &b, kind) == 2 && b < c.layers) {
    Layer &y = m->L[b];
    const uint64_t id = (uint64_t)b * 16;
    if (!strcmp(kind, "attn_norm.weight")) { norm(&y.attn_norm, id + 0); return VKL_OK; }
    if (!strcmp(kind, "attn_q.weight")) { rowsplit(&y.wq, c.dim, c.dim, id + 1); return VKL_OK; }
    if (!strcmp(kind, "attn_k.weight")) { rowsplit(&y.wk, c.dim, c.dim, id + 2); return VKL_OK; }
    if (!strcmp(kind, "attn_v.weight")) { rowsplit(&y.wv, c.dim, c.dim, id + 3); return VKL_OK; }
    if (!strcmp(kind, "attn_output.weight")) { colsplit(&y.wo, c.dim, c.dim, id + 4); return VKL_OK; }
    if (!strcmp(kind, "ffn_norm.weight")) { norm(&y.ffn_norm, id + 5); return VKL_OK; }
    if (!strcmp(kind, "ffn_gate.weight")) { rowsplit(&y.gate, c.ffn, c.dim, id + 6); return VKL_OK; }
    if (!strcmp(kind, "ffn_up.weight")) { rowsplit(&y.up, c.ffn, c.dim, id + 7); return VKL_OK; }
    if (!strcmp(kind, "ffn_down.weight")) { colsplit(&y.down, c.dim, c.ffn, id + 8); return VKL_OK; }
  }
  return fail(VKL_INVALID_ARGUMENT, "model: tensor name '%s' is not part of a Llama-2 model with %u blocks", name, c.layers);
}

const char *kLayerNames[9] = {"attn_norm", "attn_q", "attn_k", "attn_v", "attn_output", "ffn_norm", "ffn_gate", "ffn_up", "ffn_down"};

}  // namespace

extern "C" {

int vkl_model_create(vkl_device *dev, const vkl_model_config *cfg, vkl_model **out) {
  if (!dev || !cfg || !out) return fail(VKL_INVALID_ARGUMENT, "model_create: null argument");
  const vkl_model_config &c = *cfg;
  if (!c.dim || !c.heads || !c.ffn || !c.vocab || !c.maxlen || c.dim % c.heads)
    return fail(VKL_INVALID_ARGUMENT, "model_create: bad dimensions (dim %u, heads %u, ffn %u, vocab %u, maxlen %u)", c.dim, c.heads, c.ffn, c.vocab, c.maxlen);
  if (c.weight_dtype != VKL_Q8_0 && c.weight_dtype != VKL_FP16) return fail(VKL_INVALID_ARGUMENT, "model_create: weight dtype %d is unsupported (Q8_0 or FP16)", c.weight_dtype);
  const uint32_t hd = c.dim / c.heads;
  if (hd > 128 || (hd & 7)) return fail(VKL_UNIMPLEMENTED, "model_create: head dim %u is unsupported (multiple of 8, at most 128)", hd);
  const uint32_t tp = c.tp_size < 1 ? 1 : c.tp_size;
  if (c.tp_rank < 0 || (uint32_t)c.tp_rank >= tp) return fail(VKL_INVALID_ARGUMENT, "model_create: tp_rank %d outside tp_size %u", c.tp_rank, tp);
  if (c.heads % tp || (c.ffn / tp) % 32 || c.ffn % tp || (c.dim / tp) % 32 || c.vocab % tp)
    return fail(VKL_INVALID_ARGUMENT, "model_create: tp_size %u does not divide heads/ffn/dim/vocab on 32-column boundaries", tp);
  if (c.weight_dtype == VKL_FP16 && ((c.dim & 7) || (c.ffn & 7))) return fail(VKL_UNIMPLEMENTED, "model_create: FP16 weights need widths that are multiples of 8");
  if (tp > 8) return fail(VKL_UNIMPLEMENTED, "model_create: at most 8 tensor-parallel ranks");
  if (tp > 1 && c.weight_dtype != VKL_Q8_0) return fail(VKL_UNIMPLEMENTED, "model_create: tensor parallelism is built for Q8_0 weights");
  VKL_CUDA(cudaSetDevice(dev->ordinal));
  vkl_model *m = new vkl_model();
  m->dev = dev;
  m->cfg = c;
  m->cfg.tp_size = tp;
  m->head_dim = hd;
  m->heads_l = c.heads / tp;
  m->dim_l = m->heads_l * hd;
  m->ffn_l = c.ffn / tp;
  m->vocab_l = c.vocab / tp;
  m->L.resize(c.layers);
  auto bail = [&](int st) {
    delete m;
    return st;
  };
  cudaError_t e = cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) return bail(fail(VKL_INTERNAL, "cudaStreamCreate: %s", cudaGetErrorString(e)));
  dev->add_stream(m->stream);
  cudaEventCreate(&m->ev0);
  cudaEventCreate(&m->ev1);
  cudaEventCreate(&m->ev2);
  for (auto &l : m->L) {
    if (int st = tensor_new(dev, m->heads_l, c.maxlen, hd, VKL_FP16, &l.kcache)) return bail(st);
    if (int st = tensor_new(dev, m->heads_l, c.maxlen, hd, VKL_FP16, &l.vcache)) return bail(st);
    cudaMemsetAsync(l.kcache->data(), 0, l.kcache->device_bytes(), m->stream);
    cudaMemsetAsync(l.vcache->data(), 0, l.vcache->device_bytes(), m->stream);
  }
  // Positions up to 2*maxlen are valid, the size the reference gives its tables (rope.cpp:73-76).
  if (int st = rope_tables(dev, m->stream, hd, 2 * c.maxlen, &m->fc, &m->fs)) return bail(st);
  m->splits = 8;
  m->out_cap = 2 * c.maxlen + 16;
  int st = VKL_OK;
  if ((st = tensor_new(dev, 1, 1, m->vocab_l, VKL_FP16, &m->logits16)) || (st = tensor_new(dev, 1, 1, m->vocab_l, VKL_FP32, &m->logits32)) ||
      (st = tensor_new(dev, 1, 1, 8, VKL_UINT32, &m->state)) || (st = tensor_new(dev, 1, 1, c.maxlen, VKL_UINT32, &m->forced)) || (st = tensor_new(dev, 1, 1, m->out_cap, VKL_UINT32, &m->out_ids)) ||
      (st = tensor_new(dev, 1, 1, argop_partials_bytes(1, m->vocab_l) / 4 + 2, VKL_FP32, &m->argpart)) ||
      (st = tensor_new(dev, 1, 1, m->heads_l, VKL_UINT32, &m->attn_counters)))
    return bail(st);
  cudaMemsetAsync(m->state->data(), 0, 32, m->stream);
  if (tp > 1) {
    m->tp_flag_off = 4 * tp * c.dim;  // partial sums: [2 parities][tp][dim] words of {fp32 sum, sequence number}
    m->tp_bytes = ((size_t)m->tp_flag_off + 64) * 4;
    m->tp_pf_rows = std::min(c.maxlen, 1024u);
    m->tp_pf_off = (m->tp_bytes + 255) / 256 * 256;
    m->tp_pf_flag_off = m->tp_pf_off + 2 * (size_t)m->tp_pf_rows * c.dim * 4;
    m->tp_bytes = m->tp_pf_flag_off + 64;
    if (cudaMalloc(&m->tp_buf, m->tp_bytes) != cudaSuccess) return bail(fail(VKL_RESOURCE_EXHAUSTED, "model_create: exchange buffer allocation failed"));
    cudaMemsetAsync(m->tp_buf, 0, m->tp_bytes, m->stream);
    m->tp_peer[c.tp_rank] = m->tp_buf;
  }
  cudaMemsetAsync(m->attn_counters->data(), 0, m->attn_counters->device_bytes(), m->stream);
  if ((st = ensure_rows(m, 1))) return bail(st);
  e = cudaStreamSynchronize(m->stream);
  if (e != cudaSuccess) return bail(fail(VKL_INTERNAL, "model_create: %s", cudaGetErrorString(e)));
  *out = m;
  return VKL_OK;
}

int vkl_model_destroy(vkl_model *m) {
  if (!m) return VKL_OK;
  cudaSetDevice(m->dev->ordinal);
  cudaStreamSynchronize(m->stream);
  delete m;
  return VKL_OK;
}

// New weights: the decode kernel's packed copies and tables, if already built, are stale.
static void drop_packed(vkl_model *m) {
  if (m->mega_packed.empty() && !m->mega_tried) return;
  cudaStreamSynchronize(m->stream);
  for (vkl_tensor *t : m->mega_packed) vkl_tensor_release(t);
  m->mega_packed.clear();
  for (vkl_tensor **t : {&m->mega_ops, &m->mega_sync, &m->mega_arg, &m->mega_attn, &m->mega_stages, &m->mega_counts, &m->mega_ll}) {
    vkl_tensor_release(*t);
    *t = nullptr;
  }
  m->mega_ready = m->mega_tried = false;
}

int vkl_model_set_weight(vkl_model *m, const char *name, int dtype, const void *data, size_t bytes) {
  if (!m || !name || !data) return fail(VKL_INVALID_ARGUMENT, "model_set_weight: null argument");
  VKL_CUDA(cudaSetDevice(m->dev->ordinal));
  drop_packed(m);
  Slot s;
  VKL_OKAY(find_slot(m, name, &s));
  if (s.norm) {
    if (dtype != VKL_FP32) return fail(VKL_INVALID_ARGUMENT, "model_set_weight: %s must be FP32 (rms_norm.cpp:33), got dtype %d", name, dtype);
    if (bytes != (size_t)s.cols * 4) return fail(VKL_INVALID_ARGUMENT, "model_set_weight: %s takes %zu bytes, got %zu", name, (size_t)s.cols * 4, bytes);
    VKL_OKAY(ensure_tensor(m->dev, s.dst, 1, 1, s.cols, VKL_FP32));
    VKL_CUDA(cudaMemcpyAsync((*s.dst)->data(), data, bytes, cudaMemcpyHostToDevice, m->stream));
    VKL_CUDA(cudaStreamSynchronize(m->stream));
    return VKL_OK;
  }
  if (dtype != m->cfg.weight_dtype) return fail(VKL_INVALID_ARGUMENT, "model_set_weight: %s has dtype %d but the model was created for %d", name, dtype, m->cfg.weight_dtype);
  const bool isq = dtype == VKL_Q8_0;
  const size_t row_b = isq ? (size_t)(s.cols / 32) * 34 : (size_t)s.cols * 2;
  if (isq && s.cols % 32) return fail(VKL_UNIMPLEMENTED, "model_set_weight: Q8_0 rows must be whole blocks");
  if (bytes != row_b * s.rows) return fail(VKL_INVALID_ARGUMENT, "model_set_weight: %s takes %zu bytes, got %zu", name, row_b * s.rows, bytes);
  // Cut this rank's window out of the full tensor on the host (block aligned).
  const size_t win_row_b = isq ? (size_t)(s.nc / 32) * 34 : (size_t)s.nc * 2;
  const size_t col_off = isq ? (size_t)(s.c0 / 32) * 34 : (size_t)s.c0 * 2;
  const uint8_t *src = (const uint8_t *)data;
  std::vector<uint8_t> win;
  const uint8_t *up = src + (size_t)s.r0 * row_b;
  if (s.nc != s.cols) {
    win.resize(win_row_b * s.nr);
    for (uint32_t r = 0; r < s.nr; ++r) memcpy(&win[r * win_row_b], src + (size_t)(s.r0 + r) * row_b + col_off, win_row_b);
    up = win.data();
  }
  VKL_OKAY(ensure_tensor(m->dev, s.dst, 1, s.nr, s.nc, dtype));
  if (isq) {
    void *tmp = nullptr;
    VKL_OKAY(m->dev->alloc(win_row_b * s.nr, &tmp));
    cudaError_t e = cudaMemcpyAsync(tmp, up, win_row_b * s.nr, cudaMemcpyHostToDevice, m->stream);
    if (e == cudaSuccess) e = launch_q8_repack((const uint8_t *)tmp, (*s.dst)->data(), s.nr, s.nc, m->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(m->stream);
    m->dev->release(tmp, win_row_b * s.nr);
    count_launches(1);
    if (e != cudaSuccess) return fail(VKL_INTERNAL, "model_set_weight: %s", cudaGetErrorString(e));
  } else {
    VKL_CUDA(cudaMemcpyAsync((*s.dst)->data(), up, win_row_b * s.nr, cudaMemcpyHostToDevice, m->stream));
    VKL_CUDA(cudaStreamSynchronize(m->stream));
  }
  return VKL_OK;
}

int vkl_model_synth_weights(vkl_model *m, uint64_t seed, float wstd, float nstd) {
  if (!m) return fail(VKL_INVALID_ARGUMENT, "model_synth_weights: null model");
  VKL_CUDA(cudaSetDevice(m->dev->ordinal));
  drop_packed(m);
  std::vector<std::string> names = {"token_embd.weight", "output_norm.weight", "output.weight"};
  for (uint32_t l = 0; l < m->cfg.layers; ++l)
    for (const char *k : kLayerNames) names.push_back("blk." + std::to_string(l) + "." + k + ".weight");
  void *tmp = nullptr;
  size_t tmp_b = 0;
  for (auto &nm : names) {
    Slot s;
    VKL_OKAY(find_slot(m, nm.c_str(), &s));
    if (s.norm) {
      VKL_OKAY(ensure_tensor(m->dev, s.dst, 1, 1, s.cols, VKL_FP32));
      VKL_LAUNCH(1, launch_synth_f32((float *)(*s.dst)->data(), seed, s.synth_id, 0, s.cols, 1.f, nstd, m->stream));
      continue;
    }
    VKL_OKAY(ensure_tensor(m->dev, s.dst, 1, s.nr, s.nc, m->cfg.weight_dtype));
    if (q8(m)) {
      const size_t need = (size_t)s.nr * (s.nc / 32) * 34;
      if (need > tmp_b) {
        if (tmp) {
          VKL_CUDA(cudaStreamSynchronize(m->stream));
          m->dev->release(tmp, tmp_b);
        }
        VKL_OKAY(m->dev->alloc(need, &tmp));
        tmp_b = need;
      }
      VKL_LAUNCH(1, launch_synth_q8((uint8_t *)tmp, seed, s.synth_id, s.nr, s.nc, 0.f, wstd, s.r0, s.c0, s.cols, m->stream));
      VKL_LAUNCH(1, launch_q8_repack((const uint8_t *)tmp, (*s.dst)->data(), s.nr, s.nc, m->stream));
    } else {
      if (s.nc != s.cols) return fail(VKL_UNIMPLEMENTED, "model_synth_weights: column-split FP16 shards are not generated on the device");
      VKL_LAUNCH(1, launch_synth_f16((__half *)(*s.dst)->data(), seed, s.synth_id, (uint64_t)s.r0 * s.cols, (uint64_t)s.nr * s.cols, 0.f, wstd, m->stream));
    }
  }
  VKL_CUDA(cudaStreamSynchronize(m->stream));
  if (tmp) m->dev->release(tmp, tmp_b);
  return VKL_OK;
}

int vkl_model_forward(vkl_model *m, const uint32_t *toks, size_t n, size_t offset, float *logits_out) {
  VKL_OKAY(check_ready(m));
  if (!toks || !logits_out) return fail(VKL_INVALID_ARGUMENT, "model_forward: null argument");
  if (n == 0) return fail(VKL_INVALID_ARGUMENT, "model_forward: no tokens");
  if (n > m->cfg.maxlen) return fail(VKL_OUT_OF_RANGE, "model_forward: %zu tokens exceed the context length %u", n, m->cfg.maxlen);
  if (offset + n > (size_t)2 * m->cfg.maxlen) return fail(VKL_OUT_OF_RANGE, "model_forward: position %zu is beyond the RoPE table (2*maxlen)", offset + n);
  VKL_CUDA(cudaSetDevice(m->dev->ordinal));
  VKL_OKAY(ensure_rows(m, (uint32_t)n));
  if (n == 1 || m->cfg.tp_size > 1) VKL_OKAY(prepare_decode(m));
  if (n > 1 && m->cfg.tp_size > 1) {
    // Sharded model, several tokens: all but the last fill the caches (many-token passes where they are long
    // enough for the tensor-core path, else token by token through the decode kernel, which feeds itself the
    // next id), the last goes through the decode kernel and leaves this rank's slice of its logits. The last
    // block's query is rotated at its own position here, not at the call's first (the single-GPU form keeps the
    // reference's quirk, this one does not).
    if (!m->mega_ready) return fail(VKL_UNIMPLEMENTED, "model_forward: tensor-parallel models need the persistent decode kernel");
    if (offset + n > m->cfg.maxlen) return fail(VKL_OUT_OF_RANGE, "model_forward: multi-token calls of a tensor-parallel model must end inside the context length");
    if (m->tp_failed) return decode_step(m);  // reports the state
    const uint32_t st[2] = {(uint32_t)offset, 0};
    const uint32_t nf = (uint32_t)(offset + n);
    VKL_CUDA(cudaMemcpyAsync(m->state->data(), st, 8, cudaMemcpyHostToDevice, m->stream));
    VKL_CUDA(cudaMemcpyAsync((uint32_t *)m->state->data() + 5, &nf, 4, cudaMemcpyHostToDevice, m->stream));
    VKL_CUDA(cudaMemcpyAsync(m->toks->data(), toks, n * 4, cudaMemcpyHostToDevice, m->stream));
    VKL_CUDA(cudaMemcpyAsync((uint32_t *)m->forced->data() + offset, toks, n * 4, cudaMemcpyHostToDevice, m->stream));
    size_t done = 0;
    while (n - 1 - done >= gemm_min_rows(q8(m))) {
      const uint32_t T = (uint32_t)std::min<size_t>(n - 1 - done, m->tp_pf_rows);
      if (!use_gemm(m, T)) break;
      const uint32_t at = (uint32_t)(offset + done);
      VKL_CUDA(cudaMemcpyAsync(m->state->data(), &at, 4, cudaMemcpyHostToDevice, m->stream));
      VKL_OKAY(run_tokens(m, T, false, nullptr, true, (uint32_t)done));
      done += T;
    }
    if (done) {
      const uint32_t at = (uint32_t)(offset + done);
      VKL_CUDA(cudaMemcpyAsync(m->state->data(), &at, 4, cudaMemcpyHostToDevice, m->stream));
      VKL_CUDA(cudaMemcpyAsync(m->toks->data(), (const uint32_t *)m->toks->data() + done, 4, cudaMemcpyDeviceToDevice, m->stream));
    }
    for (size_t i = done; i < n; ++i) VKL_OKAY(decode_step(m));
    VKL_CUDA(cudaMemcpyAsync(logits_out, m->logits32->data(), (size_t)m->vocab_l * 4, cudaMemcpyDeviceToHost, m->stream));
    VKL_CUDA(cudaStreamSynchronize(m->stream));
    VKL_OKAY(check_gemm(m));
    return check_mega(m);
  }
  if (n == 1) {
    // The per-token call of a host-driven loop: one small launch sets the step up, the logits and the decode
    // kernel's error word come back through pinned memory behind one synchronisation.
    const size_t lb = (size_t)m->vocab_l * 4;
    if (!m->pin) VKL_CUDA(cudaHostAlloc((void **)&m->pin, lb + 16, cudaHostAllocDefault));
    begin_token_kernel<<<1, 1, 0, m->stream>>>((uint32_t *)m->state->data(), (uint32_t *)m->toks->data(), (uint32_t)offset, toks[0]);
    VKL_LAUNCH(1, cudaGetLastError());
    VKL_OKAY(decode_step(m));
    VKL_CUDA(cudaMemcpyAsync(m->pin, m->logits32->data(), lb, cudaMemcpyDeviceToHost, m->stream));
    uint32_t *errw = (uint32_t *)(m->pin + lb);
    *errw = 0;
    if (m->mega_ready) VKL_CUDA(cudaMemcpyAsync(errw, m->mp.error, 4, cudaMemcpyDeviceToHost, m->stream));
    VKL_CUDA(cudaStreamSynchronize(m->stream));
    memcpy(logits_out, m->pin, lb);
    if (*errw) VKL_OKAY(check_mega(m));  // (reads the word again, resets the kernel's state, reports)
    VKL_OKAY(check_gemm(m));
    return VKL_OK;
  }
  VKL_CUDA(cudaMemsetAsync((uint32_t *)m->state->data() + 5, 0, 4, m->stream));
  const uint32_t st[2] = {(uint32_t)offset, 0};
  VKL_CUDA(cudaMemcpyAsync(m->state->data(), st, 8, cudaMemcpyHostToDevice, m->stream));
  VKL_CUDA(cudaMemcpyAsync(m->toks->data(), toks, n * 4, cudaMemcpyHostToDevice, m->stream));
  if (n == 1) {
    VKL_OKAY(decode_step(m));
  } else {
    VKL_OKAY(run_tokens(m, (uint32_t)n, false));
  }
  VKL_CUDA(cudaMemcpyAsync(logits_out, m->logits32->data(), (size_t)m->vocab_l * 4, cudaMemcpyDeviceToHost, m->stream));
  VKL_CUDA(cudaStreamSynchronize(m->stream));
  if (n == 1) VKL_OKAY(check_mega(m));
  VKL_OKAY(check_gemm(m));
  return VKL_OK;
}

int vkl_model_generate(vkl_model *m, const uint32_t *prompt, size_t n_prompt, size_t n_gen, uint32_t *out_ids, float *prefill_ms,
                       float *decode_ms) {
  VKL_OKAY(check_ready(m));
  if (!prompt || !out_ids) return fail(VKL_INVALID_ARGUMENT, "model_generate: null argument");
  if (n_prompt == 0 || n_gen == 0) return fail(VKL_INVALID_ARGUMENT, "model_generate: empty prompt or nothing to generate");
  if (n_prompt > m->cfg.maxlen) return fail(VKL_OUT_OF_RANGE, "model_generate: prompt of %zu tokens exceeds the context length %u", n_prompt, m->cfg.maxlen);
  if (n_prompt + n_gen > (size_t)2 * m->cfg.maxlen || n_gen > m->out_cap)
    return fail(VKL_OUT_OF_RANGE, "model_generate: %zu + %zu tokens run past the RoPE table (2*maxlen)", n_prompt, n_gen);
  VKL_CUDA(cudaSetDevice(m->dev->ordinal));
  VKL_OKAY(ensure_rows(m, (uint32_t)n_prompt));
  VKL_OKAY(prepare_decode(m));
  const uint32_t st[2] = {0, 0};
  VKL_CUDA(cudaMemcpyAsync(m->state->data(), st, 8, cudaMemcpyHostToDevice, m->stream));
  VKL_CUDA(cudaMemcpyAsync(m->toks->data(), prompt, n_prompt * 4, cudaMemcpyHostToDevice, m->stream));
  // Tensor-parallel models (and VKLLAMA_PREFILL=sequential) prefill token by token through
  // the persistent decode kernel: while the position is inside the prompt the kernel feeds
  // itself the next prompt id instead of its arg-max.
  const char *pf = getenv("VKLLAMA_PREFILL");
  const bool by_token = pf && !strcmp(pf, "sequential");
  const bool sequential = m->mega_ready && n_prompt > 1 && (m->cfg.tp_size > 1 || by_token);
  if (m->cfg.tp_size > 1 && !m->mega_ready) return fail(VKL_UNIMPLEMENTED, "model_generate: tensor-parallel models need the persistent decode kernel");
  if (m->tp_failed) return decode_step(m);  // reports the state
  const uint32_t nf = sequential ? (uint32_t)n_prompt : 0u;
  VKL_CUDA(cudaMemcpyAsync((uint32_t *)m->state->data() + 5, &nf, 4, cudaMemcpyHostToDevice, m->stream));
  if (sequential) VKL_CUDA(cudaMemcpyAsync(m->forced->data(), prompt, n_prompt * 4, cudaMemcpyHostToDevice, m->stream));
  VKL_CUDA(cudaEventRecord(m->ev0, m->stream));
  if (sequential) {
    // A sharded model first fills the caches for all but the last prompt tokens in many-token passes on the
    // tensor-core GEMMs (chunks of at most tp_pf_rows tokens, each with enough rows for that path); what is
    // left, the last prompt token at least, goes through the decode kernel, which also yields the first id.
    size_t done = 0;
    if (m->cfg.tp_size > 1 && !by_token) {
      while (n_prompt - 1 - done >= gemm_min_rows(q8(m))) {
        const uint32_t T = (uint32_t)std::min<size_t>(n_prompt - 1 - done, m->tp_pf_rows);
        if (!use_gemm(m, T)) break;
        const uint32_t at = (uint32_t)done;
        VKL_CUDA(cudaMemcpyAsync(m->state->data(), &at, 4, cudaMemcpyHostToDevice, m->stream));
        VKL_OKAY(run_tokens(m, T, false, nullptr, true, at));
        done += T;
      }
      if (done) {
        const uint32_t at = (uint32_t)done;
        VKL_CUDA(cudaMemcpyAsync(m->state->data(), &at, 4, cudaMemcpyHostToDevice, m->stream));
        VKL_CUDA(cudaMemcpyAsync(m->toks->data(), (const uint32_t *)m->toks->data() + done, 4, cudaMemcpyDeviceToDevice, m->stream));
      }
    }
    for (size_t i = done; i < n_prompt; ++i) VKL_OKAY(decode_step(m));
  } else if (n_prompt == 1) {
    VKL_OKAY(decode_step(m));
  } else {
    VKL_OKAY(run_tokens(m, (uint32_t)n_prompt, false));
    VKL_OKAY(launch_advance(m, (uint32_t)n_prompt));
  }
  VKL_CUDA(cudaEventRecord(m->ev1, m->stream));
  for (size_t i = 1; i < n_gen; ++i) VKL_OKAY(decode_step(m));
  VKL_CUDA(cudaEventRecord(m->ev2, m->stream));
  VKL_CUDA(cudaMemcpyAsync(out_ids, m->out_ids->data(), n_gen * 4, cudaMemcpyDeviceToHost, m->stream));
  VKL_CUDA(cudaStreamSynchronize(m->stream));
  float ms = 0.f;
  if (prefill_ms) {
    VKL_CUDA(cudaEventElapsedTime(&ms, m->ev0, m->ev1));
    *prefill_ms = ms;
  }
  if (decode_ms) {
    VKL_CUDA(cudaEventElapsedTime(&ms, m->ev1, m->ev2));
    *decode_ms = ms;
  }
  VKL_OKAY(check_gemm(m));
  return check_mega(m);
}

int vkl_model_last_token(vkl_model *m, uint32_t *id) {
  if (!m || !id) return fail(VKL_INVALID_ARGUMENT, "model_last_token: null argument");
  VKL_CUDA(cudaSetDevice(m->dev->ordinal));
  VKL_CUDA(cudaMemcpyAsync(id, (uint32_t *)m->state->data() + 2, 4, cudaMemcpyDeviceToHost, m->stream));
  VKL_CUDA(cudaStreamSynchronize(m->stream));
  return VKL_OK;
}

int vkl_model_topk(vkl_model *m, uint32_t k, float *values, uint32_t *ids) {
  if (!m || !values || !ids) return fail(VKL_INVALID_ARGUMENT, "model_topk: null argument");
  if (k < 1 || k > 64 || k > m->vocab_l) return fail(VKL_INVALID_ARGUMENT, "model_topk: k = %u (1..64, at most the vocabulary)", k);
  if (m->cfg.tp_size > 1) return fail(VKL_UNIMPLEMENTED, "model_topk: the output layer of a tensor-parallel model is split over ranks");
  VKL_CUDA(cudaSetDevice(m->dev->ordinal));
  void *buf = nullptr;
  VKL_OKAY(m->dev->alloc(64 * 8, &buf));
  float *dv = (float *)buf;
  uint32_t *di = (uint32_t *)buf + 64;
  cudaError_t e = launch_topk_f32((const float *)m->logits32->data(), m->vocab_l, k, dv, di, m->stream);
  if (e == cudaSuccess) e = cudaMemcpyAsync(values, dv, k * 4, cudaMemcpyDeviceToHost, m->stream);
  if (e == cudaSuccess) e = cudaMemcpyAsync(ids, di, k * 4, cudaMemcpyDeviceToHost, m->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(m->stream);
  m->dev->release(buf, 64 * 8);
  count_launches(1);
  if (e != cudaSuccess) return fail(VKL_INTERNAL, "model_topk: %s", cudaGetErrorString(e));
  return VKL_OK;
}

int vkl_model_read_kv(vkl_model *m, uint32_t layer, void *kcache, void *vcache) {
  if (!m || layer >= m->cfg.layers) return fail(VKL_INVALID_ARGUMENT, "model_read_kv: bad model or layer");
  VKL_CUDA(cudaSetDevice(m->dev->ordinal));
  Layer &y = m->L[layer];
  if (kcache) VKL_CUDA(cudaMemcpyAsync(kcache, y.kcache->data(), y.kcache->device_bytes(), cudaMemcpyDeviceToHost, m->stream));
  if (vcache) VKL_CUDA(cudaMemcpyAsync(vcache, y.vcache->data(), y.vcache->device_bytes(), cudaMemcpyDeviceToHost, m->stream));
  VKL_CUDA(cudaStreamSynchronize(m->stream));
  return VKL_OK;
}
int vkl_model_write_kv(vkl_model *m, uint32_t layer, const void *kcache, const void *vcache) {
  if (!m || layer >= m->cfg.layers) return fail(VKL_INVALID_ARGUMENT, "model_write_kv: bad model or layer");
  VKL_CUDA(cudaSetDevice(m->dev->ordinal));
  Layer &y = m->L[layer];
  if (kcache) VKL_CUDA(cudaMemcpyAsync(y.kcache->data(), kcache, y.kcache->device_bytes(), cudaMemcpyHostToDevice, m->stream));
  if (vcache) VKL_CUDA(cudaMemcpyAsync(y.vcache->data(), vcache, y.vcache->device_bytes(), cudaMemcpyHostToDevice, m->stream));
  VKL_CUDA(cudaStreamSynchronize(m->stream));
  return VKL_OK;
}

int vkl_model_block_forward(vkl_model *m, uint32_t layer, const void *x_fp16, size_t T, size_t offset, void *out_fp16) {
  if (!m || layer >= m->cfg.layers || !x_fp16 || !out_fp16 || T == 0) return fail(VKL_INVALID_ARGUMENT, "model_block_forward: bad argument");
  if (T > m->cfg.maxlen || offset + T > (size_t)2 * m->cfg.maxlen) return fail(VKL_OUT_OF_RANGE, "model_block_forward: rows or position out of range");
  Layer &y = m->L[layer];
  if (!y.attn_norm || !y.ffn_norm || !y.wq || !y.wk || !y.wv || !y.wo || !y.gate || !y.up || !y.down)
    return fail(VKL_FAILED_PRECONDITION, "model_block_forward: weights of block %u are incomplete", layer);
  VKL_CUDA(cudaSetDevice(m->dev->ordinal));
  VKL_OKAY(ensure_rows(m, (uint32_t)T));
  // Run the model path on a one-block view of this model.
  const uint32_t st[2] = {(uint32_t)offset, 0};
  VKL_CUDA(cudaMemcpyAsync(m->state->data(), st, 8, cudaMemcpyHostToDevice, m->stream));
  const size_t D = m->cfg.dim;
  cudaStream_t s = m->stream;
  __half *x = (__half *)m->x->data(), *xn = (__half *)m->xn->data();
  VKL_CUDA(cudaMemcpyAsync(x, x_fp16, T * D * 2, cudaMemcpyHostToDevice, s));
  const bool dec = T == 1;
  MvParams p = mv(m, y.wk, dec ? x : xn, (__half *)m->k->data(), (uint32_t)T);
  p.codes[1] = y.wq->data(); p.codes[2] = y.wv->data();
  if (q8(m)) { p.scales[1] = y.wq->scales(); p.scales[2] = y.wv->scales(); }
  p.out[1] = (__half *)m->q->data(); p.out[2] = (__half *)m->v->data();
  p.nmat = 3;
  if (dec) {
    p.norm_w = (const float *)y.attn_norm->data();
    p.eps = m->cfg.eps;
    VKL_LAUNCH(1, launch_matvec(p, EPI_PLAIN, true, s));
  } else {
    VKL_LAUNCH(1, launch_rms_norm(x, (const float *)y.attn_norm->data(), xn, (uint32_t)T, (uint32_t)D, m->cfg.eps, s));
    VKL_LAUNCH((T + 63) / 64, launch_matvec(p, EPI_PLAIN, false, s));
  }
  AttnParams a = {};
  a.q = (__half *)m->q->data(); a.k = (const __half *)m->k->data(); a.v = (const __half *)m->v->data();
  a.kcache = (__half *)y.kcache->data(); a.vcache = (__half *)y.vcache->data();
  a.out = (__half *)m->ao->data();
  a.freqc = (const float *)m->fc->data(); a.freqs = (const float *)m->fs->data();
  a.pos_dev = m->pos_dev();
  a.scratch = (float *)m->attn_scratch->data(); a.counters = (uint32_t *)m->attn_counters->data();
  a.T = (uint32_t)T; a.heads = m->heads_l; a.dim = m->head_dim; a.maxlen = m->cfg.maxlen;
  a.splits = dec ? m->splits : 1;
  VKL_LAUNCH(dec ? 1 : 2, launch_attention(a, s));
  MvParams o = mv(m, y.wo, (__half *)m->ao->data(), x, (uint32_t)T);
  o.residual = x;
  VKL_LAUNCH((T + 63) / 64, launch_matvec(o, EPI_ADD, false, s));
  MvParams f = mv(m, y.gate, dec ? x : xn, (__half *)m->t->data(), (uint32_t)T);
  f.codes[1] = y.up->data();
  if (q8(m)) f.scales[1] = y.up->scales();
  if (dec) {
    f.norm_w = (const float *)y.ffn_norm->data();
    f.eps = m->cfg.eps;
    VKL_LAUNCH(1, launch_matvec(f, EPI_SWIGLU, true, s));
  } else {
    VKL_LAUNCH(1, launch_rms_norm(x, (const float *)y.ffn_norm->data(), xn, (uint32_t)T, (uint32_t)D, m->cfg.eps, s));
    VKL_LAUNCH((T + 63) / 64, launch_matvec(f, EPI_SWIGLU, false, s));
  }
  MvParams d = mv(m, y.down, (__half *)m->t->data(), x, (uint32_t)T);
  d.residual = x;
  VKL_LAUNCH((T + 63) / 64, launch_matvec(d, EPI_ADD, false, s));
  VKL_CUDA(cudaMemcpyAsync(out_fp16, x, T * D * 2, cudaMemcpyDeviceToHost, s));
  VKL_CUDA(cudaStreamSynchronize(s));
  return VKL_OK;
}

int vkl_model_decode_profile(vkl_model *m, uint32_t token, size_t offset, float out_us[20]) {
  VKL_OKAY(check_ready(m));
  if (!out_us) return fail(VKL_INVALID_ARGUMENT, "model_decode_profile: null output");
  if (offset + 1 > (size_t)2 * m->cfg.maxlen) return fail(VKL_OUT_OF_RANGE, "model_decode_profile: position out of range");
  VKL_CUDA(cudaSetDevice(m->dev->ordinal));
  VKL_OKAY(prepare_decode(m));
  const uint32_t st[2] = {(uint32_t)offset, 0};
  VKL_CUDA(cudaMemcpyAsync(m->state->data(), st, 8, cudaMemcpyHostToDevice, m->stream));
  VKL_CUDA(cudaMemcpyAsync(m->toks->data(), &token, 4, cudaMemcpyHostToDevice, m->stream));
  for (int i = 0; i < 20; ++i) out_us[i] = 0.f;
  if (m->mega_ready) {
    if (!m->sm_mhz) {
      void *cb = nullptr;
      VKL_OKAY(m->dev->alloc(16, &cb));
      unsigned long long r[2] = {0, 0};
      clock_probe_kernel<<<1, 1, 0, m->stream>>>((unsigned long long *)cb);
      cudaError_t ce = cudaMemcpyAsync(r, cb, 16, cudaMemcpyDeviceToHost, m->stream);
      if (ce == cudaSuccess) ce = cudaStreamSynchronize(m->stream);
      m->dev->release(cb, 16);
      count_launches(1);
      if (ce != cudaSuccess) return fail(VKL_INTERNAL, "model_decode_profile: %s", cudaGetErrorString(ce));
      m->sm_mhz = r[1] ? (uint32_t)(r[0] * 1000ull / r[1]) : 0u;
      if (m->sm_mhz < 100u) m->sm_mhz = (uint32_t)(m->dev->prop.clockRate / 1000);
    }
    // Timeline of CTA 0 of the persistent kernel: per op, work and barrier wait.
    const size_t n = m->mp.nops;
    void *buf = nullptr;
    VKL_OKAY(m->dev->alloc(n * 24, &buf));
    MegaParams p = m->mp;
    p.timing = (unsigned long long *)buf;
    p.sm_mhz = m->sm_mhz;
    p.timing_mode = (getenv("VKLLAMA_DEBUG_PROLOGUE") ? 1 : 0) | (getenv("VKLLAMA_DEBUG_NOCOPY") ? 2 : 0) | (getenv("VKLLAMA_DEBUG_NOMATH") ? 4 : 0) | (getenv("VKLLAMA_DEBUG_EPILOGUE") ? 8 : 0) |
                    (getenv("VKLLAMA_DEBUG_LOOP") ? 32 : 0) | (getenv("VKLLAMA_DEBUG_NOBODY") ? 64 : 0) |
                    (getenv("VKLLAMA_DEBUG_NOHANDSHAKE") ? 128 : 0);
    std::vector<unsigned long long> tl(3 * n);
    std::vector<MegaOp> ops(n);
    cudaError_t e = cudaMemsetAsync(buf, 0, n * 24, m->stream);
    if (e == cudaSuccess) e = launch_decode_mega(p, m->mega_grid, m->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(tl.data(), buf, n * 24, cudaMemcpyDeviceToHost, m->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(ops.data(), m->mp.ops, n * sizeof(MegaOp), cudaMemcpyDeviceToHost, m->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(m->stream);
    m->dev->release(buf, n * 24);
    count_launches(1);
    if (e != cudaSuccess) return fail(VKL_INTERNAL, "model_decode_profile: %s", cudaGetErrorString(e));
    // Classes: 0 embedding, 1 norm+QKV, 2 attention, 3 o_proj, 4 gate/up, 5 down, 6 lm head,
    // 7 arg-max, 8 tensor-parallel all-reduce. A mat-vec's class follows from what it is:
    // three matrices = QKV, SwiGLU epilogue = gate/up, arg-max tracking = lm head, and of the
    // two residual projections the one right after the attention op is o_proj.
    bool after_attn = false;
    for (size_t i = 0; i < n; ++i) {
      int cls = 0;
      switch (ops[i].kind) {
        case MK_EMBED: cls = 0; break;
        case MK_ATTN_PART:
        case MK_ATTN_COMBINE: cls = 2; after_attn = true; break;
        case MK_ARGMAX: cls = 7; break;
        case MK_ALLREDUCE: cls = 8; break;
        default:
          if (ops[i].track_argmax) cls = 6;
          else if (ops[i].nmat == 3) cls = 1;
          else if (ops[i].epi == EPI_SWIGLU) cls = 4;
          else if (after_attn) { cls = 3; after_attn = false; }
          else cls = 5;
      }
      out_us[cls] += (float)(tl[2 * i] + tl[2 * i + 1]) * 1e-3f;
      out_us[10 + cls] += (float)tl[2 * i + 1] * 1e-3f;
      if (getenv("VKLLAMA_DEBUG_LOOP")) {  // diagnostic: [cls] = loop time, [10+cls] = stages of CTA 0
        out_us[cls] += (float)(tl[2 * n + i] >> 16) * 1e-3f - (float)(tl[2 * i] + tl[2 * i + 1]) * 1e-3f;
        out_us[10 + cls] += (float)(tl[2 * n + i] & 0xffff) - (float)tl[2 * i + 1] * 1e-3f;
      }
      if (getenv("VKLLAMA_DEBUG_RING")) out_us[10 + cls] = out_us[10 + cls] - (float)tl[2 * i + 1] * 1e-3f + (float)tl[2 * n + i] * 1e-3f;
    }
    return check_mega(m);
  }
  Marker mk;
  mk.s = m->stream;
  int rc = run_tokens(m, 1, false, &mk);
  cudaError_t e = cudaStreamSynchronize(m->stream);
  for (size_t i = 1; i < mk.ev.size(); ++i) {
    float ms = 0.f;
    if (rc == VKL_OK && e == cudaSuccess && cudaEventElapsedTime(&ms, mk.ev[i - 1], mk.ev[i]) == cudaSuccess && mk.cls[i] >= 0)
      out_us[mk.cls[i]] += ms * 1000.f;
  }
  for (cudaEvent_t ev : mk.ev) cudaEventDestroy(ev);
  if (rc != VKL_OK) return rc;
  if (e != cudaSuccess) return fail(VKL_INTERNAL, "model_decode_profile: %s", cudaGetErrorString(e));
  return VKL_OK;
}

int vkl_model_decode_trace(vkl_model *m, uint32_t token, size_t offset, unsigned long long *out, size_t cap, uint32_t *nops, uint32_t *grid, uint32_t *kinds) {
  VKL_OKAY(check_ready(m));
  if (!nops || !grid) return fail(VKL_INVALID_ARGUMENT, "model_decode_trace: null argument");
  if (offset + 1 > (size_t)2 * m->cfg.maxlen) return fail(VKL_OUT_OF_RANGE, "model_decode_trace: position out of range");
  VKL_CUDA(cudaSetDevice(m->dev->ordinal));
  VKL_OKAY(prepare_decode(m));
  if (!m->mega_ready) return fail(VKL_FAILED_PRECONDITION, "model_decode_trace: the persistent decode kernel is not in use for this model");
  const size_t n = m->mp.nops, G = (size_t)m->mega_grid, words = n * G * 8;
  *nops = (uint32_t)n;
  *grid = (uint32_t)G;
  if (!out) return VKL_OK;  // size query
  if (cap < words) return fail(VKL_INVALID_ARGUMENT, "model_decode_trace: %zu words needed, %zu given", words, cap);
  const uint32_t st[2] = {(uint32_t)offset, 0};
  VKL_CUDA(cudaMemcpyAsync(m->state->data(), st, 8, cudaMemcpyHostToDevice, m->stream));
  VKL_CUDA(cudaMemcpyAsync(m->toks->data(), &token, 4, cudaMemcpyHostToDevice, m->stream));
  void *buf = nullptr;
  VKL_OKAY(m->dev->alloc(words * 8, &buf));
  MegaParams p = m->mp;
  p.timing = (unsigned long long *)buf;
  p.timing_mode = 256u;
  p.sm_mhz = 1000;
  cudaError_t e = cudaMemsetAsync(buf, 0, words * 8, m->stream);
  if (e == cudaSuccess) e = launch_decode_mega(p, m->mega_grid, m->stream);
  if (e == cudaSuccess) e = cudaMemcpyAsync(out, buf, words * 8, cudaMemcpyDeviceToHost, m->stream);
  if (e == cudaSuccess && kinds) {
    std::vector<MegaOp> ops(n);
    e = cudaMemcpyAsync(ops.data(), m->mp.ops, n * sizeof(MegaOp), cudaMemcpyDeviceToHost, m->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(m->stream);
    for (size_t i = 0; i < n; ++i) kinds[i] = ops[i].kind | (ops[i].nmat << 8) | (ops[i].epi << 16);
  }
  if (e == cudaSuccess) e = cudaStreamSynchronize(m->stream);
  m->dev->release(buf, words * 8);
  count_launches(1);
  if (e != cudaSuccess) return fail(VKL_INTERNAL, "model_decode_trace: %s", cudaGetErrorString(e));
  return check_mega(m);
}

int vkl_model_tp_buffer(vkl_model *m, void **local_ptr, size_t *bytes) {
  if (!m || !local_ptr || !bytes) return fail(VKL_INVALID_ARGUMENT, "model_tp_buffer: null argument");
  if (m->cfg.tp_size <= 1) return fail(VKL_FAILED_PRECONDITION, "model_tp_buffer: the model is not tensor parallel");
  *local_ptr = m->tp_buf;
  *bytes = m->tp_bytes;
  return VKL_OK;
}
int vkl_model_tp_connect(vkl_model *m, void *const *peer_ptrs, int n) {
  if (!m || !peer_ptrs) return fail(VKL_INVALID_ARGUMENT, "model_tp_connect: null argument");
  if (n != m->cfg.tp_size) return fail(VKL_INVALID_ARGUMENT, "model_tp_connect: %d pointers for %d ranks", n, m->cfg.tp_size);
  for (int i = 0; i < n; ++i) {
    if (i == m->cfg.tp_rank) continue;
    if (!peer_ptrs[i]) return fail(VKL_INVALID_ARGUMENT, "model_tp_connect: null pointer for rank %d", i);
    m->tp_peer[i] = peer_ptrs[i];
  }
  m->tp_connected = true;
  // (Re)connection: every rank calls this while no rank has a kernel in flight (host barrier before and
  // after), so the exchange buffer and the sequence counters restart from zero on all ranks together.
  VKL_CUDA(cudaSetDevice(m->dev->ordinal));
  VKL_CUDA(cudaStreamSynchronize(m->stream));
  VKL_CUDA(cudaMemsetAsync(m->tp_buf, 0, m->tp_bytes, m->stream));
  VKL_CUDA(cudaMemsetAsync((uint32_t *)m->state->data() + 3, 0, 8, m->stream));  // all-reduces done, arg-max exchanges done
  VKL_CUDA(cudaStreamSynchronize(m->stream));
  m->tp_failed = false;
  m->tp_pf_seq = 0;
  if (m->mega_ready)
    for (int i = 0; i < 8; ++i) m->mp.tp_peer[i] = m->tp_peer[i];
  return VKL_OK;
}
int vkl_model_set_wait_limit(vkl_model *m, uint32_t polls) {
  if (!m) return fail(VKL_INVALID_ARGUMENT, "model_set_wait_limit: null model");
  if (polls && polls < 256) return fail(VKL_INVALID_ARGUMENT, "model_set_wait_limit: at least 256 polls (0 restores the default)");
  m->wait_limit = polls;
  if (m->mega_ready) m->mp.wait_limit = polls ? polls : (m->cfg.tp_size > 1 ? (1u << 24) : (1u << 21));
  return VKL_OK;
}
int vkl_ipc_export(void *device_ptr, unsigned char handle[64]) {
  if (!device_ptr || !handle) return fail(VKL_INVALID_ARGUMENT, "ipc_export: null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaIpcMemHandle_t h;
  VKL_CUDA(cudaIpcGetMemHandle(&h, device_ptr));
  memcpy(handle, &h, 64);
  return VKL_OK;
}
int vkl_ipc_open(vkl_device *dev, const unsigned char handle[64], void **device_ptr) {
  if (!dev || !handle || !device_ptr) return fail(VKL_INVALID_ARGUMENT, "ipc_open: null argument");
  VKL_CUDA(cudaSetDevice(dev->ordinal));
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  VKL_CUDA(cudaIpcOpenMemHandle(device_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return VKL_OK;
}

}  // extern "C"
