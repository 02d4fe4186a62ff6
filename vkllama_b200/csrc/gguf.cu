// GGUF container reader and the host samplers: the two callers either side of the
// token loop (app/llama2_infer.cpp:46-73 reads the checkpoint through gguflib and hands
// Model::init the key and tensor maps; :141-210 samples every token from the logits).
//
// The reader memory-maps the file and indexes the metadata keys and tensor infos of
// GGUF versions 2 and 3 (little endian). Only what Model::init consumes is interpreted
// (models/llama2.h:367-370 the llama.* keys, :382-397 the tensor types 0/1/8 = F32/F16/
// Q8_0, :401-403 and :486-512 the tensor names); everything else is skipped by size.
// Tensor data is handed out as pointers into the mapping, exactly as gguflib does, and
// vkl_model_load_gguf feeds them to vkl_model_set_weight, which uploads and shards.
#include <errno.h>
#include <fcntl.h>
#include <math.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <random>
#include <string>
#include <vector>

#include "runtime.h"

using namespace vkl;

namespace {

enum GgufType : uint32_t { GT_U8 = 0, GT_I8, GT_U16, GT_I16, GT_U32, GT_I32, GT_F32, GT_BOOL, GT_STRING, GT_ARRAY, GT_U64, GT_I64, GT_F64 };

size_t scalar_size(uint32_t t) {
  switch (t) {
    case GT_U8: case GT_I8: case GT_BOOL: return 1;
    case GT_U16: case GT_I16: return 2;
    case GT_U32: case GT_I32: case GT_F32: return 4;
    case GT_U64: case GT_I64: case GT_F64: return 8;
    default: return 0;
  }
}

struct Key {
  std::string name;
  uint32_t type;
  const uint8_t *val;  // scalars: the value; strings: the u64 length; arrays: the element type word
};
struct TensorInfo {
  std::string name;
  uint32_t ndim;
  uint64_t dim[4];
  uint32_t type;
  uint64_t offset;  // from the start of the data section
  size_t bytes;
};

}  // namespace

struct vkl_gguf {
  int fd = -1;
  const uint8_t *base = nullptr;
  size_t size = 0;
  uint32_t version = 0;
  uint64_t alignment = 32;
  size_t data_start = 0;
  std::vector<Key> keys;
  std::vector<TensorInfo> tensors;
  ~vkl_gguf() {
    if (base) munmap((void *)base, size);
    if (fd >= 0) close(fd);
  }
};

namespace {

// Bounds-checked cursor over the mapping.
struct Cur {
  const uint8_t *p, *end;
  bool ok = true;
  template <typename T>
  T get() {
    T v{};
    if (!ok || (size_t)(end - p) < sizeof(T)) {
      ok = false;
      return v;
    }
    memcpy(&v, p, sizeof(T));
    p += sizeof(T);
    return v;
  }
  bool skip(uint64_t n) {
    if (!ok || (uint64_t)(end - p) < n) return ok = false;
    p += n;
    return true;
  }
  bool str(std::string *out) {
    const uint64_t n = get<uint64_t>();
    if (!ok || (uint64_t)(end - p) < n) return ok = false;
    if (out) out->assign((const char *)p, (size_t)n);
    p += n;
    return true;
  }
  // skips one value of `type` (arrays recursively)
  bool value(uint32_t type, int depth = 0) {
    if (type == GT_STRING) return str(nullptr);
    if (type == GT_ARRAY) {
      if (depth > 4) return ok = false;
      const uint32_t et = get<uint32_t>();
      const uint64_t n = get<uint64_t>();
      if (!ok) return false;
      const size_t es = scalar_size(et);
      if (es) return skip(n * es);
      for (uint64_t i = 0; i < n && ok; ++i) value(et, depth + 1);
      return ok;
    }
    const size_t s = scalar_size(type);
    if (!s) return ok = false;
    return skip(s);
  }
};

// bytes of a tensor of `type` with `n` elements whose rows have dim0 elements (GGML types 0, 1, 8)
bool tensor_bytes(uint32_t type, uint64_t n, uint64_t dim0, size_t *out) {
  switch (type) {
    case 0: *out = n * 4; return true;
    case 1: *out = n * 2; return true;
    case 8:
      if (dim0 % 32) return false;
      *out = n / 32 * 34;
      return true;
    default: return false;
  }
}

const Key *find_key(const vkl_gguf *g, const char *name) {
  for (const Key &k : g->keys)
    if (k.name == name) return &k;
  return nullptr;
}
const TensorInfo *find_tensor(const vkl_gguf *g, const std::string &name) {
  for (const TensorInfo &t : g->tensors)
    if (t.name == name) return &t;
  return nullptr;
}

int to_dtype(uint32_t ggml_type) {  // models/llama2.h:382-397
  return ggml_type == 0 ? VKL_FP32 : ggml_type == 1 ? VKL_FP16 : ggml_type == 8 ? VKL_Q8_0 : -1;
}

}  // namespace

extern "C" {

int vkl_gguf_open(const char *path, vkl_gguf **out) {
  if (!path || !out) return fail(VKL_INVALID_ARGUMENT, "gguf_open: null argument");
  std::unique_ptr<vkl_gguf> g(new vkl_gguf());
  g->fd = open(path, O_RDONLY);
  if (g->fd < 0) return fail(VKL_NOT_FOUND, "gguf_open: %s: %s", path, strerror(errno));
  struct stat st;
  if (fstat(g->fd, &st) != 0 || st.st_size < 24) return fail(VKL_INVALID_ARGUMENT, "gguf_open: %s is too short to be a GGUF file", path);
  g->size = (size_t)st.st_size;
  void *m = mmap(nullptr, g->size, PROT_READ, MAP_PRIVATE, g->fd, 0);
  if (m == MAP_FAILED) return fail(VKL_INTERNAL, "gguf_open: mmap of %s failed: %s", path, strerror(errno));
  g->base = (const uint8_t *)m;
  Cur c{g->base, g->base + g->size};
  if (memcmp(c.p, "GGUF", 4) != 0) return fail(VKL_INVALID_ARGUMENT, "gguf_open: %s has no GGUF magic", path);
  c.skip(4);
  g->version = c.get<uint32_t>();
  if (g->version < 2 || g->version > 3) return fail(VKL_UNIMPLEMENTED, "gguf_open: GGUF version %u is unsupported (2 or 3)", g->version);
  const uint64_t nt = c.get<uint64_t>(), nk = c.get<uint64_t>();
  if (nt > (1u << 20) || nk > (1u << 20)) return fail(VKL_INVALID_ARGUMENT, "gguf_open: implausible header (%llu tensors, %llu keys)", (unsigned long long)nt, (unsigned long long)nk);
  for (uint64_t i = 0; i < nk; ++i) {
    Key k;
    if (!c.str(&k.name)) break;
    k.type = c.get<uint32_t>();
    k.val = c.p;
    if (!c.value(k.type)) break;
    if (k.name == "general.alignment" && k.type == GT_U32) {
      uint32_t a;
      memcpy(&a, k.val, 4);
      if (a && !(a & (a - 1))) g->alignment = a;
    }
    g->keys.push_back(std::move(k));
  }
  if (!c.ok) return fail(VKL_INVALID_ARGUMENT, "gguf_open: %s: the metadata section is truncated or malformed", path);
  for (uint64_t i = 0; i < nt; ++i) {
    TensorInfo t{};
    if (!c.str(&t.name)) break;
    t.ndim = c.get<uint32_t>();
    if (!c.ok || t.ndim < 1 || t.ndim > 4) {
      c.ok = false;
      break;
    }
    uint64_t n = 1;
    for (uint32_t d = 0; d < 4; ++d) t.dim[d] = 1;
    for (uint32_t d = 0; d < t.ndim; ++d) {
      t.dim[d] = c.get<uint64_t>();
      n *= t.dim[d];
    }
    t.type = c.get<uint32_t>();
    t.offset = c.get<uint64_t>();
    if (!c.ok) break;
    if (!tensor_bytes(t.type, n, t.dim[0], &t.bytes)) t.bytes = 0;  // a type the model path does not take: listed, not loadable
    g->tensors.push_back(std::move(t));
  }
  if (!c.ok) return fail(VKL_INVALID_ARGUMENT, "gguf_open: %s: the tensor table is truncated or malformed", path);
  const size_t pos = (size_t)(c.p - g->base);
  g->data_start = (pos + g->alignment - 1) / g->alignment * g->alignment;
  for (const TensorInfo &t : g->tensors)
    if (t.bytes && (g->data_start + t.offset > g->size || t.bytes > g->size - g->data_start - t.offset))
      return fail(VKL_OUT_OF_RANGE, "gguf_open: tensor %s runs past the end of %s", t.name.c_str(), path);
  *out = g.release();
  return VKL_OK;
}

int vkl_gguf_close(vkl_gguf *g) {
  delete g;
  return VKL_OK;
}

int vkl_gguf_counts(const vkl_gguf *g, uint32_t *version, size_t *n_keys, size_t *n_tensors) {
  if (!g) return fail(VKL_INVALID_ARGUMENT, "gguf_counts: null handle");
  if (version) *version = g->version;
  if (n_keys) *n_keys = g->keys.size();
  if (n_tensors) *n_tensors = g->tensors.size();
  return VKL_OK;
}

int vkl_gguf_get_u32(const vkl_gguf *g, const char *key, uint32_t *out) {
  if (!g || !key || !out) return fail(VKL_INVALID_ARGUMENT, "gguf_get_u32: null argument");
  const Key *k = find_key(g, key);
  if (!k) return fail(VKL_NOT_FOUND, "gguf: key %s is missing", key);
  if (k->type == GT_U32 || k->type == GT_I32) {
    memcpy(out, k->val, 4);
  } else if (k->type == GT_U64 || k->type == GT_I64) {
    uint64_t v;
    memcpy(&v, k->val, 8);
    *out = (uint32_t)v;
  } else if (k->type == GT_U16) {
    uint16_t v;
    memcpy(&v, k->val, 2);
    *out = v;
  } else {
    return fail(VKL_INVALID_ARGUMENT, "gguf: key %s has type %u, not an integer", key, k->type);
  }
  return VKL_OK;
}

int vkl_gguf_get_f32(const vkl_gguf *g, const char *key, float *out) {
  if (!g || !key || !out) return fail(VKL_INVALID_ARGUMENT, "gguf_get_f32: null argument");
  const Key *k = find_key(g, key);
  if (!k) return fail(VKL_NOT_FOUND, "gguf: key %s is missing", key);
  if (k->type == GT_F32) {
    memcpy(out, k->val, 4);
  } else if (k->type == GT_F64) {
    double v;
    memcpy(&v, k->val, 8);
    *out = (float)v;
  } else {
    return fail(VKL_INVALID_ARGUMENT, "gguf: key %s has type %u, not a float", key, k->type);
  }
  return VKL_OK;
}

int vkl_gguf_get_string(const vkl_gguf *g, const char *key, char *buf, size_t cap) {
  if (!g || !key || !buf || !cap) return fail(VKL_INVALID_ARGUMENT, "gguf_get_string: null argument");
  const Key *k = find_key(g, key);
  if (!k) return fail(VKL_NOT_FOUND, "gguf: key %s is missing", key);
  if (k->type != GT_STRING) return fail(VKL_INVALID_ARGUMENT, "gguf: key %s has type %u, not a string", key, k->type);
  uint64_t n;
  memcpy(&n, k->val, 8);
  const size_t m = std::min<size_t>((size_t)n, cap - 1);
  memcpy(buf, k->val + 8, m);
  buf[m] = 0;
  return VKL_OK;
}

int vkl_gguf_tensor(const vkl_gguf *g, size_t index, const char *name, char *name_out, size_t name_cap, uint32_t *ndim, uint64_t dims[4],
                    uint32_t *ggml_type, const void **data, size_t *bytes) {
  if (!g) return fail(VKL_INVALID_ARGUMENT, "gguf_tensor: null handle");
  const TensorInfo *t = nullptr;
  if (name) {
    t = find_tensor(g, name);
    if (!t) return fail(VKL_NOT_FOUND, "gguf: tensor %s is missing", name);
  } else {
    if (index >= g->tensors.size()) return fail(VKL_OUT_OF_RANGE, "gguf_tensor: index %zu of %zu", index, g->tensors.size());
    t = &g->tensors[index];
  }
  if (name_out && name_cap) {
    const size_t m = std::min(t->name.size(), name_cap - 1);
    memcpy(name_out, t->name.data(), m);
    name_out[m] = 0;
  }
  if (ndim) *ndim = t->ndim;
  if (dims)
    for (int d = 0; d < 4; ++d) dims[d] = t->dim[d];
  if (ggml_type) *ggml_type = t->type;
  if (data) *data = g->base + g->data_start + t->offset;
  if (bytes) *bytes = t->bytes;
  return VKL_OK;
}

int vkl_model_load_gguf(vkl_device *dev, const vkl_gguf *g, uint32_t maxlen, int tp_rank, int tp_size, vkl_model **out) {
  if (!dev || !g || !out) return fail(VKL_INVALID_ARGUMENT, "model_load_gguf: null argument");
  vkl_model_config c = {};
  // models/llama2.h:367-370
  VKL_OKAY(vkl_gguf_get_u32(g, "llama.attention.head_count", &c.heads));
  VKL_OKAY(vkl_gguf_get_u32(g, "llama.block_count", &c.layers));
  VKL_OKAY(vkl_gguf_get_f32(g, "llama.attention.layer_norm_rms_epsilon", &c.eps));
  uint32_t ctx = 0;
  VKL_OKAY(vkl_gguf_get_u32(g, "llama.context_length", &ctx));
  c.maxlen = maxlen ? std::min(maxlen, ctx) : ctx;
  c.final_eps = 1e-6f;  // hard-coded for the output norm: models/llama2.h:268
  // shapes from the tensors, as Model::init takes them (llama2.h:401-412: [1, dim[1], dim[0]])
  const TensorInfo *emb = find_tensor(g, "token_embd.weight"), *outw = find_tensor(g, "output.weight");
  if (!emb || !outw || !find_tensor(g, "output_norm.weight")) return fail(VKL_NOT_FOUND, "model_load_gguf: token_embd / output / output_norm tensors are missing");
  const TensorInfo *gate = c.layers ? find_tensor(g, "blk.0.ffn_gate.weight") : nullptr;
  if (c.layers && !gate) return fail(VKL_NOT_FOUND, "model_load_gguf: blk.0.ffn_gate.weight is missing");
  c.dim = (uint32_t)emb->dim[0];
  c.vocab = (uint32_t)emb->dim[1];
  c.ffn = gate ? (uint32_t)gate->dim[1] : c.dim;
  c.weight_dtype = to_dtype(outw->type);
  if (c.weight_dtype != VKL_Q8_0 && c.weight_dtype != VKL_FP16) return fail(VKL_UNIMPLEMENTED, "model_load_gguf: weight type %u is unsupported (F16 = 1 or Q8_0 = 8)", outw->type);
  c.tp_rank = tp_rank;
  c.tp_size = tp_size < 1 ? 1 : tp_size;
  uint32_t kv_heads = c.heads;
  if (find_key(g, "llama.attention.head_count_kv")) VKL_OKAY(vkl_gguf_get_u32(g, "llama.attention.head_count_kv", &kv_heads));
  if (kv_heads != c.heads) return fail(VKL_UNIMPLEMENTED, "model_load_gguf: grouped-query attention (%u KV heads for %u heads) is outside the Llama-2 path of the reference", kv_heads, c.heads);
  vkl_model *m = nullptr;
  VKL_OKAY(vkl_model_create(dev, &c, &m));
  auto load = [&](const std::string &name) -> int {
    const TensorInfo *t = find_tensor(g, name);
    if (!t) return fail(VKL_NOT_FOUND, "model_load_gguf: tensor %s is missing", name.c_str());
    const int dt = to_dtype(t->type);
    if (dt < 0 || !t->bytes) return fail(VKL_UNIMPLEMENTED, "model_load_gguf: tensor %s has GGML type %u (F32, F16 and Q8_0 are supported)", name.c_str(), t->type);
    return vkl_model_set_weight(m, name.c_str(), dt, g->base + g->data_start + t->offset, t->bytes);
  };
  static const char *kBlock[9] = {"attn_norm", "attn_q", "attn_k", "attn_v", "attn_output", "ffn_norm", "ffn_gate", "ffn_up", "ffn_down"};
  int st = VKL_OK;
  for (const char *n : {"token_embd.weight", "output_norm.weight", "output.weight"})
    if (st == VKL_OK) st = load(n);
  for (uint32_t b = 0; b < c.layers && st == VKL_OK; ++b)
    for (const char *k : kBlock)
      if (st == VKL_OK) st = load("blk." + std::to_string(b) + "." + k + ".weight");
  if (st != VKL_OK) {
    vkl_model_destroy(m);
    return st;
  }
  *out = m;
  return VKL_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------
// Samplers (models/samplers.cpp). The reference sorts all (logit, index) pairs descending,
// keeps the first k (TopkSampler, :37-64) or the shortest prefix whose softmax mass reaches
// p (TopPSampler, :67-101), applies a softmax over the kept logits and draws from it with
// std::discrete_distribution over a std::mt19937. Ties: std::sort leaves their order
// unspecified; here equal logits keep index order (lowest first), which is also what the
// device arg-max does. seed 0 seeds from std::random_device as the reference does.
// ---------------------------------------------------------------------------------------
struct vkl_sampler {
  int kind = 0;  // 0 top-k, 1 top-p
  size_t k = 40;
  float p = 1.f;
  std::mt19937 gen;
  std::vector<std::pair<float, int>> tmp;
  std::vector<float> probs;
};

namespace {

void softmax_pairs(std::vector<std::pair<float, int>> &v, size_t n) {  // samplers.cpp:16-33: max = first (sorted) entry
  const float m = v[0].first;
  float acc = 0.f;
  for (size_t i = 0; i < n; ++i) {
    v[i].first = std::exp(v[i].first - m);
    acc += v[i].first;
  }
  for (size_t i = 0; i < n; ++i) v[i].first /= acc;
}

int draw(vkl_sampler *s, size_t n) {
  s->probs.resize(n);
  for (size_t i = 0; i < n; ++i) s->probs[i] = s->tmp[i].first;
  std::discrete_distribution<> dis(s->probs.begin(), s->probs.end());
  return s->tmp[(size_t)dis(s->gen)].second;
}

bool pair_before(const std::pair<float, int> &a, const std::pair<float, int> &b) {
  return a.first > b.first || (a.first == b.first && a.second < b.second);
}

}  // namespace

extern "C" {

int vkl_sampler_create(int kind, size_t topk, float topp, uint64_t seed, vkl_sampler **out) {
  if (!out) return fail(VKL_INVALID_ARGUMENT, "sampler_create: null argument");
  if (kind != 0 && kind != 1) return fail(VKL_INVALID_ARGUMENT, "sampler_create: kind %d (0 = top-k, 1 = top-p)", kind);
  if (kind == 0 && topk == 0) return fail(VKL_INVALID_ARGUMENT, "sampler_create: top-k of 0");
  if (kind == 1 && !(topp > 0.f)) return fail(VKL_INVALID_ARGUMENT, "sampler_create: top-p must be positive");
  vkl_sampler *s = new vkl_sampler();
  s->kind = kind;
  s->k = topk;
  s->p = topp;
  if (seed) {
    s->gen.seed((uint32_t)(seed ^ (seed >> 32)));
  } else {
    std::random_device rd;
    s->gen.seed(rd());
  }
  *out = s;
  return VKL_OK;
}

int vkl_sampler_destroy(vkl_sampler *s) {
  delete s;
  return VKL_OK;
}

int vkl_sampler_sample(vkl_sampler *s, const float *logits, size_t n, int *id) {
  if (!s || !logits || !id || n == 0) return fail(VKL_INVALID_ARGUMENT, "sampler_sample: null or empty argument");
  s->tmp.resize(n);
  for (size_t i = 0; i < n; ++i) s->tmp[i] = std::make_pair(logits[i], (int)i);
  if (s->kind == 0) {
    const size_t k = std::min(s->k, n);
    std::partial_sort(s->tmp.begin(), s->tmp.begin() + k, s->tmp.end(), pair_before);  // the first k of the full sort
    softmax_pairs(s->tmp, k);
    *id = draw(s, k);
    return VKL_OK;
  }
  std::sort(s->tmp.begin(), s->tmp.end(), pair_before);
  // prefix whose mass under the softmax over ALL logits reaches p (samplers.cpp:82-91; fp32 as there)
  const float m = s->tmp[0].first;
  float total = 0.f;
  for (size_t i = 0; i < n; ++i) total += std::exp(s->tmp[i].first - m);
  float acc = 0.f;
  size_t keep = 0;
  for (; keep < n && acc < s->p; ++keep) acc += std::exp(s->tmp[keep].first - m) / total;
  softmax_pairs(s->tmp, keep);
  *id = draw(s, keep);
  return VKL_OK;
}

int vkl_sampler_sample_candidates(vkl_sampler *s, const float *values, const uint32_t *ids, size_t k, int *id) {
  if (!s || !values || !ids || !id || k == 0) return fail(VKL_INVALID_ARGUMENT, "sampler_sample_candidates: null or empty argument");
  if (s->kind != 0) return fail(VKL_FAILED_PRECONDITION, "sampler_sample_candidates: only the top-k sampler draws from a candidate list (top-p needs all logits)");
  const size_t n = std::min(s->k, k);
  s->tmp.resize(n);
  for (size_t i = 0; i < n; ++i) s->tmp[i] = std::make_pair(values[i], (int)ids[i]);  // already sorted descending by the device top-k
  softmax_pairs(s->tmp, n);
  *id = draw(s, n);
  return VKL_OK;
}

}  // extern "C"
