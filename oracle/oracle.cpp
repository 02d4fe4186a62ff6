// CPU oracle for the Llama-2 token loop of ComingToy/vkllama.
//
// TEST INFRASTRUCTURE ONLY. This file is the checker that the CUDA path is
// compared against (tests, the smoke check and the cpu_baseline / reference
// arm of the benchmark). It is never linked into, imported by or called from
// the product library.
//
// Every function restates one piece of the reference in plain C++ and cites
// the reference file:line it follows (paths relative to the vkllama tree).
// GLSL subgroup reductions are restated as a fixed 32-lane partition followed
// by a sequential lane sum; fp32 accumulation and fp16 rounding at every op
// boundary are kept exactly where the shaders have them.
//
// Pinning: the Q8_0 quantizer is checked byte-for-byte against the
// reference's own src/core/quants.h compiled into oracle/_ref (see
// oracle/Makefile and tests/golden/). The reference holds no golden vectors
// or CPU implementation for the other ops (its tests draw inputs from
// std::random_device and need a Vulkan device), so for those ops parity is
// pinned on the shader sources only: "parity unpinned" beyond the quantizer.
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <cmath>
#include <vector>

typedef _Float16 f16;

#define ORC_API extern "C" __attribute__((visibility("default")))

static inline float h2f(uint16_t u) {
  f16 h;
  memcpy(&h, &u, 2);
  return (float)h;
}
// IEEE round-to-nearest-even, what `float16_t(v)` does in the shaders.
static inline uint16_t f2h(float f) {
  f16 h = (f16)f;
  uint16_t u;
  memcpy(&u, &h, 2);
  return u;
}

// Host threads of the OpenMP loops below (a launcher may have pinned OMP_NUM_THREADS to 1).
#include <omp.h>
ORC_API int orc_threads(void) { return omp_get_max_threads(); }
ORC_API void orc_set_threads(int n) {
  if (n > 0) omp_set_num_threads(n);
}

// ---------------------------------------------------------------------------
// Seeded synthetic data (stands in for real checkpoints). Integer-only up to
// one fp32 fma, so a device implementation reproduces it bit for bit.
// value(seed, tensor, i) = fma(z, std, mean), z = (sum of twelve 16-bit
// uniforms - 393210) / 65536  (Irwin-Hall, unit variance).
// ---------------------------------------------------------------------------
static inline uint64_t mix64(uint64_t z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
static inline uint64_t synth_key(uint64_t seed, uint64_t tensor) {
  return mix64(seed * 0x9E3779B97F4A7C15ull + tensor * 0xD1B54A32D192ED03ull +
               0x2545F4914F6CDD1Dull);
}
static inline float synth_z(uint64_t key, uint64_t i) {
  uint32_t s = 0;
  for (int j = 0; j < 3; ++j) {
    uint64_t h = mix64(key + (3 * i + j + 1) * 0x9E3779B97F4A7C15ull);
    s += (uint32_t)(h & 0xFFFF) + (uint32_t)((h >> 16) & 0xFFFF) +
         (uint32_t)((h >> 32) & 0xFFFF) + (uint32_t)((h >> 48) & 0xFFFF);
  }
  return (float)((int32_t)s - 393210) * (1.0f / 65536.0f);
}

ORC_API void orc_synth_normal_f32(uint64_t seed, uint64_t tensor, uint64_t first,
                                  uint64_t n, float mean, float stdv, float *out) {
  const uint64_t key = synth_key(seed, tensor);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i)
    out[i] = fmaf(synth_z(key, first + i), stdv, mean);
}

ORC_API void orc_synth_normal_f16(uint64_t seed, uint64_t tensor, uint64_t first,
                                  uint64_t n, float mean, float stdv, uint16_t *out) {
  const uint64_t key = synth_key(seed, tensor);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i)
    out[i] = f2h(fmaf(synth_z(key, first + i), stdv, mean));
}

ORC_API void orc_synth_tokens(uint64_t seed, uint64_t tensor, uint64_t n,
                              uint32_t vocab, uint32_t *out) {
  const uint64_t key = synth_key(seed, tensor);
  for (uint64_t i = 0; i < n; ++i)
    out[i] = (uint32_t)((mix64(key + (i + 1) * 0x9E3779B97F4A7C15ull) >> 11) % vocab);
}

// ---------------------------------------------------------------------------
// Q8_0 quantizer. src/core/quants.h:37-96 (qint8_0_quantize_row): per block of
// 32, absmax; scale = absmax/127.0f; inverse = scale > 0 ? 127.0f/absmax : 0;
// code = (int8)roundf(x*inverse); tail elements beyond n are code 0. The host
// layout is [fp32 scale][32 x int8] = 36 bytes (quants.cpp:14).
// ---------------------------------------------------------------------------
ORC_API void orc_q8_0_quantize_row36(const float *src, uint8_t *dst, uint64_t n) {
  const uint64_t nb = (n + 31) / 32;
  for (uint64_t b = 0; b < nb; ++b) {
    const uint64_t start = b * 32, end = start + 32;
    float amax = fabsf(src[start]);
    for (uint64_t i = start; i < end && i < n; ++i) amax = std::max(fabsf(src[i]), amax);
    const float scale = amax / 127.0f;
    const float inv = scale > 0 ? 127.0f / amax : .0f;
    uint8_t *blk = dst + b * 36;
    memcpy(blk, &scale, 4);
    for (uint64_t i = start; i < end; ++i)
      blk[4 + (i - start)] = i >= n ? 0 : (uint8_t)(int8_t)roundf(src[i] * inv);
  }
}

// Device/GGUF layout used by every Q8_0 shader: [fp16 scale][32 x int8] = 34
// bytes (src/shaders/common.h:8-10). The reference never narrows a scale
// itself (model files already hold fp16 scales); this build defines the fp16
// scale as the round-to-nearest-even of the fp32 scale above.
ORC_API void orc_q8_0_quantize_row34(const float *src, uint8_t *dst, uint64_t n) {
  const uint64_t nb = (n + 31) / 32;
  std::vector<uint8_t> tmp(nb * 36);
  orc_q8_0_quantize_row36(src, tmp.data(), n);
  for (uint64_t b = 0; b < nb; ++b) {
    float s;
    memcpy(&s, &tmp[b * 36], 4);
    const uint16_t hs = f2h(s);
    memcpy(dst + b * 34, &hs, 2);
    memcpy(dst + b * 34 + 2, &tmp[b * 36 + 4], 32);
  }
}

// src/core/quants.h:143-158 (qint8_0_quantize): row by row.
ORC_API void orc_q8_0_quantize34(const float *src, uint8_t *dst, uint64_t h, uint64_t w) {
  const uint64_t rb = ((w + 31) / 32) * 34;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < (int64_t)h; ++r) orc_q8_0_quantize_row34(src + r * w, dst + r * rb, w);
}
ORC_API void orc_q8_0_quantize36(const float *src, uint8_t *dst, uint64_t h, uint64_t w) {
  const uint64_t rb = ((w + 31) / 32) * 36;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < (int64_t)h; ++r) orc_q8_0_quantize_row36(src + r * w, dst + r * rb, w);
}

// src/core/quants.h:98-140 (qint8_0_dequantize_row) on the 34-byte layout.
ORC_API void orc_q8_0_dequantize34(const uint8_t *src, float *dst, uint64_t h, uint64_t w) {
  const uint64_t nb = (w + 31) / 32;
  for (uint64_t r = 0; r < h; ++r)
    for (uint64_t b = 0; b < nb; ++b) {
      const uint8_t *blk = src + (r * nb + b) * 34;
      uint16_t hs;
      memcpy(&hs, blk, 2);
      const float d = h2f(hs);
      for (uint64_t i = 0; i < 32 && b * 32 + i < w; ++i)
        dst[r * w + b * 32 + i] = (float)(int8_t)blk[2 + i] * d;
    }
}

// Synthetic Q8_0 weight matrix [rows, K]: N(mean,std) fp32 -> 34-byte blocks.
ORC_API void orc_synth_q8_0(uint64_t seed, uint64_t tensor, uint64_t rows, uint64_t K,
                            float mean, float stdv, uint8_t *dst) {
  const uint64_t key = synth_key(seed, tensor);
  const uint64_t rb = ((K + 31) / 32) * 34;
#pragma omp parallel
  {
    std::vector<float> row(K);
#pragma omp for schedule(static)
    for (int64_t r = 0; r < (int64_t)rows; ++r) {
      for (uint64_t k = 0; k < K; ++k) row[k] = fmaf(synth_z(key, r * K + k), stdv, mean);
      orc_q8_0_quantize_row34(row.data(), dst + r * rb, K);
    }
  }
}

// ---------------------------------------------------------------------------
// Operators. Activations are fp16 bit patterns (uint16_t), row-major.
// ---------------------------------------------------------------------------

// One output of the Q8_0 shaders' inner loop: lane (ix = lane/4, il = lane%4)
// walks blocks ix, ix+8, ... and within a block the 8 items il*8..il*8+7,
// `sums += sum_b * d`; then subgroupAdd over the 32 lanes.
// src/shaders/matmul_b0_fp16_x_q8_0.comp:85-123 (same loop in
// kqv_fp16_x_q8_0.comp:78-119 and ffn_up_and_gate_q8_0.comp:81-118).
static inline float q8_row_dot(const float *x, const uint8_t *wrow, uint32_t K) {
  const uint32_t nb = (K + 31) / 32;
  float lane[32];
  for (int i = 0; i < 32; ++i) lane[i] = 0.f;
  for (uint32_t b = 0; b < nb; ++b) {
    const uint8_t *blk = wrow + (size_t)b * 34;
    uint16_t hs;
    memcpy(&hs, blk, 2);
    const float d = h2f(hs);
    const int8_t *q = (const int8_t *)(blk + 2);
    const float *xb = x + b * 32;
    const int ix = b & 7;
    for (int il = 0; il < 4; ++il) {
      float s = 0.f;
      for (int i = 0; i < 8; ++i) s += xb[il * 8 + i] * (float)q[il * 8 + i];
      lane[ix * 4 + il] += s * d;
    }
  }
  float v = 0.f;
  for (int i = 0; i < 32; ++i) v += lane[i];
  return v;
}

static void to_float(const uint16_t *x, float *xf, size_t n, size_t padded) {
  for (size_t i = 0; i < n; ++i) xf[i] = h2f(x[i]);
  for (size_t i = n; i < padded; ++i) xf[i] = 0.f;
}

// MatMul with a Q8_0 weight [N,K] (transpose_b): Y = fp16(act(X.W^T*scale+bias)),
// act 1 = SiLU as v/(1+exp(-v)). src/shaders/matmul_b0_fp16_x_q8_0.comp:50-140,
// host side src/ops/mat_mul.cpp:160-228.
ORC_API void orc_matmul_q8_0(const uint16_t *x, const uint8_t *w, uint16_t *y, uint32_t M,
                             uint32_t N, uint32_t K, float scale, float bias, int act) {
  const uint32_t Kp = ((K + 31) / 32) * 32;
  const size_t rb = (size_t)(Kp / 32) * 34;
  std::vector<float> xf((size_t)M * Kp);
  for (uint32_t m = 0; m < M; ++m) to_float(x + (size_t)m * K, &xf[(size_t)m * Kp], K, Kp);
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < (int64_t)N; ++n)
    for (uint32_t m = 0; m < M; ++m) {
      float v = q8_row_dot(&xf[(size_t)m * Kp], w + n * rb, K) * scale + bias;
      if (act == 1) v = v / (1.0f + expf(-v));
      y[(size_t)m * N + n] = f2h(v);
    }
}

// K,Q,V projections in one pass. src/shaders/kqv_fp16_x_q8_0.comp:42-139,
// launched at src/ops/multiheadattention_v2.cpp:190-202.
ORC_API void orc_kqv_q8_0(const uint16_t *x, const uint8_t *wk, const uint8_t *wq,
                          const uint8_t *wv, uint16_t *k, uint16_t *q, uint16_t *v,
                          uint32_t M, uint32_t N, uint32_t K) {
  orc_matmul_q8_0(x, wk, k, M, N, K, 1.f, 0.f, 0);
  orc_matmul_q8_0(x, wq, q, M, N, K, 1.f, 0.f, 0);
  orc_matmul_q8_0(x, wv, v, M, N, K, 1.f, 0.f, 0);
}

// t = fp16( silu(x.Wgate^T) * (x.Wup^T) ). src/shaders/ffn_up_and_gate_q8_0.comp:
// 120-133 (`v0.y / (1.0 + exp(-v0.y)) * v0.x`, x = up, y = gate).
ORC_API void orc_ffn_up_gate_q8_0(const uint16_t *x, const uint8_t *wup, const uint8_t *wgate,
                                  uint16_t *t, uint32_t M, uint32_t N, uint32_t K) {
  const uint32_t Kp = ((K + 31) / 32) * 32;
  const size_t rb = (size_t)(Kp / 32) * 34;
  std::vector<float> xf((size_t)M * Kp);
  for (uint32_t m = 0; m < M; ++m) to_float(x + (size_t)m * K, &xf[(size_t)m * Kp], K, Kp);
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < (int64_t)N; ++n)
    for (uint32_t m = 0; m < M; ++m) {
      const float up = q8_row_dot(&xf[(size_t)m * Kp], wup + n * rb, K);
      const float gate = q8_row_dot(&xf[(size_t)m * Kp], wgate + n * rb, K);
      t[(size_t)m * N + n] = f2h(gate / (1.0f + expf(-gate)) * up);
    }
}

// FeedForward: down( up_gate(x) ). src/ops/feed_forward.cpp:88-133; ctor order
// (w1 = gate, w2 = down, w3 = up) feed_forward.cpp:14-22, models/llama2.h:128-130.
ORC_API void orc_feed_forward_q8_0(const uint16_t *x, const uint8_t *w1_gate,
                                   const uint8_t *w2_down, const uint8_t *w3_up, uint16_t *y,
                                   uint32_t M, uint32_t dim, uint32_t hidden) {
  std::vector<uint16_t> t((size_t)M * hidden);
  orc_ffn_up_gate_q8_0(x, w3_up, w1_gate, t.data(), M, hidden, dim);
  orc_matmul_q8_0(t.data(), w2_down, y, M, dim, hidden, 1.f, 0.f, 0);
}

// Batched A.B^T on fp16 with element strides (channel, row) per operand.
// src/shaders/matmul_b0_tb_fp16_v2.comp:38-120: 64-wide K blocks, lane
// (ix, il) takes a 16-element slice of block ix, ix+8, ...
ORC_API void orc_matmul_tb_f16(const uint16_t *a, const uint16_t *b, uint16_t *c, uint32_t C,
                               uint32_t M, uint32_t N, uint32_t K, uint64_t a_cs, uint64_t a_hs,
                               uint64_t b_cs, uint64_t b_hs, uint64_t c_cs, uint64_t c_hs,
                               float scale, float bias, int act) {
  const uint32_t nblk = (K + 63) / 64;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t ch = 0; ch < (int64_t)C; ++ch)
    for (int64_t n = 0; n < (int64_t)N; ++n)
      for (uint32_t m = 0; m < M; ++m) {
        const uint16_t *ar = a + ch * a_cs + m * a_hs;
        const uint16_t *br = b + ch * b_cs + n * b_hs;
        float lane[32];
        for (int i = 0; i < 32; ++i) lane[i] = 0.f;
        for (uint32_t bi = 0; bi < nblk; ++bi)
          for (int il = 0; il < 4; ++il) {
            float s = 0.f;
            for (int i = 0; i < 16; ++i) {
              const uint32_t k = bi * 64 + il * 16 + i;
              if (k < K) s += h2f(ar[k]) * h2f(br[k]);
            }
            lane[(bi & 7) * 4 + il] += s;
          }
        float v = 0.f;
        for (int i = 0; i < 32; ++i) v += lane[i];
        v = v * scale + bias;
        if (act == 1) v = v / (1.0f + expf(-v));
        c[ch * c_cs + m * c_hs + n] = f2h(v);
      }
}

// One fp16 row dot with the 32-lane partition of the fp16 shaders: lane (ix, il) owns the
// 16-element slice il of K blocks ix, ix+8, ...; lanes are summed in index order.
static float f16_row_dot(const uint16_t *ar, const uint16_t *br, uint32_t K) {
  const uint32_t nblk = (K + 63) / 64;
  float lane[32];
  for (int i = 0; i < 32; ++i) lane[i] = 0.f;
  for (uint32_t bi = 0; bi < nblk; ++bi)
    for (int il = 0; il < 4; ++il) {
      float s = 0.f;
      for (int i = 0; i < 16; ++i) {
        const uint32_t k = bi * 64 + il * 16 + i;
        if (k < K) s += h2f(ar[k]) * h2f(br[k]);
      }
      lane[(bi & 7) * 4 + il] += s;
    }
  float v = 0.f;
  for (int i = 0; i < 32; ++i) v += lane[i];
  return v;
}

// FeedForward with FP16 weights: t = fp16(silu(gate.x) * (up.x)) on unrounded fp32 dots
// (src/shaders/ffn_up_and_gate_fp16.comp:58-125), then the down MatMul
// (src/ops/feed_forward.cpp:88-133). Weights are [out,in].
ORC_API void orc_feed_forward_f16(const uint16_t *x, const uint16_t *w1_gate, const uint16_t *w2_down,
                                  const uint16_t *w3_up, uint16_t *y, uint32_t M, uint32_t dim,
                                  uint32_t hidden) {
  std::vector<uint16_t> t((size_t)M * hidden);
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < (int64_t)hidden; ++n)
    for (uint32_t m = 0; m < M; ++m) {
      const float up = f16_row_dot(x + (size_t)m * dim, w3_up + (size_t)n * dim, dim);
      const float gate = f16_row_dot(x + (size_t)m * dim, w1_gate + (size_t)n * dim, dim);
      t[(size_t)m * hidden + n] = f2h(gate / (1.0f + expf(-gate)) * up);
    }
  orc_matmul_tb_f16(t.data(), w2_down, y, 1, M, dim, hidden, (uint64_t)M * hidden, hidden,
                    (uint64_t)dim * hidden, hidden, (uint64_t)M * dim, dim, 1.f, 0.f, 0);
}

// Batched A.B (B not transposed). src/shaders/matmul_broadcast0_fp16_v2.comp:
// 37-105 with transpose_b = 0: lane i strides K by 32.
ORC_API void orc_matmul_nn_f16(const uint16_t *a, const uint16_t *b, uint16_t *c, uint32_t C,
                               uint32_t M, uint32_t N, uint32_t K, uint64_t a_cs, uint64_t a_hs,
                               uint64_t b_cs, uint64_t b_hs, uint64_t c_cs, uint64_t c_hs,
                               float scale, float bias, int act) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t ch = 0; ch < (int64_t)C; ++ch)
    for (int64_t n = 0; n < (int64_t)N; ++n)
      for (uint32_t m = 0; m < M; ++m) {
        const uint16_t *ar = a + ch * a_cs + m * a_hs;
        const uint16_t *bc = b + ch * b_cs + n;
        float lane[32];
        for (int l = 0; l < 32; ++l) {
          float s = 0.f;
          for (uint32_t k = l; k < K; k += 32) s += h2f(ar[k]) * h2f(bc[(uint64_t)k * b_hs]);
          lane[l] = s;
        }
        float v = 0.f;
        for (int i = 0; i < 32; ++i) v += lane[i];
        v = v * scale + bias;
        if (act == 1) v = v / (1.0f + expf(-v));
        c[ch * c_cs + m * c_hs + n] = f2h(v);
      }
}

// Row softmax with optional causal mask `col > row + offset` -> 0; the max is
// taken over the whole row including masked columns.
// src/shaders/softmax_fp16.comp:22-76; host src/ops/softmax.cpp:53-92.
ORC_API void orc_softmax_f16(const uint16_t *in, uint16_t *out, uint32_t C, uint32_t H,
                             uint32_t W, int seq_mask, uint32_t offset) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t c = 0; c < (int64_t)C; ++c)
    for (int64_t h = 0; h < (int64_t)H; ++h) {
      const uint16_t *r = in + ((size_t)c * H + h) * W;
      uint16_t *o = out + ((size_t)c * H + h) * W;
      float mx = h2f(r[0]);
      for (uint32_t i = 0; i < W; ++i) mx = std::max(mx, h2f(r[i]));
      float lane[32];
      for (int l = 0; l < 32; ++l) {
        float s = 0.f;
        for (uint32_t i = l; i < W; i += 32) {
          if (seq_mask > 0 && i > h + offset) continue;
          s += expf(h2f(r[i]) - mx);
        }
        lane[l] = s;
      }
      float sum = 0.f;
      for (int l = 0; l < 32; ++l) sum += lane[l];
      for (uint32_t i = 0; i < W; ++i)
        o[i] = (seq_mask > 0 && i > h + offset) ? (uint16_t)0 : f2h(expf(h2f(r[i]) - mx) / sum);
    }
}

// cos/sin tables. src/ops/rope.cpp:19-47 (compute_freq): freq_k =
// 1/pow(10000, 2k/dim) in fp32, angle = freq_k * float(pos).
ORC_API void orc_rope_table(uint32_t dim, uint32_t maxlen, float *freqc, float *freqs) {
  std::vector<float> freq(dim / 2);
  float n = .0f;
  for (uint32_t k = 0; k < dim / 2; ++k) {
    freq[k] = 1.0f / std::pow(10000.0f, n / dim);
    n += 2.0;
  }
  for (uint32_t i = 0; i < maxlen; ++i)
    for (uint32_t k = 0; k < dim / 2; ++k) {
      const float f = freq[k] * static_cast<float>(i);
      freqc[(size_t)i * (dim / 2) + k] = std::cos(f);
      freqs[(size_t)i * (dim / 2) + k] = std::sin(f);
    }
}

// In-place rotation of adjacent pairs. src/shaders/rope_fp16.comp:18-49.
ORC_API void orc_rope_f16(uint16_t *x, uint32_t C, uint32_t H, uint32_t W, uint32_t offset,
                          const float *freqc, const float *freqs) {
  for (uint32_t c = 0; c < C; ++c)
    for (uint32_t h = 0; h < H; ++h)
      for (uint32_t i = 0; i < W / 2; ++i) {
        const size_t fi = (size_t)(h + offset) * (W / 2) + i;
        const float fc = freqc[fi], fs = freqs[fi];
        uint16_t *p = x + ((size_t)c * H + h) * W + 2 * i;
        const float q0 = h2f(p[0]), q1 = h2f(p[1]);
        p[0] = f2h(q0 * fc - q1 * fs);
        p[1] = f2h(q0 * fs + q1 * fc);
      }
}

// cache[c, (offset+y) % HO, :] = kv[c, y, :]. src/shaders/update_kvcache_fp16.comp:21-39.
ORC_API void orc_update_kvcache_f16(uint16_t *cache, const uint16_t *kv, uint32_t C, uint32_t H,
                                    uint32_t W, uint32_t HO, uint32_t WO, uint32_t offset) {
  for (uint32_t c = 0; c < C; ++c)
    for (uint32_t y = 0; y < H; ++y)
      memcpy(cache + ((size_t)c * HO + (offset + y) % HO) * WO, kv + ((size_t)c * H + y) * W,
             (size_t)W * 2);
}

// y = fp16(x*w*alpha), alpha = 1/sqrt(sum(x^2)/W + eps); 512 strided partial
// sums then a halving tree. src/shaders/rms_norm_fp16.comp:33-78.
ORC_API void orc_rms_norm_f16(const uint16_t *x, const float *w, uint16_t *y, uint32_t rows,
                              uint32_t W, float eps) {
  for (uint32_t r = 0; r < rows; ++r) {
    const uint16_t *xr = x + (size_t)r * W;
    float part[512];
    for (int t = 0; t < 512; ++t) {
      float s = 0.f;
      for (uint32_t i = t; i < W; i += 512) {
        const float v = h2f(xr[i]);
        s += v * v;
      }
      part[t] = s;
    }
    for (int i = 256; i > 0; i /= 2)
      for (int t = 0; t < i; ++t) part[t] += part[t + i];
    const float alpha = 1.0f / sqrtf(part[0] / (float)W + eps);
    for (uint32_t i = 0; i < W; ++i) y[(size_t)r * W + i] = f2h(h2f(xr[i]) * w[i] * alpha);
  }
}

// y <- fp16(x + y), written into the second operand.
// src/shaders/element_wise_fp16.comp:19-31 (op_type 0); src/ops/elementwise.cpp:68-102.
ORC_API void orc_add_f16(const uint16_t *x, uint16_t *y, uint64_t n) {
  for (uint64_t i = 0; i < n; ++i) y[i] = f2h(h2f(x[i]) + h2f(y[i]));
}

// Row gather with dequantisation; ids >= vocab map to UNK.
// src/shaders/embedding_q8_0.comp:39-85; src/ops/embedding.cpp:58-114.
ORC_API void orc_embedding_q8_0(const uint8_t *vocab, const uint32_t *ids, uint16_t *out,
                                uint32_t T, uint32_t VH, uint32_t VW, uint32_t unk) {
  const uint32_t nb = (VW + 31) / 32;
  for (uint32_t t = 0; t < T; ++t) {
    uint32_t tok = ids[t];
    if (tok >= VH) tok = unk;
    for (uint32_t b = 0; b < nb; ++b) {
      const uint8_t *blk = vocab + ((size_t)tok * nb + b) * 34;
      uint16_t hs;
      memcpy(&hs, blk, 2);
      const float d = h2f(hs);
      for (uint32_t i = 0; i < 32 && b * 32 + i < VW; ++i)
        out[(size_t)t * VW + b * 32 + i] = f2h((float)(int8_t)blk[2 + i] * d);
    }
  }
}
// src/shaders/embedding_fp16.comp:29-59.
ORC_API void orc_embedding_f16(const uint16_t *vocab, const uint32_t *ids, uint16_t *out,
                               uint32_t T, uint32_t VH, uint32_t VW, uint32_t unk) {
  for (uint32_t t = 0; t < T; ++t) {
    uint32_t tok = ids[t];
    if (tok >= VH) tok = unk;
    memcpy(out + (size_t)t * VW, vocab + (size_t)tok * VW, (size_t)VW * 2);
  }
}

// Row arg-max, strict compare so the lowest index wins a tie.
// src/shaders/argmax_stage0_fp16.comp:69-76 and argmax_stage1.comp:40-52.
ORC_API void orc_argmax_f16(const uint16_t *x, uint32_t *out, uint32_t rows, uint32_t W) {
  for (uint32_t r = 0; r < rows; ++r) {
    const uint16_t *p = x + (size_t)r * W;
    float v = h2f(p[0]);
    uint32_t idx = 0;
    for (uint32_t i = 1; i < W; ++i)
      if (h2f(p[i]) > v) {
        v = h2f(p[i]);
        idx = i;
      }
    out[r] = idx;
  }
}
// Greedy pick over fp32 logits, lowest index on ties (TopkSampler(1):
// models/samplers.cpp:37-64 sorts descending; the tie order there is unspecified).
ORC_API uint32_t orc_argmax_f32(const float *x, uint32_t W) {
  uint32_t idx = 0;
  for (uint32_t i = 1; i < W; ++i)
    if (x[i] > x[idx]) idx = i;
  return idx;
}

// [C,H,W] -> [H,C,W]. src/shaders/transpose_type0_fp16.comp.
static void transpose_chw_hcw(const uint16_t *in, uint16_t *out, uint32_t C, uint32_t H,
                              uint32_t W) {
  for (uint32_t c = 0; c < C; ++c)
    for (uint32_t h = 0; h < H; ++h)
      memcpy(out + ((size_t)h * C + c) * W, in + ((size_t)c * H + h) * W, (size_t)W * 2);
}
ORC_API void orc_transpose_f16(const uint16_t *in, uint16_t *out, uint32_t C, uint32_t H,
                               uint32_t W) {
  transpose_chw_hcw(in, out, C, H, W);
}

// ---------------------------------------------------------------------------
// Attention sub-block. src/ops/multiheadattention_v2.cpp:140-325:
// kqv -> [T,heads,dim] -> (clip Q to the last token) -> transpose to
// [heads,T,dim] -> rope(Q), rope(K) at `offset` -> cache append -> K,V = cache
// view of min(offset+T, maxlen) rows -> QK^T/sqrt(dim) -> masked softmax with
// offset W-H -> P.V -> transpose back -> o_proj.
// ---------------------------------------------------------------------------
struct OrcAttn {
  uint32_t heads, dim, maxlen, width;  // width = heads*dim
  std::vector<uint16_t> kcache, vcache;
  std::vector<float> freqc, freqs;
};

static void attn_init(OrcAttn &a, uint32_t heads, uint32_t dim, uint32_t maxlen) {
  a.heads = heads;
  a.dim = dim;
  a.maxlen = maxlen;
  a.width = heads * dim;
  a.kcache.assign((size_t)heads * maxlen * dim, 0);
  a.vcache.assign((size_t)heads * maxlen * dim, 0);
  // The reference sizes its tables for 2*maxlen positions but uploads only the
  // first maxlen rows (src/ops/rope.cpp:73-96: the byte count uses sizeof(fp16)
  // on fp32 data), so positions >= maxlen read uninitialised memory there. Here
  // all 2*maxlen rows are computed: defined behaviour where the reference has none.
  a.freqc.resize((size_t)2 * maxlen * dim / 2);
  a.freqs.resize((size_t)2 * maxlen * dim / 2);
  orc_rope_table(dim, 2 * maxlen, a.freqc.data(), a.freqs.data());
}

// Everything after the KQV projection and before o_proj; k,q,v are [T, heads*dim].
static void attn_core(OrcAttn &a, const uint16_t *k, const uint16_t *q, const uint16_t *v,
                      uint32_t T, uint32_t offset, bool clip, uint16_t *concat /*[Tq, width]*/) {
  const uint32_t H = a.heads, D = a.dim;
  const uint32_t Tq = clip ? 1 : T;
  std::vector<uint16_t> tk((size_t)H * T * D), tq((size_t)H * Tq * D), tv((size_t)H * T * D);
  transpose_chw_hcw(k, tk.data(), T, H, D);
  transpose_chw_hcw(v, tv.data(), T, H, D);
  transpose_chw_hcw(clip ? q + (size_t)(T - 1) * a.width : q, tq.data(), Tq, H, D);
  // Rope on the clipped Q uses row index 0 + offset (multiheadattention_v2.cpp:251):
  // the reference passes the same `offset` for Q and K even when Q was clipped.
  orc_rope_f16(tq.data(), H, Tq, D, offset, a.freqc.data(), a.freqs.data());
  orc_rope_f16(tk.data(), H, T, D, offset, a.freqc.data(), a.freqs.data());
  orc_update_kvcache_f16(a.kcache.data(), tk.data(), H, T, D, a.maxlen, D, offset);
  orc_update_kvcache_f16(a.vcache.data(), tv.data(), H, T, D, a.maxlen, D, offset);
  const uint32_t L = std::min(offset + T, a.maxlen);
  std::vector<uint16_t> s((size_t)H * Tq * L), p((size_t)H * Tq * L), o((size_t)H * Tq * D);
  const uint64_t ccs = (uint64_t)a.maxlen * D;
  orc_matmul_tb_f16(tq.data(), a.kcache.data(), s.data(), H, Tq, L, D, (uint64_t)Tq * D, D, ccs,
                    D, (uint64_t)Tq * L, L, 1.0f / std::sqrt(static_cast<float>(D)), 0.f, 0);
  orc_softmax_f16(s.data(), p.data(), H, Tq, L, 1, L - Tq);
  orc_matmul_nn_f16(p.data(), a.vcache.data(), o.data(), H, Tq, D, L, (uint64_t)Tq * L, L, ccs,
                    D, (uint64_t)Tq * D, D, 1.f, 0.f, 0);
  transpose_chw_hcw(o.data(), concat, H, Tq, D);
}

ORC_API void *orc_attn_create(uint32_t heads, uint32_t dim, uint32_t maxlen) {
  OrcAttn *a = new OrcAttn();
  attn_init(*a, heads, dim, maxlen);
  return a;
}
ORC_API void orc_attn_destroy(void *h) { delete (OrcAttn *)h; }
// Caches are [heads, maxlen, dim] fp16.
ORC_API uint16_t *orc_attn_kcache(void *h) { return ((OrcAttn *)h)->kcache.data(); }
ORC_API uint16_t *orc_attn_vcache(void *h) { return ((OrcAttn *)h)->vcache.data(); }

ORC_API void orc_attn_forward_q8_0(void *h, const uint16_t *x, const uint8_t *wk,
                                   const uint8_t *wq, const uint8_t *wv, const uint8_t *wo,
                                   uint32_t T, uint32_t offset, int clip, uint16_t *out) {
  OrcAttn &a = *(OrcAttn *)h;
  const uint32_t Wd = a.width, Tq = clip ? 1 : T;
  std::vector<uint16_t> k((size_t)T * Wd), q((size_t)T * Wd), v((size_t)T * Wd),
      cc((size_t)Tq * Wd);
  orc_kqv_q8_0(x, wk, wq, wv, k.data(), q.data(), v.data(), T, Wd, Wd);
  attn_core(a, k.data(), q.data(), v.data(), T, offset, clip != 0, cc.data());
  orc_matmul_q8_0(cc.data(), wo, out, Tq, Wd, Wd, 1.f, 0.f, 0);
}

// ---------------------------------------------------------------------------
// Decoder block and model. models/llama2.h:160-213 (Llama2Block::operator()),
// 283-298 (OutputLayer), 683-843 (Model::operator()).
// ---------------------------------------------------------------------------
struct OrcLayer {
  const float *attn_norm, *ffn_norm;
  const uint8_t *wq, *wk, *wv, *wo, *gate, *up, *down;
  OrcAttn attn;
};
struct OrcModel {
  uint32_t dim, heads, head_dim, ffn, vocab, layers, maxlen;
  float eps, final_eps;
  std::vector<OrcLayer> L;
  const uint8_t *tok_embd, *output;
  const float *output_norm;
  bool fp16 = false;  // weights are dense fp16 [out,in] instead of Q8_0 blocks
  std::vector<std::vector<uint8_t>> owned8;
  std::vector<std::vector<float>> owned32;
};

ORC_API void *orc_model_create(uint32_t dim, uint32_t heads, uint32_t ffn, uint32_t vocab,
                               uint32_t layers, uint32_t maxlen, float eps, float final_eps) {
  OrcModel *m = new OrcModel();
  m->dim = dim;
  m->heads = heads;
  m->head_dim = dim / heads;
  m->ffn = ffn;
  m->vocab = vocab;
  m->layers = layers;
  m->maxlen = maxlen;
  m->eps = eps;
  m->final_eps = final_eps;
  m->L.resize(layers);
  for (auto &l : m->L) attn_init(l.attn, heads, m->head_dim, maxlen);
  return m;
}
ORC_API void orc_model_destroy(void *h) { delete (OrcModel *)h; }

// Tensor ids of the synthetic model: layer*16 + slot; globals use layer = n_layers.
enum { S_ATTN_NORM = 0, S_WQ, S_WK, S_WV, S_WO, S_FFN_NORM, S_GATE, S_UP, S_DOWN };
enum { G_TOK_EMBD = 0, G_OUT_NORM, G_OUTPUT };

// Weights N(0, wstd) -> Q8_0 (or, for an fp16 model, rounded to fp16); norm weights 1 + N(0, nstd).
static void model_synth(OrcModel &m, uint64_t seed, float wstd, float nstd) {
  auto q8 = [&](uint64_t id, uint32_t rows, uint32_t K) {
    if (m.fp16) {
      m.owned8.emplace_back((size_t)rows * K * 2);
      orc_synth_normal_f16(seed, id, 0, (uint64_t)rows * K, 0.f, wstd, (uint16_t *)m.owned8.back().data());
    } else {
      m.owned8.emplace_back((size_t)rows * ((K + 31) / 32) * 34);
      orc_synth_q8_0(seed, id, rows, K, 0.f, wstd, m.owned8.back().data());
    }
    return (const uint8_t *)m.owned8.back().data();
  };
  auto nw = [&](uint64_t id, uint32_t n) {
    m.owned32.emplace_back(n);
    orc_synth_normal_f32(seed, id, 0, n, 1.f, nstd, m.owned32.back().data());
    return (const float *)m.owned32.back().data();
  };
  for (uint32_t l = 0; l < m.layers; ++l) {
    OrcLayer &y = m.L[l];
    const uint64_t b = (uint64_t)l * 16;
    y.attn_norm = nw(b + S_ATTN_NORM, m.dim);
    y.wq = q8(b + S_WQ, m.dim, m.dim);
    y.wk = q8(b + S_WK, m.dim, m.dim);
    y.wv = q8(b + S_WV, m.dim, m.dim);
    y.wo = q8(b + S_WO, m.dim, m.dim);
    y.ffn_norm = nw(b + S_FFN_NORM, m.dim);
    y.gate = q8(b + S_GATE, m.ffn, m.dim);
    y.up = q8(b + S_UP, m.ffn, m.dim);
    y.down = q8(b + S_DOWN, m.dim, m.ffn);
  }
  const uint64_t g = (uint64_t)m.layers * 16;
  m.tok_embd = q8(g + G_TOK_EMBD, m.vocab, m.dim);
  m.output_norm = nw(g + G_OUT_NORM, m.dim);
  m.output = q8(g + G_OUTPUT, m.vocab, m.dim);
}
ORC_API void orc_model_synth(void *h, uint64_t seed, float wstd, float nstd) {
  OrcModel &m = *(OrcModel *)h;
  m.fp16 = false;
  model_synth(m, seed, wstd, nstd);
}
// The FP16-weights build of the model (models/llama2.h picks the dtype per GGUF tensor).
ORC_API void orc_model_synth_f16(void *h, uint64_t seed, float wstd, float nstd) {
  OrcModel &m = *(OrcModel *)h;
  m.fp16 = true;
  model_synth(m, seed, wstd, nstd);
}

// Raw 34-byte-block bytes of one weight, for upload to the device under test.
ORC_API const void *orc_model_weight(void *h, uint32_t layer, uint32_t slot, uint64_t *bytes) {
  OrcModel &m = *(OrcModel *)h;
  const size_t q = m.fp16 ? (size_t)m.dim * 2 : (size_t)(m.dim / 32) * 34, qf = m.fp16 ? (size_t)m.ffn * 2 : (size_t)(m.ffn / 32) * 34;
  if (layer < m.layers) {
    OrcLayer &y = m.L[layer];
    switch (slot) {
      case S_ATTN_NORM: *bytes = (uint64_t)m.dim * 4; return y.attn_norm;
      case S_WQ: *bytes = m.dim * q; return y.wq;
      case S_WK: *bytes = m.dim * q; return y.wk;
      case S_WV: *bytes = m.dim * q; return y.wv;
      case S_WO: *bytes = m.dim * q; return y.wo;
      case S_FFN_NORM: *bytes = (uint64_t)m.dim * 4; return y.ffn_norm;
      case S_GATE: *bytes = m.ffn * q; return y.gate;
      case S_UP: *bytes = m.ffn * q; return y.up;
      case S_DOWN: *bytes = m.dim * qf; return y.down;
    }
  } else {
    switch (slot) {
      case G_TOK_EMBD: *bytes = m.vocab * q; return m.tok_embd;
      case G_OUT_NORM: *bytes = (uint64_t)m.dim * 4; return m.output_norm;
      case G_OUTPUT: *bytes = m.vocab * q; return m.output;
    }
  }
  *bytes = 0;
  return nullptr;
}

ORC_API uint16_t *orc_model_kcache(void *h, uint32_t layer) {
  return ((OrcModel *)h)->L[layer].attn.kcache.data();
}
ORC_API uint16_t *orc_model_vcache(void *h, uint32_t layer) {
  return ((OrcModel *)h)->L[layer].attn.vcache.data();
}

// One block on hidden states x [T, dim] -> out [To, dim], To = 1 when `clip`
// (the last block keeps only the last token: models/llama2.h:181-191).
// y[M,N] = x[M,K] . w[N,K]^T with dense fp16 weights (matmul_b0_tb_fp16_v2.comp).
static void linear_f16(const uint16_t *x, const uint8_t *w, uint16_t *y, uint32_t M, uint32_t N, uint32_t K) {
  orc_matmul_tb_f16(x, (const uint16_t *)w, y, 1, M, N, K, (uint64_t)M * K, K, (uint64_t)N * K, K, (uint64_t)M * N, N, 1.f, 0.f, 0);
}

static void block_forward(OrcModel &m, OrcLayer &y, const uint16_t *x, uint32_t T,
                          uint32_t offset, bool clip, uint16_t *out) {
  const uint32_t D = m.dim, To = clip ? 1 : T;
  std::vector<uint16_t> normed((size_t)T * D), added((size_t)To * D), normed2((size_t)To * D),
      feed((size_t)To * D), attn((size_t)To * D);
  orc_rms_norm_f16(x, y.attn_norm, normed.data(), T, D, m.eps);
  if (m.fp16) {
    // MultiHeadAttentionV2 with FP16 weights: three MatMuls, the shared core, o_proj
    // (src/ops/multiheadattention_v2.cpp:186-300)
    std::vector<uint16_t> k((size_t)T * D), q((size_t)T * D), v((size_t)T * D), cc((size_t)To * D);
    linear_f16(normed.data(), y.wk, k.data(), T, D, D);
    linear_f16(normed.data(), y.wq, q.data(), T, D, D);
    linear_f16(normed.data(), y.wv, v.data(), T, D, D);
    attn_core(y.attn, k.data(), q.data(), v.data(), T, offset, clip, cc.data());
    linear_f16(cc.data(), y.wo, attn.data(), To, D, D);
  } else {
    orc_attn_forward_q8_0(&y.attn, normed.data(), y.wk, y.wq, y.wv, y.wo, T, offset, clip,
                          attn.data());
  }
  // add_op_(transformed, in): in <- fp16(transformed + in)   (llama2.h:193-196)
  memcpy(added.data(), clip ? x + (size_t)(T - 1) * D : x, (size_t)To * D * 2);
  orc_add_f16(attn.data(), added.data(), (size_t)To * D);
  orc_rms_norm_f16(added.data(), y.ffn_norm, normed2.data(), To, D, m.eps);
  if (m.fp16)
    orc_feed_forward_f16(normed2.data(), (const uint16_t *)y.gate, (const uint16_t *)y.down, (const uint16_t *)y.up, feed.data(), To, D,
                         m.ffn);
  else
    orc_feed_forward_q8_0(normed2.data(), y.gate, y.down, y.up, feed.data(), To, D, m.ffn);
  // add_op2_(feed, added): added <- fp16(feed + added)        (llama2.h:209)
  memcpy(out, added.data(), (size_t)To * D * 2);
  orc_add_f16(feed.data(), out, (size_t)To * D);
}

ORC_API void orc_block_forward(void *h, uint32_t layer, const uint16_t *x, uint32_t T,
                               uint32_t offset, int clip, uint16_t *out) {
  OrcModel &m = *(OrcModel *)h;
  block_forward(m, m.L[layer], x, T, offset, clip != 0, out);
}

// Model::operator()(toks, offset) -> fp32 logits of the last token.
// Optionally also returns the final hidden state (fp16, [dim]) for diagnostics.
ORC_API void orc_model_forward(void *h, const uint32_t *toks, uint32_t T, uint32_t offset,
                               float *logits, uint16_t *hidden_out) {
  OrcModel &m = *(OrcModel *)h;
  const uint32_t D = m.dim;
  std::vector<uint16_t> x((size_t)T * D), nx((size_t)T * D);
  if (m.fp16)
    orc_embedding_f16((const uint16_t *)m.tok_embd, toks, x.data(), T, m.vocab, D, 0);
  else
    orc_embedding_q8_0(m.tok_embd, toks, x.data(), T, m.vocab, D, 0);
  for (uint32_t l = 0; l < m.layers; ++l) {
    const bool clip = l == m.layers - 1;
    block_forward(m, m.L[l], x.data(), T, offset, clip, nx.data());
    x.swap(nx);
  }
  if (hidden_out) memcpy(hidden_out, x.data(), (size_t)D * 2);
  std::vector<uint16_t> normed(D), lg(m.vocab);
  orc_rms_norm_f16(x.data(), m.output_norm, normed.data(), 1, D, m.final_eps);
  if (m.fp16)
    linear_f16(normed.data(), m.output, lg.data(), 1, m.vocab, D);
  else
    orc_matmul_q8_0(normed.data(), m.output, lg.data(), 1, m.vocab, D, 1.f, 0.f, 0);
  for (uint32_t i = 0; i < m.vocab; ++i) logits[i] = h2f(lg[i]);  // Cast fp16->fp32
}

// llama2_infer's loop shape: prefill, then n one-token steps with greedy pick
// (app/llama2_infer.cpp:141-210). Returns the generated ids and, per step, the
// gap between the two largest logits (for diagnosing ties).
ORC_API void orc_model_generate(void *h, const uint32_t *prompt, uint32_t P, uint32_t n_gen,
                                uint32_t *out_ids, float *out_gap) {
  OrcModel &m = *(OrcModel *)h;
  std::vector<float> logits(m.vocab);
  auto pick = [&](uint32_t step) {
    const uint32_t id = orc_argmax_f32(logits.data(), m.vocab);
    float second = -INFINITY;
    for (uint32_t i = 0; i < m.vocab; ++i)
      if (i != id && logits[i] > second) second = logits[i];
    out_ids[step] = id;
    if (out_gap) out_gap[step] = logits[id] - second;
    return id;
  };
  orc_model_forward(h, prompt, P, 0, logits.data(), nullptr);
  uint32_t tok = pick(0);
  for (uint32_t i = 1; i < n_gen; ++i) {
    orc_model_forward(h, &tok, 1, P + i - 1, logits.data(), nullptr);
    tok = pick(i);
  }
}
