// Small HBM/latency-bound kernels around the weight stream: layout repack,
// quantizer, synthetic data, RMSNorm, residual add, embedding gather, arg-max,
// softmax, RoPE, KV-cache append, transpose, slice, casts and the generic
// batched fp16 mat-mul of the operator API.
#include <mutex>

#include "common.cuh"
#include "kernels.h"
#include "runtime.h"

namespace vkl {
namespace {

// ------------------------------------------------------------ layout repack
// 34-byte block: [fp16 d][32 x int8] (src/shaders/common.h:8-10).
__global__ void q8_repack_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst,
                                 Q8Layout L) {
  const size_t nvec = (size_t)L.tiles * L.groups * 4 * 32;  // 16-byte code vectors
  const size_t nsc = (size_t)L.tiles * L.groups * 8;        // 16-byte scale vectors
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < nvec) {
    const uint32_t lane = i & 31, b = (i >> 5) % (L.groups * 4), tile = (i >> 5) / (L.groups * 4);
    const uint32_t g = lane >> 2, t = lane & 3;
    uint8_t v[16];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const uint32_t row = tile * 16 + g + half * 8;
      const bool ok = row < L.N && b < L.blocks;
      const uint8_t *blk = src + ((size_t)row * L.blocks + b) * 34 + 2 + t * 8;
#pragma unroll
      for (int k = 0; k < 8; ++k) v[half * 8 + q8_byte_pos(k)] = ok ? (uint8_t)(blk[k] ^ 0x80) : (uint8_t)0x80;
    }
    *reinterpret_cast<uint4 *>(dst + i * 16) = *reinterpret_cast<uint4 *>(v);
  } else if (i < nvec + nsc) {
    const size_t j = i - nvec;
    const uint32_t g = j & 7, grp = (j >> 3) % L.groups, tile = (j >> 3) / L.groups;
    uint16_t v[8];
#pragma unroll
    for (int half = 0; half < 2; ++half)
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t row = tile * 16 + g + half * 8, b = grp * 4 + k;
        uint16_t d = 0;
        if (row < L.N && b < L.blocks) {
          const uint8_t *blk = src + ((size_t)row * L.blocks + b) * 34;
          d = (uint16_t)blk[0] | ((uint16_t)blk[1] << 8);
        }
        v[half * 4 + k] = d;
      }
    *reinterpret_cast<uint4 *>(dst + L.codes_bytes() + j * 16) = *reinterpret_cast<uint4 *>(v);
  }
}

__global__ void q8_unpack_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst,
                                 Q8Layout L) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per block34
  if (i >= (size_t)L.N * L.blocks) return;
  const uint32_t b = i % L.blocks, row = i / L.blocks;
  const uint32_t tile = row >> 4, r = row & 15, g = r & 7, half = r >> 3;
  const uint16_t *sc = reinterpret_cast<const uint16_t *>(src + L.codes_bytes());
  const uint16_t d = sc[(((size_t)tile * L.groups + (b >> 2)) * 8 + g) * 8 + half * 4 + (b & 3)];
  uint8_t *o = dst + i * 34;
  o[0] = d & 0xff;
  o[1] = d >> 8;
  for (uint32_t t = 0; t < 4; ++t) {
    const uint8_t *c = src + (((size_t)tile * L.groups * 4 + b) * 32 + g * 4 + t) * 16 + half * 8;
    for (int k = 0; k < 8; ++k) o[2 + t * 8 + k] = c[q8_byte_pos(k)] ^ 0x80;
  }
}

// ---------------------------------------------------------------- quantizer
// One warp per 32-value block; arithmetic of src/core/quants.h:58-92:
// scale = absmax/127.0f, inverse = scale > 0 ? 127.0f/absmax : 0,
// code = (int8)roundf(x*inverse); the stored scale is fp16 (nearest even).
__device__ __forceinline__ void quantize_block_store(float x, bool valid, uint8_t *blk, int lane) {
  float amax = warp_max(valid ? fabsf(x) : 0.f);
  const float scale = amax / 127.0f;
  const float inv = scale > 0 ? 127.0f / amax : 0.f;
  const int8_t q = valid ? (int8_t)roundf(x * inv) : (int8_t)0;
  // Blocks are 34 bytes: every block start is 2-byte aligned, so the scale is one
  // 16-bit store.
  if (lane == 0) *reinterpret_cast<__half *>(blk) = __float2half_rn(scale);
  blk[2 + lane] = (uint8_t)q;
}

__global__ void q8_quantize_kernel(const float *__restrict__ src, uint8_t *__restrict__ dst,
                                   uint32_t N, uint32_t K) {
  const uint32_t blocks = (K + 31) / 32;
  const size_t wid = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= (size_t)N * blocks) return;
  const uint32_t b = wid % blocks, row = wid / blocks;
  const uint32_t k = b * 32 + lane;
  const bool valid = k < K;
  const float x = valid ? src[(size_t)row * K + k] : 0.f;
  quantize_block_store(x, valid, dst + wid * 34, lane);
}

// ------------------------------------------------------------ synthetic data
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
__host__ __device__ inline uint64_t synth_key_mix(uint64_t z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
__device__ __forceinline__ float synth_z(uint64_t key, uint64_t i) {
  uint32_t s = 0;
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    const uint64_t h = mix64(key + (3 * i + j + 1) * 0x9E3779B97F4A7C15ull);
    s += (uint32_t)(h & 0xFFFF) + (uint32_t)((h >> 16) & 0xFFFF) + (uint32_t)((h >> 32) & 0xFFFF) +
         (uint32_t)((h >> 48) & 0xFFFF);
  }
  return (float)((int32_t)s - 393210) * (1.0f / 65536.0f);
}
inline uint64_t synth_key(uint64_t seed, uint64_t tensor) {
  return synth_key_mix(seed * 0x9E3779B97F4A7C15ull + tensor * 0xD1B54A32D192ED03ull +
                       0x2545F4914F6CDD1Dull);
}

__global__ void synth_f32_kernel(float *dst, uint64_t key, uint64_t first, uint64_t n, float mean,
                                 float stdv) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (uint64_t)gridDim.x * blockDim.x)
    dst[i] = __fmaf_rn(synth_z(key, first + i), stdv, mean);
}
__global__ void synth_f16_kernel(__half *dst, uint64_t key, uint64_t first, uint64_t n,
                                 float mean, float stdv) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (uint64_t)gridDim.x * blockDim.x)
    dst[i] = __float2half_rn(__fmaf_rn(synth_z(key, first + i), stdv, mean));
}
__global__ void synth_q8_kernel(uint8_t *dst, uint64_t key, uint32_t N, uint32_t K, float mean,
                                float stdv, uint32_t row0, uint32_t col0, uint32_t ld_full) {
  const uint32_t blocks = (K + 31) / 32;
  const int lane = threadIdx.x & 31;
  const size_t nw = (size_t)N * blocks;
  for (size_t wid = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; wid < nw;
       wid += ((size_t)gridDim.x * blockDim.x) >> 5) {
    const uint32_t b = wid % blocks, row = wid / blocks;
    const uint32_t k = b * 32 + lane;
    const bool valid = k < K;
    const float x = valid ? __fmaf_rn(synth_z(key, (uint64_t)(row0 + row) * ld_full + col0 + k), stdv, mean) : 0.f;
    quantize_block_store(x, valid, dst + wid * 34, lane);
  }
}

// ------------------------------------------------------------------ RMSNorm
// y = fp16(x*w*alpha), alpha = 1/sqrt(mean(x^2)+eps). src/shaders/rms_norm_fp16.comp:33-78.
__global__ void __launch_bounds__(256) rms_norm_kernel(const __half *__restrict__ x,
                                                       const float *__restrict__ w,
                                                       __half *__restrict__ y, uint32_t W,
                                                       float eps) {
  __shared__ float ssum[8];
  const __half *xr = x + (size_t)blockIdx.x * W;
  __half *yr = y + (size_t)blockIdx.x * W;
  float s = 0.f;
  for (uint32_t i = threadIdx.x; i < W; i += 256) {
    const float v = __half2float(xr[i]);
    s += v * v;
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) ssum[threadIdx.x >> 5] = s;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += ssum[i];
  const float alpha = 1.0f / sqrtf(tot / (float)W + eps);
  for (uint32_t i = threadIdx.x; i < W; i += 256)
    yr[i] = __float2half_rn(__half2float(xr[i]) * w[i] * alpha);
}

// y <- fp16(x op y). src/shaders/element_wise_fp16.comp:19-48.
__global__ void elementwise_kernel(const __half *__restrict__ x, __half *y, uint64_t n, int op) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float a = __half2float(x[i]), b = __half2float(y[i]);
  float r = a + b;
  if (op == 1) r = a - b;
  if (op == 2) r = a * b;
  if (op == 3) r = a / b;
  y[i] = __float2half_rn(r);
}

// x <- fp16(x op alpha). src/shaders/element_wise_constant_fp16.comp:19-44 (fp32 arithmetic form).
__global__ void elementwise_scalar_kernel(__half *x, uint64_t n, int op, float alpha) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float a = __half2float(x[i]);
  float r = a + alpha;
  if (op == 1) r = a - alpha;
  if (op == 2) r = a * alpha;
  if (op == 3) r = a / alpha;
  x[i] = __float2half_rn(r);
}

// out[c, h, w + off_w ...] = in[c, h, w]: one input of a concatenation copied to its place
// (src/shaders/concat_fp16.comp:27-49: element offset OFFSET inside the output's [c][h][w] strides).
__global__ void concat_copy_kernel(const __half *__restrict__ in, __half *__restrict__ out, uint32_t C, uint32_t H, uint32_t W,
                                   uint64_t ocs, uint64_t ohs, uint64_t offset) {
  const uint64_t n = (uint64_t)C * H * W, i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const uint32_t w = (uint32_t)(i % W), h = (uint32_t)((i / W) % H), c = (uint32_t)(i / ((uint64_t)W * H));
  out[c * ocs + h * ohs + w + offset] = in[i];
}

// One warp per row: sum / max / min over the row, times mean_scale (src/shaders/reduce_fp16.comp:24-76:
// lane-strided partial results, then a subgroup reduction; max and min start from the row's first value).
__global__ void reduce_kernel(const __half *__restrict__ in, __half *__restrict__ out, uint32_t rows, uint32_t W, int op, float mean_scale) {
  const uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const __half *x = in + (size_t)row * W;
  float r = op == 0 ? 0.f : __half2float(x[0]);
  for (uint32_t w = lane; w < W; w += 32) {
    const float v = __half2float(x[w]);
    r = op == 0 ? r + v : op == 1 ? fmaxf(r, v) : fminf(r, v);
  }
  // lanes combined in lane order (a subgroup reduction has no defined order; the oracle sums the same way)
  float tot = __shfl_sync(0xffffffffu, r, 0);
  for (int l = 1; l < 32; ++l) {
    const float v = __shfl_sync(0xffffffffu, r, l);
    tot = op == 0 ? tot + v : op == 1 ? fmaxf(tot, v) : fminf(tot, v);
  }
  if (lane == 0) out[row] = __float2half_rn(tot * mean_scale);
}

// out[c, y, :] = cache[c, (y + offset) % H, :]. src/shaders/read_kvcache_fp16.comp.
__global__ void read_kvcache_kernel(const __half *__restrict__ cache, __half *__restrict__ out, uint32_t C, uint32_t H, uint32_t W, uint32_t offset,
                                    uint32_t len) {
  const uint64_t n = (uint64_t)C * len * W, i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const uint32_t w = (uint32_t)(i % W), y = (uint32_t)((i / W) % len), c = (uint32_t)(i / ((uint64_t)W * len));
  out[i] = cache[((size_t)c * H + (y + offset) % H) * W + w];
}

// ---------------------------------------------------------------- embedding
// out[t,:] = dequant(vocab[tok_t,:]); tok >= VH -> UNK. embedding_q8_0.comp:39-85.
__global__ void embedding_q8_kernel(const uint8_t *__restrict__ planes,
                                    const uint32_t *__restrict__ ids, __half *__restrict__ out,
                                    Q8Layout L, uint32_t unk) {
  uint32_t tok = ids[blockIdx.x];
  if (tok >= L.N) tok = unk;
  const uint32_t tile = tok >> 4, r = tok & 15, g = r & 7, half = r >> 3;
  const uint16_t *sc = reinterpret_cast<const uint16_t *>(planes + L.codes_bytes());
  for (uint32_t k = threadIdx.x; k < L.K; k += blockDim.x) {
    const uint32_t b = k >> 5, t = (k >> 3) & 3, i = k & 7;
    const uint8_t c = planes[(((size_t)tile * L.groups * 4 + b) * 32 + g * 4 + t) * 16 + half * 8 + q8_byte_pos(i)];
    const uint16_t d = sc[(((size_t)tile * L.groups + (b >> 2)) * 8 + g) * 8 + half * 4 + (b & 3)];
    const float q = (float)((int)c - 128);
    out[(size_t)blockIdx.x * L.K + k] = __float2half_rn(q * __half2float(__ushort_as_half(d)));
  }
}
__global__ void embedding_f16_kernel(const __half *__restrict__ vocab,
                                     const uint32_t *__restrict__ ids, __half *__restrict__ out,
                                     uint32_t VH, uint32_t VW, uint32_t unk) {
  uint32_t tok = ids[blockIdx.x];
  if (tok >= VH) tok = unk;
  for (uint32_t k = threadIdx.x; k < VW; k += blockDim.x)
    out[(size_t)blockIdx.x * VW + k] = vocab[(size_t)tok * VW + k];
}

// ------------------------------------------------------------------ arg-max
// Stage 0: best (value, index) of each 1024-wide chunk; stage 1: scan the
// chunk winners. Strict compares: the lowest index wins a tie
// (argmax_stage0_fp16.comp:69-76, argmax_stage1.comp:40-52).
struct Pair {
  uint32_t i;
  float v;
};
__device__ __forceinline__ bool better(float v, uint32_t i, float bv, uint32_t bi, int op) {
  if (op == 0) return v > bv || (v == bv && i < bi);
  return v < bv || (v == bv && i < bi);
}
__global__ void __launch_bounds__(256) argop0_kernel(const __half *__restrict__ x, Pair *part,
                                                     uint32_t W, uint32_t chunks, int op) {
  const uint32_t row = blockIdx.y, chunk = blockIdx.x;
  const __half *xr = x + (size_t)row * W;
  const uint32_t base = chunk * 1024;
  float bv = op == 0 ? -INFINITY : INFINITY;
  uint32_t bi = 0xffffffffu;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t i = base + j * 256 + threadIdx.x;
    if (i < W) {
      const float v = __half2float(xr[i]);
      if (bi == 0xffffffffu || better(v, i, bv, bi, op)) {
        bv = v;
        bi = i;
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (oi != 0xffffffffu && (bi == 0xffffffffu || better(ov, oi, bv, bi, op))) {
      bv = ov;
      bi = oi;
    }
  }
  __shared__ float sv[8];
  __shared__ uint32_t si[8];
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = bv;
    si[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (si[w] != 0xffffffffu && (bi == 0xffffffffu || better(sv[w], si[w], bv, bi, op))) {
        bv = sv[w];
        bi = si[w];
      }
    part[(size_t)row * chunks + chunk].i = bi;
    part[(size_t)row * chunks + chunk].v = bv;
  }
}
__global__ void argop1_kernel(const Pair *part, uint32_t *out, uint32_t rows, uint32_t chunks,
                              int op) {
  const uint32_t row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  float bv = part[(size_t)row * chunks].v;
  uint32_t bi = part[(size_t)row * chunks].i;
  for (uint32_t c = 1; c < chunks; ++c) {
    const Pair q = part[(size_t)row * chunks + c];
    if ((op == 0 && q.v > bv) || (op == 1 && q.v < bv)) {
      bv = q.v;
      bi = q.i;
    }
  }
  out[row] = bi;
}

// ------------------------------------------------------------------ softmax
// One warp per row; max over the whole row (masked columns included), masked
// columns (col > row + offset) excluded from the sum and written as 0.
// src/shaders/softmax_fp16.comp:22-76.
__global__ void softmax_kernel(const __half *__restrict__ in, __half *__restrict__ out,
                               uint32_t rows, uint32_t H, uint32_t W, int seq_mask,
                               uint32_t offset) {
  const uint32_t row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (row >= rows) return;
  const uint32_t h = row % H;
  const __half *r = in + (size_t)row * W;
  __half *o = out + (size_t)row * W;
  float mx = __half2float(r[0]);
  for (uint32_t i = lane; i < W; i += 32) mx = fmaxf(mx, __half2float(r[i]));
  mx = warp_max(mx);
  float s = 0.f;
  for (uint32_t i = lane; i < W; i += 32) {
    if (seq_mask > 0 && i > h + offset) continue;
    s += expf(__half2float(r[i]) - mx);
  }
  s = warp_sum(s);
  for (uint32_t i = lane; i < W; i += 32)
    o[i] = (seq_mask > 0 && i > h + offset) ? __ushort_as_half(0)
                                            : __float2half_rn(expf(__half2float(r[i]) - mx) / s);
}

// --------------------------------------------------------------------- RoPE
// Adjacent pairs (2i, 2i+1), tables indexed by row+offset. rope_fp16.comp:18-49.
__global__ void rope_kernel(__half *x, uint32_t C, uint32_t H, uint32_t W, uint64_t cs,
                            uint64_t hs, const uint32_t *pos_dev, uint32_t offset,
                            const float *__restrict__ fc, const float *__restrict__ fs) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  const uint32_t h = blockIdx.y, c = blockIdx.z;
  if (2 * i >= W) return;
  const uint32_t pos = (pos_dev ? *pos_dev : 0u) + offset + h;
  const size_t fi = (size_t)pos * (W / 2) + i;
  const float co = fc[fi], si = fs[fi];
  __half *p = x + c * cs + h * hs + 2 * i;
  const float q0 = __half2float(p[0]), q1 = __half2float(p[1]);
  p[0] = __float2half_rn(q0 * co - q1 * si);
  p[1] = __float2half_rn(q0 * si + q1 * co);
}

// cache[c,(offset+y)%HO,:] = kv[c,y,:]. update_kvcache_fp16.comp:21-39.
__global__ void update_kvcache_kernel(__half *cache, const __half *__restrict__ kv, uint32_t H,
                                      uint32_t W, uint32_t HO, uint32_t WO, uint32_t offset) {
  const uint32_t x = blockIdx.x * blockDim.x + threadIdx.x, y = blockIdx.y, c = blockIdx.z;
  if (x >= W) return;
  cache[((size_t)c * HO + (offset + y) % HO) * WO + x] = kv[((size_t)c * H + y) * W + x];
}

// [C,H,W] -> [H,C,W]. transpose_type0_fp16.comp.
__global__ void transpose_kernel(const __half *__restrict__ in, __half *__restrict__ out,
                                 uint32_t C, uint32_t H, uint32_t W) {
  const uint32_t x = blockIdx.x * blockDim.x + threadIdx.x, h = blockIdx.y, c = blockIdx.z;
  if (x >= W) return;
  out[((size_t)h * C + c) * W + x] = in[((size_t)c * H + h) * W + x];
}

// 3-D sub-block copy. slice_fp16.comp.
__global__ void slice_kernel(const __half *__restrict__ in, __half *__restrict__ out, uint32_t H,
                             uint32_t W, uint32_t c0, uint32_t h0, uint32_t w0, uint32_t EH,
                             uint32_t EW) {
  const uint32_t x = blockIdx.x * blockDim.x + threadIdx.x, h = blockIdx.y, c = blockIdx.z;
  if (x >= EW) return;
  out[((size_t)c * EH + h) * EW + x] = in[((size_t)(c + c0) * H + h + h0) * W + x + w0];
}

__global__ void cast_f16_f32_kernel(const __half *__restrict__ in, float *__restrict__ out,
                                    uint64_t n) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __half2float(in[i]);
}
__global__ void cast_f32_f16_kernel(const float *__restrict__ in, __half *__restrict__ out,
                                    uint64_t n) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __float2half_rn(in[i]);
}

// Generic batched fp16 mat-mul of the operator API (Q.K^T and P.V when the ops
// are used one by one): one warp per output element, fp32 accumulation.
// matmul_b0_tb_fp16_v2.comp:38-120 / matmul_broadcast0_fp16_v2.comp:37-105.
__global__ void bmm_f16_kernel(const __half *__restrict__ a, const __half *__restrict__ b,
                               __half *__restrict__ c, uint32_t M, uint32_t N, uint32_t K,
                               uint64_t a_cs, uint64_t a_hs, uint64_t b_cs, uint64_t b_hs,
                               uint64_t c_cs, uint64_t c_hs, int tb, float scale, float bias,
                               int act) {
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const uint32_t m = blockIdx.y, ch = blockIdx.z;
  if (n >= N) return;
  const __half *ar = a + ch * a_cs + m * a_hs;
  float s = 0.f;
  if (tb) {
    const __half *br = b + ch * b_cs + n * b_hs;
    for (uint32_t k = lane; k < K; k += 32) s += __half2float(ar[k]) * __half2float(br[k]);
  } else {
    const __half *bc = b + ch * b_cs + n;
    for (uint32_t k = lane; k < K; k += 32) s += __half2float(ar[k]) * __half2float(bc[(uint64_t)k * b_hs]);
  }
  s = warp_sum(s);
  if (lane == 0) {
    float v = s * scale + bias;
    if (act == 1) v = v / (1.0f + expf(-v));
    c[ch * c_cs + m * c_hs + n] = __float2half_rn(v);
  }
}

inline unsigned nblk(uint64_t n, unsigned per) { return (unsigned)((n + per - 1) / per); }

}  // namespace

cudaError_t launch_q8_repack(const uint8_t *src, uint8_t *dst, uint32_t N, uint32_t K,
                             cudaStream_t s) {
  const Q8Layout L = q8_layout(N, K);
  const size_t n = (size_t)L.tiles * L.groups * (4 * 32 + 8);
  q8_repack_kernel<<<nblk(n, 256), 256, 0, s>>>(src, dst, L);
  return cudaGetLastError();
}
cudaError_t launch_q8_unpack(const uint8_t *src, uint8_t *dst, uint32_t N, uint32_t K,
                             cudaStream_t s) {
  const Q8Layout L = q8_layout(N, K);
  q8_unpack_kernel<<<nblk((size_t)N * L.blocks, 256), 256, 0, s>>>(src, dst, L);
  return cudaGetLastError();
}
cudaError_t launch_q8_quantize(const float *src, uint8_t *dst, uint32_t N, uint32_t K,
                               cudaStream_t s) {
  const size_t warps = (size_t)N * ((K + 31) / 32);
  q8_quantize_kernel<<<nblk(warps * 32, 256), 256, 0, s>>>(src, dst, N, K);
  return cudaGetLastError();
}
cudaError_t launch_synth_f32(float *dst, uint64_t seed, uint64_t tensor, uint64_t first,
                             uint64_t n, float mean, float stdv, cudaStream_t s) {
  if (!n) return cudaSuccess;
  synth_f32_kernel<<<std::min(nblk(n, 256), 148u * 32), 256, 0, s>>>(dst, synth_key(seed, tensor), first, n, mean, stdv);
  return cudaGetLastError();
}
cudaError_t launch_synth_f16(__half *dst, uint64_t seed, uint64_t tensor, uint64_t first,
                             uint64_t n, float mean, float stdv, cudaStream_t s) {
  if (!n) return cudaSuccess;
  synth_f16_kernel<<<std::min(nblk(n, 256), 148u * 32), 256, 0, s>>>(dst, synth_key(seed, tensor), first, n, mean, stdv);
  return cudaGetLastError();
}
cudaError_t launch_synth_q8(uint8_t *dst, uint64_t seed, uint64_t tensor, uint32_t N, uint32_t K,
                            float mean, float stdv, uint32_t row0, uint32_t col0, uint32_t ld_full,
                            cudaStream_t s) {
  const size_t warps = (size_t)N * ((K + 31) / 32);
  synth_q8_kernel<<<std::min(nblk(warps * 32, 256), 148u * 64), 256, 0, s>>>(dst, synth_key(seed, tensor), N, K, mean, stdv, row0, col0, ld_full);
  return cudaGetLastError();
}
cudaError_t launch_rms_norm(const __half *x, const float *w, __half *y, uint32_t rows,
                            uint32_t W, float eps, cudaStream_t s) {
  if (!rows) return cudaSuccess;
  rms_norm_kernel<<<rows, 256, 0, s>>>(x, w, y, W, eps);
  return cudaGetLastError();
}
cudaError_t launch_add(const __half *x, __half *y, uint64_t n, int op, cudaStream_t s) {
  if (!n) return cudaSuccess;
  elementwise_kernel<<<nblk(n, 256), 256, 0, s>>>(x, y, n, op);
  return cudaGetLastError();
}
cudaError_t launch_scalar_op(__half *x, uint64_t n, int op, float alpha, cudaStream_t s) {
  if (!n) return cudaSuccess;
  elementwise_scalar_kernel<<<nblk(n, 256), 256, 0, s>>>(x, n, op, alpha);
  return cudaGetLastError();
}
cudaError_t launch_concat_copy(const __half *in, __half *out, uint32_t C, uint32_t H, uint32_t W, uint64_t ocs, uint64_t ohs, uint64_t offset,
                               cudaStream_t s) {
  const uint64_t n = (uint64_t)C * H * W;
  if (!n) return cudaSuccess;
  concat_copy_kernel<<<nblk(n, 256), 256, 0, s>>>(in, out, C, H, W, ocs, ohs, offset);
  return cudaGetLastError();
}
cudaError_t launch_reduce(const __half *in, __half *out, uint32_t rows, uint32_t W, int op, float mean_scale, cudaStream_t s) {
  if (!rows) return cudaSuccess;
  reduce_kernel<<<(rows + 7) / 8, 256, 0, s>>>(in, out, rows, W, op, mean_scale);
  return cudaGetLastError();
}
cudaError_t launch_read_kvcache(const __half *cache, __half *out, uint32_t C, uint32_t H, uint32_t W, uint32_t offset, uint32_t len,
                                cudaStream_t s) {
  const uint64_t n = (uint64_t)C * len * W;
  if (!n) return cudaSuccess;
  read_kvcache_kernel<<<nblk(n, 256), 256, 0, s>>>(cache, out, C, H, W, offset, len);
  return cudaGetLastError();
}
cudaError_t launch_embedding(const uint8_t *vocab, int is_q8, const uint32_t *ids, __half *out,
                             uint32_t T, uint32_t VH, uint32_t VW, uint32_t unk, cudaStream_t s) {
  if (!T) return cudaSuccess;
  if (is_q8)
    embedding_q8_kernel<<<T, 256, 0, s>>>(vocab, ids, out, q8_layout(VH, VW), unk);
  else
    embedding_f16_kernel<<<T, 256, 0, s>>>(reinterpret_cast<const __half *>(vocab), ids, out, VH, VW, unk);
  return cudaGetLastError();
}
size_t argop_partials_bytes(uint32_t rows, uint32_t W) { return (size_t)rows * ((W + 1023) / 1024) * sizeof(Pair); }
cudaError_t launch_argop(const __half *x, uint32_t *out, void *partials, uint32_t rows,
                         uint32_t W, int op, cudaStream_t s) {
  if (!rows || !W) return cudaSuccess;
  const uint32_t chunks = (W + 1023) / 1024;
  argop0_kernel<<<dim3(chunks, rows), 256, 0, s>>>(x, (Pair *)partials, W, chunks, op);
  argop1_kernel<<<nblk(rows, 128), 128, 0, s>>>((const Pair *)partials, out, rows, chunks, op);
  return cudaGetLastError();
}
cudaError_t launch_softmax(const __half *in, __half *out, uint32_t C, uint32_t H, uint32_t W,
                           int seq_mask, uint32_t offset, cudaStream_t s) {
  const uint32_t rows = C * H;
  if (!rows) return cudaSuccess;
  softmax_kernel<<<nblk((uint64_t)rows * 32, 128), 128, 0, s>>>(in, out, rows, H, W, seq_mask, offset);
  return cudaGetLastError();
}
cudaError_t launch_rope(__half *x, uint32_t C, uint32_t H, uint32_t W, uint64_t cs, uint64_t hs,
                        const uint32_t *pos_dev, uint32_t offset, const float *fc, const float *fs,
                        cudaStream_t s) {
  if (!C || !H) return cudaSuccess;
  rope_kernel<<<dim3(nblk(W / 2, 64), H, C), 64, 0, s>>>(x, C, H, W, cs, hs, pos_dev, offset, fc, fs);
  return cudaGetLastError();
}
cudaError_t launch_update_kvcache(__half *cache, const __half *kv, uint32_t C, uint32_t H,
                                  uint32_t W, uint32_t HO, uint32_t WO, uint32_t offset,
                                  cudaStream_t s) {
  if (!C || !H) return cudaSuccess;
  update_kvcache_kernel<<<dim3(nblk(W, 128), H, C), 128, 0, s>>>(cache, kv, H, W, HO, WO, offset);
  return cudaGetLastError();
}
cudaError_t launch_transpose(const __half *in, __half *out, uint32_t C, uint32_t H, uint32_t W,
                             cudaStream_t s) {
  if (!C || !H) return cudaSuccess;
  transpose_kernel<<<dim3(nblk(W, 128), H, C), 128, 0, s>>>(in, out, C, H, W);
  return cudaGetLastError();
}
cudaError_t launch_slice(const __half *in, __half *out, uint32_t C, uint32_t H, uint32_t W,
                         uint32_t c0, uint32_t h0, uint32_t w0, uint32_t EC, uint32_t EH,
                         uint32_t EW, cudaStream_t s) {
  (void)C;
  if (!EC || !EH || !EW) return cudaSuccess;
  slice_kernel<<<dim3(nblk(EW, 128), EH, EC), 128, 0, s>>>(in, out, H, W, c0, h0, w0, EH, EW);
  return cudaGetLastError();
}
cudaError_t launch_cast_f16_f32(const __half *in, float *out, uint64_t n, cudaStream_t s) {
  if (!n) return cudaSuccess;
  cast_f16_f32_kernel<<<nblk(n, 256), 256, 0, s>>>(in, out, n);
  return cudaGetLastError();
}
cudaError_t launch_cast_f32_f16(const float *in, __half *out, uint64_t n, cudaStream_t s) {
  if (!n) return cudaSuccess;
  cast_f32_f16_kernel<<<nblk(n, 256), 256, 0, s>>>(in, out, n);
  return cudaGetLastError();
}
cudaError_t launch_bmm_f16(const __half *a, const __half *b, __half *c, uint32_t C, uint32_t M,
                           uint32_t N, uint32_t K, uint64_t a_cs, uint64_t a_hs, uint64_t b_cs,
                           uint64_t b_hs, uint64_t c_cs, uint64_t c_hs, int tb, float scale,
                           float bias, int act, cudaStream_t s) {
  if (!C || !M || !N) return cudaSuccess;
  bmm_f16_kernel<<<dim3(nblk(N, 4), M, C), 128, 0, s>>>(a, b, c, M, N, K, a_cs, a_hs, b_cs, b_hs,
                                                        c_cs, c_hs, tb, scale, bias, act);
  return cudaGetLastError();
}

}  // namespace vkl

// ---------------------------------------------------------------------------
// Arg-max without any allocation.
//
// vkl_argmax_noalloc is for callers that may not allocate device memory at the
// point where they need the greedy pick: a serving loop that handed its whole
// memory budget out at start-up, code running while a stream is being captured, or
// a host runtime that forbids cudaMalloc after initialisation (it synchronises the
// device and can fail late). The two-stage arg-max needs a scratch buffer for the
// per-chunk winners; here that buffer is a fixed array in the library's device
// image instead of an allocation.
//
// The array below is resident on every GPU that loads this library, from load until
// the process exits. It is shared by all calls and keeps whatever the previous call
// left in it; the arg-max overwrites every entry it later reads, so nothing has to be
// cleared between calls. Two calls that overlap on the GPU (different streams, or
// different host threads without ordering) race on it and must be serialised by the
// caller.
// ---------------------------------------------------------------------------
namespace {
constexpr size_t kNoAllocScratchBytes = 64 * 1024;  // 8192 (index, value) pairs
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];
std::mutex g_noalloc_mu;
void *g_noalloc_ptr[64] = {};  // device address of the array, per device ordinal
}  // namespace

extern "C" int vkl_argmax_noalloc(const void *x_fp16, uint32_t rows, uint32_t width, uint32_t *out_idx, void *cuda_stream) {
  using namespace vkl;
  if (!x_fp16 || !out_idx) return fail(VKL_INVALID_ARGUMENT, "argmax_noalloc: null input or output pointer");
  if (rows == 0 || width == 0) return fail(VKL_INVALID_ARGUMENT, "argmax_noalloc: empty input (%u rows of %u)", rows, width);
  const size_t need = argop_partials_bytes(rows, width);
  if (need > kNoAllocScratchBytes)
    return fail(VKL_OUT_OF_RANGE,
                "argmax_noalloc: %u rows of %u values need %zu bytes of scratch, the built-in buffer holds %zu "
                "(rows * ceil(width/1024) must not exceed %zu); use the ArgMax op for larger inputs",
                rows, width, need, kNoAllocScratchBytes, kNoAllocScratchBytes / 8);
  int dev = 0;
  VKL_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(VKL_UNIMPLEMENTED, "argmax_noalloc: device ordinal %d is beyond the 64 this entry point tracks", dev);
  // The scratch address is looked up for the CURRENT device: input and output must live there
  // too, or the kernels would be handed another GPU's address. (A host-side query, no allocation.)
  for (const void *ptr : {x_fp16, (const void *)out_idx}) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, ptr) != cudaSuccess) {
      cudaGetLastError();
      return fail(VKL_INVALID_ARGUMENT, "argmax_noalloc: %p is not a CUDA pointer", ptr);
    }
    if (at.type != cudaMemoryTypeDevice && at.type != cudaMemoryTypeManaged)
      return fail(VKL_INVALID_ARGUMENT, "argmax_noalloc: %p is not device memory", ptr);
    if (at.type == cudaMemoryTypeDevice && at.device != dev)
      return fail(VKL_INVALID_ARGUMENT, "argmax_noalloc: %p lives on device %d but device %d is current; make the buffers' device current on every call", ptr, at.device, dev);
  }
  void *scratch = nullptr;
  {
    // Set-up, once per device, with that device current: the array's name is only a
    // host-side handle, the kernel needs the address the symbol has on this device.
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (!g_noalloc_ptr[dev]) {
      void *p = nullptr;
      VKL_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
      if (!p) return fail(VKL_INTERNAL, "argmax_noalloc: the scratch symbol has no address on device %d", dev);
      g_noalloc_ptr[dev] = p;
    }
    scratch = g_noalloc_ptr[dev];
  }
  VKL_LAUNCH(2, launch_argop(static_cast<const __half *>(x_fp16), out_idx, scratch, rows, width, 0, static_cast<cudaStream_t>(cuda_stream)));
  return VKL_OK;
}

// ---------------------------------------------------------------------------------------
// Device top-k over one row of fp32 logits, for the top-k sampler (models/samplers.cpp:37-64
// sorts all pairs on the host after a 128 KB download). One CTA; pick i is the largest
// (value, then lowest index) element that comes strictly after pick i-1 in that order, so
// nothing has to be marked as taken: k passes over the row, which stays in L2.
// ---------------------------------------------------------------------------------------
namespace vkl {
namespace {
__device__ __forceinline__ bool topk_before(float v, uint32_t i, float w, uint32_t j) {  // (v,i) sorts before (w,j)
  return v > w || (v == w && i < j);
}
__global__ void __launch_bounds__(1024) topk_f32_kernel(const float *__restrict__ x, uint32_t n, uint32_t k, float *vals, uint32_t *ids) {
  __shared__ float sv[32];
  __shared__ uint32_t si[32];
  __shared__ float pv;
  __shared__ uint32_t pi;
  const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float prev_v = INFINITY;
  uint32_t prev_i = 0;
  bool first = true;
  for (uint32_t pick = 0; pick < k; ++pick) {
    float bv = -INFINITY;
    uint32_t bi = 0xffffffffu;
    for (uint32_t i = tid; i < n; i += 1024) {
      const float v = x[i];
      const bool after = first || topk_before(prev_v, prev_i, v, i);
      if (after && (bi == 0xffffffffu || topk_before(v, i, bv, bi))) {
        bv = v;
        bi = i;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi != 0xffffffffu && (bi == 0xffffffffu || topk_before(ov, oi, bv, bi))) {
        bv = ov;
        bi = oi;
      }
    }
    if (lane == 0) {
      sv[warp] = bv;
      si[warp] = bi;
    }
    __syncthreads();
    if (warp == 0) {
      bv = sv[lane];
      bi = si[lane];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi != 0xffffffffu && (bi == 0xffffffffu || topk_before(ov, oi, bv, bi))) {
          bv = ov;
          bi = oi;
        }
      }
      if (lane == 0) {
        pv = bv;
        pi = bi;
        vals[pick] = bv;
        ids[pick] = bi;  // 0xffffffff when the row has fewer than k comparable values
      }
    }
    __syncthreads();
    prev_v = pv;
    prev_i = pi;
    first = false;
    if (prev_i == 0xffffffffu) break;
  }
}
}  // namespace
cudaError_t launch_topk_f32(const float *x, uint32_t n, uint32_t k, float *vals, uint32_t *ids, cudaStream_t s) {
  topk_f32_kernel<<<1, 1024, 0, s>>>(x, n, k, vals, ids);
  return cudaGetLastError();
}
}  // namespace vkl
