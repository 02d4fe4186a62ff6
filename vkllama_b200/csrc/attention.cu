// Attention core of the model path: RoPE(q), RoPE(k), KV-cache append, causal
// softmax(q.K^T/sqrt(d)).V over the fp16 cache, split over the KV length with a
// fixed-order combine. One kernel for decode (T = 1); for multi-token calls a
// small rotate-and-append kernel runs first.
//
// Replaces this op chain of the reference (src/ops/multiheadattention_v2.cpp:
// 236-309): Transpose x3, Rope x2 (rope_fp16.comp), UpdateKVCache x2
// (update_kvcache_fp16.comp), MatMul Q.K^T (matmul_b0_tb_fp16_v2.comp), Softmax
// (softmax_fp16.comp), MatMul P.V (matmul_broadcast0_fp16_v2.comp), Transpose.
// Rounding points kept: roped q and k are fp16, the scaled score is rounded to
// fp16 before the softmax, the head output is fp16. The probabilities are kept
// in fp32 here (the reference stores them as fp16 between two dispatches).
#include "common.cuh"
#include "kernels.h"

namespace vkl {
namespace {

constexpr int kAttnThreads = 128;

__device__ __forceinline__ void rope_pair(float x0, float x1, float c, float s, __half &o0,
                                          __half &o1) {
  o0 = __float2half_rn(x0 * c - x1 * s);
  o1 = __float2half_rn(x0 * s + x1 * c);
}

// Multi-token calls: cache[h,(pos+m)%maxlen,:] = rope(k[m,h,:]) and v likewise.
__global__ void rope_append_kernel(const AttnParams p) {
  const uint32_t h = blockIdx.x, m = blockIdx.y, i = threadIdx.x;  // i: pair index
  if (2 * i >= p.dim) return;
  const uint32_t pos = *p.pos_dev + m;
  const size_t fi = (size_t)pos * (p.dim / 2) + i;
  const float c = p.freqc[fi], s = p.freqs[fi];
  const size_t src = (size_t)m * p.heads * p.dim + (size_t)h * p.dim + 2 * i;
  const size_t dst = ((size_t)h * p.maxlen + pos % p.maxlen) * p.dim + 2 * i;
  __half k0, k1;
  rope_pair(__half2float(p.k[src]), __half2float(p.k[src + 1]), c, s, k0, k1);
  p.kcache[dst] = k0;
  p.kcache[dst + 1] = k1;
  p.vcache[dst] = p.v[src];
  p.vcache[dst + 1] = p.v[src + 1];
}

// grid (heads, T, splits), 128 threads. FUSED: T == 1, the CTA whose column
// range holds the new position rotates k, uses it and writes both cache rows.
template <bool FUSED>
__global__ void __launch_bounds__(kAttnThreads) attention_kernel(const AttnParams p) {
  extern __shared__ __align__(16) float sm[];
  const uint32_t h = blockIdx.x, m = p.clip ? p.T - 1 : blockIdx.y, split = blockIdx.z;
  const uint32_t D = p.dim, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float *q_s = sm;                 // [D] roped query, fp16-rounded values
  float *kn_s = sm + D;            // [D] roped new key (FUSED)
  float *red_s = sm + 2 * D;       // [2*D + 8] reduction scratch
  float *s_s = sm + 4 * D + 8;     // [chunk] scores, then probabilities

  if (p.use_pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint32_t pos0 = *p.pos_dev;
  const uint32_t L = min(pos0 + p.T, p.maxlen);
  const uint32_t vis = min(L, m + (L - p.T) + 1);  // causal: col <= row + (W - H)
  uint32_t chunk = (vis + p.splits - 1) / p.splits;
  chunk = (chunk + 31) & ~31u;
  const uint32_t c0 = min(split * chunk, vis), c1 = min(c0 + chunk, vis);
  const uint32_t jn = pos0 % p.maxlen;  // FUSED: physical column of the new token
  const bool owns_new = FUSED && jn >= c0 && jn < c1;

  const size_t row_in = (size_t)m * p.heads * D + (size_t)h * D;
  if (2 * tid < D) {
    const size_t fi = (size_t)(pos0 + (p.clip ? 0u : m)) * (D / 2) + tid;
    const float c = p.freqc[fi], s = p.freqs[fi];
    __half r0, r1;
    rope_pair(__half2float(p.q[row_in + 2 * tid]), __half2float(p.q[row_in + 2 * tid + 1]), c, s, r0, r1);
    q_s[2 * tid] = __half2float(r0);
    q_s[2 * tid + 1] = __half2float(r1);
    if (owns_new) {
      rope_pair(__half2float(p.k[row_in + 2 * tid]), __half2float(p.k[row_in + 2 * tid + 1]), c, s, r0, r1);
      kn_s[2 * tid] = __half2float(r0);
      kn_s[2 * tid + 1] = __half2float(r1);
      const size_t dst = ((size_t)h * p.maxlen + jn) * D + 2 * tid;
      p.kcache[dst] = r0;
      p.kcache[dst + 1] = r1;
      p.vcache[dst] = p.v[row_in + 2 * tid];
      p.vcache[dst + 1] = p.v[row_in + 2 * tid + 1];
    }
  }
  __syncthreads();

  // ---- scores: one column per lane ----------------------------------------
  const float scale = 1.0f / sqrtf((float)D);
  const __half *kc = p.kcache + (size_t)h * p.maxlen * D;
  float lmax = -INFINITY;
  for (uint32_t j = c0 + tid; j < c1; j += kAttnThreads) {
    float acc = 0.f;
    if (owns_new && j == jn) {
      for (uint32_t d = 0; d < D; ++d) acc = fmaf(q_s[d], kn_s[d], acc);
    } else {
      const uint4 *kr = reinterpret_cast<const uint4 *>(kc + (size_t)j * D);
#pragma unroll 4
      for (uint32_t d8 = 0; d8 < D / 8; ++d8) {
        const uint4 kv = __ldg(kr + d8);
        const float4 qa = *reinterpret_cast<const float4 *>(q_s + d8 * 8);
        const float4 qb = *reinterpret_cast<const float4 *>(q_s + d8 * 8 + 4);
        const float2 k0 = __half22float2(*reinterpret_cast<const __half2 *>(&kv.x));
        const float2 k1 = __half22float2(*reinterpret_cast<const __half2 *>(&kv.y));
        const float2 k2 = __half22float2(*reinterpret_cast<const __half2 *>(&kv.z));
        const float2 k3 = __half22float2(*reinterpret_cast<const __half2 *>(&kv.w));
        acc = fmaf(qa.x, k0.x, acc);
        acc = fmaf(qa.y, k0.y, acc);
        acc = fmaf(qa.z, k1.x, acc);
        acc = fmaf(qa.w, k1.y, acc);
        acc = fmaf(qb.x, k2.x, acc);
        acc = fmaf(qb.y, k2.y, acc);
        acc = fmaf(qb.z, k3.x, acc);
        acc = fmaf(qb.w, k3.y, acc);
      }
    }
    const float sc = round_h(acc * scale);
    s_s[j - c0] = sc;
    lmax = fmaxf(lmax, sc);
  }
  lmax = warp_max(lmax);
  if (lane == 0) red_s[warp] = lmax;
  __syncthreads();
  const float mloc = fmaxf(fmaxf(red_s[0], red_s[1]), fmaxf(red_s[2], red_s[3]));
  __syncthreads();
  float lsum = 0.f;
  for (uint32_t j = c0 + tid; j < c1; j += kAttnThreads) {
    const float pj = expf(s_s[j - c0] - mloc);
    s_s[j - c0] = pj;
    lsum += pj;
  }
  lsum = warp_sum(lsum);
  if (lane == 0) red_s[4 + warp] = lsum;
  __syncthreads();
  const float lloc = red_s[4] + red_s[5] + red_s[6] + red_s[7];

  // ---- P.V: thread = (column parity group, dim pair) ----------------------
  const uint32_t npair = D / 2;  // <= 64
  const uint32_t grp = tid / 64, dp = tid % 64;
  float2 acc = make_float2(0.f, 0.f);
  if (dp < npair) {
    const __half *vc = p.vcache + (size_t)h * p.maxlen * D + 2 * dp;
    for (uint32_t j = c0 + grp; j < c1; j += 2) {
      float2 vv;
      if (owns_new && j == jn)
        vv = __half22float2(*reinterpret_cast<const __half2 *>(p.v + row_in + 2 * dp));
      else
        vv = __half22float2(*reinterpret_cast<const __half2 *>(vc + (size_t)j * D));
      const float pj = s_s[j - c0];
      acc.x = fmaf(pj, vv.x, acc.x);
      acc.y = fmaf(pj, vv.y, acc.y);
    }
  }
  __syncthreads();
  if (grp == 1 && dp < npair) {
    red_s[8 + 2 * dp] = acc.x;
    red_s[8 + 2 * dp + 1] = acc.y;
  }
  __syncthreads();
  if (grp == 0 && dp < npair) {
    acc.x += red_s[8 + 2 * dp];
    acc.y += red_s[8 + 2 * dp + 1];
  }
  if (p.use_pdl) asm volatile("griddepcontrol.launch_dependents;");

  __half *orow = p.out + (p.clip ? (size_t)h * D : row_in);
  if (p.splits == 1) {
    if (grp == 0 && dp < npair) {
      orow[2 * dp] = __float2half_rn(acc.x / lloc);
      orow[2 * dp + 1] = __float2half_rn(acc.y / lloc);
    }
    return;
  }
  // ---- split combine: last CTA to arrive sums the partials in split order --
  const size_t unit = (size_t)blockIdx.y * p.heads + h;
  float *part = p.scratch + (unit * p.splits + split) * (D + 2);
  if (grp == 0 && dp < npair) {
    part[2 * dp] = acc.x;
    part[2 * dp + 1] = acc.y;
  }
  if (tid == 0) {
    part[D] = mloc;
    part[D + 1] = lloc;
  }
  __threadfence();
  __syncthreads();
  __shared__ uint32_t s_last;
  if (tid == 0) s_last = atomicAdd(&p.counters[unit], 1u) == p.splits - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const float *base = p.scratch + unit * p.splits * (D + 2);
  float M = -INFINITY;
  for (uint32_t s = 0; s < p.splits; ++s) M = fmaxf(M, __ldcg(base + s * (D + 2) + D));
  float den = 0.f;
  for (uint32_t s = 0; s < p.splits; ++s) {
    const float ms = __ldcg(base + s * (D + 2) + D), ls = __ldcg(base + s * (D + 2) + D + 1);
    if (ls > 0.f) den += ls * expf(ms - M);
  }
  for (uint32_t d = tid; d < D; d += kAttnThreads) {
    float num = 0.f;
    for (uint32_t s = 0; s < p.splits; ++s) {
      const float ms = __ldcg(base + s * (D + 2) + D), ls = __ldcg(base + s * (D + 2) + D + 1);
      if (ls > 0.f) num += __ldcg(base + s * (D + 2) + d) * expf(ms - M);
    }
    orow[d] = __float2half_rn(num / den);
  }
  if (tid == 0) p.counters[unit] = 0;
}

size_t attn_smem(const AttnParams &p) {
  uint32_t chunk = (p.maxlen + p.splits - 1) / p.splits;
  chunk = ((chunk + 31) & ~31u) + 32;
  return (size_t)(4 * p.dim + 8 + chunk) * sizeof(float);
}

}  // namespace

size_t attention_scratch_bytes(uint32_t T, uint32_t heads, uint32_t dim, uint32_t splits) {
  return (size_t)T * heads * splits * (dim + 2) * sizeof(float);
}

cudaError_t launch_attention(const AttnParams &p, cudaStream_t s) {
  if (p.dim > 128 || (p.dim & 7) || p.T == 0) return cudaErrorInvalidValue;
  if (p.T > 1) {
    rope_append_kernel<<<dim3(p.heads, p.T), 64, 0, s>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  const size_t smem = attn_smem(p);
  auto kern = p.T == 1 ? attention_kernel<true> : attention_kernel<false>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.heads, p.clip ? 1 : p.T, p.splits);
  cfg.blockDim = dim3(kAttnThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (p.use_pdl && p.T == 1) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, p);
}

}  // namespace vkl
