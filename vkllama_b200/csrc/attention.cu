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
#include <cstdlib>
#include <cstring>

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
#pragma unroll 16  // the whole row in flight: one memory round trip per column
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
    constexpr uint32_t UN = 8;  // cache rows in flight per thread
    for (uint32_t jb = c0 + grp; jb < c1; jb += 2 * UN) {
      uint32_t raw[UN];
#pragma unroll
      for (uint32_t u = 0; u < UN; ++u) {
        const uint32_t j = jb + 2 * u;
        raw[u] = 0;
        if (j < c1)
          raw[u] = (owns_new && j == jn) ? *reinterpret_cast<const uint32_t *>(p.v + row_in + 2 * dp)
                                         : __ldg(reinterpret_cast<const uint32_t *>(vc + (size_t)j * D));
      }
#pragma unroll
      for (uint32_t u = 0; u < UN; ++u) {
        const uint32_t j = jb + 2 * u;
        if (j < c1) {
          const float2 vv = __half22float2(*reinterpret_cast<const __half2 *>(&raw[u]));
          const float pj = s_s[j - c0];
          acc.x = fmaf(pj, vv.x, acc.x);
          acc.y = fmaf(pj, vv.y, acc.y);
        }
      }
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


// ---- multi-token calls with many rows: 64 query rows of one head per CTA ----------------------
// The per-row kernel above re-reads the head's K and V rows for every query row. This one stages
// a 64-position K/V tile in shared memory once for 64 query rows and runs both products on the
// tensor cores (mma.sync m16n8k16, fp32 accumulate): S = Q.K^T per warp of 16 rows, the scaled
// score rounded to fp16 as the reference's softmax input is, a running (max, sum) per row, the
// probabilities as fp16 MMA operands (the reference stores them as fp16 between two dispatches),
// O += P.V with V fragments transposed by ldmatrix. Columns are physical cache rows 0..L-1 with
// the reference's mask col <= row + (L - T) (softmax_fp16.comp:52-60), so a wrapped ring behaves
// as in the per-row kernel.
__device__ __forceinline__ void mma16816_h(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  const __half2 v = __halves2half2(__float2half_rn(lo), __float2half_rn(hi));
  return *reinterpret_cast<const uint32_t *>(&v);
}

template <int D>
__global__ void __launch_bounds__(128) attention_tile_kernel(const AttnParams p) {
  constexpr int QT = 64, KT = 64, LD = D + 8;  // padded rows: conflict-free fragment loads
  extern __shared__ __align__(16) __half smh[];
  __half *q_s = smh;             // [QT][LD] roped queries
  __half *k_s = q_s + QT * LD;   // [KT][LD]
  __half *v_s = k_s + KT * LD;   // [KT][LD]
  const uint32_t h = blockIdx.x, m0 = blockIdx.y * QT, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const uint32_t T = p.T, pos0 = *p.pos_dev;
  const uint32_t L = min(pos0 + T, p.maxlen), shift = L - T;
  for (uint32_t i = tid; i < QT * (D / 2); i += 128) {  // rotate the query tile at positions pos0 + row
    const uint32_t r = i / (D / 2), pr = i % (D / 2), m = m0 + r;
    __half r0 = __float2half_rn(0.f), r1 = r0;
    if (m < T) {
      const size_t fi = (size_t)(pos0 + m) * (D / 2) + pr, src = (size_t)m * p.heads * D + (size_t)h * D + 2 * pr;
      rope_pair(__half2float(p.q[src]), __half2float(p.q[src + 1]), p.freqc[fi], p.freqs[fi], r0, r1);
    }
    q_s[r * LD + 2 * pr] = r0;
    q_s[r * LD + 2 * pr + 1] = r1;
  }
  const uint32_t r_lo = m0 + warp * 16 + g, r_hi = r_lo + 8;
  const uint32_t vis_lo = r_lo < T ? min(L, r_lo + shift + 1) : 0u, vis_hi = r_hi < T ? min(L, r_hi + shift + 1) : 0u;
  const uint32_t jmax = min(L, min(m0 + QT, T) + shift);  // columns any row of this tile can see
  const float scale = 1.0f / sqrtf((float)D);
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  const __half *kc = p.kcache + (size_t)h * p.maxlen * D, *vc = p.vcache + (size_t)h * p.maxlen * D;
  const __half *qw = q_s + (warp * 16 + g) * LD + 2 * t;
  for (uint32_t j0 = 0; j0 < jmax; j0 += KT) {
    __syncthreads();  // the previous tile is consumed (and, first time, the query tile is written)
    for (uint32_t i = tid; i < KT * (D / 8); i += 128) {
      const uint32_t r = i / (D / 8), c8 = i % (D / 8), j = j0 + r;
      uint4 kv = make_uint4(0, 0, 0, 0), vv = kv;
      if (j < L) {
        kv = __ldg(reinterpret_cast<const uint4 *>(kc + (size_t)j * D) + c8);
        vv = __ldg(reinterpret_cast<const uint4 *>(vc + (size_t)j * D) + c8);
      }
      *reinterpret_cast<uint4 *>(k_s + r * LD + c8 * 8) = kv;
      *reinterpret_cast<uint4 *>(v_s + r * LD + c8 * 8) = vv;
    }
    __syncthreads();
    // ---- S = Q.K^T: 16 rows x 64 columns per warp
    float sc[KT / 8][4];
#pragma unroll
    for (int nt = 0; nt < KT / 8; ++nt) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const uint32_t a0 = *reinterpret_cast<const uint32_t *>(qw + kk * 16), a1 = *reinterpret_cast<const uint32_t *>(qw + 8 * LD + kk * 16);
      const uint32_t a2 = *reinterpret_cast<const uint32_t *>(qw + kk * 16 + 8), a3 = *reinterpret_cast<const uint32_t *>(qw + 8 * LD + kk * 16 + 8);
#pragma unroll
      for (int nt = 0; nt < KT / 8; ++nt) {
        const __half *kr = k_s + (nt * 8 + g) * LD + kk * 16 + 2 * t;
        mma16816_h(sc[nt], a0, a1, a2, a3, *reinterpret_cast<const uint32_t *>(kr), *reinterpret_cast<const uint32_t *>(kr + 8));
      }
    }
    // ---- scaled fp16 scores, mask, running max and sum
    float tmax_lo = -INFINITY, tmax_hi = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < KT / 8; ++nt) {
      const uint32_t c = j0 + nt * 8 + 2 * t;
      sc[nt][0] = c < vis_lo ? round_h(sc[nt][0] * scale) : -INFINITY;
      sc[nt][1] = c + 1 < vis_lo ? round_h(sc[nt][1] * scale) : -INFINITY;
      sc[nt][2] = c < vis_hi ? round_h(sc[nt][2] * scale) : -INFINITY;
      sc[nt][3] = c + 1 < vis_hi ? round_h(sc[nt][3] * scale) : -INFINITY;
      tmax_lo = fmaxf(tmax_lo, fmaxf(sc[nt][0], sc[nt][1]));
      tmax_hi = fmaxf(tmax_hi, fmaxf(sc[nt][2], sc[nt][3]));
    }
    tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 1));
    tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 2));
    tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 1));
    tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 2));
    const float mn_lo = fmaxf(m_lo, tmax_lo), mn_hi = fmaxf(m_hi, tmax_hi);
    const float corr_lo = m_lo == -INFINITY ? 0.f : expf(m_lo - mn_lo), corr_hi = m_hi == -INFINITY ? 0.f : expf(m_hi - mn_hi);
    float rs_lo = 0.f, rs_hi = 0.f;
#pragma unroll
    for (int nt = 0; nt < KT / 8; ++nt) {
      sc[nt][0] = sc[nt][0] == -INFINITY ? 0.f : expf(sc[nt][0] - mn_lo);
      sc[nt][1] = sc[nt][1] == -INFINITY ? 0.f : expf(sc[nt][1] - mn_lo);
      sc[nt][2] = sc[nt][2] == -INFINITY ? 0.f : expf(sc[nt][2] - mn_hi);
      sc[nt][3] = sc[nt][3] == -INFINITY ? 0.f : expf(sc[nt][3] - mn_hi);
      rs_lo += sc[nt][0] + sc[nt][1];
      rs_hi += sc[nt][2] + sc[nt][3];
    }
    rs_lo += __shfl_xor_sync(0xffffffffu, rs_lo, 1);
    rs_lo += __shfl_xor_sync(0xffffffffu, rs_lo, 2);
    rs_hi += __shfl_xor_sync(0xffffffffu, rs_hi, 1);
    rs_hi += __shfl_xor_sync(0xffffffffu, rs_hi, 2);
    l_lo = l_lo * corr_lo + rs_lo;
    l_hi = l_hi * corr_hi + rs_hi;
    m_lo = mn_lo;
    m_hi = mn_hi;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= corr_lo;
      o[i][1] *= corr_lo;
      o[i][2] *= corr_hi;
      o[i][3] *= corr_hi;
    }
    // ---- O += P.V: 16 cache rows per step, V fragments transposed by ldmatrix
#pragma unroll
    for (int j16 = 0; j16 < KT / 16; ++j16) {
      const uint32_t a0 = pack_h2(sc[2 * j16][0], sc[2 * j16][1]), a1 = pack_h2(sc[2 * j16][2], sc[2 * j16][3]);
      const uint32_t a2 = pack_h2(sc[2 * j16 + 1][0], sc[2 * j16 + 1][1]), a3 = pack_h2(sc[2 * j16 + 1][2], sc[2 * j16 + 1][3]);
      // lane l gives the address of row l % 8 of matrix l / 8: matrices (rows +0, cols +0), (rows +8, cols +0), (rows +0, cols +8), (rows +8, cols +8)
      const __half *vrow = v_s + (j16 * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + ((lane >> 4) & 1) * 8;
#pragma unroll
      for (int dt = 0; dt < D / 16; ++dt) {
        uint32_t b0, b1, b2, b3;
        const uint32_t addr = (uint32_t)__cvta_generic_to_shared(vrow + dt * 16);
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(addr));
        mma16816_h(o[2 * dt], a0, a1, a2, a3, b0, b1);
        mma16816_h(o[2 * dt + 1], a0, a1, a2, a3, b2, b3);
      }
    }
  }
  // ---- out[m, h*D + d] = fp16(O / sum)
  const float inv_lo = l_lo > 0.f ? 1.0f / l_lo : 0.f, inv_hi = l_hi > 0.f ? 1.0f / l_hi : 0.f;
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) {
    const uint32_t d = nt * 8 + 2 * t;
    if (r_lo < T) *reinterpret_cast<uint32_t *>(p.out + (size_t)r_lo * p.heads * D + (size_t)h * D + d) = pack_h2(o[nt][0] * inv_lo, o[nt][1] * inv_lo);
    if (r_hi < T) *reinterpret_cast<uint32_t *>(p.out + (size_t)r_hi * p.heads * D + (size_t)h * D + d) = pack_h2(o[nt][2] * inv_hi, o[nt][3] * inv_hi);
  }
}

constexpr uint32_t kTileMinRows = 32;  // below this the per-row kernel is used

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
  static const bool tile_off = [] { const char *e = getenv("VKLLAMA_PREFILL_ATTENTION"); return e && !strcmp(e, "rows"); }();
  if (!tile_off && p.T >= kTileMinRows && !p.clip && (p.dim == 64 || p.dim == 128)) {
    const size_t tsmem = (size_t)3 * 64 * (p.dim + 8) * sizeof(__half);
    auto tk = p.dim == 128 ? attention_tile_kernel<128> : attention_tile_kernel<64>;
    cudaError_t e = cudaFuncSetAttribute(tk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tsmem);
    if (e != cudaSuccess) return e;
    tk<<<dim3(p.heads, (p.T + 63) / 64), 128, tsmem, s>>>(p);
    return cudaGetLastError();
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
