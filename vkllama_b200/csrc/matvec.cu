// Weight-streaming mat-vec / skinny mat-mul: Y[M,N] = epilogue(X[M,K] . W[N,K]^T)
// for Q8_0 weights (fused dequantisation) and FP16 weights.
//
// Replaces the reference's four weight shaders
//   src/shaders/matmul_b0_fp16_x_q8_0.comp, kqv_fp16_x_q8_0.comp,
//   ffn_up_and_gate_q8_0.comp, matmul_b0_tb_fp16_v2.comp / ffn_up_and_gate_fp16.comp
// with one HBM-bound kernel: 16-row tiles dealt evenly to a grid that fits the GPU in one
// wave (a CTA takes every gridDim.x-th tile and requests its next tile's first weights
// before it reduces the current one), eight warps splitting K,
// every lane streaming 128-bit weight loads that are already MMA A-fragments
// (see Q8Layout), exact int8->fp16 conversion, m16n8k16 tensor-core products
// with fp32 accumulation, the block scale applied in fp32 per 32-column block
// (as the shaders do: `sums += sum_b * d`), a fixed-order cross-warp reduction
// and the fused epilogue (scale/bias/SiLU, residual add, or SwiGLU).
// The optional prologue fuses RMSNorm of the input row (decode path).
#include <algorithm>

#include "common.cuh"
#include "kernels.h"

namespace vkl {

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
#ifndef VKL_MV_DEPTH
#define VKL_MV_DEPTH 2
#endif
constexpr int kDepth = VKL_MV_DEPTH;  // 4-block groups kept in flight per warp

template <bool Q8, int NW>
struct Stage {
  uint4 c[NW][Q8 ? 4 : 8];
  uint4 s[NW];
};

template <int MT, int EPI, bool XS, bool Q8>
__global__ void __launch_bounds__(kThreads) mv_kernel(const MvParams p) {
  constexpr int NW = (EPI == EPI_SWIGLU) ? 2 : 1;
  extern __shared__ __align__(16) unsigned char smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const uint32_t mat = blockIdx.y, ntiles = (p.N + 15) / 16;
  uint32_t tile = blockIdx.x;
  const uint32_t blocks = (p.K + 31) / 32, groups = (blocks + 3) / 4;
  const uint32_t g0 = (warp * groups) / kWarps, g1 = ((warp + 1) * groups) / kWarps;

  const uint8_t *cb[NW];
  const uint8_t *sb[NW];
  uint32_t row_g = 0;
  auto set_tile = [&](uint32_t tl) {  // where the loads of tile `tl` read
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const uint32_t mi = (EPI == EPI_SWIGLU) ? w : mat;
      if (Q8) {
        cb[w] = p.codes[mi] + (size_t)tl * groups * 2048 + lane * 16;
        sb[w] = p.scales[mi] + (size_t)tl * groups * 128 + g * 16;
      } else {
        cb[w] = p.codes[mi];
        sb[w] = nullptr;
      }
    }
    row_g = tl * 16 + g;
  };
  set_tile(tile);

  auto load = [&](Stage<Q8, NW> &st, uint32_t grp) {
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      if (Q8) {
#pragma unroll
        for (int j = 0; j < 4; ++j) st.c[w][j] = ldg_stream(cb[w] + (size_t)grp * 2048 + j * 512);
        st.s[w] = ldg_stream(sb[w] + (size_t)grp * 128);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t k = (grp * 4 + j) * 32 + t * 8;
          const bool kin = k < p.K;
          st.c[w][2 * j] = (kin && row_g < p.N)
                               ? ldg_stream(cb[w] + ((size_t)row_g * p.K + k) * 2)
                               : make_uint4(0, 0, 0, 0);
          st.c[w][2 * j + 1] = (kin && row_g + 8 < p.N)
                                   ? ldg_stream(cb[w] + ((size_t)(row_g + 8) * p.K + k) * 2)
                                   : make_uint4(0, 0, 0, 0);
        }
      }
    }
  };

  // FP16 weights: 16-byte fragments, twice the registers per stage; one stage in flight per warp
  // and more resident CTAs measured faster than two stages (7B FP16 decode 240 -> 277 tok/s)
  constexpr int KD = !Q8 ? 1 : kDepth;
  Stage<Q8, NW> st[KD];
#pragma unroll
  for (int d = 0; d < KD; ++d)
    if (g0 + d < g1) load(st[d], g0 + d);

  // ---- input rows -------------------------------------------------------
  // XS: rows staged in shared memory (optionally RMS-normalised on the way,
  // rounded to fp16 exactly where the reference's RMSNorm op rounds).
  const uint32_t xs_ld = p.K + 32;  // +64 B keeps 8 token rows on distinct banks
  __half *xs = reinterpret_cast<__half *>(smem);
  float *red = reinterpret_cast<float *>(smem + (XS ? ((size_t)p.M * xs_ld * 2 + 15) / 16 * 16 : 0));
  if (XS) {
    if (p.use_pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float ssum[kWarps];
    for (uint32_t m = 0; m < p.M; ++m) {
      const __half *xr = p.x + (size_t)m * p.x_ld;
      float alpha = 1.f;
      if (p.norm_w) {
        float s = 0.f;
        for (uint32_t i = threadIdx.x; i < p.K; i += kThreads) {
          const float v = __half2float(xr[i]);
          s += v * v;
        }
        s = warp_sum(s);
        if (lane == 0) ssum[warp] = s;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) tot += ssum[w];
        alpha = 1.0f / sqrtf(tot / (float)p.K + p.eps);
        __syncthreads();
      }
      for (uint32_t i = threadIdx.x; i < p.K; i += kThreads) {
        const float v = __half2float(xr[i]);
        xs[(size_t)m * xs_ld + i] = p.norm_w ? __float2half_rn(v * p.norm_w[i] * alpha) : xr[i];
      }
    }
    __syncthreads();
  } else {
    if (p.use_pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
  }
  const bool vec_ok = XS || ((p.x_ld & 7) == 0);

  auto xfrag = [&](uint32_t m, uint32_t k) -> uint4 {
    if (m >= p.M || k >= p.K) return make_uint4(0, 0, 0, 0);
    if (XS) {
      if (k + 8 <= p.K) return *reinterpret_cast<const uint4 *>(xs + (size_t)m * xs_ld + k);
    } else if (vec_ok && k + 8 <= p.K) {
      return __ldg(reinterpret_cast<const uint4 *>(p.x + (size_t)m * p.x_ld + k));
    }
    __half h[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const __half z = __ushort_as_half(0);
      h[i] = (k + i < p.K) ? (XS ? xs[(size_t)m * xs_ld + k + i] : p.x[(size_t)m * p.x_ld + k + i]) : z;
    }
    return *reinterpret_cast<uint4 *>(h);
  };

  for (;; tile += gridDim.x) {  // this CTA's tiles
  float acc[NW][MT][4];
#pragma unroll
  for (int w = 0; w < NW; ++w)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[w][mt][i] = 0.f;

  auto process = [&](const Stage<Q8, NW> &sg, uint32_t grp) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t k = (grp * 4 + j) * 32 + t * 8;
      uint4 X[MT];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) X[mt] = xfrag(mt * 8 + g, k);
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        uint32_t A0[4], A1[4];
        float dg = 1.f, dg8 = 1.f;
        if (Q8) {
          const uint4 cw = sg.c[w][j];
          A0[0] = codes_to_h2(cw.x, false);
          A0[1] = codes_to_h2(cw.z, false);
          A0[2] = codes_to_h2(cw.x, true);
          A0[3] = codes_to_h2(cw.z, true);
          A1[0] = codes_to_h2(cw.y, false);
          A1[1] = codes_to_h2(cw.w, false);
          A1[2] = codes_to_h2(cw.y, true);
          A1[3] = codes_to_h2(cw.w, true);
          const uint32_t sa = (j < 2) ? sg.s[w].x : sg.s[w].y;
          const uint32_t sb8 = (j < 2) ? sg.s[w].z : sg.s[w].w;
          dg = __half2float(__ushort_as_half((unsigned short)((j & 1) ? (sa >> 16) : (sa & 0xffff))));
          dg8 = __half2float(__ushort_as_half((unsigned short)((j & 1) ? (sb8 >> 16) : (sb8 & 0xffff))));
        } else {
          const uint4 r0 = sg.c[w][2 * j], r8 = sg.c[w][2 * j + 1];
          A0[0] = r0.x; A0[1] = r8.x; A0[2] = r0.y; A0[3] = r8.y;
          A1[0] = r0.z; A1[1] = r8.z; A1[2] = r0.w; A1[3] = r8.w;
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          if (Q8) {
            float c[4] = {0.f, 0.f, 0.f, 0.f};
            mma16816(c, A0[0], A0[1], A0[2], A0[3], X[mt].x, X[mt].y);
            mma16816(c, A1[0], A1[1], A1[2], A1[3], X[mt].z, X[mt].w);
            acc[w][mt][0] = fmaf(c[0], dg, acc[w][mt][0]);
            acc[w][mt][1] = fmaf(c[1], dg, acc[w][mt][1]);
            acc[w][mt][2] = fmaf(c[2], dg8, acc[w][mt][2]);
            acc[w][mt][3] = fmaf(c[3], dg8, acc[w][mt][3]);
          } else {
            mma16816(acc[w][mt], A0[0], A0[1], A0[2], A0[3], X[mt].x, X[mt].y);
            mma16816(acc[w][mt], A1[0], A1[1], A1[2], A1[3], X[mt].z, X[mt].w);
          }
        }
      }
    }
  };

  for (uint32_t base = g0; base < g1; base += KD) {
#pragma unroll
    for (int d = 0; d < KD; ++d) {
      const uint32_t grp = base + d;
      if (grp < g1) {
        process(st[d], grp);
        if (grp + KD < g1) load(st[d], grp + KD);
      }
    }
  }
  // the next tile's first groups are requested now: the weight stream keeps going through the reduction below
  const bool more = tile + gridDim.x < ntiles;
  if (more) {
    set_tile(tile + gridDim.x);
#pragma unroll
    for (int d = 0; d < KD; ++d)
      if (g0 + d < g1) load(st[d], g0 + d);
  } else if (p.use_pdl) {
    asm volatile("griddepcontrol.launch_dependents;");
  }

  // ---- fixed-order cross-warp reduction + epilogue ------------------------
#pragma unroll
  for (int w = 0; w < NW; ++w)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i)
        red[(((warp * NW + w) * MT + mt) * 4 + i) * 32 + lane] = acc[w][mt][i];
  __syncthreads();

  for (uint32_t idx = threadIdx.x; idx < 128u * MT; idx += kThreads) {
    const uint32_t r = idx & 15, c = (idx >> 4) & 7, mt = idx >> 7;
    const uint32_t m = mt * 8 + c, n = tile * 16 + r;
    if (m >= p.M || n >= p.N) continue;
    const uint32_t ln = (r & 7) * 4 + (c >> 1), i = (r >> 3) * 2 + (c & 1);
    float v[NW];
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      float s = 0.f;
#pragma unroll
      for (int wp = 0; wp < kWarps; ++wp) s += red[(((wp * NW + w) * MT + mt) * 4 + i) * 32 + ln];
      v[w] = s;
    }
    const size_t o = (size_t)m * p.out_ld + n;
    if (EPI == EPI_SWIGLU) {
      const float gate = v[0], up = v[NW - 1];
      p.out[0][o] = __float2half_rn(gate / (1.0f + expf(-gate)) * up);
    } else if (EPI == EPI_ADD) {
      const float y = round_h(v[0] * p.scale + p.bias);
      p.out[0][o] = __float2half_rn(y + __half2float(p.residual[o]));
    } else {
      float y = v[0] * p.scale + p.bias;
      if (p.act == 1) y = y / (1.0f + expf(-y));
      const __half hy = __float2half_rn(y);
      p.out[mat][o] = hy;
      if (p.out_f32) p.out_f32[o] = __half2float(hy);
    }
  }
  if (!more) break;
  __syncthreads();  // `red` is free for the next tile
  }
}

template <int MT, int EPI, bool XS, bool Q8>
cudaError_t launch_t(const MvParams &p, cudaStream_t s) {
  constexpr int NW = (EPI == EPI_SWIGLU) ? 2 : 1;
  size_t smem = (size_t)kWarps * NW * MT * 4 * 32 * 4;
  if (XS) smem += ((size_t)p.M * (p.K + 32) * 2 + 15) / 16 * 16;
  auto kern = mv_kernel<MT, EPI, XS, Q8>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  // One wave: the CTAs that fit the GPU at once, each with the same number of tiles (or one less).
  static int sms = 0, dev_cached = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev != dev_cached) {
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    dev_cached = dev;
  }
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, smem) != cudaSuccess || per_sm < 1) per_sm = 1;
  const uint32_t ntiles = (p.N + 15) / 16, nmat = EPI == EPI_SWIGLU ? 1u : p.nmat;
  const uint32_t slots = std::max(1u, (uint32_t)(sms * per_sm) / nmat);
  const uint32_t per_cta = (ntiles + slots - 1) / slots;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((ntiles + per_cta - 1) / per_cta, nmat, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.use_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, p);
}

template <int EPI, bool XS, bool Q8>
cudaError_t launch_m(const MvParams &p, cudaStream_t s) {
  if (p.M <= 8) return launch_t<1, EPI, XS, Q8>(p, s);
  if (XS) return cudaErrorInvalidValue;
  if (p.M <= 16) return launch_t<2, EPI, false, Q8>(p, s);
  if (p.M <= 32) return launch_t<4, EPI, false, Q8>(p, s);
  // Wider inputs: passes of 64 rows (the weights are re-streamed per pass).
  for (uint32_t m0 = 0; m0 < p.M; m0 += 64) {
    MvParams q = p;
    q.M = (p.M - m0 < 64) ? p.M - m0 : 64;
    q.x = p.x + (size_t)m0 * p.x_ld;
    for (int i = 0; i < 3; ++i)
      if (p.out[i]) q.out[i] = p.out[i] + (size_t)m0 * p.out_ld;
    if (p.out_f32) q.out_f32 = p.out_f32 + (size_t)m0 * p.out_ld;
    if (p.residual) q.residual = p.residual + (size_t)m0 * p.out_ld;
    cudaError_t e = (q.M <= 8)    ? launch_t<1, EPI, false, Q8>(q, s)
                    : (q.M <= 16) ? launch_t<2, EPI, false, Q8>(q, s)
                    : (q.M <= 32) ? launch_t<4, EPI, false, Q8>(q, s)
                                  : launch_t<8, EPI, false, Q8>(q, s);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

template <bool XS, bool Q8>
cudaError_t launch_e(const MvParams &p, int epi, cudaStream_t s) {
  switch (epi) {
    case EPI_PLAIN: return launch_m<EPI_PLAIN, XS, Q8>(p, s);
    case EPI_ADD: return launch_m<EPI_ADD, XS, Q8>(p, s);
    case EPI_SWIGLU: return launch_m<EPI_SWIGLU, XS, Q8>(p, s);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t launch_matvec(const MvParams &p, int epilogue, bool fuse_norm_smem, cudaStream_t s) {
  if (p.M == 0 || p.N == 0) return cudaSuccess;
  if (p.fp16_weights && (p.K & 7)) return cudaErrorInvalidValue;
  if (fuse_norm_smem)
    return p.fp16_weights ? launch_e<true, false>(p, epilogue, s) : launch_e<true, true>(p, epilogue, s);
  return p.fp16_weights ? launch_e<false, false>(p, epilogue, s) : launch_e<false, true>(p, epilogue, s);
}

}  // namespace vkl
