// All-reduce of a [rows, dim] block of fp32 partial sums over the tensor-parallel ranks, for the
// many-token pass that fills the KV caches of a sharded model (the o_proj and down projections are
// split along K, llama2.h:193-196 and 227-230 give each their residual add).
//
// Every rank's GEMM writes its partial sums into its own exchange region; `tp_signal_kernel`, next in
// the stream, publishes that by storing the all-reduce's sequence number into a flag word of every
// rank; `tp_reduce_rows_kernel` waits (bounded) until all ranks' numbers have arrived in this rank's
// flags, then reads the partial sums of all ranks with plain peer loads, adds them in rank order (the
// same order on every rank, so the ranks' residual streams stay bit-identical), rounds as the one-token
// path does and adds the residual. Two regions alternate: a rank rewrites a region only after it has
// seen every rank's signal for the all-reduce in between, which a rank sends after its reads of the
// region are complete.
#include <algorithm>

#include "kernels.h"

namespace vkl {
namespace {

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float round_h(float v) { return __half2float(__float2half_rn(v)); }

__global__ void tp_signal_kernel(TpRowsParams p) {
  if (threadIdx.x < p.tp) {
    __threadfence_system();
    st_release_sys(p.flags[threadIdx.x] + p.rank, p.seq);
  }
}

__global__ void __launch_bounds__(256) tp_reduce_rows_kernel(TpRowsParams p) {
  __shared__ uint32_t failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  if (threadIdx.x < p.tp) {
    // sequence numbers only grow, and a rank may already have signalled its next all-reduce
    const uint32_t *f = p.flags[p.rank] + threadIdx.x;
    bool ok = false;
    for (uint32_t it = 0; it < p.wait_limit; ++it) {
      if ((int32_t)(ld_acquire_sys(f) - p.seq) >= 0) {
        ok = true;
        break;
      }
      if (it > 4096u) __nanosleep(200);
      if ((it & 1023u) == 1023u && *(volatile uint32_t *)p.error != 0u) break;
    }
    if (!ok) {
      failed = 1;
      atomicCAS(p.error, 0u, 16u);
    }
  }
  __syncthreads();
  if (failed) return;
  const size_t n8 = p.n / 8;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (uint32_t r = 0; r < p.tp; ++r) {
      const float4 a = __ldcg(reinterpret_cast<const float4 *>(p.part[r]) + 2 * i);
      const float4 b = __ldcg(reinterpret_cast<const float4 *>(p.part[r]) + 2 * i + 1);
      s[0] += a.x; s[1] += a.y; s[2] += a.z; s[3] += a.w;
      s[4] += b.x; s[5] += b.y; s[6] += b.z; s[7] += b.w;
    }
    union {
      uint4 u;
      __half h[8];
    } x;
    x.u = *(reinterpret_cast<const uint4 *>(p.x) + i);
#pragma unroll
    for (int j = 0; j < 8; ++j) x.h[j] = __float2half_rn(round_h(s[j]) + __half2float(x.h[j]));
    *(reinterpret_cast<uint4 *>(p.x) + i) = x.u;
  }
}

}  // namespace

cudaError_t launch_tp_reduce_rows(const TpRowsParams &p, int sms, cudaStream_t s) {
  if (p.tp < 2 || p.tp > 8 || (p.n % 8) || !p.error) return cudaErrorInvalidValue;
  tp_signal_kernel<<<1, 32, 0, s>>>(p);
  const size_t n8 = p.n / 8;
  const int grid = (int)std::min<size_t>((size_t)sms * 4, (n8 + 255) / 256);
  tp_reduce_rows_kernel<<<grid, 256, 0, s>>>(p);
  return cudaGetLastError();
}

}  // namespace vkl
