// Dense FP16 GEMM for multi-token (prefill) passes on the 5th-generation tensor cores:
// C[M,N] = A[M,K] . W[N,K]^T with fp32 accumulation in tensor memory (TMEM).
//
// Replaces, for FP16 weights and many rows, the reference's matmul_b0_tb_fp16_v2.comp
// (src/ops/mat_mul.cpp:71-82), which re-reads the whole weight matrix for every input row.
//
// One CTA computes a 128 x 128 output tile. Per 64-wide K block the four warps copy the
// A and W tiles into shared memory in the 128-byte-swizzled K-major layout that the
// tensor core's shared-memory descriptors address, one elected thread issues four
// tcgen05.mma (M128 N128 K16, kind::f16) that accumulate into 128 TMEM columns, and
// tcgen05.commit arrives on an mbarrier when the MMAs have consumed the stage, so the copy
// of the next K block overlaps the math (two stages). The epilogue reads the accumulator
// back with tcgen05.ld (each warp its 32 lanes), applies the op's rounding and writes fp16
// (optionally after a residual add) or raw fp32. Every mbarrier wait is bounded; on a
// time-out the kernel raises the error word, still frees its TMEM and returns.
#include "common.cuh"
#include "kernels.h"

namespace vkl {
namespace {

constexpr int BM = 128, BN = 128, BK = 64;
constexpr int STAGES = 2;
constexpr uint32_t TILE_BYTES = BM * BK * 2;  // 16 KB per operand tile
constexpr uint32_t GEMM_WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t sa(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < GEMM_WAIT_LIMIT; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);  // start address, 16-byte units
  d |= (uint64_t)1 << 16;                   // leading-dimension offset (unused with swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;         // stride between 8-row groups
  d |= (uint64_t)1 << 46;                   // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                   // 128-byte swizzle
  return d;
}

// kind::f16 instruction descriptor: fp16 x fp16 -> fp32, both operands K-major, M x N tile.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t m, uint32_t n) {
  return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// Copies rows [row0, row0+128) x columns [k0, k0+64) of a row-major fp16 matrix (ld = K) into
// the swizzled tile: 16-byte chunk c of row r lands at r*128 + ((c ^ (r & 7)) * 16).
__device__ __forceinline__ void load_tile(unsigned char *tile, const __half *src, uint32_t rows, uint32_t row0, uint32_t K,
                                          uint32_t k0) {
  for (uint32_t i = threadIdx.x; i < BM * 8; i += blockDim.x) {
    const uint32_t r = i >> 3, c = i & 7;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row0 + r < rows) v = __ldg(reinterpret_cast<const uint4 *>(src + (size_t)(row0 + r) * K + k0) + c);
    *reinterpret_cast<uint4 *>(tile + r * 128 + ((c ^ (r & 7)) << 4)) = v;
  }
}

__global__ void __launch_bounds__(128, 1) gemm_f16_tcgen05_kernel(const GemmParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // 1024-byte alignment for the swizzle atoms
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char *a_tiles = smem;                         // [STAGES][16 KB]
  unsigned char *b_tiles = smem + STAGES * TILE_BYTES;   // [STAGES][16 KB]
  __shared__ __align__(8) uint64_t stage_free[STAGES];   // arrives when the MMAs have read the stage
  __shared__ __align__(8) uint64_t acc_ready;
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t failed_s;

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(sa(&stage_free[s])) : "memory");
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(sa(&acc_ready)) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    failed_s = 0;
  }
  if (warp == 0) {  // one warp allocates 128 TMEM columns (the fp32 accumulator of the tile)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sa(&tmem_base_s)), "r"(128u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_acc = tmem_base_s;

  const uint32_t nkb = p.K / BK;
  constexpr uint32_t idesc = instr_desc(BM, BN);
  for (uint32_t kb = 0; kb < nkb; ++kb) {
    const uint32_t s = kb % STAGES;
    if (kb >= STAGES) {  // the MMAs of k-block kb-STAGES must have finished reading this stage
      if (!failed_s && !mbar_wait_bounded(sa(&stage_free[s]), ((kb / STAGES) - 1) & 1u)) failed_s = 1;
    }
    load_tile(a_tiles + s * TILE_BYTES, p.a, p.M, m0, p.K, kb * BK);
    load_tile(b_tiles + s * TILE_BYTES, p.w, p.N, n0, p.K, kb * BK);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> tensor-core reads
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0 && !failed_s) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t a_addr = sa(a_tiles + s * TILE_BYTES), b_addr = sa(b_tiles + s * TILE_BYTES);
#pragma unroll
      for (uint32_t k = 0; k < BK / 16; ++k) {
        const uint64_t da = smem_desc(a_addr + k * 32), db = smem_desc(b_addr + k * 32);
        const uint32_t accumulate = (kb | k) ? 1u : 0u;
        asm volatile(
            "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(tmem_acc),
            "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
            : "memory");
      }
      // arrives on the barrier once every MMA issued so far has completed
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(sa(&stage_free[s])) : "memory");
      if (kb + 1 == nkb)
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(sa(&acc_ready)) : "memory");
    }
  }
  __syncthreads();
  if (!failed_s && nkb > 0 && !mbar_wait_bounded(sa(&acc_ready), 0)) failed_s = 1;
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

  if (!failed_s) {
    // ---- epilogue: warp w owns TMEM lanes 32w..32w+31 = output rows m0 + 32w + lane
    const uint32_t row = m0 + warp * 32 + lane;
#pragma unroll 1
    for (uint32_t cc = 0; cc < BN; cc += 32) {
      uint32_t r[32];
      const uint32_t taddr = tmem_acc + ((warp * 32u) << 16) + cc;
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
          "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
          : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
            "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
            "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
            "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
          : "r"(taddr)
          : "memory");
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (row < p.M) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const uint32_t n = n0 + cc + j;
          if (n >= p.N) break;
          float v = __uint_as_float(r[j]) * p.scale + p.bias;
          if (p.act == 1) v = v / (1.0f + expf(-v));
          const size_t o = (size_t)row * p.N + n;
          if (p.c_f32) {
            p.c_f32[o] = v;
          } else if (p.residual) {
            p.c[o] = __float2half_rn(round_h(v) + __half2float(p.residual[o]));
          } else {
            p.c[o] = __float2half_rn(v);
          }
        }
      }
    }
  } else if (threadIdx.x == 0 && p.error) {
    atomicExch(p.error, 1u);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(128u) : "memory");
}

// y <- fp16( silu(gate) * up ) on fp32 inputs: the epilogue of ffn_up_and_gate_fp16.comp.
__global__ void swiglu_f32_kernel(const float *__restrict__ gate, const float *__restrict__ up, __half *__restrict__ out, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float g = gate[i];
  out[i] = __float2half_rn(g / (1.0f + expf(-g)) * up[i]);
}

}  // namespace

bool gemm_tcgen05_supported(uint32_t M, uint32_t N, uint32_t K) { return M >= 1 && K % BK == 0 && K >= BK && (N % 8) == 0; }

cudaError_t launch_gemm_f16_tcgen05(const GemmParams &p, cudaStream_t s) {
  if (!gemm_tcgen05_supported(p.M, p.N, p.K)) return cudaErrorInvalidValue;
  const size_t smem = 2 * STAGES * TILE_BYTES + 1024;
  cudaError_t e = cudaFuncSetAttribute(gemm_f16_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  gemm_f16_tcgen05_kernel<<<dim3((p.N + BN - 1) / BN, (p.M + BM - 1) / BM), 128, smem, s>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_swiglu_f32(const float *gate, const float *up, __half *out, size_t n, cudaStream_t s) {
  if (!n) return cudaSuccess;
  swiglu_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(gate, up, out, n);
  return cudaGetLastError();
}

}  // namespace vkl
