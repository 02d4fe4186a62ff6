// Dense GEMM for multi-token (prefill) passes on the 5th-generation tensor cores:
// C[M,N] = A[M,K] . W[N,K]^T with fp32 accumulation in tensor memory (TMEM), W in FP16 or Q8_0.
//
// Replaces, for many rows, the reference's matmul_b0_tb_fp16_v2.comp and matmul_b0_fp16_x_q8_0.comp
// (src/ops/mat_mul.cpp:71-103), which re-read the whole weight matrix for every input row.
//
// Q8_0 weights are dequantised on the way into shared memory: sixteen extra warps, in two groups that take
// alternating K steps, fetch the codes and scales of their stage's W tile (tiled planes, common.cuh) with
// ordered asynchronous copies, turn every code into the fp16 value fp16(q * d) and store it where a
// 128-byte-swizzled tensor copy would have put it, so the MMA loop is the same as for FP16 weights.
// q * d has up to 19 significant bits: this path rounds every weight once to fp16 (relative 2^-12), where
// the reference multiplies in fp32; the rows-at-a-time kernel (matvec.cu) keeps the exact form and is used
// below GEMM_Q8_MIN_ROWS rows.
//
// One CTA computes a 128 x BN output tile (BN = 32 ... 256, picked per launch) with these kinds of warps:
//   warp 0    producer: one lane issues TMA tensor copies (cp.async.bulk.tensor.2d, 128-byte
//             swizzle) of the A and W tiles of each 64-wide K block into a ring of shared-
//             memory stages; the copies complete on the stage's "full" mbarrier.
//   warp 1    MMA: allocates the TMEM accumulator (BN columns); one lane waits for a full
//             stage and issues four tcgen05.mma (M128 N{BN} K16, kind::f16) on shared-memory
//             descriptors; tcgen05.commit arrives on the stage's "empty" mbarrier when the
//             tensor core has read the stage, and on "acc_ready" after the last K block.
//   warps 2-5 epilogue: each reads its 32 TMEM lanes (= 32 output rows) with tcgen05.ld,
//             applies the op's rounding (scale, bias, SiLU, residual add) and stores fp16 or
//             raw fp32 rows with 128-bit stores.
// Every mbarrier wait is bounded; on a time-out the kernel raises the error word, lets
// copies in flight land, frees its TMEM and returns.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"

#ifndef VKL_GEMM_TRACE
#define VKL_GEMM_TRACE 0  // diagnostic build: CTA (0,0) stamps the global timer at fixed points of every K step
#endif
#if VKL_GEMM_TRACE
__device__ unsigned long long g_gemm_trace[8 * 512];
extern "C" int vkl_debug_gemm_trace_clear() {
  static unsigned long long zeros[8 * 512];
  return (int)cudaMemcpyToSymbol(g_gemm_trace, zeros, sizeof(zeros));
}
extern "C" int vkl_debug_gemm_trace(unsigned long long *out, size_t n) {
  return (int)cudaMemcpyFromSymbol(out, g_gemm_trace, (n < 8 * 512 ? n : 8 * 512) * sizeof(unsigned long long));
}
#define GEMM_STAMP(kb, k)                                                                       \
  do {                                                                                          \
    if (blockIdx.x == 0 && blockIdx.y == 0 && (kb) < 512) {                                     \
      unsigned long long t_;                                                                    \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                    \
      g_gemm_trace[(kb) * 8 + (k)] = t_;                                                        \
    }                                                                                           \
  } while (0)
#else
#define GEMM_STAMP(kb, k) \
  do {                    \
  } while (0)
#endif

namespace vkl {
namespace {

#ifndef VKL_GEMM_NACC2
#define VKL_GEMM_NACC2 1
#endif
#ifndef VKL_GEMM_TESTWAIT
#define VKL_GEMM_TESTWAIT 0
#endif
#ifndef VKL_GEMM_MMAONLY
#define VKL_GEMM_MMAONLY 0  // diagnostic build: the MMA lane runs alone on whatever the shared memory holds
#endif
constexpr int BM = 128, BK = 64;
constexpr uint32_t A_TILE_BYTES = BM * BK * 2;  // 16 KB
constexpr uint32_t GEMM_WAIT_LIMIT = 1u << 22;
constexpr int GEMM_THREADS = 192;          // FP16 weights: TMA producer, MMA, four epilogue warps
#ifndef VKL_GEMM_NDW
#define VKL_GEMM_NDW 16
#endif
constexpr int NDW = VKL_GEMM_NDW;               // warps dequantising the W tile: one warp issues an instruction every five cycles or so
                                                // (a dependent chain of permutes, multiplies and stores), so it takes several per SM
                                                // sub-partition to keep up with the weight stream
#ifndef VKL_GEMM_NG
#define VKL_GEMM_NG 2
#endif
constexpr int NG = VKL_GEMM_NG;                 // the dequantising warps work in NG groups on alternating K steps: a warp's pass over
                                                // one K step is a serial chain of waits, loads, conversion, stores and a proxy fence
                                                // (about half a microsecond), so several K steps have to be in work at a time
// The MMA lane (warp 1) issues some sixty instructions per K step and the whole CTA waits on it. A warp's scheduler
// is warp % 4: the dequantising warps that would share warp 1's scheduler (every fourth) are left idle, or that
// lane gets an issue slot every twenty-odd cycles and a K step takes 0.58 us instead of 0.3.
__host__ __device__ constexpr int skipped_below(int w) { return w < 9 ? 0 : (w - 9) / 4 + 1; }  // warps 9, 13, 17, ... below warp w
constexpr int NDW_ACTIVE = NDW - skipped_below(6 + NDW);                      // the launched warps 6 .. 5 + NDW, less those
constexpr int NDWG = NDW_ACTIVE / NG;           // warps per group = arrivals per stage
static_assert(NDW_ACTIVE % NG == 0, "whole groups");
constexpr int GEMM_THREADS_Q8 = 192 + 32 * NDW;

// Q8_0 weights: what a dequantising warp keeps in flight from DRAM, in shared memory (asynchronous 16-byte
// copies, waited for in order): Q8_UNITS_AHEAD units of 512 bytes of codes + 128 bytes of scales per warp.
constexpr uint32_t Q8_UNIT_STAGING = 512 + 128, Q8_UNITS_AHEAD = NDW_ACTIVE >= 16 ? 4 : 6;
constexpr uint32_t Q8_STAGING_BYTES = NDW_ACTIVE * Q8_UNITS_AHEAD * Q8_UNIT_STAGING;  // 45 KB

template <int BN, bool Q8 = false> struct Cfg {
  static constexpr uint32_t B_TILE_BYTES = BN * BK * 2;
  static constexpr uint32_t STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
  static constexpr int RING_BYTES = 192 * 1024 - (Q8 ? (int)Q8_STAGING_BYTES : 0);  // up to 192 KB of stages (and staging)
  static constexpr int STAGES = (RING_BYTES / (int)STAGE_BYTES) < 8 ? (RING_BYTES / (int)STAGE_BYTES) : 8;
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + (Q8 ? Q8_STAGING_BYTES : 0) + 1024;
};

__device__ __forceinline__ uint32_t sa(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Bounded wait. `sleep_ns`: pause between polls, for the waits that are long by design (the epilogue warps wait
// for the whole K loop): a warp that spins takes issue slots from the warps that work on the same sub-partition.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint32_t sleep_ns = 0) {
  for (uint32_t i = 0; i < GEMM_WAIT_LIMIT; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
    if (sleep_ns) __nanosleep(sleep_ns);
  }
  return false;
}

// The same with the non-blocking test (mbarrier.test_wait), for the MMA lane: try_wait may suspend the thread.
__device__ __forceinline__ bool mbar_spin_bounded(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < (GEMM_WAIT_LIMIT << 4); ++i) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
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

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t x, uint32_t y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
               "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
               : "memory");
}

template <int COLS> __device__ __forceinline__ void tmem_alloc(uint32_t dst_smem) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"((uint32_t)COLS) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
        "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
        "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// One Q8_0 unit (16 rows x 32 columns, 512 bytes of codes) -> fp16 values q * d in the swizzled W tile.
// Lane (g, t) holds 8 codes of row g and 8 codes of row g + 8 at columns 8 t .. 8 t + 7 (common.cuh). 128-byte
// swizzle of a K-major tile with 128-byte rows: 16-byte chunk c of row r sits at chunk c ^ (r % 8); the two store
// offsets depend on the warp's unit, not on the K step, and are worked out beforehand.
__device__ __forceinline__ void dequant_unit_at(unsigned char *wtile, uint32_t off_a, uint32_t off_b, uint4 w, uint32_t d_lo, uint32_t d_hi) {
  const __half2 dl = __half2half2(__ushort_as_half((unsigned short)d_lo)), dh = __half2half2(__ushort_as_half((unsigned short)d_hi));
  uint32_t a[4], b[4];
  a[0] = codes_to_h2(w.x, false); a[1] = codes_to_h2(w.x, true); a[2] = codes_to_h2(w.y, false); a[3] = codes_to_h2(w.y, true);
  b[0] = codes_to_h2(w.z, false); b[1] = codes_to_h2(w.z, true); b[2] = codes_to_h2(w.w, false); b[3] = codes_to_h2(w.w, true);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __half2 x = __hmul2(*reinterpret_cast<__half2 *>(&a[i]), dl), y = __hmul2(*reinterpret_cast<__half2 *>(&b[i]), dh);
    a[i] = *reinterpret_cast<uint32_t *>(&x);
    b[i] = *reinterpret_cast<uint32_t *>(&y);
  }
  *reinterpret_cast<uint4 *>(wtile + off_a) = make_uint4(a[0], a[1], a[2], a[3]);
  *reinterpret_cast<uint4 *>(wtile + off_b) = make_uint4(b[0], b[1], b[2], b[3]);
}

template <int BN, bool Q8>
__global__ void __launch_bounds__(Q8 ? GEMM_THREADS_Q8 : GEMM_THREADS, 1)
    gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, const GemmParams p) {
  using C = Cfg<BN, Q8>;
  extern __shared__ unsigned char smem_raw[];
  // swizzle atoms are 1024 bytes: align the stage ring
  unsigned char *stages = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full[C::STAGES];   // TMA bytes of the stage have landed
  __shared__ __align__(8) uint64_t empty[C::STAGES];  // the MMAs have read the stage
  __shared__ __align__(8) uint64_t acc_ready;
#if VKL_GEMM_TRACE
  __shared__ __align__(8) uint64_t full_a[C::STAGES];  // diagnostic build, Q8_0: the A tile's copy completes on a barrier of its own
#endif
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile uint32_t failed_s;

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  const uint32_t nkb = p.K / BK;
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(sa(&full[s])), "r"(Q8 ? 1u + NDWG : 1u) : "memory");  // the TMA lane (+ one lane per dequantising warp)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(sa(&empty[s])) : "memory");
#if VKL_GEMM_TRACE
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(sa(&full_a[s])) : "memory");
#endif
    }
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(sa(&acc_ready)) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    failed_s = 0;
  }
  // Tiles of up to 128 columns accumulate the even and the odd 16-wide K slices in two TMEM accumulators, added in
  // the epilogue: a tcgen05.mma of so few columns takes about 110 cycles however narrow it is when it has to
  // follow the one before it on the same accumulator; two independent chains hide half of that.
  constexpr uint32_t NACC = VKL_GEMM_NACC2 && BN <= 128 ? 2 : 1;
  if (warp == 1) tmem_alloc<NACC * BN>(sa(&tmem_base_s));
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_acc = tmem_base_s;

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0 && !VKL_GEMM_MMAONLY) {
      for (uint32_t kb = 0; kb < nkb; ++kb) {
        const uint32_t s = kb % C::STAGES, use = kb / C::STAGES;
        if (use > 0 && !mbar_wait_bounded(sa(&empty[s]), (use - 1) & 1u)) {
          failed_s = 1;
          break;
        }
        if (failed_s) break;
        GEMM_STAMP(kb, 0);  // the stage is free: its A tile is requested now
#if VKL_GEMM_TRACE
        const uint32_t bar = Q8 ? sa(&full_a[s]) : sa(&full[s]);
        if (Q8) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(sa(&full[s])) : "memory");  // the producer's share of the count
#else
        const uint32_t bar = sa(&full[s]);
#endif
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(Q8 ? A_TILE_BYTES : C::STAGE_BYTES) : "memory");
        unsigned char *st = stages + (size_t)s * C::STAGE_BYTES;
        tma_load_2d(sa(st), &map_a, kb * BK, m0, bar);
        if (!Q8) tma_load_2d(sa(st + A_TILE_BYTES), &map_w, kb * BK, n0, bar);
      }
    }
  } else if (Q8 && warp >= 6 && (warp & 3u) != 1u && !VKL_GEMM_MMAONLY) {
    // ------------------------------------------- W tile: Q8_0 -> fp16 in shared memory
    // BN rows x 64 columns = (BN / 16) row tiles x 2 blocks: units of 512 bytes of codes, dealt round robin to
    // the dequantising warps. The scales of a row tile and 4-block group are 8 x 16 bytes: row g's four blocks, then row g + 8's.
    const uint32_t dw = (warp - 6) - (uint32_t)skipped_below((int)warp), g = lane >> 2, t = lane & 3;  // index among the active dequantising warps
    const uint32_t grp = dw % NG, wi = dw / NG;  // this warp's group (its K steps: grp, grp + NG, ...) and place in it
    const uint32_t tiles16 = (p.N + 15) / 16, groups = ((p.K + 31) / 32 + 3) / 4;
    constexpr uint32_t UNITS = (BN / 16) * 2, UPQ = (UNITS + NDWG - 1) / NDWG;  // units per stage, and of those at most this warp's
    constexpr uint32_t PF = Q8_UNITS_AHEAD / UPQ;                              // of its own K steps, how many are requested ahead
    static_assert(UPQ <= Q8_UNITS_AHEAD && PF >= 1, "staging holds at least one stage of a warp's units");
    // The codes of a stage come from DRAM (a microsecond away), so the warp's next PF stages' units are kept in
    // flight. They travel as asynchronous copies into this warp's own staging area, which complete in order
    // (cp.async groups): loads into registers would share the warp's few scoreboards, and the wait for the oldest
    // would also wait for the youngest.
    unsigned char *stg = stages + (size_t)C::STAGES * C::STAGE_BYTES + (size_t)dw * Q8_UNITS_AHEAD * Q8_UNIT_STAGING;
    // What does not change from K step to K step is worked out once per unit of this warp: where its codes and its
    // scales start in the planes (they advance by 1024 bytes per K step and by 128 bytes per two K steps), where
    // its two stores go in the W tile (128-byte swizzle), which half of the block pair it is.
    const unsigned char *cbase[UPQ], *sbase[UPQ];
    uint32_t off_a[UPQ], off_b[UPQ], bl[UPQ];
    bool valid[UPQ];
#pragma unroll
    for (uint32_t j = 0; j < UPQ; ++j) {
      const uint32_t u = wi + NDWG * j, tile = n0 / 16 + (u >> 1);
      bl[j] = u & 1u;
      valid[j] = u < UNITS && tile < tiles16;
      cbase[j] = p.w_codes + (((size_t)tile * groups * 4 + bl[j]) * 32 + lane) * 16;
      sbase[j] = p.w_scales + ((size_t)tile * groups * 8 + g) * 16;
      const uint32_t ra = (u >> 1) * 16 + g, rb = ra + 8, c = bl[j] * 4 + t;
      off_a[j] = ra * 128 + ((c ^ (ra & 7)) << 4);
      off_b[j] = rb * 128 + ((c ^ (rb & 7)) << 4);
    }
    auto request = [&](uint32_t kb, uint32_t slot) {
#pragma unroll
      for (uint32_t j = 0; j < UPQ; ++j) {
        if (valid[j] && kb < nkb) {
          const uint32_t dst = sa(stg + (slot * UPQ + j) * Q8_UNIT_STAGING);
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + lane * 16), "l"(cbase[j] + (size_t)kb * 1024) : "memory");
          if (t == 0)  // the 4-block group's scales of rows g and g + 8: 16 bytes
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 512 + g * 16), "l"(sbase[j] + (size_t)(kb >> 1) * 128) : "memory");
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");  // one group per stage, also when it is empty
    };
#pragma unroll
    for (uint32_t i = 0; i < PF; ++i) request(grp + NG * i, i);
    for (uint32_t kb0 = grp; kb0 < nkb; kb0 += NG * PF) {
      bool stop = false;
#pragma unroll
      for (uint32_t i = 0; i < PF; ++i) {  // staging slots are indexed by compile-time constants
        const uint32_t kb = kb0 + NG * i;
        if (kb >= nkb || stop) continue;
        const uint32_t s = kb % C::STAGES, use = kb / C::STAGES;
        uint32_t ok = 1;
        if (wi == 0 && lane == 0) GEMM_STAMP(kb, 1);  // a dequantising warp turns to the stage
        if (lane == 0 && use > 0) ok = mbar_wait_bounded(sa(&empty[s]), (use - 1) & 1u, 100) ? 1u : 0u;
        ok = __shfl_sync(0xffffffffu, ok, 0);
#if !VKL_GEMM_TRACE
        if (wi == 0 && lane == 0) GEMM_STAMP(kb, 2);  // ... has the stage
#endif
        if (!ok) {
          if (lane == 0) failed_s = 4;
          stop = true;
          continue;
        }
        if (failed_s) {
          stop = true;
          continue;
        }
        asm volatile("cp.async.wait_group %0;" ::"n"(PF - 1) : "memory");  // this stage's copies (the oldest group) have landed
        __syncwarp();
        if (wi == 0 && lane == 0) GEMM_STAMP(kb, 3);  // ... has its codes
        unsigned char *wt = stages + (size_t)s * C::STAGE_BYTES + A_TILE_BYTES;
#pragma unroll
        for (uint32_t j = 0; j < UPQ; ++j) {
          if (wi + NDWG * j >= UNITS) continue;
          uint4 w = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);  // code 0 (stored biased by 128): rows beyond the matrix
          uint32_t lo = 0, hi = 0;
          if (valid[j]) {
            const unsigned char *src = stg + (i * UPQ + j) * Q8_UNIT_STAGING;
            w = *reinterpret_cast<const uint4 *>(src + lane * 16);
            // row g's four block scales, then row g + 8's: this unit's block of the four is ((kb & 1) << 1) | bl
            const unsigned short *d = reinterpret_cast<const unsigned short *>(src + 512 + g * 16) + (((kb & 1u) << 1) | bl[j]);
            lo = d[0];
            hi = d[4];
          }
          dequant_unit_at(wt, off_a[j], off_b[j], w, lo, hi);
        }
        // the tensor core reads shared memory through the async proxy: order this warp's stores before its arrival.
        // (The fence waits for the thread's memory operations in flight: the refill below comes after it.)
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();          // every lane has fenced, and has read the staging slot
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(sa(&full[s])) : "memory");
        if (wi == 0 && lane == 0) GEMM_STAMP(kb, 4);  // ... has written and published its part of the W tile
#if VKL_GEMM_TRACE
        if (lane == 0 && blockIdx.x == 0 && blockIdx.y == 0 && kb < 512) {  // [7]: the last warp of the group to publish
          unsigned long long t_;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));
          atomicMax(&g_gemm_trace[kb * 8 + 7], t_);
        }
#endif
        request(kb + NG * PF, i);   // refill the slot for this warp's stage PF steps ahead
      }
      if (stop) break;
    }
    asm volatile("cp.async.wait_all;" ::: "memory");  // nothing of this warp may still be landing when the CTA exits
  } else if (warp == 1) {
    // --------------------------------------------------------------------- MMA
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc(BM, BN);
      for (uint32_t kb = 0; kb < nkb; ++kb) {
        const uint32_t s = kb % C::STAGES, use = kb / C::STAGES;
        if (!VKL_GEMM_MMAONLY && !(VKL_GEMM_TESTWAIT ? mbar_spin_bounded(sa(&full[s]), use & 1u) : mbar_wait_bounded(sa(&full[s]), use & 1u))) {
          failed_s = 2;
          break;
        }
        if (failed_s) break;
#if VKL_GEMM_TRACE
        GEMM_STAMP(kb, 2);  // (diagnostic build: reuses slot 2) the MMA lane has the W tile
        if (Q8 && !mbar_wait_bounded(sa(&full_a[s]), use & 1u)) {
          failed_s = 2;
          break;
        }
#endif
        GEMM_STAMP(kb, 5);  // the MMA lane has the full stage
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = sa(stages + (size_t)s * C::STAGE_BYTES), b_addr = a_addr + A_TILE_BYTES;
#pragma unroll
        for (uint32_t k = 0; k < BK / 16; ++k) {
          const uint64_t da = smem_desc(a_addr + k * 32), db = smem_desc(b_addr + k * 32);
          const uint32_t accumulate = NACC == 2 ? ((kb | (k >> 1)) ? 1u : 0u) : ((kb | k) ? 1u : 0u);
          asm volatile(
              "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(tmem_acc + (NACC == 2 ? (k & 1u) * BN : 0u)),
              "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
              : "memory");
        }
        // arrives once every MMA issued so far has completed (implies fence::before_thread_sync)
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(sa(&empty[s])) : "memory");
        GEMM_STAMP(kb, 6);  // ... has issued the stage's MMAs and the commit
        if (kb + 1 == nkb)
          asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(sa(&acc_ready)) : "memory");
      }
    }
  } else if (warp >= 2 && warp < 6) {
    // ---------------------------------------------------------------- epilogue
    // a warp may only touch TMEM lanes 32*(warp % 4) .. +31
    const uint32_t quad = warp & 3u;
    const uint32_t row = m0 + quad * 32 + lane;
    uint32_t ok = 1;
    if (lane == 0) ok = mbar_wait_bounded(sa(&acc_ready), 0, 1000) ? 1u : 0u;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (!ok) {
      if (lane == 0) failed_s = 3;
    } else if (!failed_s) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
      for (uint32_t cc = 0; cc < (uint32_t)BN; cc += 32) {
        if (n0 + cc >= p.N) break;  // uniform over the warp
        uint32_t r[32];
        tmem_ld32(tmem_acc + ((quad * 32u) << 16) + cc, r);
        if (NACC == 2) {
          uint32_t r2[32];
          tmem_ld32(tmem_acc + ((quad * 32u) << 16) + BN + cc, r2);
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(r2[j]));
        }
        if (row < p.M) {
          const size_t o = (size_t)row * p.N + n0 + cc;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (n0 + cc + j >= p.N) break;  // N is a multiple of 8
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              v[i] = __uint_as_float(r[j + i]) * p.scale + p.bias;
              if (p.act == 1) v[i] = v[i] / (1.0f + expf(-v[i]));
            }
            if (p.c_f32) {
              *reinterpret_cast<float4 *>(p.c_f32 + o + j) = make_float4(v[0], v[1], v[2], v[3]);
              *reinterpret_cast<float4 *>(p.c_f32 + o + j + 4) = make_float4(v[4], v[5], v[6], v[7]);
            } else {
              union {
                uint4 u;
                __half h[8];
              } out, res;
              if (p.residual) {
                res.u = *reinterpret_cast<const uint4 *>(p.residual + o + j);
#pragma unroll
                for (int i = 0; i < 8; ++i) out.h[i] = __float2half_rn(round_h(v[i]) + __half2float(res.h[i]));
              } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) out.h[i] = __float2half_rn(v[i]);
              }
              *reinterpret_cast<uint4 *>(p.c + o + j) = out.u;
            }
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (failed_s) {
    if (threadIdx.x == 0 && p.error) atomicExch(p.error, failed_s);
    // let tensor copies that are still in flight land before the shared memory is given back
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
    __syncthreads();
  }
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"((uint32_t)(NACC * BN)) : "memory");
}

// y <- fp16( silu(gate) * up ) on fp32 inputs: the epilogue of ffn_up_and_gate_fp16.comp.
__global__ void swiglu_f32_kernel(const float *__restrict__ gate, const float *__restrict__ up, __half *__restrict__ out, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float g = gate[i];
  out[i] = __float2half_rn(g / (1.0f + expf(-g)) * up[i]);
}

using EncodeTiled = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                 const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
  static EncodeTiled fn = [] {
    void *f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) f = nullptr;
    return reinterpret_cast<EncodeTiled>(f);
  }();
  return fn;
}

// Tensor map over a row-major fp16 matrix [rows, K]: boxes of 64 columns x box_rows rows,
// 128-byte swizzle, rows beyond the matrix read as zero.
bool make_map(CUtensorMap *map, const __half *base, uint32_t rows, uint32_t K, uint32_t box_rows) {
  EncodeTiled enc = encode_tiled();
  if (!enc) return false;
  const cuuint64_t dims[2] = {K, rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {BK, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, bool Q8> cudaError_t launch_bn(const GemmParams &p, cudaStream_t s) {
  CUtensorMap ma, mw;
  if (!make_map(&ma, p.a, p.M, p.K, BM)) return cudaErrorInvalidValue;
  if (Q8) {
    mw = ma;  // unused: the W tile is written by the dequantising warps
  } else if (!make_map(&mw, p.w, p.N, p.K, BN)) {
    return cudaErrorInvalidValue;
  }
  cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, Q8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<BN, Q8>::SMEM);
  if (e != cudaSuccess) return e;
  // x = row tile, so that the CTAs sharing one tile of W run together and W crosses HBM once
  gemm_tcgen05_kernel<BN, Q8><<<dim3((p.M + BM - 1) / BM, (p.N + BN - 1) / BN), Q8 ? GEMM_THREADS_Q8 : GEMM_THREADS, Cfg<BN, Q8>::SMEM, s>>>(ma, mw, p);
  return cudaGetLastError();
}

}  // namespace

// SMs of the current device (the tile shape is chosen so that the grid still fills them).
static size_t sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
  return (size_t)n;
}

bool gemm_tcgen05_supported(uint32_t M, uint32_t N, uint32_t K) { return M >= 1 && K % BK == 0 && K >= BK && (N % 8) == 0; }

// W-tile width. A grid runs in waves of one CTA per SM, and a last wave that fills a fraction of the SMs takes
// as long as a full one: pick the width with the smallest waves x (time of one tile). A tile's time is a fixed
// part (the K loop's pipeline latencies, the A tile's copies, the epilogue) plus a part that grows with the
// width; the fixed part dominates, most of all for FP16 weights.
static int forced_bn() {
  static const int forced = [] { const char *e = getenv("VKLLAMA_GEMM_BN"); return e ? atoi(e) : 0; }();  // experiments
  return forced == 256 || forced == 128 || forced == 64 || forced == 32 ? forced : 0;
}
static int pick_bn(const GemmParams &p, bool q8) {
  if (int f = forced_bn()) return (q8 || f >= 128) ? f : 128;
  const size_t mt = (p.M + BM - 1) / BM, sms = sm_count();
  int best = 0;
  double best_cost = 0.0;
  for (int bn : {256, 128, 64, 32}) {
    if (!q8 && bn < 128) break;
    const size_t ctas = mt * ((p.N + bn - 1) / bn), waves = (ctas + sms - 1) / sms;
    // measured time of one wave at K = 4096, us: Q8_0 30.9 / 31.2 / 43.0 / 73.4 for 32 / 64 / 128 / 256 columns, FP16 27 + 0.022 bn
    const double wave = q8 ? (bn == 32 ? 30.9 : bn == 64 ? 31.2 : bn == 128 ? 43.0 : 73.4) : 27.0 + 0.022 * bn;
    const double cost = (double)waves * wave;
    if (!best || cost < best_cost) {
      best = bn;
      best_cost = cost;
    }
  }
  return best;
}

cudaError_t launch_gemm_f16_tcgen05(const GemmParams &p, cudaStream_t s) {
  if (!gemm_tcgen05_supported(p.M, p.N, p.K)) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(p.a) | reinterpret_cast<uintptr_t>(p.w)) & 15) return cudaErrorMisalignedAddress;
  return pick_bn(p, false) == 256 ? launch_bn<256, false>(p, s) : launch_bn<128, false>(p, s);
}

cudaError_t launch_gemm_q8_tcgen05(const GemmParams &p, cudaStream_t s) {
  if (!gemm_tcgen05_supported(p.M, p.N, p.K) || !p.w_codes || !p.w_scales) return cudaErrorInvalidValue;
  if (reinterpret_cast<uintptr_t>(p.a) & 15) return cudaErrorMisalignedAddress;
  switch (pick_bn(p, true)) {
    case 256: return launch_bn<256, true>(p, s);
    case 128: return launch_bn<128, true>(p, s);
    case 64: return launch_bn<64, true>(p, s);
    default: return launch_bn<32, true>(p, s);
  }
}

cudaError_t launch_swiglu_f32(const float *gate, const float *up, __half *out, size_t n, cudaStream_t s) {
  if (!n) return cudaSuccess;
  swiglu_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(gate, up, out, n);
  return cudaGetLastError();
}

}  // namespace vkl
