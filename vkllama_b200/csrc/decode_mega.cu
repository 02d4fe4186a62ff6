// One persistent kernel per decode token (Q8_0 weights, batch 1).
//
// The reference records 19 Vulkan dispatches per layer per token
// (models/llama2.h:160-213, src/ops/multiheadattention_v2.cpp:190-319) and stalls
// the weight stream at every one of them. Here the whole token is one
// cooperative launch of one CTA per SM:
//
//   * a producer warp walks the static schedule of this CTA's weight tiles for
//     ALL mat-vec ops of the token and streams them with bulk-copy TMA
//     (cp.async.bulk + mbarrier) into a shared-memory ring, one copy per stage: what a
//     CTA reads of an op is one consecutive range of the op's packed stream. Weights never
//     depend on activations, so the producer runs ahead across op boundaries and HBM
//     stays busy while the consumers sit in a norm, an attention op or a wait;
//   * eleven consumer warps take their units (one Q8_0 block x 32 rows) of every ring
//     stage, put the codes into the tensor cores as fp16 subnormals (exact, one byte permute
//     per pair), multiply (m16n8k16, fp32 accumulate), apply block scales in fp32, reduce
//     across warps in fixed order and run the fused epilogue (RMSNorm prologue, residual add,
//     SwiGLU, fp32 logits, running arg-max). What they cost is instruction issue, not the
//     tensor pipe (12 % busy; mma.sync m16n8k16 (f16) and m16n8k32 (s8) both issue every 8
//     cycles per scheduler on this GPU). A warp's scheduler is warp % 4: eleven or fifteen
//     consumer warps (+ the producer) load the four schedulers evenly, every other count is
//     15-25 % slower; eleven (24 KB stages, seven of them, 168 registers) measured 1.5 %
//     faster than fifteen (32 KB stages, five, 128 registers). An int8 variant on three exact
//     byte slices of the input was 30 % slower for its integer-to-float conversions;
//   * activations cross CTAs as tagged words (value + sequence tag in one 32-bit word) that
//     the readers poll; only the output layer's arg-max needs a grid barrier.
//
// Tiles of op i go to CTA (tile + rot_i) mod grid; rot_i advances by the op's
// tile count so the uneven remainder rotates over the SMs.
// Every wait is bounded; on a time-out the kernel raises *error, stops issuing
// copies, drains the copies in flight and leaves through the normal path.
#include <cooperative_groups.h>

#include <algorithm>

#include "common.cuh"
#include "kernels.h"

namespace vkl {
namespace {

constexpr int NCW = (int)MEGA_NCW;     // consumer warps (11 + 1 producer warp = 384 threads of 168 registers)
constexpr int CT = NCW * 32;           // consumer threads
constexpr int THREADS = CT + 32;       // + producer warp
constexpr int UPW = (int)MEGA_UPW;     // units (one Q8_0 block x 32 rows) per consumer warp and ring stage
constexpr int SU = NCW * UPW;          // units per ring stage
static_assert(SU == (int)MEGA_SU, "host and device agree on the stage size");
constexpr uint32_t UNIT_CODES = MEGA_UNIT_CODES, UNIT_SCALES = MEGA_UNIT_SCALES;
constexpr uint32_t UNIT_BYTES = UNIT_CODES + UNIT_SCALES;  // a unit's codes, then its 32 scales
constexpr uint32_t STAGE_BYTES = SU * UNIT_BYTES;          // 32640
static_assert(STAGE_BYTES == MEGA_STAGE_BYTES, "host and device agree on the stage size");
constexpr uint32_t XB_BYTES = 64;      // the input vector in shared memory: fp16, 64 bytes per block of 32 inputs
constexpr int MAX_NST = 12;            // ring stages are a launch parameter (whatever fits), at most this many
// Every wait of the kernel is bounded by MegaParams::wait_limit polls (about half a microsecond each): the host
// picks the bound, the same for all waits, so that no wait gives up while another one it depends on is still
// legitimately waiting (for a slower tensor-parallel rank, say).

__device__ __forceinline__ uint32_t s32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t a, uint32_t n) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a), "r"(n) : "memory");
}
__device__ __forceinline__ void mbar_expect(uint32_t a, uint32_t tx) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(a), "r"(tx) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t a) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(a) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try(uint32_t a, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(a), "r"(parity)
      : "memory");
  return ok;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t mbar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(__cvta_generic_to_global(src)), "r"(bytes), "r"(mbar)
               : "memory");
}
__device__ __forceinline__ void cons_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CT) : "memory"); }
__device__ __forceinline__ uint32_t ld_acq_sys_u32(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_rel_sys_u32(uint32_t *p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// ---- tagged activation words: fp16 value | (low 16 bits of the producing op's sequence number) << 16
__device__ __forceinline__ uint32_t ll_pack(__half v, uint32_t tag) { return (uint32_t)__half_as_ushort(v) | (tag << 16); }
__device__ __forceinline__ __half ll_half(uint32_t w) { return __ushort_as_half((unsigned short)(w & 0xffffu)); }
__device__ __forceinline__ uint32_t ld_vol_u32(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint2 ld_vol_v2(const uint32_t *p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_vol_v4(const uint32_t *p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// Read-only 128-bit load that keeps its place among the volatile polls around it (a plain
// __ldg may be scheduled after them, behind a spin).
__device__ __forceinline__ float4 ldg_f4_ordered(const float4 *p) {
  float4 v;
  asm volatile("ld.global.nc.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ uint64_t ld_acq_u64(const unsigned long long *p) {
  uint64_t v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ bool getenv_prologue(const MegaParams &p) { return (p.timing_mode & 1u) != 0; }
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Trace mode (timing_mode bit 256, TIMED instances): thread 0 of EVERY CTA stamps the global
// timer at fixed points of every op: [0] op entered, [1] input vector complete (after the
// norm), [2] this warp's stream done, [3] all warps' streams done, [4] results stored,
// [5] end-of-op synchronisation passed. Layout: trace[(op * grid + cta) * 8 + k].
#define VKL_TRACE(k)                                                   \
  do {                                                                 \
    if (TIMED && trace) trace[k] = gtime();                            \
  } while (0)

// The spin loops of the bounded waits. They are inlined like everything else in this kernel: kept out
// of line (to make the code smaller) they cost 10 % of the token time, the calls forcing the polled
// words through local memory and registers to be saved around every wait.
struct Ctx;
#define VKL_SLOW __forceinline__
__device__ VKL_SLOW bool slow_mbar_wait(volatile uint32_t *abort_s, uint32_t *error, uint32_t limit, uint32_t bar, uint32_t parity, uint32_t code, uint32_t sleep_ns) {
#pragma unroll 1
  for (uint32_t i = 0; i < limit; ++i) {
    if (sleep_ns) __nanosleep(sleep_ns);  // keep a waiting warp off the shared-memory pipe the working warps need
    if (mbar_try(bar, parity)) return true;
    if ((i & 255u) == 255u && (*(volatile uint32_t *)error != 0u || *abort_s != 0)) {
      *abort_s = 1;
      return false;
    }
  }
  *abort_s = 1;
  atomicCAS(error, 0u, code);
  return false;
}
__device__ VKL_SLOW uint32_t slow_ll_wait1(volatile uint32_t *abort_s, uint32_t *error, uint32_t limit, const uint32_t *src, uint32_t tag) {
  uint32_t w = 0;
#pragma unroll 1
  for (uint32_t i = 0; i < limit; ++i) {
    w = ld_vol_u32(src);
    if ((w >> 16) == tag) return w;
    if ((i & 255u) == 255u && (*(volatile uint32_t *)error != 0u || *abort_s != 0)) {
      *abort_s = 1;
      return w;
    }
  }
  *abort_s = 1;
  atomicCAS(error, 0u, 6u);
  return w;
}
__device__ VKL_SLOW uint2 slow_ll_wait2(volatile uint32_t *abort_s, uint32_t *error, uint32_t limit, const uint32_t *src, uint32_t tag) {
  uint2 w = make_uint2(0, 0);
#pragma unroll 1
  for (uint32_t i = 0; i < limit; ++i) {
    w = ld_vol_v2(src);
    if (((w.x >> 16) == tag) & ((w.y >> 16) == tag)) return w;
    if ((i & 255u) == 255u && (*(volatile uint32_t *)error != 0u || *abort_s != 0)) {
      *abort_s = 1;
      return w;
    }
  }
  *abort_s = 1;
  atomicCAS(error, 0u, 6u);
  return w;
}
__device__ __forceinline__ bool ll_ready8(const uint4 &a, const uint4 &b, uint32_t tag) {
  return ((a.x >> 16) == tag) & ((a.y >> 16) == tag) & ((a.z >> 16) == tag) & ((a.w >> 16) == tag) & ((b.x >> 16) == tag) &
         ((b.y >> 16) == tag) & ((b.z >> 16) == tag) & ((b.w >> 16) == tag);
}
// polls eight consecutive tagged words until all carry `tag`; the words come back through a, b
__device__ VKL_SLOW void slow_ll_wait8(volatile uint32_t *abort_s, uint32_t *error, uint32_t limit, const uint32_t *src, uint32_t tag, uint4 &a, uint4 &b) {
#pragma unroll 1
  for (uint32_t i = 0; i < limit; ++i) {
    a = ld_vol_v4(src);
    b = ld_vol_v4(src + 4);
    if (ll_ready8(a, b, tag)) return;
    if ((i & 255u) == 255u && (*(volatile uint32_t *)error != 0u || *abort_s != 0)) {
      *abort_s = 1;  // give up quietly: another wait has already raised the error
      return;
    }
  }
  *abort_s = 1;
  atomicCAS(error, 0u, 6u);
}

struct Ctx {
  const MegaParams &p;
  volatile uint32_t *abort_s;  // shared flag: some wait of this CTA timed out or *error was seen
  __device__ __forceinline__ bool aborted() const { return *abort_s != 0; }
  // Under tensor parallelism an input may sit behind an all-reduce that is itself waiting for a slow
  // rank: the input's wait must outlast that one (four times its polls), so that the error names the wait that really failed.
  __device__ __forceinline__ uint32_t ll_limit() const { return p.tp_size > 1 ? (p.wait_limit < 0x40000000u ? 4u * p.wait_limit : 0xffffffffu) : p.wait_limit; }
  __device__ __forceinline__ void raise(uint32_t code) const {
    *abort_s = 1;
    atomicCAS(p.error, 0u, code);
  }
  // Bounded mbarrier wait; false (and the abort flag set) on time-out.
  __device__ __forceinline__ bool wait(uint32_t bar, uint32_t parity, uint32_t code, uint32_t sleep_ns = 0) const {
    if (mbar_try(bar, parity)) return true;  // fast path: the phase is already complete
    if (aborted()) return false;
    return slow_mbar_wait(abort_s, p.error, p.wait_limit, bar, parity, code, sleep_ns);
  }
  // One tagged word, polled (bounded) until its tag is `tag`. Returns the word; on a time-out
  // or an abort returns what it last read (the caller's results are discarded on abort).
  __device__ __forceinline__ uint32_t ll_wait1(const uint32_t *src, uint32_t tag) const {
    const uint32_t w = ld_vol_u32(src);
    if ((w >> 16) == tag) return w;
    return slow_ll_wait1(abort_s, p.error, ll_limit(), src, tag);
  }
  // Two consecutive tagged words (8-byte aligned), already requested once.
  __device__ __forceinline__ uint2 ll_wait2(const uint32_t *src, uint2 w, uint32_t tag) const {
    if (((w.x >> 16) == tag) & ((w.y >> 16) == tag)) return w;
    return slow_ll_wait2(abort_s, p.error, ll_limit(), src, tag);
  }
  // Eight consecutive tagged words (32-byte aligned) -> eight packed halves, polled the same way.
  __device__ __forceinline__ uint4 ll_wait8(const uint32_t *src, uint4 a, uint4 b, uint32_t tag) const {
    if (!ll_ready8(a, b, tag)) slow_ll_wait8(abort_s, p.error, ll_limit(), src, tag, a, b);
    return make_uint4((a.x & 0xffffu) | (a.y << 16), (a.z & 0xffffu) | (a.w << 16), (b.x & 0xffffu) | (b.y << 16), (b.z & 0xffffu) | (b.w << 16));
  }
};

// ------------------------------------------------------------------ producer
// The producer warp walks this CTA's precomputed stage table (one entry per ring
// stage of the whole token, in consumer order). Lane 0 keeps the shared-memory ring
// full with bulk copies; the other lanes only fetch table chunks.
__device__ __forceinline__ void producer(const Ctx &c, unsigned char *ring, uint64_t *full, uint64_t *empty,
                                         MegaStage *tabs /* [128] in shared memory */) {
  const MegaParams &p = c.p;
  const uint32_t lane = threadIdx.x & 31;
  const MegaStage *table = p.stages + (size_t)blockIdx.x * p.stage_stride;
  const uint32_t n = p.stage_count[blockIdx.x];
  const uint32_t NST = p.nst;
  if (lane < min(n, 32u)) tabs[lane] = table[lane];
  __syncwarp();
  uint32_t it = 0, slot = 0, ph = 0;
  uint32_t issued = 0;  // ring stages issued so far (table entries and stages differ: a KV entry is 0..n stages)
  bool stop = false;
  // this CTA's (head, split) and row range of the attention ops: the same for every layer of the token
  const uint32_t pos0 = p.state[0];
  const uint32_t Lnow = min(pos0 + 1, p.maxlen);
  const uint32_t S_eff = mega_splits(Lnow, p.splits, p.split_rows);
  uint32_t kv_c0 = 0, kv_c1 = 0;
  if (blockIdx.x < p.heads * S_eff) mega_kv_range(Lnow, S_eff, blockIdx.x % S_eff, kv_c0, kv_c1);
  const uint32_t kv_head = blockIdx.x / S_eff, kv_rps = mega_kv_rows_per_stage(p.head_dim);
  for (uint32_t base = 0; base < n && !stop; base += 32) {
    // chunk base/32 is in tabs[(base/32 % 4)*32 ..]; fetch the next one behind it. The table is a
    // ring of four chunks because the consumers, up to a ring depth of stages behind, still read
    // their stages' entries.
    if (base + 32 + lane < n) tabs[((base / 32 + 1) & 3) * 32 + lane] = table[base + 32 + lane];
    __syncwarp();
    if (lane == 0) {
      const uint32_t end = min(base + 32, n);
      for (; it < end; ++it) {
        const MegaStage &e = tabs[it & 127];
        if (e.n0 == MEGA_KV_MARK) {
          // K rows, then V rows, of this CTA's split of an attention op: whole cache rows,
          // contiguous in [heads, maxlen, head_dim], up to kv_rps rows per stage
          const uint32_t rowb = p.head_dim * 2u;
          for (uint32_t kv = 0; kv < 2 && !stop; ++kv) {
            const uint8_t *src = (kv ? e.src2 : e.src) + ((size_t)kv_head * p.maxlen + kv_c0) * rowb;
            for (uint32_t r0 = kv_c0; r0 < kv_c1; r0 += kv_rps) {
              if (issued >= NST && !(p.timing_mode & 128u) && !c.wait(s32(&empty[slot]), ph ^ 1u, 2, 0)) {
                stop = true;
                break;
              }
              const uint32_t fb = s32(&full[slot]), bytes = min(kv_rps, kv_c1 - r0) * rowb;
              if (p.timing_mode & 2u) {
                mbar_arrive(fb);
              } else {
                mbar_expect(fb, bytes);
                bulk_g2s(s32(ring + (size_t)slot * STAGE_BYTES), src + (size_t)(r0 - kv_c0) * rowb, bytes, fb);
              }
              ++issued;
              if (++slot == NST) {
                slot = 0;
                ph ^= 1u;
              }
            }
          }
          if (stop) break;
          continue;
        }
        if (issued >= NST && !(p.timing_mode & 128u) && !c.wait(s32(&empty[slot]), ph ^ 1u, 2, 0)) {
          stop = true;
          break;
        }
        const uint32_t fb = s32(&full[slot]);
        ++issued;
        if (p.timing_mode & 2u) {  // diagnostic: consumer speed without the weight stream
          mbar_arrive(fb);
        } else {
          // a CTA's units of an op are consecutive in memory, across its tiles: one copy per stage
          const uint32_t bytes = (e.n0 + e.n1) * UNIT_BYTES;
          mbar_expect(fb, bytes);
          bulk_g2s(s32(ring + (size_t)slot * STAGE_BYTES), e.src, bytes, fb);
        }
        if (++slot == NST) {
          slot = 0;
          ph ^= 1u;
        }
      }
    }
    stop = __shfl_sync(0xffffffffu, stop ? 1 : 0, 0) != 0;
  }
  // Nothing may still be landing in this CTA's shared memory when it exits.
  if (lane == 0) {
    const uint32_t lo = issued > NST ? issued - NST : 0;
    for (uint32_t j = lo; j < issued; ++j) {
      const uint32_t fb = s32(&full[j % NST]), ph2 = (j / NST) & 1u;
    #pragma unroll 1
      // (not the caller's bound, which a test may have made very short: a copy in flight lands within microseconds)
      for (uint32_t i = 0; i < max(p.wait_limit, 1u << 20) && !mbar_try(fb, ph2); ++i) {
      }
    }
  }
}

// ------------------------------------------------------------ grid barrier
__device__ VKL_SLOW bool grid_barrier(const Ctx &c, uint64_t target, uint32_t round, volatile uint32_t *seen_s) {
  cons_sync();  // every consumer store of this op is issued
  // Lane 0 of the first POLLERS warps poll the counter, each a fraction of a memory round trip
  // after the previous one, so that the last arrival is seen a fraction of a round trip after it
  // lands instead of half a round trip on average. `seen_s` holds the last round (1, 2, ... within
  // this launch) that one of them has seen complete.
  const uint32_t POLLERS = c.p.barrier_pollers;
  const uint32_t w = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0 && w < POLLERS && !c.aborted()) {
    if (w == 0) {
      // release-add without a return value: orders this CTA's stores (made visible to
      // thread 0 by the bar.sync above) before the arrival, one L2 trip instead of two
      asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(c.p.bar), "l"(1ull) : "memory");
    } else {
      __nanosleep(160 * w);
    }
    const uint32_t tgt = round;
    bool ok = false;
  #pragma unroll 1
    // (under tensor parallelism a CTA without a tile of the projections runs ahead to this barrier while others
    // wait for another rank's partial sums: the barrier's wait outlasts theirs, so that the error names theirs)
    const uint32_t limit = c.p.tp_size > 1 ? (c.p.wait_limit < 0x10000000u ? 16u * c.p.wait_limit : 0xffffffffu) : c.p.wait_limit;
    for (uint32_t i = 0; i < limit; ++i) {
      if (*seen_s == tgt || ld_acq_u64(c.p.bar) >= target) {
        ok = true;
        break;
      }
      if (i > 100000u) __nanosleep(64);
      if ((i & 1023u) == 1023u && *(volatile uint32_t *)c.p.error != 0u) break;
    }
    if (ok)
      *seen_s = tgt;
    else
      c.raise(3);
    __threadfence();
  }
  cons_sync();
  return !c.aborted();
}

__device__ __forceinline__ float ldcg_h(const __half *p) {
  return __half2float(__ushort_as_half(__ldcg(reinterpret_cast<const unsigned short *>(p))));
}

// ------------------------------------------------------------------ mat-vec
struct Best {
  float v;
  uint32_t i;
};
__device__ __forceinline__ bool better(float v, uint32_t i, const Best &b) {
  return b.i == 0xffffffffu || v > b.v || (v == b.v && i < b.i);
}

// Two stored codes (bytes 0 and 2, or 1 and 3, of a plane word) as a pair of fp16 subnormals u * 2^-24.
__device__ __forceinline__ uint32_t codes_sub_h2(uint32_t w, bool hi) { return __byte_perm(w, 0u, hi ? 0x4341u : 0x4240u); }

// One mat-vec op of the token: y = W . x for the op's packed weight stream (MegaOp).
//
// Arithmetic. The stored codes u = q + 128 go into the tensor core as fp16 subnormals u * 2^-24
// (one byte permute per pair, no arithmetic): products and their fp32 sums are exact up to the
// accumulator's rounding, and sum_k u_k x_k = sum_k q_k x_k + 128 * sum_k x_k, so a block's
// result is 2^24 * acc - 128 * sum(x of the block), scaled by the block's fp16 scale in fp32 as
// the reference does (matmul_b0_fp16_x_q8_0.comp:99-133). The input is column 0 of the B operand,
// the other columns read zeros. (An integer path, dp4a on three byte planes of the input, was
// measured 30 % slower: dp4a issues at about 16 lanes per clock and SM on this GPU.)
template <bool TIMED, bool DBG>
__device__ __forceinline__ void matvec_op(const Ctx &c, const MegaOp &op_global, uint32_t &it, uint32_t &slot, uint32_t &ph,
                                          unsigned char *ring, uint64_t *full, uint64_t *empty, const MegaStage *tabs, __half *xs, float *xbias,
                                          const __half *zero16, float *red, float *ssum, Best &best, unsigned long long *tw, uint32_t ar_seq,
                                          uint32_t tag_in, uint32_t tag_out, uint32_t tag_res, unsigned long long *trace) {
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const uint32_t G = gridDim.x, cta = blockIdx.x;
  // The op's entry sits in shared memory: fields are read where they are used (the prologue, then again
  // in the epilogue) instead of being carried in registers through the streaming loop, which needs them all.
  const MegaOp &op = op_global;
  const uint32_t K = op.K, tiles = op.tiles, NST = c.p.nst;
  const uint32_t tile0 = (cta + G - (op.rot % G)) % G;
  const uint32_t tl = tile0 < tiles ? (tiles - tile0 + G - 1) / G : 0u;  // this CTA's tiles
  // No tile here: nothing to read either. (It must not wait for the input: nobody waits for this
  // CTA's results, so by the time it looked the producers of a later op may have re-tagged the words.)
  if (tl == 0) return;
  const uint32_t nstages = op_global.stages_per_cta[cta];  // requested here, together with the input: needed when the stream starts
  // ---- input vector -> shared memory (RMSNorm fused, rounded to fp16 where the
  // reference's RMSNorm op rounds: rms_norm_fp16.comp:70-77). Norm weights and input are
  // requested together: one memory round trip.
  {
    constexpr int MAXV = (2048 + CT - 1) / CT;  // 8-half vectors per thread: K <= 16384
    uint4 v[MAXV];
    const uint32_t nv = K / 8;
    const bool norm = op.norm_w != nullptr;
    constexpr int NWV = 2;  // vectors per thread whose norm weights are requested early (K <= 7680: every norm op of the model shapes)
    float4 nw[NWV][2];
    if (norm) {  // the norm weights depend on nothing: request them before the polls, which can spin for a while
#pragma unroll
      for (int j = 0; j < NWV; ++j) {
        const uint32_t i = tid + j * CT;
        if (i < nv) {
          nw[j][0] = ldg_f4_ordered(reinterpret_cast<const float4 *>(op.norm_w) + 2 * i);
          nw[j][1] = ldg_f4_ordered(reinterpret_cast<const float4 *>(op.norm_w) + 2 * i + 1);
        }
      }
    }
    {
      // the first loads together (one memory round trip when the producers are done), then the tag checks
      constexpr int LFIRST = (11008 / 8 + CT - 1) / CT;  // K <= 11008 (the largest input of the model shapes) in one round trip
      uint4 la[LFIRST], lb[LFIRST];
#pragma unroll
      for (int j = 0; j < LFIRST; ++j) {
        const uint32_t i = tid + j * CT;
        if (i < nv) {
          la[j] = ld_vol_v4(op.in + 8 * i);
          lb[j] = ld_vol_v4(op.in + 8 * i + 4);
        }
      }
#pragma unroll
      for (int j = 0; j < MAXV; ++j) {
        const uint32_t i = tid + j * CT;
        v[j] = make_uint4(0, 0, 0, 0);
        if (i < nv) {
          if (j < LFIRST)
            v[j] = c.ll_wait8(op.in + 8 * i, la[j], lb[j], tag_in);
          else
            v[j] = c.ll_wait8(op.in + 8 * i, ld_vol_v4(op.in + 8 * i), ld_vol_v4(op.in + 8 * i + 4), tag_in);
        }
      }
    }
    for (uint32_t i = tid; i < tl * NCW * 32; i += CT) red[i] = 0.f;  // warps that get no unit of a tile leave zeros
    float alpha = 1.f;
    if (norm) {
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < MAXV; ++j) {
        const __half2 *h = reinterpret_cast<const __half2 *>(&v[j]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __half22float2(h[e]);
          s += f.x * f.x + f.y * f.y;
        }
      }
      s = warp_sum(s);
      if (lane == 0) ssum[warp] = s;
      cons_sync();
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < NCW; ++w) tot += ssum[w];
      alpha = 1.0f / sqrtf(tot / (float)K + op.eps);
    }
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const uint32_t i = tid + j * CT;
      float bs = 0.f;
      if (i < nv) {
        uint4 ov = v[j];
        if (norm) {
          const float4 w0 = j < NWV ? nw[j][0] : __ldg(reinterpret_cast<const float4 *>(op.norm_w) + 2 * i);
          const float4 w1 = j < NWV ? nw[j][1] : __ldg(reinterpret_cast<const float4 *>(op.norm_w) + 2 * i + 1);
          const __half2 *h = reinterpret_cast<const __half2 *>(&v[j]);
          const float2 a = __half22float2(h[0]), b = __half22float2(h[1]), cc = __half22float2(h[2]), d = __half22float2(h[3]);
          __half2 o[4];
          o[0] = __halves2half2(__float2half_rn(a.x * w0.x * alpha), __float2half_rn(a.y * w0.y * alpha));
          o[1] = __halves2half2(__float2half_rn(b.x * w0.z * alpha), __float2half_rn(b.y * w0.w * alpha));
          o[2] = __halves2half2(__float2half_rn(cc.x * w1.x * alpha), __float2half_rn(cc.y * w1.y * alpha));
          o[3] = __halves2half2(__float2half_rn(d.x * w1.z * alpha), __float2half_rn(d.y * w1.w * alpha));
          ov = *reinterpret_cast<uint4 *>(o);
        }
        *reinterpret_cast<uint4 *>(xs + 8 * i) = ov;
        const __half2 *h = reinterpret_cast<const __half2 *>(&ov);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __half22float2(h[e]);
          bs += f.x + f.y;
        }
      }
      // a block of 32 inputs = 4 consecutive vectors = 4 consecutive lanes
      bs += __shfl_xor_sync(0xffffffffu, bs, 1);
      bs += __shfl_xor_sync(0xffffffffu, bs, 2);
      if ((lane & 3) == 0 && i < nv) xbias[i >> 2] = 128.0f * bs;
    }
    cons_sync();
  }
  // EPI_ADD: this thread's residual value, requested now so that its memory round trip is not
  // on the path between the end of the stream and the publication of the results
  float resid = 0.f;
  if ((op.epi == EPI_ADD || op.epi == EPI_REDUCE) && tid < tl * 32) {
    const uint32_t n = (tile0 + (tid >> 5) * G) * 32 + (tid & 31);
    if (n < op.N) resid = __half2float(ll_half(c.ll_wait1(op.out_ll[0] + n, tag_res)));  // (its tag is checked: the word may come from another CTA)
  }
  if (TIMED && tw) tw[1] = clock64();
  VKL_TRACE(1);

  // ---- stream this CTA's tiles. Every stage holds UPW units per consumer warp; a unit is one
  // block (32 columns) of a 32-row tile: two 16-row halves, each the A operand of two m16n8k16
  // MMAs. Stages run on across tile boundaries, so a warp's partial sums of a tile go to the
  // warp's own slot in shared memory when its units move on to the next tile, and nothing
  // synchronises until the op's single reduction at the end.
  {
    uint32_t cur = 0xffffffffu;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};  // lanes t == 0: rows g, g + 8, 16 + g, 24 + g of the tile
    auto flush = [&]() {
      if (cur != 0xffffffffu && t == 0) {
        float *slotp = red + ((size_t)cur * NCW + warp) * 32;
        slotp[g] = acc[0];
        slotp[g + 8] = acc[1];
        slotp[16 + g] = acc[2];
        slotp[24 + g] = acc[3];
      }
    };
    const __half *xbase = g == 0 ? xs + t * 8 : zero16;  // column 0 of B = the input, the other columns zeros
    const uint32_t xstep = g == 0 ? 32u : 0u;
    for (uint32_t sidx = 0; sidx < nstages; ++sidx) {
      unsigned long long w0 = 0;
      if (TIMED && tw) w0 = clock64();
      const bool ok = (DBG && (c.p.timing_mode & 128u)) ? true : c.wait(s32(&full[slot]), ph, 1);
      if (TIMED && tw) tw[0] += (clock64() - w0) * 1000ull / c.p.sm_mhz;  // SM cycles -> ns at the SM clock the host measured
      if (DBG && (c.p.timing_mode & 64u)) {  // diagnostic: handshake only
        __syncwarp();
        if (lane == 0 && !(c.p.timing_mode & 128u)) mbar_arrive(s32(&empty[slot]));
        ++it;
        if (++slot == NST) {
          slot = 0;
          ph ^= 1u;
        }
        continue;
      }
      // the stage's place in the op (tile, first block, run lengths) is in the producer's
      // table entry, which the producer wrote before it armed the stage's barrier
      const uint4 meta = *reinterpret_cast<const uint4 *>(&tabs[it & 127].n0);
      const uint32_t n0 = meta.x, n1 = meta.y, tm = meta.z, kg = meta.w;
      const unsigned char *st = ring + (size_t)slot * STAGE_BYTES;
      uint4 wa[UPW], wb[UPW];
      uint2 dsc[UPW];
      bool have[UPW];
#pragma unroll
      for (int q = 0; q < UPW; ++q) {
        const uint32_t u = warp * UPW + q;
        have[q] = ok && u < n0 + n1;
        if (have[q]) {
          wa[q] = *reinterpret_cast<const uint4 *>(st + u * UNIT_BYTES + lane * 16);        // rows g, g + 8 of the tile
          wb[q] = *reinterpret_cast<const uint4 *>(st + u * UNIT_BYTES + 512 + lane * 16);  // rows 16 + g, 24 + g
          dsc[q] = *reinterpret_cast<const uint2 *>(st + u * UNIT_BYTES + UNIT_CODES + g * 8);  // their four block scales
        }
      }
      __syncwarp();
      if (lane == 0 && ok) mbar_arrive(s32(&empty[slot]));  // this warp has read all it needs from the stage
#pragma unroll
      for (int q = 0; q < UPW; ++q) {
        if (!have[q]) continue;
        const uint32_t u = warp * UPW + q;
        const uint32_t mt = u < n0 ? tm : tm + 1, b = u < n0 ? kg + u : u - n0;
        if (mt != cur) {
          flush();
          cur = mt;
          acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
        }
        if (DBG && (c.p.timing_mode & 4u)) {  // diagnostic: ring traffic without arithmetic
          acc[0] += __uint_as_float(wa[q].x ^ wb[q].w ^ dsc[q].x);
          continue;
        }
        const uint4 X = *reinterpret_cast<const uint4 *>(xbase + b * xstep);
        const float xb = xbias[b];
        float ca[4] = {0.f, 0.f, 0.f, 0.f}, cb[4] = {0.f, 0.f, 0.f, 0.f};
        mma16816(ca, codes_sub_h2(wa[q].x, false), codes_sub_h2(wa[q].z, false), codes_sub_h2(wa[q].x, true), codes_sub_h2(wa[q].z, true), X.x, X.y);
        mma16816(cb, codes_sub_h2(wb[q].x, false), codes_sub_h2(wb[q].z, false), codes_sub_h2(wb[q].x, true), codes_sub_h2(wb[q].z, true), X.x, X.y);
        mma16816(ca, codes_sub_h2(wa[q].y, false), codes_sub_h2(wa[q].w, false), codes_sub_h2(wa[q].y, true), codes_sub_h2(wa[q].w, true), X.z, X.w);
        mma16816(cb, codes_sub_h2(wb[q].y, false), codes_sub_h2(wb[q].w, false), codes_sub_h2(wb[q].y, true), codes_sub_h2(wb[q].w, true), X.z, X.w);
        const float2 d0 = __half22float2(*reinterpret_cast<const __half2 *>(&dsc[q].x));  // rows g, g + 8
        const float2 d1 = __half22float2(*reinterpret_cast<const __half2 *>(&dsc[q].y));  // rows 16 + g, 24 + g
        acc[0] = fmaf(fmaf(ca[0], 16777216.f, -xb), d0.x, acc[0]);
        acc[1] = fmaf(fmaf(ca[2], 16777216.f, -xb), d0.y, acc[1]);
        acc[2] = fmaf(fmaf(cb[0], 16777216.f, -xb), d1.x, acc[2]);
        acc[3] = fmaf(fmaf(cb[2], 16777216.f, -xb), d1.y, acc[3]);
      }
      ++it;
      if (++slot == NST) {
        slot = 0;
        ph ^= 1u;
      }
    }
    flush();
  }
  // ---- one fixed-order reduction over the warps and the epilogue for all tiles
  VKL_TRACE(2);
  if (TIMED && tw) {
    tw[2] = clock64();
    if (c.p.timing_mode & 32u) tw[0] = (((tw[2] - tw[1]) * 1000ull / c.p.sm_mhz) << 16) | (uint64_t)min(nstages, 65535u);
  }
  cons_sync();
  VKL_TRACE(3);
  const uint32_t tpm = (op.N + 31) / 32;  // tiles per matrix (nmat = 3)
  for (uint32_t idx = tid; idx < tl * 32; idx += CT) {  // tl * 32 is a multiple of the warp size: whole warps
    const uint32_t lt = idx >> 5, r = idx & 31;
    const uint32_t gt = tile0 + lt * G;
    const float *sp = red + ((size_t)lt * NCW) * 32 + r;
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < NCW; ++w) sum += sp[w * 32];
    if (op.epi == EPI_SWIGLU) {
      // rows 0..15 of the tile are gate rows, rows 16..31 the up rows of the same outputs
      const float up = __shfl_down_sync(0xffffffffu, sum, 16);
      const uint32_t n = gt * 16 + r;
      if (r < 16 && n < op.N && !c.aborted()) op.out_ll[0][n] = ll_pack(__float2half_rn(sum / (1.0f + expf(-sum)) * up), tag_out);
      continue;
    }
    const uint32_t m = op.nmat == 3 ? gt / tpm : 0u;
    const uint32_t n = (op.nmat == 3 ? gt % tpm : gt) * 32 + r;
    if (n < op.N && !c.aborted()) {
      if (op.epi == EPI_ADD) {
        const float res = idx == tid ? resid : __half2float(ll_half(c.ll_wait1(op.out_ll[0] + n, tag_res)));
        op.out_ll[0][n] = ll_pack(__float2half_rn(round_h(sum) + res), tag_out);
      } else if (op.epi == EPI_REDUCE) {
        // this rank's share of a row-split projection, reduced in place: the row's raw fp32 sum and the all-reduce's
        // sequence number go as one 8-byte word into slot [parity][my rank] of every OTHER rank's exchange buffer
        // (plain peer stores over NVLink; the word is its own arrival flag); then this thread polls (bounded, all
        // missing words per round) the same row's words of the other ranks in its own buffer, adds in rank order (the
        // same order on every rank: bit-identical residual streams) and publishes x = fp16(fp16(sum) + x).
        const MegaParams &pp = c.p;
        const uint32_t tp = pp.tp_size, me = pp.tp_rank;
        const size_t par = (size_t)(ar_seq & 1u) * tp;
        for (uint32_t rk = 0; rk < tp; ++rk) {
          if (rk == me) continue;
          uint32_t *dst = static_cast<uint32_t *>(pp.tp_peer[rk]) + 2 * ((par + me) * pp.dim + n);
          asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(__float_as_uint(sum)), "r"(ar_seq) : "memory");
        }
        const float res = idx == tid ? resid : __half2float(ll_half(c.ll_wait1(op.out_ll[0] + n, tag_res)));
        const uint32_t *mine = static_cast<const uint32_t *>(pp.tp_peer[me]) + 2 * (par * pp.dim + n);
        float part[8];
        uint32_t missing = ((1u << tp) - 1u) & ~(1u << me);
        part[me & 7u] = sum;
        const uint32_t limit = pp.wait_limit;
      #pragma unroll 1
        for (uint32_t itw = 0; missing && itw < limit; ++itw) {
#pragma unroll
          for (uint32_t r = 0; r < 8; ++r) {
            if (missing & (1u << r)) {
              const uint2 w = ld_vol_v2(mine + 2 * (size_t)r * pp.dim);
              if (w.y == ar_seq) {
                part[r] = __uint_as_float(w.x);
                missing &= ~(1u << r);
              }
            }
          }
          if (itw > 100000u) __nanosleep(64);
          if ((itw & 1023u) == 1023u && (*(volatile uint32_t *)pp.error != 0u || c.aborted())) break;
        }
        if (missing) {
          c.raise(4);
        } else {
          float s = 0.f;
#pragma unroll
          for (uint32_t r = 0; r < 8; ++r)
            if (r < tp) s += part[r];
          op.out_ll[0][n] = ll_pack(__float2half_rn(round_h(s) + res), tag_out);
        }
      } else if (op.epi == EPI_PARTIAL) {
        // this rank's share of a row-split projection: the raw fp32 sum and the all-reduce's
        // sequence number go, as one 8-byte word, into slot [parity][my rank] of every rank's
        // exchange buffer (plain peer stores over NVLink; the word is its own arrival flag)
        const MegaParams &pp = c.p;
        for (uint32_t rk = 0; rk < pp.tp_size; ++rk) {
          uint32_t *dst = static_cast<uint32_t *>(pp.tp_peer[rk]) + 2 * (((size_t)(ar_seq & 1u) * pp.tp_size + pp.tp_rank) * pp.dim + n);
          asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(__float_as_uint(sum)), "r"(ar_seq) : "memory");
        }
      } else {
        const __half h0 = __float2half_rn(sum);
        uint32_t *o = m == 0 ? op.out_ll[0] : m == 1 ? op.out_ll[1] : op.out_ll[2];
        if (o) {
          o[n] = ll_pack(h0, tag_out);
        } else {
          op.out[0][n] = h0;
        }
        if (op.out_f32) op.out_f32[n] = __half2float(h0);
        if (op.track_argmax && better(__half2float(h0), n, best)) {
          best.v = __half2float(h0);
          best.i = n;
        }
      }
    }
  }
}

// ---------------------------------------------------------------- attention
__device__ __forceinline__ void rope_pair(float x0, float x1, float cs, float sn, __half &o0, __half &o1) {
  o0 = __float2half_rn(x0 * cs - x1 * sn);
  o1 = __float2half_rn(x0 * sn + x1 * cs);
}

// One (head, split) per CTA: RoPE(q), RoPE(k) + cache append by the split that
// owns the new column, scores over its column range, partial softmax and P.V.
// Same arithmetic as attention_kernel<true> (attention.cu). The cached K and V rows of the
// split come through the weight ring: they do not depend on this token (only the row of the
// new position does, and that one is taken from the fresh projections), so the producer warp
// has copied them into shared memory before q, k and v arrive.
__device__ __forceinline__ void attn_part_op(const Ctx &c, const MegaOp &op, float *sm, uint32_t pos0, uint32_t S, uint32_t tag_in,
                                             uint32_t tag_out, uint32_t &slot, uint32_t &ph, const unsigned char *ring, uint64_t *full,
                                             uint64_t *empty) {
  const MegaParams &p = c.p;
  const uint32_t cta = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (cta >= p.heads * S) return;
  const uint32_t h = cta / S, split = cta % S, D = p.head_dim, NST = p.nst;
  float *q_s = sm, *kn_s = sm + D, *red_s = sm + 3 * D, *s_s = sm + (3 + NCW / 2) * D + 2 * NCW + 32;
  uint32_t *vn_s = reinterpret_cast<uint32_t *>(sm + 2 * D);  // the new V row as packed half pairs
  const uint32_t L = min(pos0 + 1, p.maxlen);
  uint32_t c0, c1;
  mega_kv_range(L, S, split, c0, c1);
  const uint32_t jn = pos0 % p.maxlen;
  const bool owns = jn >= c0 && jn < c1;
  const size_t row = (size_t)h * D;
  __half *kcache = op.kcache, *vcache = op.vcache;
  if (2 * tid < D) {
    const size_t fi = (size_t)pos0 * (D / 2) + tid;
    const float cs = p.freqc[fi], sn = p.freqs[fi];  // requested with the polls below: one round trip
    __half r0, r1;
    // q, k, v of this head come from the projection op before: request this thread's pairs of
    // tagged words together (one memory round trip when they are there), then poll what is missing
    const uint32_t *qp = p.q + row + 2 * tid, *kp = p.k + row + 2 * tid, *vp = p.v + row + 2 * tid;
    uint2 qw = ld_vol_v2(qp), kw = make_uint2(0, 0), vw = make_uint2(0, 0);
    if (owns) {
      kw = ld_vol_v2(kp);
      vw = ld_vol_v2(vp);
    }
    qw = c.ll_wait2(qp, qw, tag_in);
    rope_pair(__half2float(ll_half(qw.x)), __half2float(ll_half(qw.y)), cs, sn, r0, r1);
    q_s[2 * tid] = __half2float(r0);
    q_s[2 * tid + 1] = __half2float(r1);
    if (owns) {
      kw = c.ll_wait2(kp, kw, tag_in);
      vw = c.ll_wait2(vp, vw, tag_in);
      rope_pair(__half2float(ll_half(kw.x)), __half2float(ll_half(kw.y)), cs, sn, r0, r1);
      kn_s[2 * tid] = __half2float(r0);
      kn_s[2 * tid + 1] = __half2float(r1);
      const size_t dst = ((size_t)h * p.maxlen + jn) * D + 2 * tid;
      kcache[dst] = r0;
      kcache[dst + 1] = r1;
      vcache[dst] = ll_half(vw.x);
      vcache[dst + 1] = ll_half(vw.y);
      vn_s[tid] = (vw.x & 0xffffu) | (vw.y << 16);  // the new row, for this CTA's P.V
    }
  }
  cons_sync();
  const float scale = 1.0f / sqrtf((float)D);
  const uint32_t rps = mega_kv_rows_per_stage(D), rows = c1 - c0;
  // ---- scores: 16 lanes per cached row (8 dims each), two rows per warp and step
  {
    const uint32_t sub = lane & 15, hi = lane >> 4;
    const bool act = sub * 8 < D;
    float qv[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) qv[e] = act ? q_s[sub * 8 + e] : 0.f;
    for (uint32_t r0 = 0; r0 < rows; r0 += rps) {
      const bool ok = (p.timing_mode & 128u) ? true : c.wait(s32(&full[slot]), ph, 1);
      const uint32_t nr = min(rps, rows - r0);
      const unsigned char *ks = ring + (size_t)slot * STAGE_BYTES;
      for (uint32_t rb = warp * 2; rb < nr; rb += NCW * 2) {
        const uint32_t r = rb + hi, j = c0 + r0 + r;
        float a = 0.f;
        if (ok && act && r < nr) {
          if (owns && j == jn) {
#pragma unroll
            for (int e = 0; e < 8; ++e) a = fmaf(qv[e], kn_s[sub * 8 + e], a);
          } else {
            const uint4 kv = *reinterpret_cast<const uint4 *>(ks + ((size_t)r * D + sub * 8) * 2);
            const float2 k0 = __half22float2(*reinterpret_cast<const __half2 *>(&kv.x));
            const float2 k1 = __half22float2(*reinterpret_cast<const __half2 *>(&kv.y));
            const float2 k2 = __half22float2(*reinterpret_cast<const __half2 *>(&kv.z));
            const float2 k3 = __half22float2(*reinterpret_cast<const __half2 *>(&kv.w));
            a = fmaf(qv[0], k0.x, a); a = fmaf(qv[1], k0.y, a); a = fmaf(qv[2], k1.x, a); a = fmaf(qv[3], k1.y, a);
            a = fmaf(qv[4], k2.x, a); a = fmaf(qv[5], k2.y, a); a = fmaf(qv[6], k3.x, a); a = fmaf(qv[7], k3.y, a);
          }
        }
        a += __shfl_xor_sync(0xffffffffu, a, 8);
        a += __shfl_xor_sync(0xffffffffu, a, 4);
        a += __shfl_xor_sync(0xffffffffu, a, 2);
        a += __shfl_xor_sync(0xffffffffu, a, 1);
        if (sub == 0 && r < nr) s_s[r0 + r] = round_h(a * scale);
      }
      __syncwarp();
      if (lane == 0 && ok && !(p.timing_mode & 128u)) mbar_arrive(s32(&empty[slot]));
      if (++slot == NST) {
        slot = 0;
        ph ^= 1u;
      }
    }
  }
  cons_sync();
  float lmax = -INFINITY;
  for (uint32_t i = tid; i < rows; i += CT) lmax = fmaxf(lmax, s_s[i]);
  lmax = warp_max(lmax);
  if (lane == 0) red_s[warp] = lmax;
  cons_sync();
  float mloc = red_s[0];
#pragma unroll
  for (int w = 1; w < NCW; ++w) mloc = fmaxf(mloc, red_s[w]);
  float lsum = 0.f;
  for (uint32_t i = tid; i < rows; i += CT) {
    const float pj = expf(s_s[i] - mloc);
    s_s[i] = pj;
    lsum += pj;
  }
  lsum = warp_sum(lsum);
  if (lane == 0) red_s[NCW + warp] = lsum;
  cons_sync();
  float lloc = 0.f;
#pragma unroll
  for (int w = 0; w < NCW; ++w) lloc += red_s[NCW + w];
  // P.V: CT/64 row groups x up to 64 dim pairs, rows of a group in ascending order
  const uint32_t npair = D / 2, grp = tid / 64, dp = tid % 64;
  constexpr uint32_t NG = CT / 64;  // threads beyond NG*64 sit this part out
  float2 acc = make_float2(0.f, 0.f);
  {
    const bool act = dp < npair && grp < NG;
    uint32_t rnext = grp;  // this thread's next row of the split (rows grp, grp + NG, ...)
    for (uint32_t r0 = 0; r0 < rows; r0 += rps) {
      const bool ok = (p.timing_mode & 128u) ? true : c.wait(s32(&full[slot]), ph, 1);
      const uint32_t nr = min(rps, rows - r0);
      const unsigned char *vs = ring + (size_t)slot * STAGE_BYTES;
      if (ok && act) {
        for (; rnext < r0 + nr; rnext += NG) {
          const uint32_t j = c0 + rnext;
          const uint32_t raw = (owns && j == jn) ? vn_s[dp] : *reinterpret_cast<const uint32_t *>(vs + ((size_t)(rnext - r0) * D + 2 * dp) * 2);
          const float2 vv = __half22float2(*reinterpret_cast<const __half2 *>(&raw));
          const float pj = s_s[rnext];
          acc.x = fmaf(pj, vv.x, acc.x);
          acc.y = fmaf(pj, vv.y, acc.y);
        }
      }
      __syncwarp();
      if (lane == 0 && ok) mbar_arrive(s32(&empty[slot]));
      if (++slot == NST) {
        slot = 0;
        ph ^= 1u;
      }
    }
  }
  cons_sync();
  float *pv = red_s + 2 * NCW;  // [CT/64 groups][D]
  if (dp < npair && grp < CT / 64) {
    pv[grp * D + 2 * dp] = acc.x;
    pv[grp * D + 2 * dp + 1] = acc.y;
  }
  cons_sync();
  float *part = p.attn_scratch + ((size_t)h * p.splits + split) * (D + 4);
  if (tid < D) {
    float s = 0.f;
#pragma unroll
    for (int gq = 0; gq < CT / 64; ++gq) s += pv[gq * D + tid];
    if (S == 1)
      p.ao[row + tid] = ll_pack(__float2half_rn(s / lloc), tag_out);  // whole row in this CTA: no combine phase
    else
      part[tid] = s;
  }
  if (tid == 0) {
    part[D] = mloc;
    part[D + 1] = lloc;
  }
  if (S > 1 && p.attn_counters) {
    // The split that finishes last merges the head's partials (in split order, so the result
    // does not depend on who is last): no separate combine op and no grid barrier before it.
    __threadfence();  // this thread's partial results before the CTA's arrival below
    cons_sync();
    volatile uint32_t *last_s = reinterpret_cast<volatile uint32_t *>(red_s);
    if (tid == 0) {
      uint32_t old;
      asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(p.attn_counters + h) : "memory");
      const bool last = old == S - 1;
      if (last) p.attn_counters[h] = 0;  // all splits of the head have arrived; its next use is a grid barrier away
      *last_s = last ? 1u : 0u;
    }
    cons_sync();
    if (*last_s && tid < D) {
      const float *base = p.attn_scratch + (size_t)h * p.splits * (D + 4);
      float M = -INFINITY;
      for (uint32_t sp = 0; sp < S; ++sp) M = fmaxf(M, __ldcg(base + sp * (D + 4) + D));
      float den = 0.f, num = 0.f;
      for (uint32_t sp = 0; sp < S; ++sp) {
        const float ms = __ldcg(base + sp * (D + 4) + D), ls = __ldcg(base + sp * (D + 4) + D + 1);
        if (ls > 0.f) {
          const float w = expf(ms - M);
          den += ls * w;
          num += __ldcg(base + sp * (D + 4) + tid) * w;
        }
      }
      p.ao[row + tid] = ll_pack(__float2half_rn(num / den), tag_out);
    }
  }
}

// One head per CTA: merge the split partials in split order.
__device__ VKL_SLOW void attn_combine_op(const Ctx &c, uint32_t tag_out) {
  const MegaParams &p = c.p;
  const uint32_t h = blockIdx.x, tid = threadIdx.x, D = p.head_dim;
  if (h >= p.heads || tid >= D) return;
  const float *base = p.attn_scratch + (size_t)h * p.splits * (D + 4);
  float M = -INFINITY;
  for (uint32_t s = 0; s < p.splits; ++s) M = fmaxf(M, __ldcg(base + s * (D + 4) + D));
  float den = 0.f, num = 0.f;
  for (uint32_t s = 0; s < p.splits; ++s) {
    const float ms = __ldcg(base + s * (D + 4) + D), ls = __ldcg(base + s * (D + 4) + D + 1);
    if (ls > 0.f) {
      const float w = expf(ms - M);
      den += ls * w;
      num += __ldcg(base + s * (D + 4) + tid) * w;
    }
  }
  p.ao[(size_t)h * D + tid] = ll_pack(__float2half_rn(num / den), tag_out);
}

// Embedding gather + dequantisation of the current token (embedding_q8_0.comp:39-85).
__device__ VKL_SLOW void embed_op(const Ctx &c, uint32_t tok, uint32_t tag_out) {
  const MegaParams &p = c.p;
  const uint32_t per = (p.dim + gridDim.x - 1) / gridDim.x;
  const uint32_t k = blockIdx.x * per + threadIdx.x;
  if (threadIdx.x >= per || k >= p.dim) return;
  if (tok >= p.embd_rows) tok = 0;  // UNK = 0 (models/llama2.h:455-458)
  const Q8Layout L = q8_layout(p.embd_rows, p.dim);
  const uint32_t tile = tok >> 4, r = tok & 15, g = r & 7, half = r >> 3;
  const uint32_t b = k >> 5, t = (k >> 3) & 3, i = k & 7;
  const uint8_t cb = p.embd[(((size_t)tile * L.groups * 4 + b) * 32 + g * 4 + t) * 16 + half * 8 + q8_byte_pos(i)];
  const uint16_t *sc = reinterpret_cast<const uint16_t *>(p.embd + L.codes_bytes());
  const uint16_t d = sc[(((size_t)tile * L.groups + (b >> 2)) * 8 + g) * 8 + half * 4 + (b & 3)];
  p.x[k] = ll_pack(__float2half_rn((float)((int)cb - 128) * __half2float(__ushort_as_half(d))), tag_out);
}

// CTA 0: best of the per-CTA candidates (lowest index on ties), then publish the id,
// feed it back and advance position, step and launch epoch.
__device__ VKL_SLOW void argmax_final_op(const Ctx &c, float *sm, uint32_t pos0, uint64_t rounds_done, uint32_t ar_done,
                                                uint32_t next_ebase) {
  const MegaParams &p = c.p;
  if (blockIdx.x != 0) return;
  const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  Best b = {0.f, 0xffffffffu};
  for (uint32_t i = tid; i < gridDim.x; i += CT) {
    const float v = __ldcg(p.arg_scratch + 2 * i);
    const uint32_t ix = __float_as_uint(__ldcg(p.arg_scratch + 2 * i + 1));
    if (ix != 0xffffffffu && better(v, ix, b)) {
      b.v = v;
      b.i = ix;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, b.v, o);
    const uint32_t oi = __shfl_xor_sync(0xffffffffu, b.i, o);
    if (oi != 0xffffffffu && better(ov, oi, b)) {
      b.v = ov;
      b.i = oi;
    }
  }
  uint32_t *si = reinterpret_cast<uint32_t *>(sm);
  if (lane == 0) {
    sm[32 + warp] = b.v;
    si[warp] = b.i;
  }
  cons_sync();
  if (tid == 0) {
    for (int w = 1; w < NCW; ++w)
      if (si[w] != 0xffffffffu && better(sm[32 + w], si[w], b)) {
        b.v = sm[32 + w];
        b.i = si[w];
      }
    if (p.tp_size > 1 && !c.aborted()) {
      // vocabulary-split lm head: exchange (value, global index) candidates with all ranks
      const uint32_t tp = p.tp_size, aseq = p.state[4] + 1;
      b.i += p.tp_rank * p.vocab;
      for (uint32_t r = 0; r < tp; ++r) {
        float *cand = static_cast<float *>(p.tp_peer[r]) + p.tp_flag_off + 32 + 2 * p.tp_rank;
        cand[0] = b.v;
        cand[1] = __uint_as_float(b.i);
      }
      __threadfence_system();
      for (uint32_t r = 0; r < tp; ++r) st_rel_sys_u32(static_cast<uint32_t *>(p.tp_peer[r]) + p.tp_flag_off + 16 + p.tp_rank, aseq);
      const uint32_t *mine = static_cast<const uint32_t *>(p.tp_peer[p.tp_rank]) + p.tp_flag_off;
      for (uint32_t r = 0; r < tp && !c.aborted(); ++r) {
        bool ok = false;
      #pragma unroll 1
        for (uint32_t i = 0; i < c.p.wait_limit; ++i) {
          if ((int32_t)(ld_acq_sys_u32(mine + 16 + r) - aseq) >= 0) {
            ok = true;
            break;
          }
          if (i > 100000u) __nanosleep(64);
        }
        if (!ok) c.raise(5);
      }
      Best gb = {0.f, 0xffffffffu};
      for (uint32_t r = 0; r < tp; ++r) {
        const float *cand = static_cast<const float *>(p.tp_peer[p.tp_rank]) + p.tp_flag_off + 32 + 2 * r;
        const float v = __ldcg(cand);
        const uint32_t ix = __float_as_uint(__ldcg(cand + 1));
        if (better(v, ix, gb)) {
          gb.v = v;
          gb.i = ix;
        }
      }
      b = gb;
      p.state[4] = aseq;
    }
    if (!c.aborted()) {
      const uint32_t step = p.state[1], n_forced = p.state[5];
      p.state[2] = b.i;
      if (pos0 + 1 < n_forced) {
        p.tok[0] = p.forced[pos0 + 1];  // still inside the prompt: feed the next prompt token
      } else {
        p.tok[0] = b.i;
        if (step < p.out_cap) p.out_ids[step] = b.i;
        p.state[1] = step + 1;
      }
      p.state[0] = pos0 + 1;
      p.state[3] = ar_done;
      p.state[7] = next_ebase;
      p.bar[1] = rounds_done;
    }
  }
}

// Tensor-parallel all-reduce, second half. The partial sums were pushed to every rank by the
// preceding row-split projection as 8-byte words {fp32 sum, all-reduce sequence number}.
// Every CTA reduces its slice of rows in rank order as soon as the words of all ranks carry
// this all-reduce's number: x <- fp16( fp16(sum_r partial_r) + x ), the same rounding as
// o_proj/down + residual add. No grid barrier and no separate flags: two parities of slots
// keep a fast rank's next push from overwriting what a slow rank still reads.
__device__ VKL_SLOW void allreduce_op(const Ctx &c, const MegaOp &op, uint32_t seq, uint32_t tag_out, uint32_t tag_res) {
  const MegaParams &p = c.p;
  const uint32_t tid = threadIdx.x, tp = p.tp_size;
  if (c.aborted()) return;
  const uint32_t per = (p.dim + gridDim.x - 1) / gridDim.x;
  const uint32_t i = blockIdx.x * per + tid;
  if (tid < per && i < p.dim) {
    // every rank pushed {partial sum, sequence number} words into this rank's buffer: poll this
    // row's word of every rank (bounded), add in rank order
    const uint32_t *part = static_cast<const uint32_t *>(p.tp_peer[p.tp_rank]) + 2 * ((size_t)(seq & 1u) * tp * p.dim);
    float s = 0.f;
    for (uint32_t r = 0; r < tp; ++r) {
      const uint32_t *src = part + 2 * ((size_t)r * p.dim + i);
      uint2 w = ld_vol_v2(src);
      if (w.y != seq) {
        bool ok = false;
      #pragma unroll 1
        for (uint32_t it = 0; it < p.wait_limit; ++it) {
          w = ld_vol_v2(src);
          if (w.y == seq) {
            ok = true;
            break;
          }
          if (it > 100000u) __nanosleep(64);
          if ((it & 1023u) == 1023u && (*(volatile uint32_t *)p.error != 0u || c.aborted())) break;
        }
        if (!ok) {
          c.raise(4);
          return;
        }
      }
      s += __uint_as_float(w.x);
    }
    const float res = __half2float(ll_half(c.ll_wait1(op.out_ll[0] + i, tag_res)));  // the residual, under the tag of the op that wrote it
    op.out_ll[0][i] = ll_pack(__float2half_rn(round_h(s) + res), tag_out);
  }
}

template <bool TIMED, bool DBG>
__global__ void __launch_bounds__(THREADS, 1) decode_mega_kernel(const __grid_constant__ MegaParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t NST = p.nst;
  unsigned char *ring = smem;
  unsigned char *xq = smem + (size_t)NST * STAGE_BYTES;  // quantised input vector; attention scratch
  float *red = reinterpret_cast<float *>(xq + p.xs_bytes);
  float *ssum = red + (size_t)p.red_slots * NCW * 32;  // [64]
  const __half *zero16 = reinterpret_cast<const __half *>(ssum + 64);  // 16 zero bytes
  MegaStage *tabs = reinterpret_cast<MegaStage *>(ssum + 68);  // [128], 16-byte aligned
  uint64_t *full = reinterpret_cast<uint64_t *>(tabs + 128);
  uint64_t *empty = full + MAX_NST;
  volatile uint32_t *abort_s = reinterpret_cast<volatile uint32_t *>(empty + MAX_NST);
  // The op table lives in global memory; reading an entry there costs a chain of L2 round trips
  // (kind, then the fields, then what they point to) at the start of every op. Three entries are
  // kept in shared memory instead: the running op, the next one (looked at when this one ends)
  // and the one after, which is copied in asynchronously while this op runs.
  MegaOp *opbuf = reinterpret_cast<MegaOp *>(reinterpret_cast<unsigned char *>(empty + MAX_NST) + 16);
  constexpr uint32_t OPV = sizeof(MegaOp) / 16;
  static_assert(sizeof(MegaOp) % 16 == 0, "MegaOp is copied in 16-byte pieces");
  if (threadIdx.x < 2 * OPV && threadIdx.x / OPV < p.nops)
    reinterpret_cast<uint4 *>(opbuf)[threadIdx.x] = reinterpret_cast<const uint4 *>(p.ops)[threadIdx.x];

  if (threadIdx.x == 0) {
    for (uint32_t i = 0; i < NST; ++i) {
      mbar_init(s32(&full[i]), 1);
      mbar_init(s32(&empty[i]), NCW);
    }
    abort_s[0] = 0;
    abort_s[1] = 0;
    *reinterpret_cast<uint4 *>(ssum + 64) = make_uint4(0, 0, 0, 0);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  const Ctx c{p, abort_s};

  if (threadIdx.x >= CT) {  // producer warp
    producer(c, ring, full, empty, tabs);
    return;
  }

  const uint32_t G = gridDim.x;
  const uint32_t pos0 = p.state[0], tok = p.tok[0];
  const uint64_t base_rounds = p.bar[1];  // barrier rounds completed by earlier launches
  uint64_t rounds = 0;
  const uint32_t seq0 = p.state[3];  // all-reduces completed by earlier launches
  uint32_t ar_i = 0;
  const uint32_t Lnow = min(pos0 + 1, p.maxlen);
  const uint32_t S_eff = mega_splits(Lnow, p.splits, p.split_rows);
  uint32_t it = 0, slot = 0, ph = 0;  // ring position, carried across the ops of the token
  const uint32_t ebase = p.state[7];  // sequence number of this launch's first op; op oi tags its results with ebase + oi
  auto tag = [&](uint32_t op_index) { return (ebase + op_index) & 0xffffu; };
  Best best = {0.f, 0xffffffffu};
  const bool tracing = TIMED && p.timing != nullptr && (p.timing_mode & 256u) != 0;
  const bool timed = TIMED && p.timing != nullptr && !tracing && blockIdx.x == 0 && threadIdx.x == 0;
  unsigned long long t0 = 0, twait[3] = {0, 0, 0}, c0 = 0;
  if (timed) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (uint32_t oi = 0; oi < p.nops; ++oi) {
    const MegaOp &op = opbuf[oi % 3];
    if (oi + 2 < p.nops && threadIdx.x < OPV) {  // entry oi + 2 replaces entry oi - 1, which every thread has left
      const uint32_t dst = s32(reinterpret_cast<uint4 *>(opbuf + (oi + 2) % 3) + threadIdx.x);
      const uint4 *src = reinterpret_cast<const uint4 *>(p.ops + oi + 2) + threadIdx.x;
      asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(__cvta_generic_to_global(src)) : "memory");
    }
    if (op.kind == MK_ATTN_COMBINE && S_eff == 1) {  // nothing to merge, no grid barrier either
      cons_sync();  // every thread has read this entry before the next op's copy may replace it
      continue;
    }
    if (timed) c0 = clock64();
    unsigned long long *trace = (tracing && threadIdx.x == 0) ? p.timing + ((size_t)oi * gridDim.x + blockIdx.x) * 8 : nullptr;
    VKL_TRACE(0);
    switch (op.kind) {
      case MK_EMBED: embed_op(c, tok, tag(oi)); break;
      case MK_MATVEC: matvec_op<TIMED, DBG>(c, op, it, slot, ph, ring, full, empty, tabs, reinterpret_cast<__half *>(xq), reinterpret_cast<float *>(xq + (size_t)p.xmax_blocks * XB_BYTES), zero16, red, ssum, best, (TIMED && timed) ? twait : nullptr, seq0 + ar_i + 1,
                         tag(op.src_op), tag(oi), tag(op.res_op), trace);
        if (op.epi == EPI_REDUCE) ++ar_i;  // (every CTA counts it, with or without a tile of the op)
        break;
      case MK_ATTN_PART:
        attn_part_op(c, op, reinterpret_cast<float *>(xq), pos0, S_eff, tag(op.src_op), tag(op.tag_op), slot, ph, ring, full, empty);
        if (blockIdx.x < p.heads * p.splits) ++it;  // this CTA's KV entry of the stage table
        break;
      case MK_ATTN_COMBINE: attn_combine_op(c, tag(oi)); break;
      case MK_ALLREDUCE:
        ++ar_i;
        allreduce_op(c, op, seq0 + ar_i, tag(oi), tag(op.res_op));
        break;
      case MK_ARGMAX:
        argmax_final_op(c, reinterpret_cast<float *>(xq), pos0, base_rounds + rounds, seq0 + ar_i, ebase + p.nops);
        break;
    }
    if (op.kind == MK_MATVEC && op.track_argmax) {
      // per-CTA arg-max candidate: every epilogue thread holds the best of its rows
      Best bb = best;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bb.v, o);
        const uint32_t oi2 = __shfl_xor_sync(0xffffffffu, bb.i, o);
        if (oi2 != 0xffffffffu && better(ov, oi2, bb)) {
          bb.v = ov;
          bb.i = oi2;
        }
      }
      float *cand = ssum;  // [NCW] values, then [NCW] indices
      cons_sync();
      if ((threadIdx.x & 31) == 0) {
        cand[threadIdx.x >> 5] = bb.v;
        cand[NCW + (threadIdx.x >> 5)] = __uint_as_float(bb.i);
      }
      cons_sync();
      if (threadIdx.x == 0) {
        for (int w = 1; w < NCW; ++w) {
          const uint32_t wi = __float_as_uint(cand[NCW + w]);
          if (wi != 0xffffffffu && better(cand[w], wi, bb)) {
            bb.v = cand[w];
            bb.i = wi;
          }
        }
        p.arg_scratch[2 * blockIdx.x] = bb.v;
        p.arg_scratch[2 * blockIdx.x + 1] = __uint_as_float(bb.i);
      }
    }
    unsigned long long t1 = 0, t2 = 0;
    VKL_TRACE(4);
    if (timed) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    if (oi + 1 < p.nops) {
      // While waiting for the other CTAs: start what the next op will need from DRAM and does not depend
      // on this op's results. The 7 GB weight stream of a token flushes everything else out of L2 between
      // two uses, so the norm weights would otherwise sit, with a DRAM round trip, at the start of the next
      // op: this prefetch is worth 7 % of the token time.
      const MegaOp &nx = opbuf[(oi + 1) % 3];
      if (nx.kind == MK_MATVEC) {
        if (nx.norm_w)
          for (uint32_t i = threadIdx.x * 32; i < nx.K; i += CT * 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(nx.norm_w + i));
      }
      asm volatile("cp.async.wait_all;" ::: "memory");  // entry oi + 2 has landed; the barrier below publishes it
      if (op.barrier_after) {
        ++rounds;
        grid_barrier(c, (base_rounds + rounds) * G, (uint32_t)rounds, abort_s + 1);
      } else {
        cons_sync();  // the next op reuses this one's shared memory; its input words carry their own arrival tags
      }
    }
    VKL_TRACE(5);
    if (timed) {
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t2));
      p.timing[2 * oi] = t1 - t0;
      p.timing[2 * oi + 1] = t2 - t1;
      const unsigned long long cend = clock64();
      p.timing[2 * p.nops + oi] = (p.timing_mode & 8u) ? (twait[2] ? (cend - twait[2]) * 1000ull / p.sm_mhz - (t2 - t1) : 0ull)
                                  : getenv_prologue(p) ? (twait[1] > c0 ? (twait[1] - c0) * 1000ull / p.sm_mhz : 0ull)
                                                        : twait[0];
      twait[2] = 0;
      twait[0] = 0;
      twait[1] = 0;
      t0 = t2;
    }
  }
}

}  // namespace

size_t decode_mega_xs_bytes(uint32_t max_blocks, uint32_t head_dim, uint32_t maxlen, uint32_t splits, uint32_t split_rows) {
  size_t x = (size_t)max_blocks * (XB_BYTES + 4);  // fp16 input + one fp32 bias term per block of 32 inputs
  // most rows a split can get: all splits at the full context, or one of fewer splits of split_rows rows
  uint32_t chunk = ((maxlen + splits - 1) / splits + 31) & ~31u;
  if (split_rows) chunk = std::max(chunk, (std::min(maxlen, split_rows) + 31) & ~31u);
  size_t a = (size_t)((3 + NCW / 2) * head_dim + 2 * NCW + 32 + chunk + 32) * 4;
  size_t b = x > a ? x : a;
  return (b + 127) / 128 * 128;
}
size_t decode_mega_smem(size_t xs_bytes, uint32_t nst, uint32_t red_slots) {
  return (size_t)nst * STAGE_BYTES + xs_bytes + ((size_t)red_slots * NCW * 32 + 68) * 4 + 128 * sizeof(MegaStage) + 2 * MAX_NST * 8 + 16 + 3 * sizeof(MegaOp) + 64;
}
int decode_mega_max_k() { return 16384; }
int decode_mega_max_stages() { return MAX_NST; }

// Packs the op's matrices from the library's tiled planes (common.cuh) into the stream layout of
// MegaOp: one CTA per (block, tile), one thread per 16-byte piece. A 32-row tile's unit is the two
// 512-byte (16 rows x 32 columns) units of the planes that hold its rows, unchanged (codes stay
// biased by +128 in MMA fragment order), followed by the 32 scales in the order the consumer lanes
// read them. Tiles are stored in the order the decode kernel's CTAs take them (mega_stream_tile), so
// that every CTA reads one consecutive range of the op.
namespace {
__global__ void __launch_bounds__(64) mega_pack_kernel(const uint8_t *p0, const uint8_t *p1, const uint8_t *p2, uint32_t nmat, int swiglu, uint32_t N,
                                                       uint32_t K, uint32_t tiles, uint32_t grid, uint8_t *stream) {
  const uint32_t b = blockIdx.x, t = blockIdx.y, blocks = K / 32;
  const uint32_t half = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t tpm = (N + 31) / 32;
  // the 16-row plane tile behind this half of the 32-row tile
  uint32_t m, tile16;
  if (swiglu) {
    m = half;  // gate rows 16 t .., then up rows 16 t ..
    tile16 = t;
  } else if (nmat == 3) {
    m = t / tpm;
    tile16 = (t % tpm) * 2 + half;
  } else {
    m = 0;
    tile16 = t * 2 + half;
  }
  const uint8_t *src = m == 0 ? p0 : m == 1 ? p1 : p2;
  const Q8Layout L = q8_layout(N, K);
  const bool in = tile16 < L.tiles;
  uint4 w = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);  // code 0, biased
  if (in) w = *reinterpret_cast<const uint4 *>(src + (((size_t)tile16 * L.groups * 4 + b) * 32 + lane) * 16);
  const size_t unit = (size_t)mega_stream_tile(t, tiles, grid) * blocks + b;
  uint8_t *dst = stream + unit * (MEGA_UNIT_CODES + MEGA_UNIT_SCALES);
  reinterpret_cast<uint4 *>(dst)[half * 32 + lane] = w;
  if (lane < 16) {
    // scales of the unit: [g][row g | g + 8 of half 0, row g | g + 8 of half 1] as fp16
    const uint32_t g = lane & 7, up8 = lane >> 3;
    unsigned short d = 0;
    if (in) {
      const unsigned short *sc = reinterpret_cast<const unsigned short *>(src + L.codes_bytes());
      d = sc[(((size_t)tile16 * L.groups + (b >> 2)) * 8 + g) * 8 + up8 * 4 + (b & 3)];
    }
    reinterpret_cast<unsigned short *>(dst + MEGA_UNIT_CODES)[g * 4 + half * 2 + up8] = d;
  }
}
}  // namespace

cudaError_t launch_mega_pack(const uint8_t *const planes[3], uint32_t nmat, int swiglu, uint32_t N, uint32_t K, uint32_t tiles, uint32_t grid,
                             uint8_t *stream, cudaStream_t s) {
  if (K % 32 || tiles == 0 || tiles > 65535u || grid == 0) return cudaErrorInvalidValue;
  mega_pack_kernel<<<dim3(K / 32, tiles), 64, 0, s>>>(planes[0], planes[1], planes[2], nmat, swiglu, N, K, tiles, grid, stream);
  return cudaGetLastError();
}

cudaError_t launch_decode_mega(const MegaParams &p, int grid, cudaStream_t s) {
  if (p.nst < 2 || p.nst > (uint32_t)MAX_NST) return cudaErrorInvalidValue;
  const size_t smem = decode_mega_smem(p.xs_bytes, p.nst, p.red_slots);
  // the diagnostic switches (no weight copies, no arithmetic) are compiled into separate instances
  const bool dbg = (p.timing_mode & (2u | 4u | 16u | 64u | 128u)) != 0;  // (16: the diagnostic instance with nothing switched off, its own baseline)
  auto kern = p.timing ? decode_mega_kernel<true, true> : dbg ? decode_mega_kernel<false, true> : decode_mega_kernel<false, false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  void *args[] = {(void *)&p};
  return cudaLaunchCooperativeKernel((void *)kern, dim3(grid), dim3(THREADS), args, smem, s);
}

cudaError_t decode_mega_occupancy(size_t smem, int *blocks_per_sm) {
  cudaError_t e = cudaFuncSetAttribute(decode_mega_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  return cudaOccupancyMaxActiveBlocksPerMultiprocessor(blocks_per_sm, decode_mega_kernel<false, false>, THREADS, smem);
}

}  // namespace vkl
