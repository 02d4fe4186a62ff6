// Shared device helpers and the private Q8_0 device layout.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace vkl {

// ---------------------------------------------------------------------------
// Private device layout of a Q8_0 matrix [N rows, K cols] ("tiled planes").
//
// The API format stays the 34-byte GGUF block (fp16 scale + 32 int8), as the
// reference's shaders read it (src/shaders/common.h:8-10). At upload the
// blocks are split into two planes, byte-for-byte the same information:
//
//   codes : [row_tile][block][lane 0..31][16 B]; a row tile is 16 rows, a
//           block is 32 columns. lane = g*4 + t holds, biased by +128 to
//           unsigned, the 8 codes of row 16*tile+g   at k = 32*b + 8*t..+7
//           followed by the 8 codes of row 16*tile+g+8 at the same k.
//           Inside every 32-bit word the four codes c0..c3 sit as bytes
//           [c0, c2, c1, c3], so `w & 0x00ff00ff` and `(w >> 8) & 0x00ff00ff`
//           are the code pairs (c0,c1) and (c2,c3) in the two 16-bit lanes:
//           one logic op each turns them into fp16 pairs (byte permutes run on
//           the slow conversion pipe of this GPU and are avoided).
//           That is exactly the A fragment of two m16n8k16 MMAs, so one
//           coalesced 128-bit load per lane feeds the tensor core.
//   scales: [row_tile][group of 4 blocks][g 0..7][8 halves]: the fp16 scales
//           of row g for blocks 4*grp..4*grp+3, then those of row g+8.
//
// Rows beyond N and blocks beyond ceil(K/32) are padded with code 0 / scale 0.
// ---------------------------------------------------------------------------
struct Q8Layout {
  uint32_t N, K;
  uint32_t tiles;   // ceil(N/16)
  uint32_t blocks;  // ceil(K/32)
  uint32_t groups;  // ceil(blocks/4)
  __host__ __device__ size_t codes_bytes() const { return (size_t)tiles * groups * 4 * 512; }
  __host__ __device__ size_t scales_bytes() const { return (size_t)tiles * groups * 128; }
  __host__ __device__ size_t total_bytes() const { return codes_bytes() + scales_bytes(); }
};

inline __host__ __device__ Q8Layout q8_layout(uint32_t N, uint32_t K) {
  Q8Layout l;
  l.N = N;
  l.K = K;
  l.tiles = (N + 15) / 16;
  l.blocks = (K + 31) / 32;
  l.groups = (l.blocks + 3) / 4;
  return l;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Round to fp16 (nearest even) and back: the reference's op-boundary rounding.
__device__ __forceinline__ float round_h(float v) { return __half2float(__float2half_rn(v)); }

// 128-bit streaming load that does not pollute L1 (weights are read once).
__device__ __forceinline__ uint4 ldg_stream(const void *p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Byte position of code i (0..7) inside the 8-byte run of one row (see Q8Layout).
__host__ __device__ inline uint32_t q8_byte_pos(uint32_t i) {
  const uint32_t k = i & 3;
  return (i & 4) + (k == 1 ? 2 : k == 2 ? 1 : k);
}

// Code pair (c0,c1) [hi = false] or (c2,c3) [hi = true] of a layout word as the
// fp16 pair (1024+u, 1024+u'): 0x6400 | u is the half 1024+u, exactly.
__device__ __forceinline__ uint32_t codes_raw_h2(uint32_t w, bool hi) {
  // one logic op for the low pair, one byte permute for the high pair
  return hi ? __byte_perm(w, 0x64646464u, 0x4341) : ((w & 0x00ff00ffu) | 0x64006400u);
}

// Same pair with the +128 bias and the 1024 removed: the signed codes as fp16, exact.
__device__ __forceinline__ uint32_t codes_to_h2(uint32_t w, bool hi) {
  const uint32_t p = codes_raw_h2(w, hi);
  const __half2 bias = __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480));
  __half2 r = __hsub2(*reinterpret_cast<const __half2 *>(&p), bias);
  return *reinterpret_cast<uint32_t *>(&r);
}

}  // namespace vkl
