// Host-callable launchers of every CUDA kernel in the library. All pointers are
// device pointers; every launcher enqueues on `stream` and returns the CUDA
// error of the launch (no synchronisation).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace vkl {

// EPI_PARTIAL (persistent decode kernel only): raw fp32 partial sums of a row-split
// projection, pushed into every tensor-parallel rank's exchange buffer.
// EPI_REDUCE (persistent decode kernel only): the same, and the thread that pushed a row's partial sum also
// waits for the other ranks' sums of that row, adds them in rank order with the residual and publishes the row:
// the all-reduce needs no op of its own.
enum MvEpilogue { EPI_PLAIN = 0, EPI_ADD = 1, EPI_SWIGLU = 2, EPI_PARTIAL = 3, EPI_REDUCE = 4 };

// Y = epilogue(X . W^T) for up to three Q8_0 (tiled planes) or FP16 (row-major)
// weight matrices [N,K] sharing one input X [M,K].
struct MvParams {
  const uint8_t *codes[3];   // Q8_0: codes plane; FP16: row-major weights
  const uint8_t *scales[3];  // Q8_0: scales plane; FP16: unused
  __half *out[3];            // fp16 [M, out_ld] per matrix (SWIGLU: out[0] only)
  float *out_f32;            // optional fp32 copy of out[0] (cast of the fp16 value)
  const __half *x;           // [M, x_ld]
  const __half *residual;    // EPI_ADD: [M, out_ld], may alias out[0]
  const float *norm_w;       // fused RMSNorm weight [K] (decode path), or null
  float eps;
  uint32_t nmat;             // 1..3 matrices (SWIGLU: codes[0]=gate, codes[1]=up, nmat=1)
  uint32_t N, K, M;
  uint32_t x_ld, out_ld;
  float scale, bias;
  int act;                   // 1 = SiLU on the PLAIN epilogue
  int fp16_weights;          // 0 = Q8_0 tiled planes, 1 = FP16 row-major
  int use_pdl;               // programmatic dependent launch: prefetch weights before waiting
};
cudaError_t launch_matvec(const MvParams &p, int epilogue, bool fuse_norm_smem, cudaStream_t s);

// 34-byte GGUF blocks <-> tiled planes (codes at dst, scales at dst + codes_bytes).
cudaError_t launch_q8_repack(const uint8_t *blocks34, uint8_t *planes, uint32_t N, uint32_t K,
                             cudaStream_t s);
cudaError_t launch_q8_unpack(const uint8_t *planes, uint8_t *blocks34, uint32_t N, uint32_t K,
                             cudaStream_t s);
// fp32 [N,K] -> 34-byte blocks on the device (same arithmetic as the host quantizer).
cudaError_t launch_q8_quantize(const float *src, uint8_t *blocks34, uint32_t N, uint32_t K,
                               cudaStream_t s);
// Seeded synthetic data, bit-identical to the host generator.
cudaError_t launch_synth_f32(float *dst, uint64_t seed, uint64_t tensor, uint64_t first,
                             uint64_t n, float mean, float stdv, cudaStream_t s);
cudaError_t launch_synth_f16(__half *dst, uint64_t seed, uint64_t tensor, uint64_t first,
                             uint64_t n, float mean, float stdv, cudaStream_t s);
// Synthetic N(mean,std) matrix quantised straight into 34-byte blocks. The [N,K]
// result is the window at (row0, col0) of a full matrix with `ld_full` columns
// (element index = (row0+r)*ld_full + col0 + k), so a shard equals a slice.
cudaError_t launch_synth_q8(uint8_t *blocks34, uint64_t seed, uint64_t tensor, uint32_t N,
                            uint32_t K, float mean, float stdv, uint32_t row0, uint32_t col0,
                            uint32_t ld_full, cudaStream_t s);

cudaError_t launch_rms_norm(const __half *x, const float *w, __half *y, uint32_t rows,
                            uint32_t W, float eps, cudaStream_t s);
cudaError_t launch_add(const __half *x, __half *y, uint64_t n, int op, cudaStream_t s);
// x <- fp16(x op alpha), op 0 add, 1 sub, 2 mul, 3 div.
cudaError_t launch_scalar_op(__half *x, uint64_t n, int op, float alpha, cudaStream_t s);
// Copies a dense [C,H,W] input to out[c * ocs + h * ohs + w + offset] (element strides).
cudaError_t launch_concat_copy(const __half *in, __half *out, uint32_t C, uint32_t H, uint32_t W, uint64_t ocs, uint64_t ohs, uint64_t offset,
                               cudaStream_t s);
// Row reduction over W: op 0 sum, 1 max, 2 min; the result is scaled by mean_scale.
cudaError_t launch_reduce(const __half *in, __half *out, uint32_t rows, uint32_t W, int op, float mean_scale, cudaStream_t s);
// out[c, y, :] = cache[c, (y + offset) % H, :] for y < len.
cudaError_t launch_read_kvcache(const __half *cache, __half *out, uint32_t C, uint32_t H, uint32_t W, uint32_t offset, uint32_t len,
                                cudaStream_t s);
// All-reduce of fp32 partial sums [n] over tensor-parallel ranks with the residual add of the K-split
// projections: x = fp16(fp16(sum over ranks, in rank order) + x). part[r] / flags[r] are rank r's partial
// sums and flag words [tp] (peer mappings; [rank] is this GPU's). A wait that runs out of `wait_limit`
// polls stores 16 into *error and leaves x as it was.
struct TpRowsParams {
  const float *part[8];
  uint32_t *flags[8];
  __half *x;
  size_t n;
  uint32_t rank, tp, seq, wait_limit;
  uint32_t *error;
};
cudaError_t launch_tp_reduce_rows(const TpRowsParams &p, int sms, cudaStream_t s);
cudaError_t launch_embedding(const uint8_t *vocab, int vocab_is_q8, const uint32_t *ids,
                             __half *out, uint32_t T, uint32_t VH, uint32_t VW, uint32_t unk,
                             cudaStream_t s);
// Two-stage arg-max/min over rows of width W; partials needs rows*ceil(W/1024)*8 bytes.
cudaError_t launch_argop(const __half *x, uint32_t *out, void *partials, uint32_t rows,
                         uint32_t W, int op_type, cudaStream_t s);
size_t argop_partials_bytes(uint32_t rows, uint32_t W);
// The k largest of n fp32 values and their indices, descending (equal values: lowest index first).
cudaError_t launch_topk_f32(const float *x, uint32_t n, uint32_t k, float *vals, uint32_t *ids, cudaStream_t s);
cudaError_t launch_softmax(const __half *in, __half *out, uint32_t C, uint32_t H, uint32_t W,
                           int seq_mask, uint32_t offset, cudaStream_t s);
cudaError_t launch_rope(__half *x, uint32_t C, uint32_t H, uint32_t W, uint64_t cs, uint64_t hs,
                        const uint32_t *pos_dev, uint32_t offset, const float *freqc,
                        const float *freqs, cudaStream_t s);
cudaError_t launch_update_kvcache(__half *cache, const __half *kv, uint32_t C, uint32_t H,
                                  uint32_t W, uint32_t HO, uint32_t WO, uint32_t offset,
                                  cudaStream_t s);
cudaError_t launch_transpose(const __half *in, __half *out, uint32_t C, uint32_t H, uint32_t W,
                             cudaStream_t s);
cudaError_t launch_slice(const __half *in, __half *out, uint32_t C, uint32_t H, uint32_t W,
                         uint32_t c0, uint32_t h0, uint32_t w0, uint32_t EC, uint32_t EH,
                         uint32_t EW, cudaStream_t s);
cudaError_t launch_cast_f16_f32(const __half *in, float *out, uint64_t n, cudaStream_t s);
cudaError_t launch_cast_f32_f16(const float *in, __half *out, uint64_t n, cudaStream_t s);
// Batched fp16 x fp16 matmul with element strides; transpose_b selects A.B^T.
cudaError_t launch_bmm_f16(const __half *a, const __half *b, __half *c, uint32_t C, uint32_t M,
                           uint32_t N, uint32_t K, uint64_t a_cs, uint64_t a_hs, uint64_t b_cs,
                           uint64_t b_hs, uint64_t c_cs, uint64_t c_hs, int transpose_b,
                           float scale, float bias, int act, cudaStream_t s);

// Fused attention core for the model path. q,k,v: [T, heads*dim] fresh projections.
// Rotates q and k at positions pos+row, appends k,v to the caches [heads,maxlen,dim]
// at (pos+row) % maxlen, then softmax(q.K^T/sqrt(dim)).V over the first
// min(pos+T, maxlen) cache rows with the causal mask; out: [T, heads*dim].
struct AttnParams {
  __half *q;
  const __half *k, *v;
  __half *kcache, *vcache;
  __half *out;
  const float *freqc, *freqs;
  const uint32_t *pos_dev;  // position of row 0, read on the device
  float *scratch;           // splits*T*heads*(dim+2) floats
  uint32_t *counters;       // T*heads, zero before first use (left zero after)
  uint32_t T, heads, dim, maxlen, splits;
  // clip: only the last row is computed and written to row 0 of `out`; its query is
  // rotated at position pos (row 0), as the reference does after clipping Q
  // (src/ops/multiheadattention_v2.cpp:223-253).
  int clip;
  int use_pdl;
};
cudaError_t launch_attention(const AttnParams &p, cudaStream_t s);
size_t attention_scratch_bytes(uint32_t T, uint32_t heads, uint32_t dim, uint32_t splits);

// ---- persistent decode step (decode_mega.cu) --------------------------------
enum MegaKind { MK_EMBED = 0, MK_MATVEC = 1, MK_ATTN_PART = 2, MK_ATTN_COMBINE = 3, MK_ARGMAX = 4, MK_ALLREDUCE = 5 };
// One entry of the token's op table. The kernel keeps the current and the next entry in shared
// memory (copied there with 16-byte asynchronous copies while the op before runs), so the size
// is a multiple of 16 bytes.
struct alignas(16) MegaOp {
  uint32_t kind, epi, nmat, rot;
  uint32_t N, K;          // rows of one matrix, columns
  uint32_t tiles, blocks; // 32-row tiles of the op's packed weight stream, Q8_0 blocks per row (K / 32)
  // The op's weights, packed for the kernel (mega_pack): per 32-row tile and block one unit of
  // MEGA_UNIT_CODES + MEGA_UNIT_SCALES bytes. Codes: the two 512-byte (16 rows x 32 columns) units of the
  // library's tiled planes (common.cuh) that hold the tile's rows, as they are: MMA A-fragment order, biased
  // by +128. Then the unit's scales: [g 0..7][rows g, g + 8, 16 + g, 24 + g] fp16. Units of a tile follow each
  // other block by block, tiles in the order of mega_stream_tile: everything one CTA reads of the op is one
  // consecutive range. Which matrix row a tile row is:
  //   one matrix         tile t, row r = matrix row 32 t + r
  //   nmat = 3 (K, Q, V) tile t = matrix t / tpm, rows 32 (t % tpm) + r, tpm = ceil(N / 32)
  //   SwiGLU (gate, up)  tile t: rows 0..15 = gate rows 16 t + r, rows 16..31 = up rows 16 t + r - 16
  const uint8_t *codes;
  const float *norm_w;  // fused RMSNorm of the input, or null
  float eps;
  uint32_t track_argmax;  // lm head: keep a per-CTA (max, index) candidate
  const uint32_t *stages_per_cta;  // [grid]: ring stages of this op per CTA
  // Activations that cross CTAs inside a token live in "tagged" buffers: one 32-bit word per
  // element, fp16 value in the low half and the low 16 bits of the producing op's sequence
  // number in the high half. A reader that knows which op produced its input polls the words
  // until every tag matches: the data is its own arrival flag, so most ops need no grid barrier.
  const uint32_t *in;     // input vector [K], tagged words
  uint32_t src_op;        // index of the op that produced `in` (MK_ATTN_PART: of the op that produced q, k, v)
  uint32_t tag_op;        // index of the op whose tag this op's tagged results carry (its own, unless a skipped op is expected)
  uint32_t res_op;        // residual add (and all-reduce): index of the op that last wrote out_ll[0], whose tag the residual words carry
  uint32_t barrier_after; // a grid barrier follows this op (its results are not tagged, or the next op needs one)
  uint32_t *out_ll[3];    // tagged outputs; EPI_ADD: out_ll[0] is also the residual
  __half *out[3];         // plain fp16 outputs (lm head)
  float *out_f32;
  __half *kcache, *vcache;  // MK_ATTN_PART
};
// One ring stage of the persistent kernel: up to MEGA_SU consecutive units (one Q8_0 block x
// 32 rows each) of a CTA's weight stream, one range of memory: the tail of one tile (n0 units)
// and, when that ends inside the stage, the head of the CTA's next tile (n1 units).
//
// An entry with n0 == MEGA_KV_MARK stands for the K and V rows of an attention op instead:
// src / src2 are the layer's K / V cache. How many ring stages it becomes depends on the
// token's KV length: producer and consumers both derive this CTA's (head, split) row range from
// the position and cut it into stages of mega_kv_rows_per_stage() rows, all K stages first.
struct MegaStage {
  const uint8_t *src, *src2;
  uint32_t n0, n1;  // units of the first and of the second tile
  uint32_t tm, kg;  // consumers' view: local tile and first block of the n0 units; the n1 units start at block 0 of local tile tm + 1
};
constexpr uint32_t MEGA_KV_MARK = 0xffffffffu;
// Where tile t of an op (of `tiles` tiles, dealt to a grid of `grid` CTAs as tile0 + lt * grid) sits in the
// op's weight stream: the tiles of one CTA are consecutive, CTAs in the order of their first tile.
__host__ __device__ inline uint32_t mega_stream_tile(uint32_t t, uint32_t tiles, uint32_t grid) {
  const uint32_t tile0 = t % grid, lt = t / grid, q = tiles / grid, r = tiles % grid;
  return tile0 * q + (tile0 < r ? tile0 : r) + lt;
}
constexpr uint32_t MEGA_UNIT_CODES = 1024, MEGA_UNIT_SCALES = 64;  // 32 rows x 32 codes, 32 fp16 scales
#ifndef VKL_MEGA_UPW
#define VKL_MEGA_UPW 2
#endif
constexpr uint32_t MEGA_UPW = VKL_MEGA_UPW;       // units per consumer warp and stage
#ifndef VKL_MEGA_NCW
#define VKL_MEGA_NCW 11
#endif
constexpr uint32_t MEGA_NCW = VKL_MEGA_NCW;       // consumer warps of the kernel
constexpr uint32_t MEGA_SU = MEGA_NCW * MEGA_UPW; // units per stage
constexpr uint32_t MEGA_STAGE_BYTES = MEGA_SU * (MEGA_UNIT_CODES + MEGA_UNIT_SCALES);
// Cache rows (head_dim fp16 values each) of one KV ring stage: whole rows, a multiple of 8.
__host__ __device__ inline uint32_t mega_kv_rows_per_stage(uint32_t head_dim) { return (MEGA_STAGE_BYTES / (head_dim * 2u)) & ~7u; }
// Splits per head at KV length L: as few as keep a split within `split_rows` cache rows. With one
// split a head needs no merge step between CTAs; more splits only pay when the rows of a head no
// longer stream through one SM fast enough.
__host__ __device__ inline uint32_t mega_splits(uint32_t L, uint32_t splits, uint32_t split_rows) {
  if (!split_rows) return splits;
  const uint32_t want = (L + split_rows - 1) / split_rows;
  return want < 1 ? 1u : (want < splits ? want : splits);
}
// The cached rows [c0, c1) that split `split` of `S` reads at KV length L.
__host__ __device__ inline void mega_kv_range(uint32_t L, uint32_t S, uint32_t split, uint32_t &c0, uint32_t &c1) {
  uint32_t chunk = (L + S - 1) / S;
  chunk = (chunk + 31) & ~31u;
  c0 = split * chunk < L ? split * chunk : L;
  c1 = c0 + chunk < L ? c0 + chunk : L;
}
// How a stage that starts at block `kg` of a tile of `blocks` blocks is cut: n0 units of this
// tile, then n1 of the next one (if the op has one for this CTA). Host and device walk the
// stream with the same rule.
struct MegaCut {
  uint32_t n0, n1;
};
__host__ __device__ inline MegaCut mega_stage_cut(uint32_t kg, uint32_t blocks, bool has_next) {
  MegaCut c;
  c.n0 = blocks - kg < MEGA_SU ? blocks - kg : MEGA_SU;
  const uint32_t rem = MEGA_SU - c.n0;
  c.n1 = has_next ? (rem < blocks ? rem : blocks) : 0u;
  return c;
}
__host__ __device__ inline void mega_stage_advance(const MegaCut &c, uint32_t blocks, uint32_t &tm, uint32_t &kg) {
  if (c.n1) {
    tm += 1;
    kg = c.n1;
  } else {
    kg += c.n0;
  }
  if (kg >= blocks) {
    kg = 0;
    tm += 1;
  }
}
struct MegaParams {
  const MegaOp *ops;
  const MegaStage *stages;       // [grid][stage_stride]: every CTA's stages in consumer order
  const uint32_t *stage_count;   // [grid]
  uint32_t stage_stride;
  uint32_t nops, nbarriers;
  uint32_t *state;    // [0] position, [1] step, [2] picked id, [3] all-reduces done, [4] arg-max exchanges done,
                      // [5] number of forced (prompt) tokens, [6] prefill GEMM error, [7] sequence number of the next launch's first op
  const uint32_t *forced;  // prompt ids: while position+1 < state[5] the next input is forced[position+1]
  uint32_t *tok;      // current token id
  uint32_t *out_ids;
  uint32_t out_cap;
  const uint8_t *embd;  // token embedding, Q8_0 tiled planes
  uint32_t embd_rows;
  uint32_t *x, *q, *k, *v, *ao;  // tagged words (see MegaOp)
  const float *freqc, *freqs;
  float *attn_scratch;      // heads*splits*(head_dim+4): per (head, split) the un-normalised P.V row, its max and its sum
  uint32_t attn_merge;      // how a head's split partials are merged: 0 combine op, 1 last-arriving split
  uint32_t *attn_counters;  // [heads] arrivals of a head's splits (the last one merges them), or null: separate combine op
  float *arg_scratch;       // grid*2
  unsigned long long *bar;  // [0] arrivals, [1] completed launches
  uint32_t *error;          // 0, or the code of the wait that timed out
  uint32_t dim, heads, head_dim, maxlen, splits, vocab;
  uint32_t xs_bytes;
  uint32_t xmax_blocks;  // largest K of any op, in blocks of 32 inputs: the input area holds that many blocks of digits
  // Tensor parallelism: every rank's exchange buffer (peer pointers, own included).
  // Layout of one buffer, in 4-byte words: partial sums [2 parities][tp][dim] x {fp32 sum, sequence number}, then
  // at word tp_flag_off: flags[16] (all-reduce sequence per source rank), arg flags[16],
  // arg candidates [16][2].
  uint32_t tp_rank, tp_size, tp_flag_off;
  void *tp_peer[8];
  uint32_t nst;               // ring stages (as many as fit beside the input and reduction areas)
  uint32_t red_slots;         // reduction slots: the most tiles one CTA gets of any op
  uint32_t split_rows;        // cache rows one attention split should hold: a token at KV length L uses min(splits, ceil(L / split_rows)) splits per head (0: always `splits`)
  uint32_t barrier_pollers;   // warps whose lane 0 polls the grid barrier counter, staggered in time
  // Optional timeline of CTA 0: per op, nanoseconds of work and of barrier wait.
  unsigned long long *timing;
  uint32_t timing_mode;  // third column of the timeline: 0 = ring wait, 1 = op prologue
  uint32_t sm_mhz;       // SM clock for the timeline's cycle counts (measured by the host before a profiled launch)
  uint32_t wait_limit;   // polls after which any wait of the kernel gives up and raises *error
};
size_t decode_mega_xs_bytes(uint32_t max_blocks, uint32_t head_dim, uint32_t maxlen, uint32_t splits, uint32_t split_rows);
// Packs up to three Q8_0 matrices (tiled planes) that share an input into one op's weight stream
// (layout and row rules at MegaOp). tiles = the stream's 32-row tiles.
cudaError_t launch_mega_pack(const uint8_t *const planes[3], uint32_t nmat, int swiglu, uint32_t N, uint32_t K, uint32_t tiles,
                             uint32_t grid, uint8_t *stream, cudaStream_t s);
size_t decode_mega_smem(size_t xs_bytes, uint32_t nst, uint32_t red_slots);
int decode_mega_max_k();
int decode_mega_max_stages();
cudaError_t decode_mega_occupancy(size_t smem_bytes, int *blocks_per_sm);
cudaError_t launch_decode_mega(const MegaParams &p, int grid, cudaStream_t s);

// ---- dense FP16 GEMM on tcgen05 tensor cores: C[M,N] = A[M,K] . W[N,K]^T (gemm_tcgen05.cu) ----
struct GemmParams {
  const __half *a;         // [M,K] row-major
  const __half *w;         // [N,K] row-major (a transposed-weight matrix of the reference); FP16 weights
  const uint8_t *w_codes;  // Q8_0 weights [N,K] as tiled planes (common.cuh): codes ...
  const uint8_t *w_scales; // ... and scales
  __half *c;               // [M,N] fp16 output, or nullptr when c_f32 is set
  float *c_f32;            // raw fp32 output (for the fused SwiGLU step)
  const __half *residual;  // optional [M,N]: c = fp16(fp16(acc) + residual)
  uint32_t *error;         // device word raised when a bounded wait ran out
  uint32_t M, N, K;
  float scale, bias;       // MatMul's scale and bias (mat_mul.cpp:39-41)
  int act;                 // 0 none, 1 SiLU
};
constexpr uint32_t GEMM_MIN_ROWS = 32;  // below this the weight-streaming mat-vec kernel is used
bool gemm_tcgen05_supported(uint32_t M, uint32_t N, uint32_t K);
cudaError_t launch_gemm_f16_tcgen05(const GemmParams &p, cudaStream_t s);
// The same GEMM with Q8_0 weights (w_codes / w_scales), dequantised into the shared-memory tiles.
constexpr uint32_t GEMM_Q8_MIN_ROWS = 64;  // below this the rows-at-a-time kernel keeps the exact fp32 scaling
cudaError_t launch_gemm_q8_tcgen05(const GemmParams &p, cudaStream_t s);
// Rows from which a weight of this kind goes to the tensor-core GEMM.
inline uint32_t gemm_min_rows(bool q8) { return q8 ? GEMM_Q8_MIN_ROWS : GEMM_MIN_ROWS; }
// Dispatch on the weight kind: w set = FP16 weights, else w_codes / w_scales = Q8_0.
inline cudaError_t launch_gemm_tcgen05(const GemmParams &p, cudaStream_t s) { return p.w ? launch_gemm_f16_tcgen05(p, s) : launch_gemm_q8_tcgen05(p, s); }
cudaError_t launch_swiglu_f32(const float *gate, const float *up, __half *out, size_t n, cudaStream_t s);

}  // namespace vkl
