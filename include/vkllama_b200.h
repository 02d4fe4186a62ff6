/* C ABI of the B200 implementation of vkllama's Llama-2 token loop.
 *
 * Every entry point is plain C: opaque handles, pointers, sizes. Functions
 * return a status code (0 = OK; the other values are absl::StatusCode numbers,
 * which is what the reference's ops return) and leave a message retrievable
 * with vkl_last_error() on the calling thread. Nothing throws across this
 * boundary. Citations name the reference interface each group replaces, by its
 * path inside the vkllama tree.
 *
 * Execution model (reference: src/core/command.h:26-483): ops only enqueue
 * work on their command's CUDA stream between vkl_command_begin() and
 * vkl_command_end(); results and host copies are valid after
 * vkl_command_wait(). Callers are single-threaded per command, as in the
 * reference. A CUDA device is required: there is no CPU fallback.
 */
#ifndef VKLLAMA_B200_H_
#define VKLLAMA_B200_H_
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct vkl_device vkl_device;
typedef struct vkl_tensor vkl_tensor;
typedef struct vkl_command vkl_command;
typedef struct vkl_op vkl_op;
typedef struct vkl_model vkl_model;
typedef struct vkl_gguf vkl_gguf;
typedef struct vkl_sampler vkl_sampler;

/* src/core/common.h:15-22 (enum DType), same numeric values. */
enum vkl_dtype { VKL_FP32 = 0, VKL_FP16 = 1, VKL_UINT32 = 2, VKL_INT8 = 3, VKL_Q8_0 = 4 };

/* absl::StatusCode values used by the reference's ops. */
enum vkl_status {
  VKL_OK = 0,
  VKL_INVALID_ARGUMENT = 3,
  VKL_NOT_FOUND = 5,
  VKL_RESOURCE_EXHAUSTED = 8,
  VKL_FAILED_PRECONDITION = 9,
  VKL_OUT_OF_RANGE = 11,
  VKL_UNIMPLEMENTED = 12,
  VKL_INTERNAL = 13
};

const char *vkl_last_error(void);
/* Number of kernels this library has launched in the calling process. */
uint64_t vkl_kernel_launches(void);

/* ---- device: GPUDevice, src/core/gpu_device.h:13-62 ---------------------- */
int vkl_device_create(int ordinal, vkl_device **out);
int vkl_device_destroy(vkl_device *dev);
/* name: at least 256 bytes. */
int vkl_device_info(vkl_device *dev, char *name, int *sm_count, size_t *total_mem);
/* Bytes of released device memory the device keeps for reuse (the counterpart of VMA's
 * block pool behind src/core/tensor.cpp:112-156). A released block is handed out again
 * only after the work that was queued on the device's streams at release time has
 * finished; the pool holds at most an eighth of the device memory. */
int vkl_device_pool_bytes(vkl_device *dev, size_t *bytes);

/* ---- tensor: Tensor, src/core/tensor.h:16-90 ------------------------------
 * Shape [c,h,w], row-major, strides in bytes (tensor.cpp:248-258). A handle is
 * reference counted (tensor.cpp:38-84, 355-366); views share the buffer and
 * keep the parent's strides (tensor.cpp:294-302). Q8_0 tensors are uploaded
 * and downloaded as GGUF blocks (fp16 scale + 32 int8 = 34 bytes,
 * src/shaders/common.h:8-10); their device layout is private. */
int vkl_tensor_create(vkl_device *dev, int c, int h, int w, int dtype, vkl_tensor **out);
int vkl_tensor_retain(vkl_tensor *t);
int vkl_tensor_release(vkl_tensor *t);
int vkl_tensor_view(vkl_tensor *t, size_t c, size_t h, size_t w, vkl_tensor **out);
int vkl_tensor_reshape(vkl_tensor *t, size_t c, size_t h, size_t w);
/* out6: c, h, w, cs, hs, ws (ShapeConstant, common.h:24-27). */
int vkl_tensor_shape(vkl_tensor *t, uint32_t out6[6]);
int vkl_tensor_dtype(vkl_tensor *t, int *dtype);
/* Bytes a host copy of the tensor takes (Q8_0: 34 per block). */
int vkl_tensor_bytes(vkl_tensor *t, size_t *bytes);
/* Raw device pointer of element (0,0,0); for interop with a caller's CUDA code. */
int vkl_tensor_device_ptr(vkl_tensor *t, void **ptr);

/* ---- command: Command, src/core/command.h:26-483 ------------------------- */
int vkl_command_create(vkl_device *dev, vkl_command **out);
int vkl_command_destroy(vkl_command *cmd);
int vkl_command_begin(vkl_command *cmd);
int vkl_command_end(vkl_command *cmd);
int vkl_command_submit(vkl_command *cmd);
int vkl_command_wait(vkl_command *cmd);
int vkl_command_submit_and_wait(vkl_command *cmd);
/* Device time between begin() and end() of the last recording, valid after wait();
 * the per-command counterpart of the timestamp queries in command.h:353-370. */
int vkl_command_elapsed_us(vkl_command *cmd, float *usec);
/* upload_bytes / download (command.h:141-260): host memory is copied through
 * pinned staging; a download lands in `host` when vkl_command_wait returns. */
/* The CUDA stream (cudaStream_t) the command enqueues on: the counterpart of the
 * queue a Command submits to (command.h:42-44), for callers that mix their own CUDA
 * work or the no-allocation entry point below with this library's ops. */
int vkl_command_stream(vkl_command *cmd, void **cuda_stream);
int vkl_command_upload(vkl_command *cmd, const void *host, size_t bytes, vkl_tensor *to);
int vkl_command_download(vkl_command *cmd, vkl_tensor *from, void *host, size_t bytes);

/* ---- ops: class Op, src/ops/op.h:14-25 ------------------------------------
 * create = constructor, vkl_op_init = Op::init(), run = operator(), vkl_op_time
 * = Op::time() (device microseconds of the op's last run, valid after wait).
 * Output tensors are owned by the op and reused while the shape is unchanged
 * (e.g. mat_mul.cpp:189-194); *out is a borrowed handle, valid until the op
 * runs with another shape or is destroyed (retain it to keep it longer). */
int vkl_op_init(vkl_op *op);
int vkl_op_time(vkl_op *op, uint64_t *usec);
int vkl_op_destroy(vkl_op *op);

/* MatMul, src/ops/mat_mul.h:12-27. weight may be NULL (two-operand form). */
int vkl_matmul_create(vkl_device *dev, vkl_command *cmd, vkl_tensor *weight, float scale,
                      float bias, int act, int broadcast_type, int transpose_b, int a_dtype,
                      int b_dtype, vkl_op **out);
int vkl_matmul_run(vkl_op *op, vkl_tensor *a, vkl_tensor *b, vkl_tensor **out);
/* Benchmark helper (no counterpart in the reference, whose tests time one op call at a time):
 * records `reps` weight-form MatMul calls on `a`, rotating over `n_ops` ops (copies of one
 * weight matrix larger than L2 in total). With `us_per_launch` non-null the calls are captured
 * into a CUDA graph, run once to warm up and once between two events, and the mean device time
 * of one call is returned (the command must be recording and the ops must have run once before,
 * so that nothing is allocated during the capture). */
int vkl_matmul_run_many(vkl_op *const *ops, size_t n_ops, vkl_tensor *a, size_t reps, float *us_per_launch);

/* FeedForward, src/ops/feed_forward.h:17-22 (w1 = gate, w2 = down, w3 = up). */
int vkl_feed_forward_create(vkl_device *dev, vkl_command *cmd, vkl_tensor *w1, vkl_tensor *w2,
                            vkl_tensor *w3, int transposed_weight, int dtype, vkl_op **out);
int vkl_feed_forward_run(vkl_op *op, vkl_tensor *x, vkl_tensor **out);

/* MultiHeadAttentionV2, src/ops/multiheadattention_v2.h:25-35. */
int vkl_mha_create(vkl_device *dev, vkl_command *cmd, vkl_tensor *wk, vkl_tensor *wq,
                   vkl_tensor *wv, vkl_tensor *wo, int maxlen, int dim, int transposed_weight,
                   int dtype, int use_kvcache, int clip_output, vkl_op **out);
int vkl_mha_run(vkl_op *op, vkl_tensor *x, size_t offset, vkl_tensor **out);
/* The op's caches [heads, maxlen, dim] (kcache_/vcache_ members); borrowed. */
int vkl_mha_caches(vkl_op *op, vkl_tensor **kcache, vkl_tensor **vcache);

/* UpdateKVCache, src/ops/update_kv_cache.h:13-18. */
int vkl_update_kvcache_create(vkl_device *dev, vkl_command *cmd, int dtype, vkl_op **out);
int vkl_update_kvcache_run(vkl_op *op, vkl_tensor *cache, vkl_tensor *kv, uint32_t offset);

/* RMSNorm, src/ops/rms_norm.h:12-16 (weight must be FP32, rms_norm.cpp:33). */
int vkl_rms_norm_create(vkl_device *dev, vkl_command *cmd, vkl_tensor *weight, float eps,
                        int dtype, vkl_op **out);
int vkl_rms_norm_run(vkl_op *op, vkl_tensor *x, vkl_tensor **out);

/* Rope, src/ops/rope.h:15-21: rotates `q` in place and returns it. */
int vkl_rope_create(vkl_device *dev, vkl_command *cmd, int maxlen, int dim, int dtype,
                    vkl_op **out);
int vkl_rope_run(vkl_op *op, vkl_tensor *q, size_t offset, vkl_tensor **out);

/* Softmax, src/ops/softmax.h:14-18 (temp is stored and unused, as in the reference). */
int vkl_softmax_create(vkl_device *dev, vkl_command *cmd, int seq_mask, float temp, int dtype,
                       vkl_op **out);
int vkl_softmax_run(vkl_op *op, vkl_tensor *a, size_t offset, vkl_tensor **out);

/* ArgOp<op_type>, src/ops/argop.h:13-156 (0 = ArgMax, 1 = ArgMin); output UINT32 [c,h,1]. */
int vkl_argop_create(vkl_device *dev, vkl_command *cmd, int op_type, int dtype, vkl_op **out);
int vkl_argop_run(vkl_op *op, vkl_tensor *in, vkl_tensor **out);

/* Embedding, src/ops/embedding.h:13-18; indices UINT32 [1,H,W] -> FP16 [H,W,VW]. */
int vkl_embedding_create(vkl_device *dev, vkl_command *cmd, vkl_tensor *vocab, uint32_t unk,
                         int dtype, vkl_op **out);
int vkl_embedding_run(vkl_op *op, vkl_tensor *indices, vkl_tensor **out);

/* ElementWise, src/ops/elementwise.h:16-21: y <- x (type) y, type 0 add, 1 sub,
 * 2 mul, 3 div; written into and returning the second operand. */
int vkl_elementwise_create(vkl_device *dev, vkl_command *cmd, int type, int dtype, vkl_op **out);
int vkl_elementwise_run(vkl_op *op, vkl_tensor *x, vkl_tensor *y, vkl_tensor **out);
/* ElementWise::operator()(Tensor x, float y), src/ops/elementwise.cpp:104-133: x <- x (type) y
 * in place (fp32 arithmetic, one rounding to fp16), returning x. */
int vkl_elementwise_run_scalar(vkl_op *op, vkl_tensor *x, float y, vkl_tensor **out);

/* Concat, src/ops/concat.h:10-17: `num` fp16 inputs joined along axis 0 (channels), 1 (rows)
 * or 2 (columns); the other two extents must agree (concat.cpp:82-113). */
int vkl_concat_create(vkl_device *dev, vkl_command *cmd, int num, int axis, int dtype, vkl_op **out);
int vkl_concat_run(vkl_op *op, vkl_tensor *const *inputs, size_t n, vkl_tensor **out);

/* Reduce, src/ops/reduce.h:18-67: over the rows of an fp16 [c,h,w] tensor -> [c,h,1];
 * op_type 0 sum, 1 max, 2 min, 3 mean; fp32 accumulation, one rounding to fp16. */
int vkl_reduce_create(vkl_device *dev, vkl_command *cmd, int op_type, int dtype, vkl_op **out);
int vkl_reduce_run(vkl_op *op, vkl_tensor *a, vkl_tensor **out);

/* ReadKVCache, src/ops/read_kvcache_op.h:10-16: the `len` rows of a ring cache
 * [heads, maxlen, dim] starting at `offset` (row (offset + y) % maxlen) -> [heads, len, dim]. */
int vkl_read_kvcache_create(vkl_device *dev, vkl_command *cmd, vkl_op **out);
int vkl_read_kvcache_run(vkl_op *op, vkl_tensor *cache, uint32_t offset, uint32_t len, vkl_tensor **out);

/* Transpose (type 0: [C,H,W] -> [H,C,W]), src/ops/transpose.h:14-19. */
int vkl_transpose_create(vkl_device *dev, vkl_command *cmd, int type, int dtype, vkl_op **out);
int vkl_transpose_run(vkl_op *op, vkl_tensor *in, vkl_tensor **out);

/* Slice, src/ops/slice.h:13-18. */
int vkl_slice_create(vkl_device *dev, vkl_command *cmd, int dtype, vkl_op **out);
int vkl_slice_run(vkl_op *op, vkl_tensor *in, const uint32_t starts[3],
                  const uint32_t extents[3], vkl_tensor **out);

/* Cast, src/ops/cast.h:15-20 (FP16 -> FP32 and FP32 -> FP16). */
int vkl_cast_create(vkl_device *dev, vkl_command *cmd, int from, int to, vkl_op **out);
int vkl_cast_run(vkl_op *op, vkl_tensor *in, vkl_tensor **out);

/* Row arg-max that allocates nothing. No counterpart in the reference.
 * For callers that cannot allocate device memory where they need the greedy pick
 * (a serving loop that gave its memory budget out at start-up, code inside a stream
 * capture, a host runtime that forbids cudaMalloc after initialisation). x_fp16 is a
 * device pointer to rows*width fp16 values, out_idx a device pointer to `rows`
 * uint32; lowest index wins ties, as ArgMax. The scratch of the two-stage reduction
 * is a fixed 64 KiB array inside the library, resident on every GPU that loads it:
 * rows * ceil(width/1024) may not exceed 8192, larger inputs are refused with
 * VKL_OUT_OF_RANGE. The first call on a device looks the array's device address up;
 * make that first call before any stream capture. The device that owns x_fp16, out_idx
 * and the stream must be the current device on EVERY call (the address is looked up
 * for the current device); pointers of another device, or host pointers, are refused
 * with VKL_INVALID_ARGUMENT before anything is launched.
 * All calls share the array: calls that overlap on the GPU race and must be
 * serialised by the caller. Enqueues on cuda_stream (cudaStream_t, may be NULL) and
 * does not synchronise. */
int vkl_argmax_noalloc(const void *x_fp16, uint32_t rows, uint32_t width, uint32_t *out_idx, void *cuda_stream);

/* ---- host Q8_0 quantizer: src/core/quants.h:37-176 ------------------------
 * blocks34: GGUF/device layout [fp16 scale][32 x int8]; blocks36: the
 * reference's host layout [fp32 scale][32 x int8] (quants.cpp:14). The fp16
 * scale is the fp32 scale rounded to nearest even. */
int vkl_q8_0_quantize(const float *src, void *blocks34, size_t h, size_t w);
int vkl_q8_0_quantize36(const float *src, void *blocks36, size_t h, size_t w);
int vkl_q8_0_dequantize(const void *blocks34, float *dst, size_t h, size_t w);
int vkl_q8_0_blocks36_to_34(const void *blocks36, void *blocks34, size_t n_blocks);
/* Same quantizer on the device: FP32 [1,h,w] tensor -> Q8_0 [1,h,w] tensor. */
int vkl_q8_0_quantize_device(vkl_command *cmd, vkl_tensor *src_fp32, vkl_tensor *dst_q8_0);

/* Seeded synthetic tensor contents (stand-ins for checkpoints, which this
 * library never ships): N(mean, std) for FP32/FP16/Q8_0 tensors, generated on
 * the device, bit-identical to the host generator of the test oracle. */
int vkl_tensor_fill_synthetic(vkl_command *cmd, vkl_tensor *t, uint64_t seed, uint64_t tensor_id,
                              float mean, float stdv);

/* ---- model: vkllama::Model, models/llama2.h:322-854 ------------------------ */
typedef struct vkl_model_config {
  uint32_t dim, heads, ffn, vocab, layers, maxlen;
  float eps;          /* llama.attention.layer_norm_rms_epsilon (llama2.h:369) */
  float final_eps;    /* the reference hard-codes 1e-6 for the output norm (llama2.h:268) */
  int weight_dtype;   /* VKL_Q8_0 or VKL_FP16 */
  int tp_rank, tp_size; /* tensor-parallel shard of this process (1 = single GPU) */
} vkl_model_config;

int vkl_model_create(vkl_device *dev, const vkl_model_config *cfg, vkl_model **out);
int vkl_model_destroy(vkl_model *m);
/* Model::init's per-tensor upload (llama2.h:401-677). `name` is the GGUF tensor
 * name the reference looks up: token_embd.weight, output.weight,
 * output_norm.weight, blk.N.{attn_norm,attn_q,attn_k,attn_v,attn_output,
 * ffn_norm,ffn_gate,ffn_up,ffn_down}.weight. Data is the raw GGUF payload of
 * the FULL tensor; a tensor-parallel rank keeps only its shard. */
int vkl_model_set_weight(vkl_model *m, const char *name, int dtype, const void *data,
                         size_t bytes);
/* Fill every weight with the seeded synthetic model (N(0,wstd) matrices,
 * 1+N(0,nstd) norm weights) without touching the host. */
int vkl_model_synth_weights(vkl_model *m, uint64_t seed, float wstd, float nstd);
/* Model::operator()(toks, offset) (llama2.h:683-843): host token ids in, fp32
 * logits of the last token out (vocab floats; a tensor-parallel rank gets its slice),
 * synchronous. A call with several tokens on a tensor-parallel model fills the caches
 * in many-token passes and takes the last token through the decode kernel: it must
 * end inside the context length, and the last block's query is rotated at the
 * token's own position (the single-device form rotates it at the call's first, as
 * the reference does after clipping Q). */
int vkl_model_forward(vkl_model *m, const uint32_t *toks, size_t n, size_t offset,
                      float *logits_out);
/* llama2_infer's loop (app/llama2_infer.cpp:141-210) with the greedy pick kept
 * on the device: prefill `prompt`, then n_gen - 1 one-token steps. With Q8_0 weights a
 * step is one launch of the persistent decode kernel (all ops of the token in one
 * cooperative launch); with FP16 weights, or under VKLLAMA_DECODE=graph, it is one replay
 * of a captured CUDA graph of five kernels per layer. out_ids receives n_gen ids.
 * prefill_ms / decode_ms, when not NULL, receive the device time of the two phases. */
int vkl_model_generate(vkl_model *m, const uint32_t *prompt, size_t n_prompt, size_t n_gen,
                       uint32_t *out_ids, float *prefill_ms, float *decode_ms);
/* The id the device picked after the last forward/generate step (greedy arg-max over the
 * whole vocabulary, also when the output layer is split over tensor-parallel ranks); the
 * device-side counterpart of TopkSampler(1)::sample (models/samplers.cpp:37-64). */
int vkl_model_last_token(vkl_model *m, uint32_t *id);
/* The k largest logits of the last forward / generate step and their token ids, sorted
 * descending (equal values: lowest id first), selected on the device so that a top-k
 * sampler needs k pairs instead of the 128 KB of logits that the reference downloads
 * per token (models/llama2.h:283-298, 835-842). 1 <= k <= 64. Single-GPU models. */
int vkl_model_topk(vkl_model *m, uint32_t k, float *values, uint32_t *ids);
/* Copy one layer's caches [heads_local, maxlen, head_dim] fp16 to / from the host. */
int vkl_model_read_kv(vkl_model *m, uint32_t layer, void *kcache, void *vcache);
int vkl_model_write_kv(vkl_model *m, uint32_t layer, const void *kcache, const void *vcache);
/* One decoder block on host hidden states (Llama2Block::operator(), llama2.h:160-213):
 * x fp16 [T, dim] -> out fp16 [T, dim] (all rows; the reference's last block keeps the last). */
int vkl_model_block_forward(vkl_model *m, uint32_t layer, const void *x_fp16, size_t T,
                            size_t offset, void *out_fp16);
/* Op::time() for the model path (models/llama2.h:816-841 prints per-op costs): one
 * decode step with a time stamp after each op. out_us[0..8]: device microseconds
 * summed over layers of 0 embedding, 1 RMSNorm+QKV, 2 RoPE+append+attention,
 * 3 o_proj+residual, 4 RMSNorm+gate/up+SwiGLU, 5 down+residual, 6 RMSNorm+lm head,
 * 7 arg-max, 8 tensor-parallel all-reduce (9 unused); out_us[10..19]: the part of each
 * spent waiting for the other CTAs after the op (the persistent kernel, timeline of its
 * first CTA; 0 on the multi-kernel path, which is timed with an event after every launch).
 * Appends to the KV cache at `offset`. */
int vkl_model_decode_profile(vkl_model *m, uint32_t token, size_t offset, float out_us[20]);
/* The same step with a global-timer stamp (ns) by every CTA of the persistent kernel at six
 * points of every op: out[(op * grid + cta) * 8 + k], k = 0 op entered, 1 input vector
 * complete, 2 the CTA's first warp finished its weight stream, 3 all its warps did,
 * 4 results stored, 5 end-of-op synchronisation passed (unset stamps are 0). With out == NULL
 * only *nops and *grid are returned (out needs nops * grid * 8 words). kinds[nops], when
 * not NULL, receives per op: kind | matrices << 8 | epilogue << 16. A profiling aid with no
 * counterpart in the reference beyond Op::time(). */
int vkl_model_decode_trace(vkl_model *m, uint32_t token, size_t offset, unsigned long long *out, size_t cap,
                           uint32_t *nops, uint32_t *grid, uint32_t *kinds);
/* Tensor-parallel set-up (no counterpart in the reference, which is single-device:
 * gpu_device.cpp:14-21). One process per GPU creates its shard (tp_rank of tp_size);
 * each exports its exchange buffer over CUDA IPC, the processes swap the 64-byte handles
 * by any means (the Python layer uses torch.distributed), open the peers' handles and
 * pass the mapped pointers, indexed by rank (own entry ignored), to vkl_model_tp_connect.
 * The decode kernel then pushes row-split partial sums into every rank's buffer with
 * plain peer stores and reduces them in rank order (one all-reduce after o_proj and one
 * after down_proj per layer), and exchanges arg-max candidates of the vocabulary-split
 * output layer. vkl_model_forward returns this rank's slice of the logits. */
int vkl_model_tp_buffer(vkl_model *m, void **local_ptr, size_t *bytes);
/* Failure detection (the reference's counterpart is the 60 s fence time-out of
 * src/core/command.h:389-395). Every wait inside the persistent decode kernel (weight
 * stage, ring slot, tagged input, grid barrier, tensor-parallel all-reduce and arg-max
 * exchange) gives up after `polls` polls of about half a microsecond each: the kernel
 * then leaves through its normal path and the call returns VKL_INTERNAL naming the wait
 * (code 1 weight stage, 2 ring slot, 3 grid barrier, 4 all-reduce, 5 arg-max exchange,
 * 6 tagged input). The device context stays usable. Default (polls = 0): 2^21, and 2^24
 * for tensor-parallel models, the same bound for every wait so that none gives up while
 * another it depends on is still waiting; ranks may start a step up to that much apart.
 * After such an error a tensor-parallel model refuses further steps
 * (VKL_FAILED_PRECONDITION) until every rank has called vkl_model_tp_connect again
 * between two host barriers, which clears the exchange buffers and restarts the
 * sequence counters on all ranks together. */
int vkl_model_set_wait_limit(vkl_model *m, uint32_t polls);
int vkl_model_tp_connect(vkl_model *m, void *const *peer_ptrs, int n);
int vkl_ipc_export(void *device_ptr, unsigned char handle[64]);
int vkl_ipc_open(vkl_device *dev, const unsigned char handle[64], void **device_ptr);


/* ---- checkpoint container: gguflib as used by app/llama2_infer.cpp:46-73 ---------------
 * Read-only view of a GGUF file (versions 2 and 3), memory mapped. Keys are the metadata
 * the reference reads (models/llama2.h:367-370: llama.attention.head_count,
 * llama.block_count, llama.attention.layer_norm_rms_epsilon, llama.context_length);
 * tensors are looked up by index (name == NULL) or by name and handed out as pointers
 * into the mapping, valid until vkl_gguf_close. dims[0] is the row length, as in GGUF;
 * ggml_type 0/1/8 = F32/F16/Q8_0 (llama2.h:382-397); bytes is 0 for other types. */
int vkl_gguf_open(const char *path, vkl_gguf **out);
int vkl_gguf_close(vkl_gguf *g);
int vkl_gguf_counts(const vkl_gguf *g, uint32_t *version, size_t *n_keys, size_t *n_tensors);
int vkl_gguf_get_u32(const vkl_gguf *g, const char *key, uint32_t *out);
int vkl_gguf_get_f32(const vkl_gguf *g, const char *key, float *out);
int vkl_gguf_get_string(const vkl_gguf *g, const char *key, char *buf, size_t cap);
int vkl_gguf_tensor(const vkl_gguf *g, size_t index, const char *name, char *name_out, size_t name_cap,
                    uint32_t *ndim, uint64_t dims[4], uint32_t *ggml_type, const void **data, size_t *bytes);
/* Model::init (models/llama2.h:348-681) from an open file: configuration from the llama.*
 * keys and the tensor shapes, every tensor uploaded (and sharded when tp_size > 1).
 * maxlen 0 keeps llama.context_length, otherwise the smaller of the two is used. */
int vkl_model_load_gguf(vkl_device *dev, const vkl_gguf *g, uint32_t maxlen, int tp_rank, int tp_size,
                        vkl_model **out);

/* ---- samplers: models/samplers.h, samplers.cpp:37-101 -----------------------------------
 * kind 0 = TopkSampler(topk): softmax over the k largest logits, one draw.
 * kind 1 = TopPSampler(topp): the shortest descending prefix whose softmax mass reaches p,
 * renormalised, one draw. seed 0 seeds the generator from std::random_device as the
 * reference does; any other seed makes the draws reproducible. Equal logits are ordered by
 * token id (the reference's std::sort leaves ties unspecified).
 * vkl_sampler_sample_candidates draws from a descending candidate list such as
 * vkl_model_topk returns (top-k samplers only). */
int vkl_sampler_create(int kind, size_t topk, float topp, uint64_t seed, vkl_sampler **out);
int vkl_sampler_destroy(vkl_sampler *s);
int vkl_sampler_sample(vkl_sampler *s, const float *logits, size_t n, int *id);
int vkl_sampler_sample_candidates(vkl_sampler *s, const float *values, const uint32_t *ids, size_t k, int *id);

#ifdef __cplusplus
}
#endif
#endif /* VKLLAMA_B200_H_ */
