/* libnfai_cuda.so -- C ABI of the B200 (sm_100a) Llama-3 forward path for NFAI.
 *
 * This library stands where the reference's NFAI.Vulkan + NFAI.Vulkan.Shaders projects stand: device context,
 * weight upload, KV cache, the per-token transformer schedule and every compute kernel. The managed side
 * (Parser, LlamaModelFactory, LlamaModel, GenericChatClient, ComputeCollection) keeps its shape and calls these
 * entry points through P/Invoke. Every comment "replaces:" cites the reference code (path within the
 * reference project : lines) whose job the entry point takes over.
 *
 * Conventions
 *  - every function returns an int status (NFAI_OK == 0) unless stated otherwise;
 *  - handles are opaque; a handle is used by one thread at a time (the reference drives its device from one
 *    managed thread: NFAI.Models.Llama3/LlamaModel.cs:99-174); different contexts may live on different threads;
 *  - host pointers are owned by the caller and are fully consumed before the call returns;
 *  - the library owns all device memory behind nfai_ctx / nfai_model handles;
 *  - nothing here exits, aborts or traps: failures come back as a status plus nfai_last_error().
 *  - entry points named nfai_op_* take DEVICE pointers and run one kernel of the path on caller-owned buffers.
 */
#ifndef NFAI_CUDA_H
#define NFAI_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct nfai_ctx nfai_ctx;
typedef struct nfai_model nfai_model;

enum {
  NFAI_OK = 0,
  NFAI_ERR_ARG = 1,          /* bad argument (null, out of range, wrong dtype, unknown tensor name) */
  NFAI_ERR_STATE = 2,        /* call made in the wrong lifecycle state */
  NFAI_ERR_OOM = 3,          /* device or pinned host allocation failed */
  NFAI_ERR_CUDA = 4,         /* a CUDA runtime call or kernel failed */
  NFAI_ERR_NCCL = 5,         /* an NCCL call failed or NCCL is not loadable */
  NFAI_ERR_CONTEXT_FULL = 6, /* position would reach the KV-cache capacity */
  NFAI_ERR_TIMEOUT = 7       /* a bounded device-side wait gave up */
};

enum { NFAI_F32 = 0, NFAI_F16 = 1 };

/* Model geometry. Mirrors what the reference reads from GGUF metadata
 * (NFAI.Models.Llama3/LlamaModel.cs:23-39) plus ModelOptions.KVCacheSize (NFAI.Models/ModelOptions.cs:3-8). */
typedef struct nfai_hparams {
  uint32_t H;        /* llama.embedding_length (= token_embd ne0) */
  uint32_t L;        /* llama.block_count */
  uint32_t qH;       /* llama.attention.head_count */
  uint32_t kvH;      /* llama.attention.head_count_kv */
  uint32_t d;        /* llama.attention.key_length (head dim) */
  uint32_t ropeDim;  /* llama.rope.dimension_count */
  uint32_t F;        /* FFN width (ffn_gate ne1) */
  uint32_t V;        /* vocabulary (token_embd ne1) */
  uint32_t ctx;      /* KV-cache capacity in positions (ModelOptions.KVCacheSize) */
  float eps;         /* RMSNorm epsilon; also the softmax guard (NFAI.Vulkan.Shaders/TransformerBlock.cs:115-116) */
  float rope_theta;  /* RoPE base; the reference hard-codes 500000 (TransformerBlock.cs:33) */
  int32_t weight_dtype; /* NFAI_F32 or NFAI_F16: how matrices are kept in HBM */
  int32_t kv_dtype;     /* NFAI_F32 (the reference's cache type) or NFAI_F16 */
  int32_t tied;         /* 1: LM head = token_embd (LlamaModel.cs:64-67); 0: output.weight is uploaded */
} nfai_hparams;

/* ---- library ------------------------------------------------------------------------------------------- */

/* Version string of the library (static storage). */
const char* nfai_version(void);

/* Text of the last failure on this context (static per context; empty string if none). ctx may be NULL, in
 * which case the last failure of a call that had no context (e.g. nfai_ctx_create) is returned.
 * replaces: generic Exception messages at NFAI.Vulkan/VulkanBufferManager.cs:61-87. */
const char* nfai_last_error(const nfai_ctx* ctx);

/* ---- device context ------------------------------------------------------------------------------------ */

/* Open CUDA device `device_ordinal`, create the stream, the pinned staging ring and the timing events.
 * replaces: LlamaModelFactory() ctor (NFAI.Models.Llama3/LlamaModelFactory.cs:15-22) and
 *           VulkanHelper.CreateVulkanInstance/PickPhysicalDevice/CreateLogicalDevice
 *           (NFAI.Vulkan/VulkanHelper.cs:11,136,153). */
int nfai_ctx_create(int device_ordinal, nfai_ctx** out);

/* Fill `out` (at least 128 bytes) with a fresh NCCL unique id; rank 0 makes it and the host shares it with the
 * other ranks by any means. No counterpart in the reference (single device). */
int nfai_tp_unique_id(void* out, size_t out_bytes);

/* Like nfai_ctx_create, for rank `rank` of a `world`-way tensor-parallel group (world in {1,2,4,8}); joins the
 * NCCL communicator named by `nccl_uid`. One context per GPU: either one process per GPU or one thread per GPU.
 * No counterpart in the reference (single device). */
int nfai_ctx_create_tp(int device_ordinal, int rank, int world, const void* nccl_uid, size_t uid_bytes,
                       nfai_ctx** out);

/* Optional, before nfai_model_finalize: let the tensor-parallel ranks exchange partial sums through each other's
 * memory over NVLink with this library's own kernel instead of NCCL all-reduces. Every rank writes a 128-byte
 * descriptor of its exchange area (nfai_tp_export_peer), the host gathers the `world` descriptors in rank order
 * and gives the array to every rank (nfai_tp_import_peers). Works across processes (CUDA IPC) and across threads
 * of one process (peer access). No counterpart in the reference (single device). */
int nfai_tp_export_peer(nfai_ctx* ctx, void* out, size_t out_bytes);
int nfai_tp_import_peers(nfai_ctx* ctx, const void* descs, int n);

/* replaces: LlamaModelFactory.Dispose (LlamaModelFactory.cs:24-32). */
int nfai_ctx_destroy(nfai_ctx* ctx);

/* Budget, in nanoseconds, of every device-side wait on another rank (exchange flags). Default one second, or the
 * environment variable NFAI_WAIT_NS at context creation. A wait that runs out makes the call return
 * NFAI_ERR_TIMEOUT; the kernel itself always returns. Takes effect for graphs captured afterwards
 * (nfai_model_finalize, nfai_model_tune).
 * replaces: nothing -- the reference waits on a fence without limit (VulkanBufferManager.cs:474-494). */
int nfai_ctx_set_wait_ns(nfai_ctx* ctx, uint64_t ns);

/* ---- model lifecycle: create -> tensors -> finalize -> prefill/decode -> destroy ----------------------- */

/* replaces: LlamaModel ctor reading hyper-parameters (LlamaModel.cs:21-41). */
int nfai_model_create(nfai_ctx* ctx, const nfai_hparams* hp, nfai_model** out);

/* Start uploading the tensor `gguf_name` (e.g. "blk.3.attn_q.weight"). `shape` is in GGUF ne order (innermost
 * first), as NFAI.GGUF/Parser.cs:252-258 reads it. `src_dtype` is the element type of the bytes that follow:
 * NFAI_F32 (what ComputeCollection.GetDataRaw yields today, halves already widened:
 * NFAI.Core/AbstractComputeCollection.cs:62-77) or NFAI_F16 (raw file bytes). Conversion to the model's
 * weight_dtype happens on the device; F32 -> F16 is exact for values that were widened from halves.
 * Under tensor parallelism the caller streams the WHOLE tensor; each rank keeps its shard.
 * replaces: ShaderProperty.SetValue(ComputeCollection) -> VulkanBufferManager.UploadDataToDeviceLocal
 *           (NFAI.Vulkan/VulkanBufferManager.cs:105-194) and the name lookups at
 *           NFAI.Vulkan.Shaders/TransformerBlock.cs:41-99, LlamaModel.cs:43,58. */
int nfai_model_tensor_begin(nfai_model* m, const char* gguf_name, int src_dtype, const uint64_t* shape, int ndim);

/* Next `nbytes` of the tensor opened by nfai_model_tensor_begin, in file order; any chunking is accepted as
 * long as nbytes is a multiple of the source element size. */
int nfai_model_tensor_chunk(nfai_model* m, const void* bytes, size_t nbytes);

/* Close the tensor; fails if fewer or more bytes arrived than the shape needs. */
int nfai_model_tensor_end(nfai_model* m);

/* All tensors are in: check completeness, build the RoPE table on the host in float32
 * (TransformerBlock.cs:33-38), allocate the KV cache and activations, capture the decode graph.
 * replaces: the buffer-aliasing graph wiring of TransformerBlock ctor (TransformerBlock.cs:49-124) and
 *           ShaderWrapper.Compile on first use (NFAI.Vulkan.Shaders/ShaderWrapper.cs:55-206). */
int nfai_model_finalize(nfai_model* m);

/* Whole-file path: memory-map a GGUF file, read header, metadata and tensor directory natively, and stream the
 * tensors of a general.architecture == "llama" model to the device in their stored type (float16 files stay
 * float16, no widening pass on the CPU); then finalize. kv_dtype: NFAI_F32, NFAI_F16, or -1 for the weights' type.
 * Equivalent to nfai_model_create + tensor_begin/chunk/end for every tensor + nfai_model_finalize.
 * replaces: Parser.Parse (NFAI.GGUF/Parser.cs:22-45,130-307) + ComputeCollection.GetDataRaw
 *           (NFAI.Core/AbstractComputeCollection.cs:36-79) + UploadDataToDeviceLocal
 *           (NFAI.Vulkan/VulkanBufferManager.cs:105-194) for hosts that want the native loader. */
int nfai_model_load_gguf(nfai_ctx* ctx, const char* path, uint32_t kv_cache_size, int kv_dtype, nfai_model** out);

/* Read only the header, metadata and tensor directory of a GGUF file and report the geometry nfai_model_load_gguf
 * would create, with every size and offset of the directory checked against the file length. Needs no device and no
 * context; `err_out` (may be null) receives the reason of a failure. A malformed or hostile file gives
 * NFAI_ERR_ARG, never a crash.
 * replaces: the header / metadata / tensor-info passes of Parser.Parse (NFAI.GGUF/Parser.cs:28-30,130-307), which
 *           trust the counts they read. */
int nfai_gguf_probe(const char* path, uint32_t kv_cache_size, nfai_hparams* out, char* err_out, size_t err_bytes);

/* The model's geometry as it was created (filled by nfai_model_load_gguf from the file). */
int nfai_model_get_hparams(const nfai_model* m, nfai_hparams* out);

/* replaces: LlamaModel.Dispose (LlamaModel.cs:70-74, which throws NotImplementedException). */
int nfai_model_destroy(nfai_model* m);

/* ---- the hot path --------------------------------------------------------------------------------------- */

/* Ingest `n` prompt tokens at positions pos..pos+n-1. If `logits_last` is non-null it receives the V float32
 * logits of the last token; if `argmax_last` is non-null it receives the lowest index of their maximum.
 * The result equals feeding the tokens one by one through nfai_decode.
 * replaces: the prompt loop of LlamaModel.RunAsync (LlamaModel.cs:103-126). */
int nfai_prefill(nfai_model* m, const uint32_t* tokens, int n, float* logits_last, uint32_t* argmax_last);

/* One token at the current position: embed -> L x block -> output norm -> LM head. `logits` (V floats) and
 * `argmax` are optional host outputs. Advances the position by one.
 * replaces: one iteration of the decode loop (LlamaModel.cs:134-173): TokenEmbedShader.Compute,
 *           TransformerBlock.Compute (NFAI.Vulkan.Shaders/TransformerBlock.cs:127-184), output RMSNorm, LM-head
 *           MatrixMultiplyShader, GetOutputs; and SamplingUtils.ArgMax (NFAI.Models.Llama3/SamplingUtils.cs:55-56). */
int nfai_decode(nfai_model* m, uint32_t token, float* logits, uint32_t* argmax);

/* Greedy generation that never leaves the device: feed `first_token`, then feed each arg-max back, `n_steps`
 * times. `out_tokens` (n_steps entries, host, optional) receives the arg-max of every step; `elapsed_ms`
 * (optional) the device time of the n_steps steps measured with CUDA events on the library's stream.
 * replaces: the decode loop of LlamaModel.RunAsync with SamplingUtils.ArgMax in place of TopP. */
int nfai_decode_greedy(nfai_model* m, uint32_t first_token, int n_steps, uint32_t* out_tokens, float* elapsed_ms);

/* Temperature / top-k / top-p sampling of the last step's logits on the device; only the token id comes back.
 * `u` in [0, 1) is the uniform random number the draw uses (the host supplies it, e.g. Random.Shared.NextSingle()).
 * Same arithmetic as SamplingUtils.TopP (defaults there: temperature 0.5, top_p 0.95, top_k 40); top_k <= 64.
 * The sampled token also becomes the token a following nfai_decode_greedy-style device step would embed.
 * replaces: lmHead.GetOutputs() (513 KB read-back) + SamplingUtils.TopP (NFAI.Models.Llama3/SamplingUtils.cs:5-33,
 *           LlamaModel.cs:128-130,165). */
int nfai_sample_top_p(nfai_model* m, float temperature, float top_p, int top_k, float u, uint32_t* token_out);

/* n_steps of decode with the draw of nfai_sample_top_p after every step, fed back on the device: logits, arg-max and
 * the drawn tokens stay in device memory until the loop is over; u[i] is the uniform number of step i (the host draws
 * them up front, e.g. from Random.Shared). The caller cuts the result at its end-of-sequence token.
 * replaces: the sampling loop of LlamaModel.RunAsync (LlamaModel.cs:134-173) with SamplingUtils.TopP inside. */
int nfai_decode_sampled(nfai_model* m, uint32_t first_token, int n_steps, float temperature, float top_p, int top_k,
                        const float* u, uint32_t* out_tokens, float* elapsed_ms);

/* Current position (number of tokens in the KV cache).
 * replaces: TransformerBlock.currentToken (TransformerBlock.cs:25,183) and
 *           MatrixMultiplyShader.currentCacheSize (NFAI.Vulkan.Shaders/MatrixMultiplyShader.cs:28). */
int nfai_position(const nfai_model* m, uint32_t* pos);

/* Position back to 0 (the KV cache content is left in place and overwritten as positions are reused).
 * replaces: MatrixMultiplyShader.ResetCache (MatrixMultiplyShader.cs:153-159). */
int nfai_reset(nfai_model* m);

/* ---- taps for parity tests ------------------------------------------------------------------------------ */

/* K and V rows (kvH*d floats each, widened to float32) of `layer` at `pos`. Under tensor parallelism the rank's
 * own KV heads come back in the first kvH*d/world floats.
 * replaces: MatrixMultiplyShader.GetCurrentCache (MatrixMultiplyShader.cs:313-316). */
int nfai_read_kv(nfai_model* m, uint32_t layer, uint32_t pos, float* k, float* v);

/* Overwrite K and V rows of `layer` at `pos` from float32 host data (used to seed long-context tests). */
int nfai_write_kv(nfai_model* m, uint32_t layer, uint32_t pos, const float* k, const float* v);
/* The same for n consecutive positions starting at pos0 (k and v hold n rows of this rank's KV width): seeds a long
 * cache for tests of long-context decoding without ingesting a long prompt. No counterpart in the reference. */
int nfai_write_kv_range(nfai_model* m, uint32_t layer, uint32_t pos0, uint32_t n, const float* k, const float* v);

/* Set the position without touching the cache (pairs with nfai_write_kv). */
int nfai_set_position(nfai_model* m, uint32_t pos);

/* Residual stream (H floats) after block `layer` for the token processed last.
 * replaces: TransformerBlock.GetOutputProperty().GetValue() (TransformerBlock.cs:210-213). */
int nfai_read_hidden(nfai_model* m, uint32_t layer, float* out);

/* ---- measurement ---------------------------------------------------------------------------------------- */

/* Time `iters` back-to-back launches of one kernel of the decode step on the library's stream with CUDA
 * events; launch i uses layer (i mod L)'s weights so that consecutive launches read different HBM.
 * which: 0 = FFN gate/up GEMV (+RMSNorm, +SiLU*up), 1 = FFN down GEMV (+residual), 2 = QKV GEMV (+RMSNorm,+RoPE),
 *        3 = O-projection GEMV (+residual), 4 = LM-head GEMV (+RMSNorm, +arg-max partials), 5 = attention.
 * avg_ms receives the mean duration of one launch; bytes_per_launch the algorithmic bytes it must move. */
int nfai_profile_kernel(nfai_model* m, int which, int iters, float* avg_ms, uint64_t* bytes_per_launch);

/* Launch shape of one GEMV kernel of the decode step (selector as in nfai_profile_kernel, 0..4).
 * mode 0: weights double-buffered in registers; rows_per_warp in {1,2,4}, depth = 16-byte loads in flight per row
 *         per lane in {2,4,8}.
 * mode 1: weights staged through per-warp shared-memory rings by bulk asynchronous copies, stages of
 *         2 rows x 2 KB; rows_per_warp = 2, depth = ring stages per warp in {1,2,3,4}, plus
 *         8 x the number of further stages per warp that are requested into L2 while the kernel waits for its input.
 * The QKV and gate/up kernels need an even rows_per_warp. ctas_per_sm bounds the persistent grid (1..16 CTAs per
 * SM; a value above 16 is taken as the grid's CTA count itself, e.g. 256 so that 8 192 work items make exactly four
 * rounds over 2 048 warps). rows_per_warp may carry the K split in its upper bits (rows + 16 * split, split in
 * {1,2,4,8}; 0 = chosen from the matrix shape). Results do not depend on the shape. After nfai_model_finalize the decode graphs are captured again.

 * No counterpart in the reference (its dispatch sizes are fixed in each shader class). */
int nfai_model_tune(nfai_model* m, int which, int mode, int rows_per_warp, int depth, int ctas_per_sm);

/* L2 look-ahead of the decode step: every kernel asks the L2 for the step's weight sequence up to
 * `lookahead_bytes` beyond the weights it consumes itself (`extra_bytes` further for kernels that read no
 * weights), so that HBM keeps streaming across kernel boundaries and during attention. 0 switches it off.
 * mode 0 = one prefetch per 128-byte line, 1 = bulk prefetches. Results do not depend on it.
 * No counterpart in the reference. */
int nfai_model_set_prefetch(nfai_model* m, uint64_t lookahead_bytes, uint64_t extra_bytes, int mode);

/* Number of kernel launches inside one decode step (the captured graph's kernel nodes). */
int nfai_step_launches(const nfai_model* m, int* out);

/* ---- single kernels on caller-owned DEVICE buffers (kernel-level parity tests, embedding in other hosts) - */

/* x_out[i] = E[H*token + i] widened to float32.
 * replaces: TokenEmbedShader (NFAI.Vulkan.Shaders/TokenEmbedShader.cs:139-158). */
int nfai_op_embed(nfai_ctx* ctx, const void* E, int dtype, uint32_t H, uint32_t V, uint32_t token, float* x_out);

/* y = W * f(x) (+ resid): W[N][K] row-major of `dtype`; f = RMSNorm with `gain` and `eps` when gain != NULL,
 * identity otherwise; resid (N floats) optional. All pointers are device pointers.
 * replaces: RMSNormShader (NFAI.Vulkan.Shaders/RMSNormShader.cs:129-150) + MatrixMultiplyShader
 *           (MatrixMultiplyShader.cs:266-288) + the host residual add (TransformerBlock.cs:151-161). */
int nfai_op_gemv(nfai_ctx* ctx, const void* W, int dtype, uint32_t N, uint32_t K, const float* x, const float* gain,
                 float eps, const float* resid, float* y);

/* Fused Q/K/V projection of one token at position `pos`: a = RMSNorm(x); q = RoPE(Wq a) -> q_out[qH*d];
 * K row = RoPE(Wk a), V row = Wv a written into row `pos` of kcache / vcache ([ctx][kvH*d] of kv_dtype).
 * Wqkv is [qH*d + 2*kvH*d][H] (Q rows, then K rows, then V rows). rope_cs is [ctx][ropeDim/2] (cos, sin) pairs.
 * replaces: attn RMSNorm + three MatrixMultiplyShader dispatches + two RoPEShader dispatches
 *           (TransformerBlock.cs:129-141, NFAI.Vulkan.Shaders/RoPEShader.cs:238-271). */
int nfai_op_qkv_rope(nfai_ctx* ctx, const void* Wqkv, int dtype, const float* x, const float* gain, float eps,
                     uint32_t H, uint32_t qH, uint32_t kvH, uint32_t d, uint32_t ropeDim, const float* rope_cs,
                     uint32_t pos, float* q_out, void* kcache, void* vcache, int kv_dtype);

/* h = up * silu(gate) with gate = Wg a, up = Wu a, a = RMSNorm(x). Wgu is [2F][H] with gate row j at 2j and up
 * row j at 2j+1.
 * replaces: ffn RMSNorm + up/gate MatrixMultiplyShader + SiLUShader + ElementWiseMultiplicationShader
 *           (TransformerBlock.cs:163-171, NFAI.Vulkan.Shaders/SiLUShader.cs:112-127,
 *           NFAI.Vulkan.Shaders/ElementWiseMultiplicationShader.cs:127-138). */
int nfai_op_ffn_gate_up(nfai_ctx* ctx, const void* Wgu, int dtype, const float* x, const float* gain, float eps,
                        uint32_t H, uint32_t F, float* h_out);

/* One new token's attention over positions 0..seq-1 of a position-major cache, all query heads:
 * out[h*d+i] = sum_t softmax_t(q_h . K[t, h/(qH/kvH)] / sqrt(d)) * V[t, h/(qH/kvH), i].
 * `scratch` is device memory for the split partial results; nfai_op_attn_scratch_bytes gives the size needed.
 * replaces: AttentionScoreCalculationShader (NFAI.Vulkan.Shaders/AttentionScoreCalculationShader.cs:170-205),
 *           AttentionSoftmaxShader (NFAI.Vulkan.Shaders/AttentionSoftmaxShader.cs:145-177) and
 *           AttentionWeightedValueSumShader (NFAI.Vulkan.Shaders/AttentionWeightedValueSumShader.cs:181-215). */
int nfai_op_attn_decode(nfai_ctx* ctx, const float* q, const void* kcache, const void* vcache, int kv_dtype,
                        uint32_t seq, uint32_t qH, uint32_t kvH, uint32_t d, float* out, void* scratch,
                        size_t scratch_bytes);
size_t nfai_op_attn_scratch_bytes(uint32_t qH, uint32_t kvH, uint32_t d, uint32_t max_seq);

/* ---- tensor-parallel exchange, one kernel at a time (tests and diagnostics) ---------------------------------------
 * Under tensor parallelism the sums after the O and down projections are not a collective call: the GEMV that
 * produces the partial rows stores them into every rank's exchange area ("push"), and the GEMV that consumes the sum
 * waits for all ranks' flags, adds the areas' slots in rank order plus the residual while it loads x ("pull").
 * These entry points run exactly those kernels on exchange areas the caller owns. All `world` areas may sit on ONE
 * GPU (nfai_op_xchg_area_bytes each, zero-filled, 256-byte aligned), which is how the exchange is tested on a single
 * GPU: rank after rank pushes, then any rank pulls. `epoch` numbers the exchange (1, 2, 3, ... per area set).
 * A pull whose flags do not arrive within `wait_ns` nanoseconds (0 = the context's budget) returns NFAI_ERR_TIMEOUT;
 * nothing faults or hangs and the context stays usable.
 * No counterpart in the reference (one device; its residual adds run on the host, TransformerBlock.cs:151-161,174-181). */
size_t nfai_op_xchg_area_bytes(void);
/* y = W * f(x) as nfai_op_gemv. pull_epoch != 0: x is not read; x = pull_resid + sum over ranks of exchange
 * pull_epoch, and the summed vector is also stored to pull_store. push_epoch != 0: y is not written; the rows go to
 * rank `rank`'s slot in every area and the exchange is published. */
int nfai_op_gemv_xchg(nfai_ctx* ctx, const void* W, int dtype, uint32_t N, uint32_t K, const float* x, const float* gain,
                      float eps, float* y, void* const* areas, int world, int rank, uint32_t pull_epoch,
                      const float* pull_resid, float* pull_store, uint32_t push_epoch, uint64_t wait_ns);
/* The vocabulary-sharded LM head: push != 0 runs rank `rank`'s shard (Vl rows starting at global row v_lo) and
 * pushes its best (value, global index) to every area; pull != 0 waits for all ranks' pairs and returns the global
 * arg-max (lowest index among equal maxima, SamplingUtils.cs:55-56) in *argmax_out (device memory). */
int nfai_op_lm_head_xchg(nfai_ctx* ctx, const void* W, int dtype, const float* x, const float* gain, float eps, uint32_t H,
                         uint32_t Vl, uint32_t v_lo, float* logits, void* const* areas, int world, int rank,
                         uint32_t epoch, int push, int pull, uint32_t* argmax_out, uint64_t wait_ns);

/* Same computation as nfai_op_attn_decode, for callers that cannot allocate device memory where they run it (a
 * host working inside a fixed device-memory budget, or a per-token loop that must avoid cudaMalloc's device-wide
 * synchronisation): the split scratch is a 256 KiB array built into the library, so the call takes no scratch
 * pointer and performs no allocation of any kind. Inputs and outputs are still the caller's device buffers.
 *  - Geometries whose scratch (nfai_op_attn_scratch_bytes) exceeds 256 KiB are rejected with NFAI_ERR_ARG
 *    (e.g. 32 query heads of dimension 128 over more than 7 680 positions).
 *  - Every GPU on which the library is loaded holds those 256 KiB until the process exits.
 *  - The first call on a device resolves the array's device address (a one-time set-up); make that first call
 *    before any stream capture is begun.
 *  - All calls share the one array: two calls whose GPU work overlaps (other streams, other threads) race on it.
 * No counterpart in the reference. */
int nfai_op_attn_decode_static(nfai_ctx* ctx, const float* q, const void* kcache, const void* vcache, int kv_dtype,
                               uint32_t seq, uint32_t qH, uint32_t kvH, uint32_t d, float* out);

/* C[M][N] (float32) = A[M][K] * W[N][K]^T with A and W float16 (K contiguous, K % 8 == 0, 16-byte aligned): the
 * tensor-core GEMM (TMA-fed tcgen05, accumulators in tensor memory) that the batched prompt path uses for the
 * Q/K/V, O, gate/up and down projections. All pointers are device pointers.
 * replaces: MatrixMultiplyShader with inputRows > 1 (NFAI.Vulkan.Shaders/MatrixMultiplyShader.cs:266-288), which
 *           the reference never dispatches with more than one row. */
int nfai_op_gemm_f16(nfai_ctx* ctx, const void* A, const void* W, uint32_t M, uint32_t N, uint32_t K, float* C);

/* logits = W * RMSNorm(x) (W[V][H]) and the lowest index of their maximum into *argmax_out (device).
 * replaces: output RMSNorm + LM-head MatrixMultiplyShader (LlamaModel.cs:58-67,160-163) and
 *           SamplingUtils.ArgMax (SamplingUtils.cs:55-56). */
int nfai_op_lm_head(nfai_ctx* ctx, const void* W, int dtype, const float* x, const float* gain, float eps, uint32_t H,
                    uint32_t V, float* logits, uint32_t* argmax_out);

/* SamplingUtils.TopP alone on a device-resident logits vector (logits, token_out: device pointers).
 * replaces: NFAI.Models.Llama3/SamplingUtils.cs:5-33. */
int nfai_op_sample_top_p(nfai_ctx* c, const float* logits, uint32_t V, float temperature, float top_p, int top_k, float u,
                         uint32_t* token_out);

/* ---- multi-turn reuse --------------------------------------------------------------------------------------
 * nfai_prefill appends at the current position, so a second turn costs only its own tokens (the reference also keeps
 * growing one cache across turns, LlamaModel.cs:17,101-102, but never rewinds and overflows silently). A snapshot
 * holds the cache rows 0 .. position-1 of every layer, the last step's logits / arg-max and the position in device
 * memory; restoring it rewinds the model to that point (a shared system prompt is ingested once). A snapshot belongs
 * to the model it was taken from and must be destroyed before that model. No counterpart in the reference. */
typedef struct nfai_kv_snapshot nfai_kv_snapshot;
int nfai_kv_snapshot_create(nfai_model* m, nfai_kv_snapshot** out);
int nfai_kv_snapshot_restore(nfai_model* m, const nfai_kv_snapshot* s);
void nfai_kv_snapshot_destroy(nfai_kv_snapshot* s);
uint32_t nfai_kv_snapshot_position(const nfai_kv_snapshot* s);

/* ---- tokenizer (host side; no GPU work) ---------------------------------------------------------------------
 * Byte-pair tokenizer with the observable behaviour of NFAI.Models.Llama3/Tokenizer.cs and a (left, right) -> rank
 * hash map in place of its scan over the whole merges list for every adjacent pair (Tokenizer.cs:130-166).
 * tokens[i] / token_lens[i]: the bytes of vocabulary entry i (tokenizer.ggml.tokens); merges[k]: "left right"
 * (tokenizer.ggml.merges). Not thread-safe per handle. */
typedef struct nfai_tokenizer nfai_tokenizer;
/* replaces: Tokenizer(Dictionary<string, object> metadata) (Tokenizer.cs:16-58) */
int nfai_tokenizer_create(const char* const* tokens, const uint32_t* token_lens, uint32_t n_tokens, const char* const* merges,
                          const uint32_t* merge_lens, uint32_t n_merges, uint32_t bos_id, uint32_t eos_id,
                          nfai_tokenizer** out);
void nfai_tokenizer_destroy(nfai_tokenizer* t);
const char* nfai_tokenizer_last_error(const nfai_tokenizer* t);
/* UTF-8 text holding special tokens <|...|>: each special token, then the byte-pair encoding of the text behind it;
 * text in front of the first special token is dropped, as the reference does (Tokenizer.cs:93-180).
 * *n_out = number of ids (also when cap is too small: NFAI_ERR_ARG, call again with a larger buffer). */
int nfai_tokenizer_encode(nfai_tokenizer* t, const char* text, size_t text_len, uint32_t* ids_out, size_t cap, size_t* n_out);
/* replaces: Tokenizer.Tokenize(prompt, addBos) (Tokenizer.cs:68-182): the chat template around the user prompt. */
int nfai_tokenizer_encode_chat(nfai_tokenizer* t, const char* prompt, size_t prompt_len, int add_bos, uint32_t* ids_out, size_t cap,
                               size_t* n_out);
/* Tap for the parity tests: the end offsets (in UTF-16 code units) of the pieces the pre-tokenisation pattern
 * (Tokenizer.cs:109-111) cuts `text` into. No counterpart in the reference. */
int nfai_tokenizer_pretokenize(nfai_tokenizer* t, const char* text, size_t text_len, uint32_t* ends_out, size_t cap, size_t* n_out);
/* replaces: Tokenizer.Detokenize (Tokenizer.cs:432-462): concatenated token bytes, U+0120 -> ' ', U+010A -> '\n'. */
int nfai_tokenizer_decode(nfai_tokenizer* t, const uint32_t* ids, size_t n, char* text_out, size_t cap, size_t* n_out);

#ifdef __cplusplus
}
#endif
#endif /* NFAI_CUDA_H */
