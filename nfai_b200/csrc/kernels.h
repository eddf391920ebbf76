// Host-side launch interface of the kernels in libnfai_cuda (internal; the public ABI is include/nfai_cuda.h).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "xchg_protocol.h"

namespace nfai {

// Tensor-parallel hooks of a GEMV launch (world <= 1: none of it is touched). The partial sums of a row-parallel
// matrix (O and down projections) never go through a separate collective kernel: the GEMV that produces them
// stores them, each value tagged with the exchange's epoch, straight into every rank's exchange area (push), and the
// GEMV that consumes the sum polls its own area for the tagged words and adds them in rank order while it loads x
// (pull). Protocol: xchg_protocol.h.
struct XchgHooks {
  xchg::View view{};                     // every rank's exchange area (own entry = local memory)
  const uint32_t* epoch_base = nullptr;  // device word: exchanges completed on this context before this step
  unsigned long long wait_ns = 1000000000ull;  // budget of the wait for a word; afterwards error bit 4 and a zero x
  int pull = 0;                          // x = pull_resid + sum over ranks of exchange pull_index of this step
  uint32_t pull_index = 0;
  const float* pull_resid = nullptr;
  float* pull_store = nullptr;           // CTA 0 also stores the summed x here (the residual stream)
  int push = 0;                          // row sums go to every rank's slot (exchange push_index) instead of y
  uint32_t push_index = 0;
};

// Kernels that stage their stream in shared memory ask for the largest shared-memory carve-out. Kernels that
// stream through registers must NOT: loads in flight occupy L1 lines, so shrinking the L1 cuts their bandwidth
// (measured: the register streamer lost 20% with the maximum carve-out).
template <typename Kern>
inline cudaError_t prefer_max_shared(Kern kernel) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
}

// Streaming multiprocessors of the current device (148 on a B200); persistent grids are sized from it.
uint32_t sm_count();

// Launch with programmatic stream serialisation: the kernel may be scheduled while its predecessor in the stream is
// still running; it must execute griddepcontrol.wait (pdl_wait) before it touches anything the predecessor wrote.
// `pdl` = false gives a plain launch (the wait is then a no-op).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, bool pdl,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
// Prompt-path kernels overlap their launch and set-up with the predecessor's tail unless NFAI_PREFILL_PDL=0.
bool prefill_pdl();

// Device-resident state of one model: the graph's kernels read and advance it so that one captured graph
// serves every position.
struct StepState {
  uint32_t pos;         // number of tokens already in the KV cache = position of the token being processed
  uint32_t cur_token;   // token the next decode step embeds (the final kernel feeds the arg-max back here)
  uint32_t prompt_idx;  // cursor into the prompt buffer for head-less prompt steps
  uint32_t last_argmax; // arg-max of the last step that ran the LM head
  uint32_t err;         // sticky error bits: 1 = token id out of range, 2 = position beyond the cache
  uint32_t steps;       // index of the next history slot (reset by nfai_decode_greedy)
  uint32_t pad[2];
};

// Weights a kernel asks the L2 to fetch for the kernels that follow it (up to two address ranges): HBM keeps
// streaming the weight sequence of the step while a kernel is waiting on its predecessor, normalising x or
// running attention. mode 0 = one prefetch per 128-byte line, 1 = bulk prefetches of kPrefetchChunk bytes.
struct PrefetchPlan {
  const char* ptr[2] = {nullptr, nullptr};
  unsigned long long bytes[2] = {0, 0};
  int mode = 1;
};
constexpr uint32_t kPrefetchChunk = 4096;


enum GemvEpilogue {
  EPI_STORE = 0,     // y = acc (+ resid)
  EPI_QKV_ROPE = 1,  // rows are [Q | K | V]; RoPE on Q and K; K,V rows go to the cache at row pos
  EPI_SILU_MUL = 2,  // rows are interleaved (gate_j, up_j); h_j = up_j * silu(gate_j)
  EPI_LOGITS = 3     // y = acc and a per-CTA (max, lowest index) partial
};

struct GemvParams {
  const void* W = nullptr;  // [N][K] row-major, float or half
  uint32_t N = 0, K = 0;
  const float* x = nullptr;     // [K]
  const float* gain = nullptr;  // [K] RMSNorm gain, or null for no normalisation
  float eps = 0.f;
  const float* resid = nullptr;  // [N] or null
  float* y = nullptr;            // [N] (EPI_STORE, EPI_LOGITS) or [N/2] (EPI_SILU_MUL)
  // EPI_QKV_ROPE
  float* q_out = nullptr;
  void* kcache = nullptr;  // [ctx][kvDim] of the kv type
  void* vcache = nullptr;
  uint32_t qDim = 0, kvDim = 0, d = 0, ropeDim = 0, ctx = 0;
  const float2* rope_cs = nullptr;  // [ctx][ropeDim/2] (cos, sin)
  // position: *state (if non-null) else pos_imm
  StepState* state = nullptr;
  uint32_t pos_imm = 0;
  // EPI_LOGITS
  float* part_val = nullptr;
  uint32_t* part_idx = nullptr;
  PrefetchPlan pf;
  uint32_t* err = nullptr;  // optional device word for error bits when there is no StepState (4 = a bounded wait gave up)
  uint32_t split_log2 = 0;  // filled in by launch_gemv: log2 of the warps that share one row block
  uint32_t l2_ahead = 0;    // ring modes: stages per warp requested into L2 beyond the ring before the dependency wait
  XchgHooks tp;             // tensor-parallel push / pull (see XchgHooks)
  // EPI_LOGITS under tensor parallelism: the CTA that finishes last (ticket in `tp_ticket`, a local word) reduces
  // the per-CTA partials to this rank's best (value, global index = v_lo + row) and pushes the pair to every rank
  // (exchange tp.push_index)
  uint32_t v_lo = 0;
  uint32_t* tp_ticket = nullptr;
};

// Tunable launch shape of the GEMV family.
struct GemvTune {
  int mode = 0;           // 0 = register double-buffered streamer, 1 = per-warp shared-memory rings fed by bulk copies
                          // (stages of 2 rows x 2 KB)
  int rows_per_warp = 2;  // mode 0: 1, 2 or 4 (EPI_QKV_ROPE and EPI_SILU_MUL need an even value); ring modes: always 2
  int unroll = 4;         // mode 0: 16-byte loads in flight per row per lane (2, 4 or 8); ring modes: stages per warp (1-4)
  int ctas_per_sm = 2;    // persistent grid = min(needed, 148 * ctas_per_sm) CTAs of 256 threads
  int split = 0;          // mode 0: warps sharing one row block (1, 2, 4, 8); 0 = chosen from the matrix shape
  int l2_ahead = 0;       // ring modes: stages per warp requested into L2 beyond the ring while the kernel waits
  int grid = 0;           // 0 = 148 * ctas_per_sm; else the CTA count (chosen so that the work items divide evenly
                          // over the grid's warps and no last round runs partly empty)
};

size_t gemv_ring_smem(const GemvParams& p, int S);
uint32_t gemv_ring_grid(const GemvParams& p, int ctas_per_sm);
cudaError_t launch_gemv_ring(cudaStream_t s, int wdtype, int kvdtype, GemvEpilogue epi, const GemvParams& p, int S,
                             int ctas_per_sm, bool pdl);

// Number of CTAs the launch will use (the LM head needs it to size its partial buffers).
uint32_t gemv_grid(int wdtype, GemvEpilogue epi, const GemvParams& p, const GemvTune& t);
cudaError_t launch_gemv(cudaStream_t s, int wdtype, int kvdtype, GemvEpilogue epi, const GemvParams& p,
                        const GemvTune& t, bool pdl);

struct AttnParams {
  const float* q = nullptr;  // [qH*d], rotated
  const void* kcache = nullptr;
  const void* vcache = nullptr;  // [ctx][kvH*d]
  uint32_t qH = 0, kvH = 0, d = 0;
  StepState* state = nullptr;  // seq = state->pos + 1 when non-null
  uint32_t seq_imm = 0;
  float* out = nullptr;        // [qH*d]
  __half* out_half = nullptr;  // when non-null the output goes here as float16 instead (prompt path: the next GEMM's A)
  float* part = nullptr;       // [qH][S_max][d+2] split partials
  uint32_t* tickets = nullptr; // [kvH * head_groups], zero between launches
  uint32_t S_max = 1;
  // Launch shape: query heads that share one pass over K and V (4 = every head of a Llama-3 KV group: K and V
  // are read once, right for long contexts; 1 = one CTA per query head: four times the CTAs and all of a short
  // context in flight at once) and the fewest positions a CTA takes before the range is split.
  uint32_t heads_per_cta = 4;  // 4, 2 or 1
  uint32_t min_chunk = 512;
  uint32_t early = 1;  // request the K/V rows of earlier positions before the dependency wait (0: wait first)
  PrefetchPlan pf;
};


constexpr uint32_t kAttnMinChunk = 512;   // fewest positions one CTA takes before the range is split
constexpr uint32_t kAttnHeadsPerCta = 4;  // query heads sharing one pass over K/V

uint32_t attn_head_groups(uint32_t qH, uint32_t kvH, uint32_t heads_per_cta = kAttnHeadsPerCta);
uint32_t attn_splits(uint32_t qH, uint32_t kvH, uint32_t max_seq, uint32_t heads_per_cta = kAttnHeadsPerCta,
                     uint32_t min_chunk = kAttnMinChunk);
size_t attn_part_floats(uint32_t qH, uint32_t d, uint32_t S_max);
cudaError_t launch_attn_decode(cudaStream_t s, int kvdtype, const AttnParams& p, bool pdl);
// Causal attention of T prompt tokens: token t (q row t of p.q, [T][qH*d]) attends to positions 0 .. p.seq_imm-1+t;
// output rows go to p.out_half ([T][qH*d] float16). One CTA per (KV head group, token), no split.
cudaError_t launch_attn_prefill(cudaStream_t s, int kvdtype, const AttnParams& p, uint32_t T);
// The same contract on the tensor cores (d = 64 or 128): a CTA owns 64 tokens of one head and walks the prefix once.
bool attn_prefill_tc_supported(uint32_t d);
cudaError_t launch_attn_prefill_tc(cudaStream_t s, int kvdtype, const AttnParams& p, uint32_t T);

// Long-context variant for a float16 cache (d = 64 or 128, four query heads per CTA): K and V staged through
// shared-memory rings by 2-D tile copies. The two tile descriptors (one K, one V per layer) are built on the host.
struct AttnTileMaps {
  alignas(64) unsigned char k[128];
  alignas(64) unsigned char v[128];
};
bool attn_ring_supported(int kvdtype, uint32_t d);
size_t attn_ring_smem(int stages);
cudaError_t attn_ring_make_maps(const void* kcache, const void* vcache, uint32_t ctx, uint32_t kvDim, uint32_t d,
                                AttnTileMaps* out);
cudaError_t launch_attn_ring(cudaStream_t s, const AttnParams& p, const AttnTileMaps& maps, bool pdl);

// Long-context variant on the tensor cores (float16 cache, d = 64 or 128, up to four query heads per CTA as the rows
// of a 16-row MMA tile): same grid, scratch and merge as the kernels above.
bool attn_mma_supported(int kvdtype, uint32_t d);
cudaError_t launch_attn_mma(cudaStream_t s, const AttnParams& p, bool pdl);

cudaError_t launch_embed(cudaStream_t s, int wdtype, const void* E, uint32_t H, uint32_t V, StepState* state,
                         const uint32_t* prompt, uint32_t token_imm, float* x_out, const PrefetchPlan& pf, bool pdl);
// Reduce the LM head's per-CTA partials to the arg-max (lowest index among maxima), feed it back as the next
// token and advance the position.
cudaError_t launch_argmax_final(cudaStream_t s, const float* part_val, const uint32_t* part_idx, uint32_t nparts,
                                StepState* state, uint32_t* argmax_out, uint32_t* history, uint32_t history_cap,
                                const PrefetchPlan& pf, uint32_t* xchg_epoch, uint32_t xchg_per_step, const XchgHooks& tp,
                                bool pdl);
// Head-less prompt step: position and prompt cursor advance by one.
// xchg_epoch (may be null) counts the tensor-parallel exchanges completed on this context; a step adds its own.
cudaError_t launch_advance(cudaStream_t s, StepState* state, uint32_t* xchg_epoch, uint32_t xchg_per_step, bool pdl);

// Temperature / top-k / top-p sampling of `logits` (V floats) on the device. `argmax` points at the index of the
// largest logit (null: found by an extra kernel). Writes the chosen token to *token_out and, if given, *cur_token;
// 0xffffffff when `argmax` does not belong to these logits.
size_t sample_scratch_bytes(uint32_t V, int* nslices_out);
cudaError_t launch_sample_top_p(cudaStream_t s, const float* logits, uint32_t V, const uint32_t* argmax, uint32_t* cur_token,
                                float temperature, float top_p, int top_k, float u, void* scratch, uint32_t* token_out);

// Scatter/convert one uploaded chunk into a matrix's final place: source element g = elem_off + e sits at
// (row, col) = (g / K, g % K); rows [row_lo,row_hi) x cols [col_lo,col_hi) are kept and land at
// dst[((row-row_lo)*row_mul + row_off) * ldd + (col-col_lo)].
struct IngestParams {
  const void* src = nullptr;
  uint64_t n = 0, elem_off = 0, K = 1;
  uint64_t row_lo = 0, row_hi = 0, col_lo = 0, col_hi = 0;
  uint64_t row_mul = 1, row_off = 0, ldd = 0;
  void* dst = nullptr;
};
cudaError_t launch_ingest(cudaStream_t s, int src_dtype, int dst_dtype, const IngestParams& p);

}  // namespace nfai
