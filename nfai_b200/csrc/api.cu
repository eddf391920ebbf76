// C ABI of libnfai_cuda.so: device context, weight upload, KV cache, the captured decode step, taps.
// The public contract is include/nfai_cuda.h; this file is the host side that stands where the reference's
// NFAI.Vulkan (buffers, staging, submit/wait) and NFAI.Vulkan.Shaders (ShaderWrapper, ShaderProperty,
// TransformerBlock wiring) projects stand.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <string>
#include <vector>

#include "../../include/nfai_cuda.h"
#include "kernels.h"
#include "gemm_tc.h"
#include "tp.h"

using namespace nfai;

namespace {

thread_local std::string g_err;  // failures of calls that have no context

constexpr size_t kStageBytes = 16u << 20;
constexpr int kStageSlots = 2;

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
size_t dtype_size(int dt) { return dt == NFAI_F16 ? 2 : 4; }

}  // namespace

struct nfai_ctx {
  int device = 0;
  int rank = 0, world = 1;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  void* stage[kStageSlots] = {nullptr, nullptr};  // pinned, device-visible
  cudaEvent_t stage_ev[kStageSlots] = {nullptr, nullptr};
  int stage_next = 0;
  uint32_t* pin_small = nullptr;  // pinned scratch for tokens / state read-back (256 bytes)
  uint32_t* dev_err = nullptr;    // device word for error bits of kernels that run outside a model step
  TpComm* tp = nullptr;
  bool pdl = true;
  bool use_graph = true;
  unsigned long long wait_ns = 1000000000ull;  // budget of every bounded device-side wait on peers (NFAI_WAIT_NS)
  std::string err;
};

namespace {

int fail(nfai_ctx* c, int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (c) c->err = buf;
  g_err = buf;
  return code;
}

#define CU(c, call)                                                                                    \
  do {                                                                                                 \
    cudaError_t e__ = (call);                                                                          \
    if (e__ != cudaSuccess)                                                                            \
      return fail((c), e__ == cudaErrorMemoryAllocation ? NFAI_ERR_OOM : NFAI_ERR_CUDA, "%s: %s (%s:%d)", #call, \
                  cudaGetErrorString(e__), __FILE__, __LINE__);                                        \
  } while (0)

struct Matrix {
  void* ptr = nullptr;
  uint64_t rows = 0, cols = 0;  // local (this rank's) shape
  size_t bytes = 0;
};

struct Gain {
  float* ptr = nullptr;
  bool done = false;
};

struct LayerW {
  Matrix qkv, o, gateup, down;
  Gain attn_norm, ffn_norm;
  bool got_q = false, got_k = false, got_v = false, got_o = false, got_gate = false, got_up = false, got_down = false;
};

// Where the tensor being uploaded goes.
struct UploadTarget {
  bool active = false;
  bool skip = false;  // accepted and ignored (output.weight on a tied model)
  std::string name;
  int src_dtype = 0, dst_dtype = 0;
  uint64_t K = 0, N = 0;  // source shape: N rows of K
  uint64_t received = 0;  // source elements so far
  IngestParams ip;
  bool* done_flag = nullptr;
};

}  // namespace

struct nfai_model {
  nfai_ctx* ctx = nullptr;
  nfai_hparams hp{};
  // local (per-rank) geometry
  uint32_t qHl = 0, kvHl = 0, qDimL = 0, kvDimL = 0, Fl = 0, Vl = 0, v_lo = 0;
  bool finalized = false;
  char* warena = nullptr;
  size_t warena_bytes = 0;
  Matrix embd, head;
  bool got_embd = false, got_head = false;
  Gain out_norm;
  std::vector<LayerW> layers;
  UploadTarget up;
  // run-time buffers (one allocation)
  char* rarena = nullptr;
  void* kc = nullptr;
  void* vc = nullptr;  // [L][ctx][kvDimL]
  float2* rope_cs = nullptr;
  float* xbuf = nullptr;  // [(2L+1)][H]: x_in(0), then per layer (after attention, after FFN)
  float* q = nullptr;
  float* attn_out = nullptr;
  float* hbuf = nullptr;
  float* logits = nullptr;
  float* part_val = nullptr;
  uint32_t* part_idx = nullptr;
  uint32_t nparts = 0, nparts_alloc = 0;
  float* attn_part = nullptr;
  uint32_t* tickets = nullptr;
  uint32_t S_max = 1;
  uint32_t attn_heads = 4;  // query heads per attention CTA in the decode step
  std::vector<AttnTileMaps> attn_maps;  // per layer, when the decode step uses the tile-staged attention kernel
  bool attn_mma = false;                // long float16 caches: the tensor-core attention kernel (default over the tile-staged one)
  StepState* state = nullptr;
  uint32_t* history = nullptr;
  uint32_t* prompt = nullptr;
  float* pin_logits = nullptr;  // pinned V floats
  float* tp_buf = nullptr;      // [H] partial sums exchanged between ranks
  void* sample_scratch = nullptr;  // per-slice sums and candidates of the on-device sampler
  cudaGraphExec_t g_full = nullptr, g_nohead = nullptr;
  int launches_full = 0;
  uint32_t pos = 0;  // host mirror of state->pos
  GemvTune tune_qkv, tune_o, tune_gateup, tune_down, tune_head;
  // batched prompt path (float16 weights, one GPU): chunk workspace
  bool prefill_gemm = false;
  uint32_t pf_chunk = 0;
  float* pfX0 = nullptr;      // [chunk][H] residual stream
  float* pfX1 = nullptr;      // [chunk][H]
  __half* pfA = nullptr;      // [chunk][max(H, qDim)] normalised activations
  float* pfQ = nullptr;       // [chunk][qDim] rotated queries
  __half* pfAO = nullptr;     // [chunk][qDim] attention output
  __half* pfH = nullptr;      // [chunk][F] SiLU(gate)*up
  float* pfPart = nullptr;    // split-K partial tiles of the prompt GEMMs
  size_t pfPartFloats = 0;
  uint32_t* pfTok = nullptr;  // [chunk]
  // L2 look-ahead: how far beyond the weights a kernel consumes the step's weight sequence is requested
  uint64_t pf_look = 0, pf_extra = 0;
  int pf_mode = 1;
};

namespace {

float* x_in(nfai_model* m, uint32_t layer) { return m->xbuf + (size_t)(2 * layer) * m->hp.H; }
float* x_mid(nfai_model* m, uint32_t layer) { return m->xbuf + (size_t)(2 * layer + 1) * m->hp.H; }

size_t kv_layer_elems(const nfai_model* m) { return (size_t)m->hp.ctx * m->kvDimL; }

int env_int(const char* name, int dflt) {
  const char* v = getenv(name);
  return v && *v ? atoi(v) : dflt;
}

bool ring_wanted(uint32_t positions) {
  const int v = env_int("NFAI_ATTN_RING", -1);
  return v < 0 ? positions > 4096 : v != 0;
}

void read_tune(const char* name, GemvTune& t, int r_default, int u_default) {
  t.rows_per_warp = r_default;
  t.unroll = u_default;
  std::string key = std::string("NFAI_TUNE_") + name;
  const char* v = getenv(key.c_str());
  if (v) {
    int r = 0, u = 0, cps = 0, mode = 0, split = 0, ahead = 0, grid = 0;
    int got = sscanf(v, "%d,%d,%d,%d,%d,%d,%d", &r, &u, &cps, &mode, &split, &ahead, &grid);
    if (got >= 2 && (r == 1 || r == 2 || r == 4) && (u == 1 || u == 2 || u == 3 || u == 4 || u == 8)) {
      t.rows_per_warp = r;
      t.unroll = u;
      if (got >= 3 && cps >= 1 && cps <= 16) t.ctas_per_sm = cps;
      if (got >= 4 && (mode == 0 || mode == 1)) t.mode = mode;
      if (got >= 5 && (split == 0 || split == 1 || split == 2 || split == 4 || split == 8)) t.split = split;
      if (got >= 6 && ahead >= 0 && ahead <= 64) t.l2_ahead = ahead;
      if (got >= 7 && grid >= 0 && grid <= 4096) t.grid = grid;
    }
  }
}

// ---- the decode step as a sequence of launches (captured into a graph or run eagerly) -------------------------
GemvParams qkv_params(nfai_model* m, uint32_t l) {
  const nfai_hparams& hp = m->hp;
  GemvParams p;
  p.W = m->layers[l].qkv.ptr;
  p.N = m->qDimL + 2 * m->kvDimL;
  p.K = hp.H;
  p.x = x_in(m, l);
  p.gain = m->layers[l].attn_norm.ptr;
  p.eps = hp.eps;
  p.q_out = m->q;
  p.kcache = (char*)m->kc + (size_t)l * kv_layer_elems(m) * dtype_size(hp.kv_dtype);
  p.vcache = (char*)m->vc + (size_t)l * kv_layer_elems(m) * dtype_size(hp.kv_dtype);
  p.qDim = m->qDimL;
  p.kvDim = m->kvDimL;
  p.d = hp.d;
  p.ropeDim = hp.ropeDim;
  p.ctx = hp.ctx;
  p.rope_cs = m->rope_cs;
  p.state = m->state;
  return p;
}

AttnParams attn_params(nfai_model* m, uint32_t l) {
  const nfai_hparams& hp = m->hp;
  AttnParams a;
  a.q = m->q;
  a.kcache = (char*)m->kc + (size_t)l * kv_layer_elems(m) * dtype_size(hp.kv_dtype);
  a.vcache = (char*)m->vc + (size_t)l * kv_layer_elems(m) * dtype_size(hp.kv_dtype);
  a.qH = m->qHl;
  a.kvH = m->kvHl;
  a.d = hp.d;
  a.state = m->state;
  a.out = m->attn_out;
  a.part = m->attn_part;
  a.tickets = m->tickets;
  a.S_max = m->S_max;
  a.heads_per_cta = m->attn_heads;
  a.min_chunk = kAttnMinChunk;
  a.early = env_int("NFAI_ATTN_EARLY", 1) != 0;
  return a;
}

GemvParams o_params(nfai_model* m, uint32_t l) {
  GemvParams p;
  p.W = m->layers[l].o.ptr;
  p.N = m->hp.H;
  p.K = m->qDimL;
  p.x = m->attn_out;
  if (m->ctx->world == 1) {
    p.resid = x_in(m, l);
    p.y = x_mid(m, l);
  } else {
    p.y = m->tp_buf;  // partial sum; the all-reduce adds the ranks and the residual
  }
  return p;
}

GemvParams gateup_params(nfai_model* m, uint32_t l) {
  GemvParams p;
  p.W = m->layers[l].gateup.ptr;
  p.N = 2 * m->Fl;
  p.K = m->hp.H;
  p.x = x_mid(m, l);
  p.gain = m->layers[l].ffn_norm.ptr;
  p.eps = m->hp.eps;
  p.y = m->hbuf;
  return p;
}

GemvParams down_params(nfai_model* m, uint32_t l) {
  GemvParams p;
  p.W = m->layers[l].down.ptr;
  p.N = m->hp.H;
  p.K = m->Fl;
  p.x = m->hbuf;
  if (m->ctx->world == 1) {
    p.resid = x_mid(m, l);
    p.y = x_in(m, l + 1);
  } else {
    p.y = m->tp_buf;
  }
  return p;
}

GemvParams head_params(nfai_model* m) {
  GemvParams p;
  const Matrix& hd = m->hp.tied ? m->embd : m->head;
  // tied: the rank's vocabulary rows of the replicated embedding matrix; untied: the rank's own shard
  p.W = m->hp.tied ? (const char*)hd.ptr + (size_t)m->v_lo * m->hp.H * dtype_size(m->hp.weight_dtype) : hd.ptr;
  p.N = m->Vl;
  p.K = m->hp.H;
  p.x = x_in(m, m->hp.L);
  p.gain = m->out_norm.ptr;
  p.eps = m->hp.eps;
  p.y = m->logits;
  p.part_val = m->part_val;
  p.part_idx = m->part_idx;
  return p;
}

// The weights of one step form a sequence in consumption order: the per-layer matrices (contiguous in the weight
// arena, in the order the kernels read them) and then the LM-head matrix. Every kernel asks the L2 for the part
// of that sequence between what earlier kernels already requested and `look` bytes beyond its own weights
// (kernels without weights reach `extra` bytes further), wrapping into the next step at the end.
struct PrefetchPlanner {
  const char* baseA = nullptr;
  uint64_t lenA = 0;
  const char* baseB = nullptr;
  uint64_t lenB = 0;
  uint64_t look = 0, extra = 0, fetched = 0;
  int mode = 1;
  uint64_t total() const { return lenA + lenB; }
  uint64_t off(const void* p) const { return (uint64_t)((const char*)p - baseA); }
  PrefetchPlan next(uint64_t cons_end, bool has_weights) {
    PrefetchPlan pl;
    pl.mode = mode;
    const uint64_t T = total();
    if (look == 0 || T == 0) return pl;
    uint64_t target = cons_end + look + (has_weights ? 0 : extra);
    uint64_t a = fetched > cons_end ? fetched : cons_end, b = target;
    if (target > fetched) fetched = target;
    if (b <= a) return pl;
    if (b - a > T) b = a + T;
    int n = 0;
    while (a < b && n < 2) {
      uint64_t w = a % T;  // position inside one step's sequence
      const bool inA = w < lenA;
      uint64_t seg_end = inA ? lenA : T;
      uint64_t len = b - a < seg_end - w ? b - a : seg_end - w;
      const char* ptr = inA ? baseA + w : baseB + (w - lenA);
      // whole 256-byte blocks: bulk prefetches need 16-byte multiples and the ranges are only hints
      uint64_t lead = (256 - ((uintptr_t)ptr & 255)) & 255;
      if (len > lead + 256) {
        pl.ptr[n] = ptr + lead;
        pl.bytes[n] = (len - lead) & ~255ull;
        ++n;
      }
      a += len;
    }
    return pl;
  }
};

PrefetchPlanner make_planner(nfai_model* m, bool with_head) {
  PrefetchPlanner pp;
  const LayerW& first = m->layers.front();
  const LayerW& last = m->layers.back();
  pp.baseA = (const char*)first.qkv.ptr;
  pp.lenA = (uint64_t)((const char*)last.ffn_norm.ptr + (size_t)m->hp.H * 4 - pp.baseA);
  if (with_head) {
    GemvParams h = head_params(m);
    pp.baseB = (const char*)h.W;
    pp.lenB = (uint64_t)h.N * h.K * dtype_size(m->hp.weight_dtype);
  }
  pp.look = m->pf_look;
  pp.extra = m->pf_extra;
  pp.mode = m->pf_mode;
  // what the tail of the previous step already requested
  uint64_t carried = pp.look + pp.extra;
  pp.fetched = carried < pp.total() ? carried : pp.total();
  return pp;
}

cudaError_t record_step(nfai_model* m, bool with_head, bool from_prompt, int* launches) {
  nfai_ctx* c = m->ctx;
  const nfai_hparams& hp = m->hp;
  cudaStream_t s = c->stream;
  const bool pdl = c->pdl;
  const int wdt = hp.weight_dtype, kvdt = hp.kv_dtype;
  int n = 0;
  cudaError_t e;
  PrefetchPlanner pp = make_planner(m, with_head);
  auto end_of = [&](const Matrix& M) { return pp.off(M.ptr) + M.bytes; };
#define STEP(call)                 \
  do {                             \
    e = (call);                    \
    if (e != cudaSuccess) return e; \
    ++n;                           \
  } while (0)
  // Tensor parallel with peer memory: the exchanges live inside the GEMV kernels (push in the epilogue of O / down /
  // LM head, pull in the prologue of the kernel that consumes the sum), so the step has the same launches as on one
  // GPU. Without peer memory: NCCL all-reduce + residual-add kernel after O and down, pair gather after the LM head.
  const bool tp_on = c->world > 1;
  const bool fused_x = tp_on && tp_push_ready(c->tp) && hp.H % 4 == 0 && hp.H <= xchg::kMaxH;
  const XchgHooks hooks = fused_x ? tp_hooks(c->tp) : XchgHooks();
  auto pull_into = [&](GemvParams& g, uint32_t index, const float* resid, float* store) {
    if (!fused_x) return;
    g.tp = hooks;
    g.tp.pull = 1;
    g.tp.pull_index = index;
    g.tp.pull_resid = resid;
    g.tp.pull_store = store;
  };
  auto push_from = [&](GemvParams& g, uint32_t index) {
    if (!fused_x) return;
    const XchgHooks keep = g.tp;
    g.tp = hooks;
    g.tp.pull = keep.pull;
    g.tp.pull_index = keep.pull_index;
    g.tp.pull_resid = keep.pull_resid;
    g.tp.pull_store = keep.pull_store;
    g.tp.push = 1;
    g.tp.push_index = index;
  };
  const bool pdl_x = pdl && (!tp_on || fused_x);  // a kernel that follows an NCCL call is launched plainly
  // the first kernel of a step must not overlap the previous step's tail: plain launch
  STEP(launch_embed(s, wdt, m->embd.ptr, hp.H, hp.V, m->state, from_prompt ? m->prompt : nullptr, 0, x_in(m, 0),
                    pp.next(0, false), false));
  for (uint32_t l = 0; l < hp.L; ++l) {
    const LayerW& LW = m->layers[l];
    GemvParams gq = qkv_params(m, l);
    gq.pf = pp.next(end_of(LW.qkv), true);
    if (l > 0) pull_into(gq, 2 * l - 1, x_mid(m, l - 1), x_in(m, l));
    STEP(launch_gemv(s, wdt, kvdt, EPI_QKV_ROPE, gq, m->tune_qkv, l > 0 ? pdl_x : pdl));
    AttnParams ga = attn_params(m, l);
    ga.pf = pp.next(end_of(LW.qkv), false);
    if (m->attn_mma) STEP(launch_attn_mma(s, ga, pdl));
    else if (!m->attn_maps.empty()) STEP(launch_attn_ring(s, ga, m->attn_maps[l], pdl));
    else STEP(launch_attn_decode(s, kvdt, ga, pdl));
    GemvParams go = o_params(m, l);
    go.pf = pp.next(end_of(LW.o), true);
    push_from(go, 2 * l);
    STEP(launch_gemv(s, wdt, kvdt, EPI_STORE, go, m->tune_o, pdl));
    if (tp_on && !fused_x) {
      e = tp_allreduce_residual(c->tp, s, m->tp_buf, x_in(m, l), x_mid(m, l), hp.H, &n);
      if (e != cudaSuccess) return e;
    }
    GemvParams gg = gateup_params(m, l);
    gg.pf = pp.next(end_of(LW.gateup), true);
    pull_into(gg, 2 * l, x_in(m, l), x_mid(m, l));
    STEP(launch_gemv(s, wdt, kvdt, EPI_SILU_MUL, gg, m->tune_gateup, pdl_x));
    GemvParams gd = down_params(m, l);
    gd.pf = pp.next(pp.off(LW.ffn_norm.ptr) + (uint64_t)hp.H * 4, true);
    push_from(gd, 2 * l + 1);
    STEP(launch_gemv(s, wdt, kvdt, EPI_STORE, gd, m->tune_down, pdl));
    if (tp_on && !fused_x) {
      e = tp_allreduce_residual(c->tp, s, m->tp_buf, x_mid(m, l), x_in(m, l + 1), hp.H, &n);
      if (e != cudaSuccess) return e;
    }
  }
  // exchanges of one step: 2 per layer, plus the arg-max pairs when the step ends with the LM head
  const uint32_t per_step = 2 * hp.L + (with_head && fused_x ? 1u : 0u);
  if (with_head) {
    GemvParams gh = head_params(m);
    gh.pf = pp.next(pp.total(), true);
    pull_into(gh, 2 * hp.L - 1, x_mid(m, hp.L - 1), x_in(m, hp.L));
    push_from(gh, 2 * hp.L);
    gh.v_lo = m->v_lo;
    if (fused_x) gh.tp_ticket = tp_ticket_ptr(c->tp);
    STEP(launch_gemv(s, wdt, kvdt, EPI_LOGITS, gh, m->tune_head, pdl_x));
    if (tp_on && !fused_x) {
      e = tp_gather_argmax(c->tp, s, m->part_val, m->part_idx, m->nparts, m->v_lo, &n);
      if (e != cudaSuccess) return e;
    }
    XchgHooks fin;
    if (fused_x) {
      fin = hooks;
      fin.pull = 1;
      fin.pull_index = 2 * hp.L;
    }
    STEP(launch_argmax_final(s, m->part_val, m->part_idx, tp_on ? (uint32_t)c->world : m->nparts, m->state,
                             nullptr, m->history, hp.ctx, pp.next(pp.total(), false), tp_on ? tp_epoch_ptr(c->tp) : nullptr, per_step,
                             fin, pdl_x));
  } else {
    // head-less prompt step under tensor parallelism: the last down projection's sum is pulled by nobody (the
    // next step starts from a fresh embedding row), which the protocol allows
    STEP(launch_advance(s, m->state, tp_on ? tp_epoch_ptr(c->tp) : nullptr, per_step, pdl_x));
  }
#undef STEP
  if (launches) *launches = n;
  return cudaSuccess;
}

int capture(nfai_model* m, bool with_head, bool from_prompt, cudaGraphExec_t* out, int* launches) {
  nfai_ctx* c = m->ctx;
  cudaGraph_t g = nullptr;
  CU(c, cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
  cudaError_t e = record_step(m, with_head, from_prompt, launches);
  cudaError_t e2 = cudaStreamEndCapture(c->stream, &g);
  if (e != cudaSuccess || e2 != cudaSuccess) {
    if (g) cudaGraphDestroy(g);
    cudaGetLastError();
    return fail(c, NFAI_ERR_CUDA, "graph capture failed: %s / %s", cudaGetErrorString(e), cudaGetErrorString(e2));
  }
  e = cudaGraphInstantiate(out, g, 0);
  cudaGraphDestroy(g);
  if (e != cudaSuccess) return fail(c, NFAI_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
  return NFAI_OK;
}

int run_step(nfai_model* m, bool with_head, bool from_prompt) {
  nfai_ctx* c = m->ctx;
  if (c->use_graph) {
    CU(c, cudaGraphLaunch(with_head ? m->g_full : m->g_nohead, c->stream));
  } else {
    CU(c, record_step(m, with_head, from_prompt, nullptr));
  }
  return NFAI_OK;
}

int check_state(nfai_model* m, StepState* host_copy) {
  nfai_ctx* c = m->ctx;
  CU(c, cudaMemcpyAsync(c->pin_small, m->state, sizeof(StepState), cudaMemcpyDeviceToHost, c->stream));
  CU(c, cudaStreamSynchronize(c->stream));
  StepState st;
  memcpy(&st, c->pin_small, sizeof st);
  if (host_copy) *host_copy = st;
  if (st.err) {
    uint32_t zero = 0;
    cudaMemcpy(&m->state->err, &zero, 4, cudaMemcpyHostToDevice);
    if (st.err & 4u) return fail(c, NFAI_ERR_TIMEOUT, "a bounded device-side wait gave up");
    if (st.err & 1u) return fail(c, NFAI_ERR_ARG, "token id out of range (>= V)");
    return fail(c, NFAI_ERR_CONTEXT_FULL, "position reached the KV-cache capacity");
  }
  return NFAI_OK;
}

int set_state_word(nfai_model* m, size_t offset, uint32_t value, int slot) {
  nfai_ctx* c = m->ctx;
  // the copy reads the pinned word when it executes: every copy that may still be pending has its own slot
  c->pin_small[32 + slot] = value;
  CU(c, cudaMemcpyAsync((char*)m->state + offset, &c->pin_small[32 + slot], 4, cudaMemcpyHostToDevice, c->stream));
  return NFAI_OK;
}

// ---- tensor name -> destination -----------------------------------------------------------------------------
int resolve_target(nfai_model* m, const char* name, int src_dtype, const uint64_t* shape, int ndim, UploadTarget* t) {
  nfai_ctx* c = m->ctx;
  const nfai_hparams& hp = m->hp;
  const uint32_t n = c->world, r = c->rank;
  const uint32_t qDim = hp.qH * hp.d, kvDim = hp.kvH * hp.d;
  std::string s(name);
  t->name = s;
  t->src_dtype = src_dtype;
  t->received = 0;
  t->skip = false;
  t->done_flag = nullptr;
  IngestParams& ip = t->ip;
  ip = IngestParams();
  auto want = [&](uint64_t K, uint64_t N) -> int {
    bool ok = (N == 1) ? (ndim == 1 && shape[0] == K) || (ndim == 2 && shape[0] == K && shape[1] == 1)
                       : (ndim == 2 && shape[0] == K && shape[1] == N);
    if (!ok) return fail(c, NFAI_ERR_ARG, "tensor %s: shape does not match the model (want ne = [%llu, %llu])", name,
                         (unsigned long long)K, (unsigned long long)N);
    t->K = K;
    t->N = N;
    ip.K = K;
    ip.row_lo = 0; ip.row_hi = N; ip.col_lo = 0; ip.col_hi = K;
    ip.row_mul = 1; ip.row_off = 0; ip.ldd = K;
    return NFAI_OK;
  };
  auto gain = [&](Gain& g) -> int {
    int rc = want(hp.H, 1);
    if (rc) return rc;
    ip.dst = g.ptr;
    t->dst_dtype = NFAI_F32;
    t->done_flag = &g.done;
    return NFAI_OK;
  };
  t->dst_dtype = hp.weight_dtype;
  if (s == "token_embd.weight") {
    int rc = want(hp.H, hp.V);
    if (rc) return rc;
    ip.dst = m->embd.ptr;
    t->done_flag = &m->got_embd;
    return NFAI_OK;
  }
  if (s == "output_norm.weight") return gain(m->out_norm);
  if (s == "output.weight") {
    int rc = want(hp.H, hp.V);
    if (rc) return rc;
    if (hp.tied) {
      t->skip = true;  // the reference never reads it (NFAI.Models.Llama3/LlamaModel.cs:64-67)
      return NFAI_OK;
    }
    ip.row_lo = m->v_lo; ip.row_hi = m->v_lo + m->Vl;
    ip.dst = m->head.ptr;
    t->done_flag = &m->got_head;
    return NFAI_OK;
  }
  if (s.rfind("blk.", 0) == 0) {
    size_t dot = s.find('.', 4);
    if (dot == std::string::npos) return fail(c, NFAI_ERR_ARG, "bad tensor name %s", name);
    char* endp = nullptr;
    long li = strtol(s.c_str() + 4, &endp, 10);
    if (endp != s.c_str() + dot || li < 0 || li >= (long)hp.L) return fail(c, NFAI_ERR_ARG, "bad layer in %s", name);
    LayerW& L = m->layers[li];
    std::string rest = s.substr(dot + 1);
    if (rest == "attn_norm.weight") return gain(L.attn_norm);
    if (rest == "ffn_norm.weight") return gain(L.ffn_norm);
    int rc;
    if (rest == "attn_q.weight") {
      if ((rc = want(hp.H, qDim))) return rc;
      ip.row_lo = (uint64_t)r * m->qDimL; ip.row_hi = ip.row_lo + m->qDimL;
      ip.dst = L.qkv.ptr; t->done_flag = &L.got_q;
      return NFAI_OK;
    }
    if (rest == "attn_k.weight") {
      if ((rc = want(hp.H, kvDim))) return rc;
      ip.row_lo = (uint64_t)r * m->kvDimL; ip.row_hi = ip.row_lo + m->kvDimL; ip.row_off = m->qDimL;
      ip.dst = L.qkv.ptr; t->done_flag = &L.got_k;
      return NFAI_OK;
    }
    if (rest == "attn_v.weight") {
      if ((rc = want(hp.H, kvDim))) return rc;
      ip.row_lo = (uint64_t)r * m->kvDimL; ip.row_hi = ip.row_lo + m->kvDimL; ip.row_off = m->qDimL + m->kvDimL;
      ip.dst = L.qkv.ptr; t->done_flag = &L.got_v;
      return NFAI_OK;
    }
    if (rest == "attn_output.weight") {
      if ((rc = want(qDim, hp.H))) return rc;
      ip.col_lo = (uint64_t)r * m->qDimL; ip.col_hi = ip.col_lo + m->qDimL; ip.ldd = m->qDimL;
      ip.dst = L.o.ptr; t->done_flag = &L.got_o;
      return NFAI_OK;
    }
    if (rest == "ffn_gate.weight" || rest == "ffn_up.weight") {
      if ((rc = want(hp.H, hp.F))) return rc;
      bool is_up = rest == "ffn_up.weight";
      ip.row_lo = (uint64_t)r * m->Fl; ip.row_hi = ip.row_lo + m->Fl; ip.row_mul = 2; ip.row_off = is_up ? 1 : 0;
      ip.dst = L.gateup.ptr; t->done_flag = is_up ? &L.got_up : &L.got_gate;
      return NFAI_OK;
    }
    if (rest == "ffn_down.weight") {
      if ((rc = want(hp.F, hp.H))) return rc;
      ip.col_lo = (uint64_t)r * m->Fl; ip.col_hi = ip.col_lo + m->Fl; ip.ldd = m->Fl;
      ip.dst = L.down.ptr; t->done_flag = &L.got_down;
      return NFAI_OK;
    }
  }
  (void)n;
  return fail(c, NFAI_ERR_ARG, "unknown tensor name %s", name);
}

float half_bits_to_float(uint16_t h) { return __half2float(__ushort_as_half(h)); }

}  // namespace

// ---- context accessors for entry points that live in other translation units ---------------------------------
namespace nfai {
int ctx_device(const nfai_ctx* c) { return c->device; }
cudaStream_t ctx_stream(const nfai_ctx* c) { return c->stream; }
int ctx_fail(nfai_ctx* c, int code, const char* message) { return fail(c, code, "%s", message); }
}  // namespace nfai

// =============================================================================================================
extern "C" {

const char* nfai_version(void) { return "nfai_cuda 0.1 (sm_100a)"; }

const char* nfai_last_error(const nfai_ctx* ctx) { return ctx ? ctx->err.c_str() : g_err.c_str(); }

static int ctx_create_common(int device, int rank, int world, const void* uid, size_t uid_bytes, nfai_ctx** out) {
  if (!out) return fail(nullptr, NFAI_ERR_ARG, "out is null");
  *out = nullptr;
  if (world != 1 && world != 2 && world != 4 && world != 8) return fail(nullptr, NFAI_ERR_ARG, "world must be 1, 2, 4 or 8");
  if (rank < 0 || rank >= world) return fail(nullptr, NFAI_ERR_ARG, "rank out of range");
  int ndev = 0;
  cudaError_t e = cudaGetDeviceCount(&ndev);
  if (e != cudaSuccess) return fail(nullptr, NFAI_ERR_CUDA, "cudaGetDeviceCount: %s", cudaGetErrorString(e));
  if (device < 0 || device >= ndev) return fail(nullptr, NFAI_ERR_ARG, "device ordinal %d out of range (%d devices)", device, ndev);
  nfai_ctx* c = new nfai_ctx();
  c->device = device;
  c->rank = rank;
  c->world = world;
  c->pdl = env_int("NFAI_PDL", 1) != 0;
  c->use_graph = env_int("NFAI_GRAPH", 1) != 0;
  if (const char* w = getenv("NFAI_WAIT_NS")) {
    const unsigned long long ns = strtoull(w, nullptr, 10);
    if (ns) c->wait_ns = ns;
  }
  auto bail = [&](int code) {
    g_err = c->err;
    nfai_ctx_destroy(c);
    return code;
  };
#define CUB(call)                                                                                            \
  do {                                                                                                       \
    cudaError_t e__ = (call);                                                                                \
    if (e__ != cudaSuccess)                                                                                  \
      return bail(fail(c, e__ == cudaErrorMemoryAllocation ? NFAI_ERR_OOM : NFAI_ERR_CUDA, "%s: %s", #call, \
                       cudaGetErrorString(e__)));                                                            \
  } while (0)
  CUB(cudaSetDevice(device));
  CUB(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
  CUB(cudaEventCreate(&c->ev0));
  CUB(cudaEventCreate(&c->ev1));
  for (int i = 0; i < kStageSlots; ++i) {
    CUB(cudaHostAlloc(&c->stage[i], kStageBytes, cudaHostAllocDefault));
    CUB(cudaEventCreateWithFlags(&c->stage_ev[i], cudaEventDisableTiming));
  }
  CUB(cudaHostAlloc((void**)&c->pin_small, 256, cudaHostAllocDefault));
  CUB(cudaMalloc((void**)&c->dev_err, 256));
  CUB(cudaMemset(c->dev_err, 0, 256));
  memset(c->pin_small, 0, 256);
#undef CUB
  if (world > 1) {
    int rc = tp_create(&c->tp, device, rank, world, uid, uid_bytes, c->stream, c->err);
    if (rc != NFAI_OK) return bail(rc);
    tp_set_wait_ns(c->tp, c->wait_ns);
  }
  *out = c;
  return NFAI_OK;
}

int nfai_ctx_create(int device_ordinal, nfai_ctx** out) { return ctx_create_common(device_ordinal, 0, 1, nullptr, 0, out); }

int nfai_tp_unique_id(void* out, size_t out_bytes) {
  std::string err;
  int rc = tp_unique_id(out, out_bytes, err);
  if (rc) g_err = err;
  return rc;
}

int nfai_ctx_create_tp(int device_ordinal, int rank, int world, const void* nccl_uid, size_t uid_bytes, nfai_ctx** out) {
  if (world > 1 && (!nccl_uid || uid_bytes < 128)) return fail(nullptr, NFAI_ERR_ARG, "nccl_uid must hold 128 bytes");
  return ctx_create_common(device_ordinal, rank, world, nccl_uid, uid_bytes, out);
}

int nfai_tp_export_peer(nfai_ctx* c, void* out, size_t out_bytes) {
  if (!c) return fail(nullptr, NFAI_ERR_ARG, "ctx is null");
  if (!c->tp) return fail(c, NFAI_ERR_STATE, "not a tensor-parallel context");
  CU(c, cudaSetDevice(c->device));
  int rc = tp_export_peer_desc(c->tp, out, out_bytes, c->err);
  return rc;
}

int nfai_tp_import_peers(nfai_ctx* c, const void* descs, int n) {
  if (!c) return fail(nullptr, NFAI_ERR_ARG, "ctx is null");
  if (!c->tp) return fail(c, NFAI_ERR_STATE, "not a tensor-parallel context");
  CU(c, cudaSetDevice(c->device));
  return tp_import_peer_descs(c->tp, descs, n, c->err);
}

int nfai_ctx_destroy(nfai_ctx* c) {
  if (!c) return NFAI_OK;
  cudaSetDevice(c->device);
  if (c->stream) cudaStreamSynchronize(c->stream);
  if (c->tp) tp_destroy(c->tp);
  for (int i = 0; i < kStageSlots; ++i) {
    if (c->stage[i]) cudaFreeHost(c->stage[i]);
    if (c->stage_ev[i]) cudaEventDestroy(c->stage_ev[i]);
  }
  if (c->pin_small) cudaFreeHost(c->pin_small);
  if (c->dev_err) cudaFree(c->dev_err);
  if (c->ev0) cudaEventDestroy(c->ev0);
  if (c->ev1) cudaEventDestroy(c->ev1);
  if (c->stream) cudaStreamDestroy(c->stream);
  delete c;
  return NFAI_OK;
}

int nfai_model_create(nfai_ctx* c, const nfai_hparams* hp, nfai_model** out) {
  if (!c) return fail(nullptr, NFAI_ERR_ARG, "ctx is null");
  if (!hp || !out) return fail(c, NFAI_ERR_ARG, "null argument");
  *out = nullptr;
  if (!hp->H || !hp->L || !hp->qH || !hp->kvH || !hp->d || !hp->F || !hp->V || !hp->ctx)
    return fail(c, NFAI_ERR_ARG, "zero-sized hyper-parameter");
  if (hp->qH % hp->kvH) return fail(c, NFAI_ERR_ARG, "qH must be a multiple of kvH");
  if (hp->d != 32 && hp->d != 64 && hp->d != 128) return fail(c, NFAI_ERR_ARG, "head dim must be 32, 64 or 128");
  if (hp->ropeDim > hp->d || (hp->ropeDim & 1)) return fail(c, NFAI_ERR_ARG, "ropeDim must be even and <= d");
  if ((hp->weight_dtype != NFAI_F32 && hp->weight_dtype != NFAI_F16) || (hp->kv_dtype != NFAI_F32 && hp->kv_dtype != NFAI_F16))
    return fail(c, NFAI_ERR_ARG, "dtype must be NFAI_F32 or NFAI_F16");
  if (!(hp->eps >= 0.f) || !(hp->rope_theta > 0.f)) return fail(c, NFAI_ERR_ARG, "bad eps or rope_theta");
  const uint32_t n = c->world;
  if (hp->kvH % n || hp->F % n || hp->V % n) return fail(c, NFAI_ERR_ARG, "kvH, F and V must divide by the tensor-parallel width");
  if ((hp->F / n) % 2 && n > 1) return fail(c, NFAI_ERR_ARG, "F / world must be even");
  CU(c, cudaSetDevice(c->device));
  nfai_model* m = new nfai_model();
  m->ctx = c;
  m->hp = *hp;
  m->kvHl = hp->kvH / n;
  m->qHl = hp->qH / n;
  m->qDimL = m->qHl * hp->d;
  m->kvDimL = m->kvHl * hp->d;
  m->Fl = hp->F / n;
  m->Vl = hp->V / n;
  m->v_lo = c->rank * m->Vl;
  m->layers.resize(hp->L);
  const size_t ws = dtype_size(hp->weight_dtype);
  // one arena for every weight
  size_t off = 0;
  auto place = [&](Matrix& M, uint64_t rows, uint64_t cols) {
    M.rows = rows; M.cols = cols; M.bytes = rows * cols * ws;
    M.ptr = (void*)off;
    off = align_up(off + M.bytes, 256);
  };
  auto place_gain = [&](Gain& g) {
    g.ptr = (float*)off;
    off = align_up(off + (size_t)hp->H * 4, 256);
  };
  place(m->embd, hp->V, hp->H);
  if (!hp->tied) place(m->head, m->Vl, hp->H);
  place_gain(m->out_norm);
  for (auto& L : m->layers) {
    place(L.qkv, m->qDimL + 2 * m->kvDimL, hp->H);
    place(L.o, hp->H, m->qDimL);
    place(L.gateup, 2 * (uint64_t)m->Fl, hp->H);
    place(L.down, hp->H, m->Fl);
    place_gain(L.attn_norm);
    place_gain(L.ffn_norm);
  }
  m->warena_bytes = off;
  cudaError_t e = cudaMalloc((void**)&m->warena, off);
  if (e != cudaSuccess) {
    delete m;
    return fail(c, NFAI_ERR_OOM, "cudaMalloc of %zu weight bytes: %s", off, cudaGetErrorString(e));
  }
  auto fix = [&](void*& p) { p = m->warena + (size_t)p; };
  auto fixg = [&](Gain& g) { g.ptr = (float*)(m->warena + (size_t)g.ptr); };
  fix(m->embd.ptr);
  if (!hp->tied) fix(m->head.ptr);
  fixg(m->out_norm);
  for (auto& L : m->layers) {
    fix(L.qkv.ptr); fix(L.o.ptr); fix(L.gateup.ptr); fix(L.down.ptr);
    fixg(L.attn_norm); fixg(L.ffn_norm);
  }
  m->pf_look = (uint64_t)env_int("NFAI_PF_MB", 0) << 20;
  m->pf_extra = (uint64_t)env_int("NFAI_PF_EXTRA_MB", 0) << 20;
  m->pf_mode = env_int("NFAI_PF_MODE", 1);
  read_tune("QKV", m->tune_qkv, 2, 4);
  read_tune("O", m->tune_o, 2, 4);
  read_tune("GATEUP", m->tune_gateup, 2, 4);
  read_tune("DOWN", m->tune_down, 2, 4);
  read_tune("HEAD", m->tune_head, 2, 4);
  *out = m;
  return NFAI_OK;
}

int nfai_model_tensor_begin(nfai_model* m, const char* name, int src_dtype, const uint64_t* shape, int ndim) {
  if (!m) return fail(nullptr, NFAI_ERR_ARG, "model is null");
  nfai_ctx* c = m->ctx;
  if (m->finalized) return fail(c, NFAI_ERR_STATE, "model already finalized");
  if (m->up.active) return fail(c, NFAI_ERR_STATE, "tensor %s is still open", m->up.name.c_str());
  if (!name || !shape || ndim < 1 || ndim > 2) return fail(c, NFAI_ERR_ARG, "bad tensor description");
  if (src_dtype != NFAI_F32 && src_dtype != NFAI_F16) return fail(c, NFAI_ERR_ARG, "source dtype must be NFAI_F32 or NFAI_F16");
  UploadTarget t;
  int rc = resolve_target(m, name, src_dtype, shape, ndim, &t);
  if (rc) return rc;
  t.active = true;
  m->up = t;
  return NFAI_OK;
}

int nfai_model_tensor_chunk(nfai_model* m, const void* bytes, size_t nbytes) {
  if (!m) return fail(nullptr, NFAI_ERR_ARG, "model is null");
  nfai_ctx* c = m->ctx;
  if (!m->up.active) return fail(c, NFAI_ERR_STATE, "no tensor is open");
  if (!bytes && nbytes) return fail(c, NFAI_ERR_ARG, "bytes is null");
  UploadTarget& t = m->up;
  const size_t es = dtype_size(t.src_dtype);
  if (nbytes % es) return fail(c, NFAI_ERR_ARG, "chunk size is not a multiple of the element size");
  const uint64_t total = t.K * t.N;
  if (t.received + nbytes / es > total) return fail(c, NFAI_ERR_ARG, "tensor %s: more data than its shape holds", t.name.c_str());
  if (t.skip) {
    t.received += nbytes / es;
    return NFAI_OK;
  }
  CU(c, cudaSetDevice(c->device));
  size_t done = 0;
  while (done < nbytes) {
    size_t piece = nbytes - done < kStageBytes ? nbytes - done : kStageBytes;
    int slot = c->stage_next;
    c->stage_next = (slot + 1) % kStageSlots;
    CU(c, cudaEventSynchronize(c->stage_ev[slot]));  // the kernel that last read this slot has finished
    memcpy(c->stage[slot], (const char*)bytes + done, piece);
    IngestParams ip = t.ip;
    ip.src = c->stage[slot];  // pinned memory is read by the kernel in place (one pass over PCIe)
    ip.n = piece / es;
    ip.elem_off = t.received;
    CU(c, launch_ingest(c->stream, t.src_dtype, t.dst_dtype, ip));
    CU(c, cudaEventRecord(c->stage_ev[slot], c->stream));
    t.received += piece / es;
    done += piece;
  }
  return NFAI_OK;
}

int nfai_model_tensor_end(nfai_model* m) {
  if (!m) return fail(nullptr, NFAI_ERR_ARG, "model is null");
  nfai_ctx* c = m->ctx;
  if (!m->up.active) return fail(c, NFAI_ERR_STATE, "no tensor is open");
  UploadTarget& t = m->up;
  t.active = false;
  if (t.received != t.K * t.N)
    return fail(c, NFAI_ERR_ARG, "tensor %s: got %llu of %llu elements", t.name.c_str(), (unsigned long long)t.received,
                (unsigned long long)(t.K * t.N));
  if (t.done_flag) *t.done_flag = true;
  return NFAI_OK;
}

int nfai_model_finalize(nfai_model* m) {
  if (!m) return fail(nullptr, NFAI_ERR_ARG, "model is null");
  nfai_ctx* c = m->ctx;
  if (m->finalized) return fail(c, NFAI_ERR_STATE, "model already finalized");
  if (m->up.active) return fail(c, NFAI_ERR_STATE, "tensor %s is still open", m->up.name.c_str());
  const nfai_hparams& hp = m->hp;
  if (!m->got_embd || !m->out_norm.done || (!hp.tied && !m->got_head)) return fail(c, NFAI_ERR_STATE, "missing token_embd / output_norm / output tensors");
  for (uint32_t l = 0; l < hp.L; ++l) {
    const LayerW& L = m->layers[l];
    if (!(L.got_q && L.got_k && L.got_v && L.got_o && L.got_gate && L.got_up && L.got_down && L.attn_norm.done && L.ffn_norm.done))
      return fail(c, NFAI_ERR_STATE, "layer %u is missing tensors", l);
  }
  CU(c, cudaSetDevice(c->device));
  CU(c, cudaStreamSynchronize(c->stream));
  // LM-head launch shape decides how many arg-max partials there are
  m->nparts = gemv_grid(hp.weight_dtype, EPI_LOGITS, [&] { GemvParams p; p.N = m->Vl; p.K = hp.H; p.W = (void*)256; return p; }(), m->tune_head);
  // short caches: one CTA per query head (K and V of a KV head are re-read from L2 by its heads, the whole
  // context is in flight at once); long caches: the heads of a KV group share one pass over K and V
  m->attn_heads = hp.ctx <= 4096 ? 1u : kAttnHeadsPerCta;
  if (env_int("NFAI_ATTN_HEADS", 0) > 0) m->attn_heads = (uint32_t)env_int("NFAI_ATTN_HEADS", 0);
  if (m->attn_heads != 1 && m->attn_heads != 2 && m->attn_heads != 4) m->attn_heads = kAttnHeadsPerCta;
  m->S_max = attn_splits(m->qHl, m->kvHl, hp.ctx, m->attn_heads, kAttnMinChunk);
  const size_t kvs = dtype_size(hp.kv_dtype);
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes, 256); return o; };
  const size_t o_kc = take((size_t)hp.L * kv_layer_elems(m) * kvs);
  const size_t o_vc = take((size_t)hp.L * kv_layer_elems(m) * kvs);
  const size_t o_rope = take((size_t)hp.ctx * (hp.ropeDim / 2) * sizeof(float2) + 16);
  const size_t o_x = take((size_t)(2 * hp.L + 1) * hp.H * 4);
  const size_t o_q = take((size_t)m->qDimL * 4);
  const size_t o_ao = take((size_t)m->qDimL * 4);
  const size_t o_h = take((size_t)m->Fl * 4);
  const size_t o_lg = take((size_t)m->Vl * 4);
  // room for every launch shape nfai_model_tune may select later (up to 16 CTAs per SM)
  const size_t npart_alloc = (size_t)sm_count() * 16;
  m->nparts_alloc = (uint32_t)npart_alloc;
  const size_t o_pv = take(npart_alloc * 4);
  const size_t o_pi = take(npart_alloc * 4);
  const uint32_t S_alloc = m->S_max;
  const size_t o_ap = take(attn_part_floats(m->qHl, hp.d, S_alloc) * 4);
  const size_t o_tk = take((size_t)m->qHl * 4);  // one ticket per (kv head, head group); at most one per query head
  const size_t o_st = take(sizeof(StepState));
  const size_t o_hi = take((size_t)hp.ctx * 4);
  const size_t o_pr = take((size_t)hp.ctx * 4);
  const size_t o_tp = take((size_t)hp.H * 4);
  // batched prompt workspace
  const bool want_pf = hp.weight_dtype == NFAI_F16 && env_int("NFAI_PREFILL_GEMM", 1) != 0 &&
                       hp.H % 8 == 0 && m->qDimL % 8 == 0 && m->Fl % 8 == 0;
  // tokens per pass of the batched prompt path: long passes amortise ~130 launches per pass and fill the GEMM grids
  uint32_t pf_want = (uint32_t)env_int("NFAI_PREFILL_CHUNK", 2048);
  if (pf_want < 8) pf_want = 8;
  if (pf_want > 8192) pf_want = 8192;
  const uint32_t pfc = want_pf ? (hp.ctx < pf_want ? hp.ctx : pf_want) : 0;
  const uint32_t amax = hp.H > m->qDimL ? hp.H : m->qDimL;
  const size_t o_px0 = take((size_t)pfc * hp.H * 4);
  const size_t o_px1 = take((size_t)pfc * hp.H * 4);
  const size_t o_pa = take((size_t)pfc * amax * 2);
  const size_t o_pq = take((size_t)pfc * m->qDimL * 4);
  const size_t o_pao = take((size_t)pfc * m->qDimL * 2);
  const size_t o_ph = take((size_t)pfc * m->Fl * 2);
  const size_t o_pt = take((size_t)pfc * 4 + 4);
  // split-K happens only below 120 output tiles of 128 x 128, with at most one CTA per SM: that many tiles of partials bound it
  const size_t pf_part_floats = want_pf && env_int("NFAI_GEMM_SPLIT", 1) ? (size_t)sm_count() * 128 * 128 * 2 : 0;
  const size_t o_pp = take(pf_part_floats * 4);
  const size_t o_ss = take(sample_scratch_bytes(m->Vl, nullptr));
  cudaError_t e = cudaMalloc((void**)&m->rarena, off);
  if (e != cudaSuccess) return fail(c, NFAI_ERR_OOM, "cudaMalloc of %zu run-time bytes (KV cache etc.): %s", off, cudaGetErrorString(e));
  CU(c, cudaMemsetAsync(m->rarena, 0, off, c->stream));
  m->kc = m->rarena + o_kc; m->vc = m->rarena + o_vc;
  // long float16 caches: attention through tile-staged rings (NFAI_ATTN_RING=0 keeps the register streamer, 1 forces it)
  m->attn_maps.clear();
  // long float16 caches: attention on the tensor cores (NFAI_ATTN_MMA=0: the tile-staged CUDA-core kernel instead)
  m->attn_mma = m->attn_heads == 4 && attn_mma_supported(hp.kv_dtype, hp.d) && ring_wanted(hp.ctx) && env_int("NFAI_ATTN_MMA", 1) != 0;
  if (!m->attn_mma && m->attn_heads == 4 && attn_ring_supported(hp.kv_dtype, hp.d) && ring_wanted(hp.ctx)) {
    m->attn_maps.resize(hp.L);
    for (uint32_t l = 0; l < hp.L; ++l) {
      const size_t lo = (size_t)l * kv_layer_elems(m) * kvs;
      if (attn_ring_make_maps((char*)m->kc + lo, (char*)m->vc + lo, hp.ctx, m->kvDimL, hp.d, &m->attn_maps[l]) != cudaSuccess) {
        m->attn_maps.clear();  // no tile descriptors on this driver: the register streamer serves every length
        break;
      }
    }
  }
  m->rope_cs = (float2*)(m->rarena + o_rope);
  m->xbuf = (float*)(m->rarena + o_x);
  m->q = (float*)(m->rarena + o_q);
  m->attn_out = (float*)(m->rarena + o_ao);
  m->hbuf = (float*)(m->rarena + o_h);
  m->logits = (float*)(m->rarena + o_lg);
  m->part_val = (float*)(m->rarena + o_pv);
  m->part_idx = (uint32_t*)(m->rarena + o_pi);
  m->attn_part = (float*)(m->rarena + o_ap);
  m->tickets = (uint32_t*)(m->rarena + o_tk);
  m->state = (StepState*)(m->rarena + o_st);
  m->history = (uint32_t*)(m->rarena + o_hi);
  m->prompt = (uint32_t*)(m->rarena + o_pr);
  m->tp_buf = (float*)(m->rarena + o_tp);
  m->prefill_gemm = want_pf && pfc > 0;
  m->pf_chunk = pfc;
  m->pfX0 = (float*)(m->rarena + o_px0);
  m->pfX1 = (float*)(m->rarena + o_px1);
  m->pfA = (__half*)(m->rarena + o_pa);
  m->pfQ = (float*)(m->rarena + o_pq);
  m->pfAO = (__half*)(m->rarena + o_pao);
  m->pfH = (__half*)(m->rarena + o_ph);
  m->pfTok = (uint32_t*)(m->rarena + o_pt);
  m->pfPart = pf_part_floats ? (float*)(m->rarena + o_pp) : nullptr;
  m->pfPartFloats = pf_part_floats;
  m->sample_scratch = m->rarena + o_ss;
  // RoPE table on the host, float32, as the reference builds its frequency table
  // (NFAI.Vulkan.Shaders/TransformerBlock.cs:33-38) and its shader forms theta = f[m] * float(pos)
  // (NFAI.Vulkan.Shaders/RoPEShader.cs:252-254); cos/sin from the host libm.
  {
    const uint32_t half = hp.ropeDim / 2;
    std::vector<float> f(half);
    for (uint32_t i = 0; i < half; ++i) f[i] = 1.0f / powf(hp.rope_theta, (float)i / ((float)hp.ropeDim / 2));
    std::vector<float2> tab((size_t)hp.ctx * half);
    for (uint32_t p = 0; p < hp.ctx; ++p)
      for (uint32_t i = 0; i < half; ++i) {
        float theta = f[i] * (float)p;
        tab[(size_t)p * half + i] = make_float2(cosf(theta), sinf(theta));
      }
    if (!tab.empty()) CU(c, cudaMemcpy(m->rope_cs, tab.data(), tab.size() * sizeof(float2), cudaMemcpyHostToDevice));
  }
  CU(c, cudaHostAlloc((void**)&m->pin_logits, (size_t)hp.V * 4, cudaHostAllocDefault));
  CU(c, cudaStreamSynchronize(c->stream));
  if (c->use_graph) {
    int rc = capture(m, true, false, &m->g_full, &m->launches_full);
    if (rc) return rc;
    rc = capture(m, false, true, &m->g_nohead, nullptr);
    if (rc) return rc;
  } else {
    m->launches_full = 3 + 5 * (int)hp.L;
  }
  m->pos = 0;
  m->finalized = true;
  return NFAI_OK;
}

int nfai_model_destroy(nfai_model* m) {
  if (!m) return NFAI_OK;
  nfai_ctx* c = m->ctx;
  cudaSetDevice(c->device);
  cudaStreamSynchronize(c->stream);
  if (m->g_full) cudaGraphExecDestroy(m->g_full);
  if (m->g_nohead) cudaGraphExecDestroy(m->g_nohead);
  if (m->pin_logits) cudaFreeHost(m->pin_logits);
  if (m->rarena) cudaFree(m->rarena);
  if (m->warena) cudaFree(m->warena);
  delete m;
  return NFAI_OK;
}

static int ready(nfai_model* m) {
  if (!m) return fail(nullptr, NFAI_ERR_ARG, "model is null");
  if (!m->finalized) return fail(m->ctx, NFAI_ERR_STATE, "model is not finalized");
  cudaError_t e = cudaSetDevice(m->ctx->device);
  if (e != cudaSuccess) return fail(m->ctx, NFAI_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(e));
  return NFAI_OK;
}

static int fetch_outputs(nfai_model* m, float* logits, uint32_t* argmax) {
  nfai_ctx* c = m->ctx;
  const nfai_hparams& hp = m->hp;
  if (logits) {
    if (c->world > 1) {
      int rc = tp_allgather_logits(c->tp, c->stream, m->logits, m->Vl, m->pin_logits, c->err);
      if (rc) return rc;
    } else {
      CU(c, cudaMemcpyAsync(m->pin_logits, m->logits, (size_t)hp.V * 4, cudaMemcpyDeviceToHost, c->stream));
    }
  }
  StepState st;
  int rc = check_state(m, &st);  // synchronises the stream
  if (rc) return rc;
  if (logits) memcpy(logits, m->pin_logits, (size_t)hp.V * 4);
  if (argmax) *argmax = st.last_argmax;
  return NFAI_OK;
}

int nfai_decode(nfai_model* m, uint32_t token, float* logits, uint32_t* argmax) {
  int rc = ready(m);
  if (rc) return rc;
  nfai_ctx* c = m->ctx;
  if (m->pos >= m->hp.ctx) return fail(c, NFAI_ERR_CONTEXT_FULL, "position %u reached the KV-cache capacity %u", m->pos, m->hp.ctx);
  if (token >= m->hp.V) return fail(c, NFAI_ERR_ARG, "token id %u out of range (V = %u)", token, m->hp.V);
  if ((rc = set_state_word(m, offsetof(StepState, cur_token), token, 0))) return rc;
  if ((rc = run_step(m, true, false))) return rc;
  m->pos += 1;
  return fetch_outputs(m, logits, argmax);
}

// Batched prompt ingestion (float16 weights): every projection of a chunk of tokens is one tensor-core GEMM, the
// causal attention one kernel per layer; K and V rows land in the cache exactly where the token-by-token path puts
// them. The LM head runs for the last token only (the reference evaluates and discards it for every prompt token:
// NFAI.Models.Llama3/LlamaModel.cs:103-126).
static int prefill_batched(nfai_model* m, const uint32_t* tokens, int n) {
  nfai_ctx* c = m->ctx;
  const nfai_hparams& hp = m->hp;
  cudaStream_t s = c->stream;
  const int kvdt = hp.kv_dtype;
  const size_t kvs = dtype_size(kvdt);
  uint32_t* err = &m->state->err;
  uint32_t pos0 = m->pos;
  const bool tp_on = c->world > 1;
  int done = 0;
  while (done < n) {
    const uint32_t T = (uint32_t)(n - done) < m->pf_chunk ? (uint32_t)(n - done) : m->pf_chunk;
    const bool last_chunk = done + (int)T == n;
    CU(c, cudaMemcpyAsync(m->pfTok, tokens + done, (size_t)T * 4, cudaMemcpyHostToDevice, s));
    CU(c, launch_embed_rows(s, (const __half*)m->embd.ptr, m->pfTok, T, hp.H, m->pfX0));
    for (uint32_t l = 0; l < hp.L; ++l) {
      const LayerW& L = m->layers[l];
      char* kcl = (char*)m->kc + (size_t)l * kv_layer_elems(m) * kvs;
      char* vcl = (char*)m->vc + (size_t)l * kv_layer_elems(m) * kvs;
      CU(c, launch_rmsnorm_to_half(s, m->pfX0, L.attn_norm.ptr, hp.eps, T, hp.H, m->pfA, tp_on && l > 0));
      GemmEpilogue eq;
      eq.kind = GEMM_EPI_QKV_ROPE;
      eq.scratch = m->pfPart; eq.scratch_floats = m->pfPartFloats;
      eq.out_f32 = m->pfQ; eq.kcache = kcl; eq.vcache = vcl; eq.kv_f16 = kvdt == NFAI_F16;
      eq.qDim = m->qDimL; eq.kvDim = m->kvDimL; eq.d = hp.d; eq.ropeDim = hp.ropeDim; eq.pos0 = pos0; eq.rope_cs = m->rope_cs;
      CU(c, launch_gemm_tc(s, m->pfA, (const __half*)L.qkv.ptr, T, m->qDimL + 2 * m->kvDimL, hp.H, eq, err));
      AttnParams a;
      a.q = m->pfQ; a.kcache = kcl; a.vcache = vcl; a.qH = m->qHl; a.kvH = m->kvHl; a.d = hp.d;
      a.seq_imm = pos0 + 1; a.out_half = m->pfAO;
      if (attn_prefill_tc_supported(hp.d) && env_int("NFAI_PREFILL_ATTN", 1) != 0) CU(c, launch_attn_prefill_tc(s, kvdt, a, T));
      else CU(c, launch_attn_prefill(s, kvdt, a, T));
      // Tensor parallel: the O and down GEMMs produce this rank's partial [T][H]; rank 0 adds the residual into its
      // partial and one NCCL all-reduce per GEMM makes the sums (bit-identical on every rank).
      const bool add_resid = !tp_on || c->rank == 0;
      GemmEpilogue eo;
      eo.kind = GEMM_EPI_STORE; eo.out_f32 = m->pfX1; eo.resid = add_resid ? m->pfX0 : nullptr;
      eo.scratch = m->pfPart; eo.scratch_floats = m->pfPartFloats;
      CU(c, launch_gemm_tc(s, m->pfAO, (const __half*)L.o.ptr, T, hp.H, m->qDimL, eo, err));
      if (tp_on) CU(c, tp_allreduce(c->tp, s, m->pfX1, (size_t)T * hp.H));
      CU(c, launch_rmsnorm_to_half(s, m->pfX1, L.ffn_norm.ptr, hp.eps, T, hp.H, m->pfA, tp_on));
      GemmEpilogue eg;
      eg.kind = GEMM_EPI_SILU_MUL; eg.out_f16 = m->pfH;
      eg.scratch = m->pfPart; eg.scratch_floats = m->pfPartFloats;
      CU(c, launch_gemm_tc(s, m->pfA, (const __half*)L.gateup.ptr, T, 2 * m->Fl, hp.H, eg, err));
      GemmEpilogue ed;
      ed.kind = GEMM_EPI_STORE; ed.out_f32 = m->pfX0; ed.resid = add_resid ? m->pfX1 : nullptr;
      ed.scratch = m->pfPart; ed.scratch_floats = m->pfPartFloats;
      CU(c, launch_gemm_tc(s, m->pfH, (const __half*)L.down.ptr, T, hp.H, m->Fl, ed, err));
      if (tp_on) CU(c, tp_allreduce(c->tp, s, m->pfX0, (size_t)T * hp.H));
      if (last_chunk)  // the last token's residual stream after this block, where the taps and the LM head expect it
        CU(c, cudaMemcpyAsync(x_in(m, l + 1), m->pfX0 + (size_t)(T - 1) * hp.H, (size_t)hp.H * 4, cudaMemcpyDeviceToDevice, s));
    }
    pos0 += T;
    done += (int)T;
  }
  // LM head + arg-max for the last token; the finishing kernel advances the position by one
  int rc = set_state_word(m, offsetof(StepState, pos), pos0 - 1, 3);
  if (rc) return rc;
  GemvParams gh = head_params(m);
  if (c->world == 1) {
    CU(c, launch_gemv(s, hp.weight_dtype, kvdt, EPI_LOGITS, gh, m->tune_head, false));
    CU(c, launch_argmax_final(s, m->part_val, m->part_idx, m->nparts, m->state, nullptr, m->history, hp.ctx, PrefetchPlan(),
                              nullptr, 0, XchgHooks(), false));
    return NFAI_OK;
  }
  // vocabulary-sharded head: the ranks' best (value, index) pairs are exchanged as in a decode step, counted as
  // one exchange of this context
  if (tp_push_ready(c->tp)) {
    gh.tp = tp_hooks(c->tp);
    gh.tp.push = 1;
    gh.tp.push_index = 0;
    gh.v_lo = m->v_lo;
    gh.tp_ticket = tp_ticket_ptr(c->tp);
    CU(c, launch_gemv(s, hp.weight_dtype, kvdt, EPI_LOGITS, gh, m->tune_head, false));
    XchgHooks fin = tp_hooks(c->tp);
    fin.pull = 1;
    fin.pull_index = 0;
    CU(c, launch_argmax_final(s, m->part_val, m->part_idx, (uint32_t)c->world, m->state, nullptr, m->history, hp.ctx,
                              PrefetchPlan(), tp_epoch_ptr(c->tp), 1, fin, false));
  } else {
    CU(c, launch_gemv(s, hp.weight_dtype, kvdt, EPI_LOGITS, gh, m->tune_head, false));
    CU(c, tp_gather_argmax(c->tp, s, m->part_val, m->part_idx, m->nparts, m->v_lo, nullptr));
    CU(c, launch_argmax_final(s, m->part_val, m->part_idx, (uint32_t)c->world, m->state, nullptr, m->history, hp.ctx,
                              PrefetchPlan(), nullptr, 0, XchgHooks(), false));
  }
  return NFAI_OK;
}

int nfai_prefill(nfai_model* m, const uint32_t* tokens, int n, float* logits_last, uint32_t* argmax_last) {
  int rc = ready(m);
  if (rc) return rc;
  nfai_ctx* c = m->ctx;
  if (!tokens || n <= 0) return fail(c, NFAI_ERR_ARG, "empty prompt");
  if ((uint64_t)m->pos + (uint64_t)n > m->hp.ctx)
    return fail(c, NFAI_ERR_CONTEXT_FULL, "prompt of %d tokens at position %u exceeds the KV-cache capacity %u", n, m->pos, m->hp.ctx);
  for (int i = 0; i < n; ++i)
    if (tokens[i] >= m->hp.V) return fail(c, NFAI_ERR_ARG, "token id %u out of range (V = %u)", tokens[i], m->hp.V);
  if (m->prefill_gemm && n >= 8) {
    if ((rc = prefill_batched(m, tokens, n))) return rc;
    m->pos += (uint32_t)n;
    return fetch_outputs(m, logits_last, argmax_last);
  }
  if (n > 1) {
    CU(c, cudaMemcpyAsync(m->prompt, tokens, (size_t)(n - 1) * 4, cudaMemcpyHostToDevice, c->stream));
    if ((rc = set_state_word(m, offsetof(StepState, prompt_idx), 0, 1))) return rc;
    for (int i = 0; i < n - 1; ++i)
      if ((rc = run_step(m, false, true))) return rc;
  }
  if ((rc = set_state_word(m, offsetof(StepState, cur_token), tokens[n - 1], 0))) return rc;
  if ((rc = run_step(m, true, false))) return rc;
  m->pos += (uint32_t)n;
  return fetch_outputs(m, logits_last, argmax_last);
}

int nfai_decode_greedy(nfai_model* m, uint32_t first_token, int n_steps, uint32_t* out_tokens, float* elapsed_ms) {
  int rc = ready(m);
  if (rc) return rc;
  nfai_ctx* c = m->ctx;
  if (n_steps <= 0) return fail(c, NFAI_ERR_ARG, "n_steps must be positive");
  if ((uint64_t)m->pos + (uint64_t)n_steps > m->hp.ctx)
    return fail(c, NFAI_ERR_CONTEXT_FULL, "%d steps from position %u exceed the KV-cache capacity %u", n_steps, m->pos, m->hp.ctx);
  if (first_token >= m->hp.V) return fail(c, NFAI_ERR_ARG, "token id %u out of range (V = %u)", first_token, m->hp.V);
  if ((rc = set_state_word(m, offsetof(StepState, cur_token), first_token, 0))) return rc;
  if ((rc = set_state_word(m, offsetof(StepState, steps), 0, 2))) return rc;
  CU(c, cudaEventRecord(c->ev0, c->stream));
  for (int i = 0; i < n_steps; ++i)
    if ((rc = run_step(m, true, false))) return rc;
  CU(c, cudaEventRecord(c->ev1, c->stream));
  m->pos += (uint32_t)n_steps;
  if ((rc = check_state(m, nullptr))) return rc;
  if (elapsed_ms) CU(c, cudaEventElapsedTime(elapsed_ms, c->ev0, c->ev1));
  if (out_tokens) CU(c, cudaMemcpy(out_tokens, m->history, (size_t)n_steps * 4, cudaMemcpyDeviceToHost));
  return NFAI_OK;
}

int nfai_model_get_hparams(const nfai_model* m, nfai_hparams* out) {
  if (!m || !out) return fail(m ? m->ctx : nullptr, NFAI_ERR_ARG, "null argument");
  *out = m->hp;
  return NFAI_OK;
}

int nfai_sample_top_p(nfai_model* m, float temperature, float top_p, int top_k, float u, uint32_t* token_out) {
  int rc = ready(m);
  if (rc) return rc;
  nfai_ctx* c = m->ctx;
  if (!token_out || !(temperature > 0.f) || !(top_p > 0.f) || top_k < 1 || top_k > 64 || !(u >= 0.f && u < 1.f))
    return fail(c, NFAI_ERR_ARG, "bad sampling parameters (temperature > 0, top_p > 0, 1 <= top_k <= 64, 0 <= u < 1)");
  if (c->world != 1) return fail(c, NFAI_ERR_STATE, "on-device sampling needs the whole vocabulary on one GPU");
  if (m->pos == 0) return fail(c, NFAI_ERR_STATE, "no step has produced logits yet");
  uint32_t* dev_tok = c->dev_err + 8;
  CU(c, launch_sample_top_p(c->stream, m->logits, m->hp.V, &m->state->last_argmax, &m->state->cur_token, temperature, top_p,
                            top_k, u, m->sample_scratch, dev_tok));
  CU(c, cudaMemcpyAsync(c->pin_small + 16, dev_tok, 4, cudaMemcpyDeviceToHost, c->stream));
  CU(c, cudaStreamSynchronize(c->stream));
  if (c->pin_small[16] == 0xffffffffu) return fail(c, NFAI_ERR_STATE, "the logits buffer and the step's arg-max are out of step");
  *token_out = c->pin_small[16];
  return NFAI_OK;
}

int nfai_decode_sampled(nfai_model* m, uint32_t first_token, int n_steps, float temperature, float top_p, int top_k,
                        const float* u, uint32_t* out_tokens, float* elapsed_ms) {
  int rc = ready(m);
  if (rc) return rc;
  nfai_ctx* c = m->ctx;
  if (n_steps <= 0 || !u) return fail(c, NFAI_ERR_ARG, "n_steps must be positive and u must hold one number per step");
  if (!(temperature > 0.f) || !(top_p > 0.f) || top_k < 1 || top_k > 64)
    return fail(c, NFAI_ERR_ARG, "bad sampling parameters (temperature > 0, top_p > 0, 1 <= top_k <= 64)");
  for (int i = 0; i < n_steps; ++i)
    if (!(u[i] >= 0.f && u[i] < 1.f)) return fail(c, NFAI_ERR_ARG, "u[%d] is outside [0, 1)", i);
  if (c->world != 1) return fail(c, NFAI_ERR_STATE, "on-device sampling needs the whole vocabulary on one GPU");
  if ((uint64_t)m->pos + (uint64_t)n_steps > m->hp.ctx)
    return fail(c, NFAI_ERR_CONTEXT_FULL, "%d steps from position %u exceed the KV-cache capacity %u", n_steps, m->pos, m->hp.ctx);
  if (first_token >= m->hp.V) return fail(c, NFAI_ERR_ARG, "token id %u out of range (V = %u)", first_token, m->hp.V);
  if ((rc = set_state_word(m, offsetof(StepState, cur_token), first_token, 0))) return rc;
  if ((rc = set_state_word(m, offsetof(StepState, steps), 0, 2))) return rc;
  CU(c, cudaEventRecord(c->ev0, c->stream));
  for (int i = 0; i < n_steps; ++i) {
    // the step leaves logits, arg-max and history[i] = arg-max; the sampler then puts the drawn token into history[i]
    // and into cur_token, which the next step embeds -- nothing returns to the host inside the loop
    if ((rc = run_step(m, true, false))) return rc;
    CU(c, launch_sample_top_p(c->stream, m->logits, m->hp.V, &m->state->last_argmax, &m->state->cur_token, temperature, top_p,
                              top_k, u[i], m->sample_scratch, m->history + i));
  }
  CU(c, cudaEventRecord(c->ev1, c->stream));
  m->pos += (uint32_t)n_steps;
  if ((rc = check_state(m, nullptr))) return rc;
  if (elapsed_ms) CU(c, cudaEventElapsedTime(elapsed_ms, c->ev0, c->ev1));
  std::vector<uint32_t> toks((size_t)n_steps);
  CU(c, cudaMemcpy(toks.data(), m->history, (size_t)n_steps * 4, cudaMemcpyDeviceToHost));
  for (int i = 0; i < n_steps; ++i)
    if (toks[i] == 0xffffffffu) return fail(c, NFAI_ERR_STATE, "step %d: the logits buffer and the step's arg-max are out of step", i);
  if (out_tokens) memcpy(out_tokens, toks.data(), (size_t)n_steps * 4);
  return NFAI_OK;
}

int nfai_position(const nfai_model* m, uint32_t* pos) {
  if (!m || !pos) return fail(m ? m->ctx : nullptr, NFAI_ERR_ARG, "null argument");
  *pos = m->pos;
  return NFAI_OK;
}

int nfai_set_position(nfai_model* m, uint32_t pos) {
  int rc = ready(m);
  if (rc) return rc;
  if (pos > m->hp.ctx) return fail(m->ctx, NFAI_ERR_ARG, "position beyond the KV-cache capacity");
  if ((rc = set_state_word(m, offsetof(StepState, pos), pos, 3))) return rc;
  CU(m->ctx, cudaStreamSynchronize(m->ctx->stream));
  m->pos = pos;
  return NFAI_OK;
}

int nfai_reset(nfai_model* m) { return nfai_set_position(m, 0); }

}  // extern "C"

// A copy of everything a later turn needs to continue from this point: the cache rows of positions 0 .. pos-1 of every
// layer, the logits and arg-max of the last step, and the position.
struct nfai_kv_snapshot {
  nfai_model* owner = nullptr;
  int device = 0;
  uint32_t pos = 0, cur_token = 0, last_argmax = 0;
  char* dev = nullptr;
  size_t row_bytes = 0;  // bytes of K (or V) of one layer: pos * kvDim * element size
};

extern "C" {

int nfai_kv_snapshot_create(nfai_model* m, nfai_kv_snapshot** out) {
  int rc = ready(m);
  if (rc) return rc;
  nfai_ctx* c = m->ctx;
  if (!out) return fail(c, NFAI_ERR_ARG, "null output");
  const nfai_hparams& hp = m->hp;
  const size_t kvs = dtype_size(hp.kv_dtype);
  StepState st;
  if ((rc = check_state(m, &st))) return rc;
  nfai_kv_snapshot* s = new nfai_kv_snapshot();
  s->owner = m;
  s->device = c->device;
  s->pos = m->pos;
  s->cur_token = st.cur_token;
  s->last_argmax = st.last_argmax;
  s->row_bytes = (size_t)m->pos * m->kvDimL * kvs;
  const size_t total = 2 * (size_t)hp.L * s->row_bytes + (size_t)m->Vl * 4;
  cudaError_t e = cudaMalloc((void**)&s->dev, total);
  if (e != cudaSuccess) {
    delete s;
    return fail(c, NFAI_ERR_OOM, "cudaMalloc of %zu snapshot bytes: %s", total, cudaGetErrorString(e));
  }
  for (uint32_t l = 0; l < hp.L && e == cudaSuccess; ++l) {
    const size_t lo = (size_t)l * kv_layer_elems(m) * kvs;
    if (s->row_bytes) {
      e = cudaMemcpyAsync(s->dev + (2 * (size_t)l) * s->row_bytes, (char*)m->kc + lo, s->row_bytes, cudaMemcpyDeviceToDevice, c->stream);
      if (e == cudaSuccess)
        e = cudaMemcpyAsync(s->dev + (2 * (size_t)l + 1) * s->row_bytes, (char*)m->vc + lo, s->row_bytes, cudaMemcpyDeviceToDevice, c->stream);
    }
  }
  if (e == cudaSuccess)
    e = cudaMemcpyAsync(s->dev + 2 * (size_t)hp.L * s->row_bytes, m->logits, (size_t)m->Vl * 4, cudaMemcpyDeviceToDevice, c->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
  if (e != cudaSuccess) {
    cudaFree(s->dev);
    delete s;
    return fail(c, NFAI_ERR_CUDA, "snapshot copy: %s", cudaGetErrorString(e));
  }
  *out = s;
  return NFAI_OK;
}

int nfai_kv_snapshot_restore(nfai_model* m, const nfai_kv_snapshot* s) {
  int rc = ready(m);
  if (rc) return rc;
  nfai_ctx* c = m->ctx;
  if (!s || s->owner != m) return fail(c, NFAI_ERR_ARG, "the snapshot was not taken from this model");
  const nfai_hparams& hp = m->hp;
  const size_t kvs = dtype_size(hp.kv_dtype);
  CU(c, cudaSetDevice(c->device));
  for (uint32_t l = 0; l < hp.L; ++l) {
    const size_t lo = (size_t)l * kv_layer_elems(m) * kvs;
    if (s->row_bytes) {
      CU(c, cudaMemcpyAsync((char*)m->kc + lo, s->dev + (2 * (size_t)l) * s->row_bytes, s->row_bytes, cudaMemcpyDeviceToDevice, c->stream));
      CU(c, cudaMemcpyAsync((char*)m->vc + lo, s->dev + (2 * (size_t)l + 1) * s->row_bytes, s->row_bytes, cudaMemcpyDeviceToDevice, c->stream));
    }
  }
  CU(c, cudaMemcpyAsync(m->logits, s->dev + 2 * (size_t)hp.L * s->row_bytes, (size_t)m->Vl * 4, cudaMemcpyDeviceToDevice, c->stream));
  if ((rc = set_state_word(m, offsetof(StepState, pos), s->pos, 3))) return rc;
  if ((rc = set_state_word(m, offsetof(StepState, cur_token), s->cur_token, 4))) return rc;
  if ((rc = set_state_word(m, offsetof(StepState, last_argmax), s->last_argmax, 5))) return rc;
  if ((rc = set_state_word(m, offsetof(StepState, err), 0, 6))) return rc;
  CU(c, cudaStreamSynchronize(c->stream));
  m->pos = s->pos;
  return NFAI_OK;
}

void nfai_kv_snapshot_destroy(nfai_kv_snapshot* s) {
  if (!s) return;
  cudaSetDevice(s->device);
  if (s->dev) cudaFree(s->dev);
  delete s;
}

uint32_t nfai_kv_snapshot_position(const nfai_kv_snapshot* s) { return s ? s->pos : 0; }

static int kv_rw(nfai_model* m, uint32_t layer, uint32_t pos, float* k, float* v, const float* kin, const float* vin) {
  int rc = ready(m);
  if (rc) return rc;
  nfai_ctx* c = m->ctx;
  if (layer >= m->hp.L || pos >= m->hp.ctx) return fail(c, NFAI_ERR_ARG, "layer or position out of range");
  const size_t kvs = dtype_size(m->hp.kv_dtype);
  const size_t off = ((size_t)layer * kv_layer_elems(m) + (size_t)pos * m->kvDimL) * kvs;
  const uint32_t nel = m->kvDimL;
  CU(c, cudaStreamSynchronize(c->stream));
  std::vector<uint16_t> tmp(nel);
  for (int which = 0; which < 2; ++which) {
    char* dev = (char*)(which == 0 ? m->kc : m->vc) + off;
    float* outp = which == 0 ? k : v;
    const float* inp = which == 0 ? kin : vin;
    if (outp) {
      if (m->hp.kv_dtype == NFAI_F32) {
        CU(c, cudaMemcpy(outp, dev, nel * 4, cudaMemcpyDeviceToHost));
      } else {
        CU(c, cudaMemcpy(tmp.data(), dev, nel * 2, cudaMemcpyDeviceToHost));
        for (uint32_t i = 0; i < nel; ++i) outp[i] = half_bits_to_float(tmp[i]);
      }
    }
    if (inp) {
      if (m->hp.kv_dtype == NFAI_F32) {
        CU(c, cudaMemcpy(dev, inp, nel * 4, cudaMemcpyHostToDevice));
      } else {
        for (uint32_t i = 0; i < nel; ++i) tmp[i] = __half_as_ushort(__float2half_rn(inp[i]));
        CU(c, cudaMemcpy(dev, tmp.data(), nel * 2, cudaMemcpyHostToDevice));
      }
    }
  }
  return NFAI_OK;
}

int nfai_read_kv(nfai_model* m, uint32_t layer, uint32_t pos, float* k, float* v) { return kv_rw(m, layer, pos, k, v, nullptr, nullptr); }
int nfai_write_kv(nfai_model* m, uint32_t layer, uint32_t pos, const float* k, const float* v) { return kv_rw(m, layer, pos, nullptr, nullptr, k, v); }

int nfai_write_kv_range(nfai_model* m, uint32_t layer, uint32_t pos0, uint32_t n, const float* k, const float* v) {
  int rc = ready(m);
  if (rc) return rc;
  nfai_ctx* c = m->ctx;
  if (!k || !v || !n || layer >= m->hp.L || pos0 >= m->hp.ctx || n > m->hp.ctx - pos0)
    return fail(c, NFAI_ERR_ARG, "layer or position range out of bounds");
  const size_t kvs = dtype_size(m->hp.kv_dtype);
  const size_t nel = (size_t)n * m->kvDimL;
  const size_t off = ((size_t)layer * kv_layer_elems(m) + (size_t)pos0 * m->kvDimL) * kvs;
  CU(c, cudaStreamSynchronize(c->stream));
  std::vector<uint16_t> tmp(m->hp.kv_dtype == NFAI_F16 ? nel : 0);
  for (int which = 0; which < 2; ++which) {
    char* dev = (char*)(which == 0 ? m->kc : m->vc) + off;
    const float* inp = which == 0 ? k : v;
    if (m->hp.kv_dtype == NFAI_F32) {
      CU(c, cudaMemcpy(dev, inp, nel * 4, cudaMemcpyHostToDevice));
    } else {
      for (size_t i = 0; i < nel; ++i) tmp[i] = __half_as_ushort(__float2half_rn(inp[i]));
      CU(c, cudaMemcpy(dev, tmp.data(), nel * 2, cudaMemcpyHostToDevice));
    }
  }
  return NFAI_OK;
}

int nfai_read_hidden(nfai_model* m, uint32_t layer, float* out) {
  int rc = ready(m);
  if (rc) return rc;
  nfai_ctx* c = m->ctx;
  if (layer >= m->hp.L || !out) return fail(c, NFAI_ERR_ARG, "layer out of range or null output");
  CU(c, cudaStreamSynchronize(c->stream));
  CU(c, cudaMemcpy(out, x_in(m, layer + 1), (size_t)m->hp.H * 4, cudaMemcpyDeviceToHost));
  return NFAI_OK;
}

int nfai_model_tune(nfai_model* m, int which, int mode, int rows_per_warp, int depth, int ctas_per_sm) {
  if (!m) return fail(nullptr, NFAI_ERR_ARG, "model is null");
  nfai_ctx* c = m->ctx;
  GemvTune* t = which == 0 ? &m->tune_gateup : which == 1 ? &m->tune_down : which == 2 ? &m->tune_qkv
              : which == 3 ? &m->tune_o : which == 4 ? &m->tune_head : nullptr;
  if (!t) return fail(c, NFAI_ERR_ARG, "kernel selector must be 0..4");
  const bool even_only = which == 0 || which == 2;
  // packed knobs: rows_per_warp = rows + 16 * K split (0 = from the shape); ctas_per_sm above 16 = the grid's CTA count
  const int split = rows_per_warp >> 4;
  rows_per_warp &= 15;
  const int grid = ctas_per_sm > 16 ? ctas_per_sm : 0;
  if (grid) ctas_per_sm = (grid + (int)sm_count() - 1) / (int)sm_count();
  bool ok = (mode == 0 || mode == 1) && ctas_per_sm >= 1 && ctas_per_sm <= 16 && !(even_only && rows_per_warp == 1) &&
            (split == 0 || split == 1 || split == 2 || split == 4 || split == 8);
  if (mode == 0)
    ok = ok && (rows_per_warp == 1 || rows_per_warp == 2 || rows_per_warp == 4) && (depth == 2 || depth == 4 || depth == 8) &&
         rows_per_warp * depth <= 16;
  else
    ok = ok && rows_per_warp == 2 && (depth & 7) >= 1 && (depth & 7) <= 4 && (depth >> 3) <= 64;
  if (!ok) return fail(c, NFAI_ERR_ARG, "unsupported launch shape");
  GemvTune old = *t;
  t->mode = mode;
  t->rows_per_warp = rows_per_warp;
  t->unroll = mode == 0 ? depth : (depth & 7);
  t->l2_ahead = mode == 0 ? 0 : (depth >> 3);
  t->ctas_per_sm = ctas_per_sm;
  t->grid = grid;
  t->split = split;
  if (!m->finalized) return NFAI_OK;
  CU(c, cudaSetDevice(c->device));
  CU(c, cudaStreamSynchronize(c->stream));
  if (which == 4) {
    GemvParams hp_ = head_params(m);
    uint32_t np = gemv_grid(m->hp.weight_dtype, EPI_LOGITS, hp_, *t);
    if (np > m->nparts_alloc) {
      *t = old;
      return fail(c, NFAI_ERR_ARG, "LM-head shape needs %u partials, %u were allocated", np, m->nparts_alloc);
    }
    m->nparts = np;
  }
  if (c->use_graph) {
    cudaGraphExec_t gf = nullptr, gn = nullptr;
    int launches = 0;
    int rc = capture(m, true, false, &gf, &launches);
    if (rc == NFAI_OK) rc = capture(m, false, true, &gn, nullptr);
    if (rc != NFAI_OK) {
      if (gf) cudaGraphExecDestroy(gf);
      *t = old;
      return rc;
    }
    cudaGraphExecDestroy(m->g_full);
    cudaGraphExecDestroy(m->g_nohead);
    m->g_full = gf;
    m->g_nohead = gn;
    m->launches_full = launches;
  }
  return NFAI_OK;
}

int nfai_model_set_prefetch(nfai_model* m, uint64_t lookahead_bytes, uint64_t extra_bytes, int mode) {
  if (!m) return fail(nullptr, NFAI_ERR_ARG, "model is null");
  nfai_ctx* c = m->ctx;
  if (mode != 0 && mode != 1) return fail(c, NFAI_ERR_ARG, "mode must be 0 (per line) or 1 (bulk)");
  m->pf_look = lookahead_bytes;
  m->pf_extra = extra_bytes;
  m->pf_mode = mode;
  if (!m->finalized || !c->use_graph) return NFAI_OK;
  CU(c, cudaSetDevice(c->device));
  CU(c, cudaStreamSynchronize(c->stream));
  cudaGraphExec_t gf = nullptr, gn = nullptr;
  int launches = 0;
  int rc = capture(m, true, false, &gf, &launches);
  if (rc == NFAI_OK) rc = capture(m, false, true, &gn, nullptr);
  if (rc != NFAI_OK) {
    if (gf) cudaGraphExecDestroy(gf);
    return rc;
  }
  cudaGraphExecDestroy(m->g_full);
  cudaGraphExecDestroy(m->g_nohead);
  m->g_full = gf;
  m->g_nohead = gn;
  m->launches_full = launches;
  return NFAI_OK;
}

int nfai_step_launches(const nfai_model* m, int* out) {
  if (!m || !out) return fail(m ? m->ctx : nullptr, NFAI_ERR_ARG, "null argument");
  *out = m->launches_full;
  return NFAI_OK;
}

int nfai_profile_kernel(nfai_model* m, int which, int iters, float* avg_ms, uint64_t* bytes_per_launch) {
  int rc = ready(m);
  if (rc) return rc;
  nfai_ctx* c = m->ctx;
  const nfai_hparams& hp = m->hp;
  if (iters <= 0 || which < 0 || which > 5) return fail(c, NFAI_ERR_ARG, "bad kernel selector or iteration count");
  if (which == 5 && m->pos == 0) return fail(c, NFAI_ERR_STATE, "attention profiling needs at least one cached position");
  const int wdt = hp.weight_dtype, kvdt = hp.kv_dtype;
  const size_t ws = dtype_size(wdt), kvs = dtype_size(kvdt);
  // the QKV kernel writes a cache row at state->pos: profile it one row below the current position
  uint32_t saved_pos = m->pos;
  if (which == 2 && saved_pos >= hp.ctx) return fail(c, NFAI_ERR_CONTEXT_FULL, "QKV profiling needs one free cache row");
  if (which == 5) {
    // attention reads positions 0..pos: make seq = pos (all of them written)
    if ((rc = set_state_word(m, offsetof(StepState, pos), saved_pos - 1, 3))) return rc;
  }
  auto one = [&](int i) -> cudaError_t {
    uint32_t l = (uint32_t)i % hp.L;
    switch (which) {
      case 0: return launch_gemv(c->stream, wdt, kvdt, EPI_SILU_MUL, gateup_params(m, l), m->tune_gateup, false);
      case 1: return launch_gemv(c->stream, wdt, kvdt, EPI_STORE, down_params(m, l), m->tune_down, false);
      case 2: return launch_gemv(c->stream, wdt, kvdt, EPI_QKV_ROPE, qkv_params(m, l), m->tune_qkv, false);
      case 3: return launch_gemv(c->stream, wdt, kvdt, EPI_STORE, o_params(m, l), m->tune_o, false);
      case 4: return launch_gemv(c->stream, wdt, kvdt, EPI_LOGITS, head_params(m), m->tune_head, false);
      default:
        if (m->attn_mma) return launch_attn_mma(c->stream, attn_params(m, l), false);
        if (!m->attn_maps.empty()) return launch_attn_ring(c->stream, attn_params(m, l), m->attn_maps[l], false);
        return launch_attn_decode(c->stream, kvdt, attn_params(m, l), false);
    }
  };
  // the launches are captured into a graph so that short kernels are timed on the device, not at the rate the
  // host can issue them
  cudaGraph_t g = nullptr;
  cudaGraphExec_t ge = nullptr;
  CU(c, cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
  cudaError_t le = cudaSuccess;
  for (int i = 0; i < iters && le == cudaSuccess; ++i) le = one(i);
  cudaError_t ee = cudaStreamEndCapture(c->stream, &g);
  if (le != cudaSuccess || ee != cudaSuccess) {
    if (g) cudaGraphDestroy(g);
    cudaGetLastError();
    return fail(c, NFAI_ERR_CUDA, "profile capture failed: %s / %s", cudaGetErrorString(le), cudaGetErrorString(ee));
  }
  le = cudaGraphInstantiate(&ge, g, 0);
  cudaGraphDestroy(g);
  if (le != cudaSuccess) return fail(c, NFAI_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(le));
  le = cudaGraphLaunch(ge, c->stream);  // warm-up
  if (le == cudaSuccess) le = cudaEventRecord(c->ev0, c->stream);
  if (le == cudaSuccess) le = cudaGraphLaunch(ge, c->stream);
  if (le == cudaSuccess) le = cudaEventRecord(c->ev1, c->stream);
  if (le == cudaSuccess) le = cudaStreamSynchronize(c->stream);
  cudaGraphExecDestroy(ge);
  if (le != cudaSuccess) return fail(c, NFAI_ERR_CUDA, "profile run failed: %s", cudaGetErrorString(le));
  if ((rc = set_state_word(m, offsetof(StepState, pos), saved_pos, 4))) return rc;
  CU(c, cudaStreamSynchronize(c->stream));
  float ms = 0.f;
  CU(c, cudaEventElapsedTime(&ms, c->ev0, c->ev1));
  if (avg_ms) *avg_ms = ms / (float)iters;
  if (bytes_per_launch) {
    uint64_t b = 0;
    switch (which) {
      case 0: b = 2ull * m->Fl * hp.H * ws + (uint64_t)hp.H * 4; break;
      case 1: b = (uint64_t)hp.H * m->Fl * ws; break;
      case 2: b = (uint64_t)(m->qDimL + 2 * m->kvDimL) * hp.H * ws + (uint64_t)hp.H * 4 + 2ull * m->kvDimL * kvs; break;
      case 3: b = (uint64_t)hp.H * m->qDimL * ws; break;
      case 4: b = (uint64_t)m->Vl * hp.H * ws + (uint64_t)hp.H * 4; break;
      default: b = 2ull * m->kvDimL * kvs * saved_pos; break;
    }
    *bytes_per_launch = b;
  }
  return NFAI_OK;
}

// ---- single kernels on caller-owned device buffers ------------------------------------------------------------

static int op_begin(nfai_ctx* c) {
  if (!c) return fail(nullptr, NFAI_ERR_ARG, "ctx is null");
  cudaError_t e = cudaSetDevice(c->device);
  if (e != cudaSuccess) return fail(c, NFAI_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(e));
  return NFAI_OK;
}

static int op_end(nfai_ctx* c, cudaError_t launch_err) {
  if (launch_err != cudaSuccess) return fail(c, launch_err == cudaErrorInvalidValue ? NFAI_ERR_ARG : NFAI_ERR_CUDA, "kernel launch: %s", cudaGetErrorString(launch_err));
  CU(c, cudaStreamSynchronize(c->stream));
  return NFAI_OK;
}

static bool bad_dtype(int dt) { return dt != NFAI_F32 && dt != NFAI_F16; }

int nfai_op_embed(nfai_ctx* c, const void* E, int dtype, uint32_t H, uint32_t V, uint32_t token, float* x_out) {
  int rc = op_begin(c);
  if (rc) return rc;
  if (!E || !x_out || bad_dtype(dtype) || !H) return fail(c, NFAI_ERR_ARG, "bad argument");
  if (token >= V) return fail(c, NFAI_ERR_ARG, "token id %u out of range (V = %u)", token, V);
  return op_end(c, launch_embed(c->stream, dtype, E, H, V, nullptr, nullptr, token, x_out, PrefetchPlan(), false));
}

int nfai_op_gemv(nfai_ctx* c, const void* W, int dtype, uint32_t N, uint32_t K, const float* x, const float* gain, float eps,
                 const float* resid, float* y) {
  int rc = op_begin(c);
  if (rc) return rc;
  if (!W || !x || !y || bad_dtype(dtype) || !N || !K) return fail(c, NFAI_ERR_ARG, "bad argument");
  GemvParams p;
  p.W = W; p.N = N; p.K = K; p.x = x; p.gain = gain; p.eps = eps; p.resid = resid; p.y = y;
  GemvTune t;
  read_tune("OP", t, 2, 4);
  return op_end(c, launch_gemv(c->stream, dtype, NFAI_F32, EPI_STORE, p, t, false));
}

int nfai_op_qkv_rope(nfai_ctx* c, const void* Wqkv, int dtype, const float* x, const float* gain, float eps, uint32_t H,
                     uint32_t qH, uint32_t kvH, uint32_t d, uint32_t ropeDim, const float* rope_cs, uint32_t pos, float* q_out,
                     void* kcache, void* vcache, int kv_dtype) {
  int rc = op_begin(c);
  if (rc) return rc;
  if (!Wqkv || !x || !rope_cs || !q_out || !kcache || !vcache || bad_dtype(dtype) || bad_dtype(kv_dtype) || !H || !qH || !kvH || !d ||
      (d & 1) || ropeDim > d || (ropeDim & 1))
    return fail(c, NFAI_ERR_ARG, "bad argument");
  GemvParams p;
  p.W = Wqkv; p.N = (qH + 2 * kvH) * d; p.K = H; p.x = x; p.gain = gain; p.eps = eps;
  p.q_out = q_out; p.kcache = kcache; p.vcache = vcache; p.qDim = qH * d; p.kvDim = kvH * d; p.d = d; p.ropeDim = ropeDim;
  p.ctx = pos + 1; p.rope_cs = (const float2*)rope_cs; p.pos_imm = pos;
  GemvTune t;
  read_tune("OP", t, 2, 4);
  return op_end(c, launch_gemv(c->stream, dtype, kv_dtype, EPI_QKV_ROPE, p, t, false));
}

int nfai_op_ffn_gate_up(nfai_ctx* c, const void* Wgu, int dtype, const float* x, const float* gain, float eps, uint32_t H, uint32_t F,
                        float* h_out) {
  int rc = op_begin(c);
  if (rc) return rc;
  if (!Wgu || !x || !h_out || bad_dtype(dtype) || !H || !F) return fail(c, NFAI_ERR_ARG, "bad argument");
  GemvParams p;
  p.W = Wgu; p.N = 2 * F; p.K = H; p.x = x; p.gain = gain; p.eps = eps; p.y = h_out;
  GemvTune t;
  read_tune("OP", t, 2, 4);
  return op_end(c, launch_gemv(c->stream, dtype, NFAI_F32, EPI_SILU_MUL, p, t, false));
}

size_t nfai_op_attn_scratch_bytes(uint32_t qH, uint32_t kvH, uint32_t d, uint32_t max_seq) {
  if (!qH || !kvH || qH % kvH || !d || !max_seq) return 0;
  uint32_t S = attn_splits(qH, kvH, max_seq);
  return align_up(attn_part_floats(qH, d, S) * 4, 256) + align_up((size_t)kvH * attn_head_groups(qH, kvH) * 4, 256);
}

int nfai_op_attn_decode(nfai_ctx* c, const float* q, const void* kcache, const void* vcache, int kv_dtype, uint32_t seq, uint32_t qH,
                        uint32_t kvH, uint32_t d, float* out, void* scratch, size_t scratch_bytes) {
  int rc = op_begin(c);
  if (rc) return rc;
  if (!q || !kcache || !vcache || !out || !scratch || bad_dtype(kv_dtype) || !seq || !qH || !kvH || qH % kvH ||
      (d != 32 && d != 64 && d != 128))
    return fail(c, NFAI_ERR_ARG, "bad argument");
  if (((uintptr_t)kcache | (uintptr_t)vcache | (uintptr_t)scratch | (uintptr_t)q) & 15) return fail(c, NFAI_ERR_ARG, "pointers must be 16-byte aligned");
  size_t need = nfai_op_attn_scratch_bytes(qH, kvH, d, seq);
  if (scratch_bytes < need) return fail(c, NFAI_ERR_ARG, "scratch too small: %zu < %zu", scratch_bytes, need);
  AttnParams a;
  a.q = q; a.kcache = kcache; a.vcache = vcache; a.qH = qH; a.kvH = kvH; a.d = d; a.seq_imm = seq; a.out = out;
  a.S_max = attn_splits(qH, kvH, seq);
  a.part = (float*)scratch;
  size_t tick_off = align_up(attn_part_floats(qH, d, a.S_max) * 4, 256);
  a.tickets = (uint32_t*)((char*)scratch + tick_off);
  CU(c, cudaMemsetAsync(a.tickets, 0, (size_t)kvH * attn_head_groups(qH, kvH) * 4, c->stream));
  if (attn_mma_supported(kv_dtype, d) && ring_wanted(seq) && env_int("NFAI_ATTN_MMA", 1) != 0)
    return op_end(c, launch_attn_mma(c->stream, a, false));
  if (attn_ring_supported(kv_dtype, d) && ring_wanted(seq)) {
    AttnTileMaps maps;
    if (attn_ring_make_maps(kcache, vcache, seq, kvH * d, d, &maps) == cudaSuccess) return op_end(c, launch_attn_ring(c->stream, a, maps, false));
  }
  return op_end(c, launch_attn_decode(c->stream, kv_dtype, a, false));
}

int nfai_op_gemm_f16(nfai_ctx* c, const void* A, const void* W, uint32_t M, uint32_t N, uint32_t K, float* C) {
  int rc = op_begin(c);
  if (rc) return rc;
  if (!A || !W || !C || !M || !N || !K) return fail(c, NFAI_ERR_ARG, "bad argument");
  if (K % 8) return fail(c, NFAI_ERR_ARG, "K must be a multiple of 8");
  if (((uintptr_t)A | (uintptr_t)W) & 15) return fail(c, NFAI_ERR_ARG, "A and W must be 16-byte aligned");
  CU(c, cudaMemsetAsync(c->dev_err, 0, 4, c->stream));
  GemmEpilogue ep;
  ep.kind = GEMM_EPI_STORE;
  ep.out_f32 = C;
  const uint32_t Z = env_int("NFAI_GEMM_SPLIT", 1) ? gemm_tc_splits(M, N, K) : 1;
  if (Z > 1) {
    ep.scratch_floats = (size_t)Z * M * N;
    CU(c, cudaMallocAsync((void**)&ep.scratch, ep.scratch_floats * 4, c->stream));
  }
  cudaError_t e = launch_gemm_tc(c->stream, (const __half*)A, (const __half*)W, M, N, K, ep, c->dev_err);
  if (ep.scratch) cudaFreeAsync(ep.scratch, c->stream);
  rc = op_end(c, e);
  if (rc) return rc;
  uint32_t err = 0;
  CU(c, cudaMemcpy(&err, c->dev_err, 4, cudaMemcpyDeviceToHost));
  if (err) return fail(c, NFAI_ERR_TIMEOUT, "a bounded wait inside the tensor-core GEMM gave up");
  return NFAI_OK;
}

int nfai_op_lm_head(nfai_ctx* c, const void* W, int dtype, const float* x, const float* gain, float eps, uint32_t H, uint32_t V,
                    float* logits, uint32_t* argmax_out) {
  int rc = op_begin(c);
  if (rc) return rc;
  if (!W || !x || !logits || !argmax_out || bad_dtype(dtype) || !H || !V) return fail(c, NFAI_ERR_ARG, "bad argument");
  GemvParams p;
  p.W = W; p.N = V; p.K = H; p.x = x; p.gain = gain; p.eps = eps; p.y = logits;
  GemvTune t;
  read_tune("OP", t, 2, 4);
  uint32_t nparts = gemv_grid(dtype, EPI_LOGITS, p, t);
  // the partials need scratch: use the (large enough) tail of the logits buffer? no -- allocate from the stream pool
  float* pv = nullptr;
  CU(c, cudaMallocAsync((void**)&pv, (size_t)nparts * 8, c->stream));
  p.part_val = pv;
  p.part_idx = (uint32_t*)(pv + nparts);
  cudaError_t e = launch_gemv(c->stream, dtype, NFAI_F32, EPI_LOGITS, p, t, false);
  if (e == cudaSuccess) e = launch_argmax_final(c->stream, p.part_val, p.part_idx, nparts, nullptr, argmax_out, nullptr, 0, PrefetchPlan(), nullptr, 0, XchgHooks(), false);
  cudaFreeAsync(pv, c->stream);
  return op_end(c, e);
}

// Hooks of an op-level call whose exchange areas all sit on this GPU (one per emulated rank). The epoch word
// (c->dev_err[16]) is zero, so index = epoch - 1; the LM head's ticket word is c->dev_err[18].
static int op_xchg_hooks(nfai_ctx* c, void* const* areas, int world, int rank, uint64_t wait_ns, XchgHooks* h) {
  if (!areas || world < 1 || world > xchg::kMaxWorld || rank < 0 || rank >= world) return fail(c, NFAI_ERR_ARG, "bad exchange geometry");
  char* bases[xchg::kMaxWorld] = {};
  for (int r = 0; r < world; ++r) {
    if (!areas[r] || ((uintptr_t)areas[r] & 255)) return fail(c, NFAI_ERR_ARG, "exchange areas must be 256-byte aligned device pointers");
    bases[r] = (char*)areas[r];
  }
  h->view = xchg::make_view(bases, rank, world);
  h->epoch_base = c->dev_err + 16;
  h->wait_ns = wait_ns ? wait_ns : c->wait_ns;
  return NFAI_OK;
}

static int op_end_xchg(nfai_ctx* c, cudaError_t launch_err) {
  int rc = op_end(c, launch_err);
  if (rc) return rc;
  uint32_t err = 0;
  CU(c, cudaMemcpy(&err, c->dev_err, 4, cudaMemcpyDeviceToHost));
  if (err) {
    CU(c, cudaMemset(c->dev_err, 0, 4));
    CU(c, cudaMemset(c->dev_err + 18, 0, 8));  // a kernel that gave up may have left its ticket word mid-count
    if (err & 4u) return fail(c, NFAI_ERR_TIMEOUT, "a bounded device-side wait gave up");
    return fail(c, NFAI_ERR_CUDA, "kernel reported error bits %u", err);
  }
  return NFAI_OK;
}

size_t nfai_op_xchg_area_bytes(void) { return xchg::kAreaBytes; }

int nfai_op_gemv_xchg(nfai_ctx* c, const void* W, int dtype, uint32_t N, uint32_t K, const float* x, const float* gain, float eps,
                      float* y, void* const* areas, int world, int rank, uint32_t pull_epoch, const float* pull_resid,
                      float* pull_store, uint32_t push_epoch, uint64_t wait_ns) {
  int rc = op_begin(c);
  if (rc) return rc;
  if (!W || bad_dtype(dtype) || !N || !K || (!pull_epoch && !x) || (!push_epoch && !y)) return fail(c, NFAI_ERR_ARG, "bad argument");
  if (pull_epoch && (!pull_resid || !pull_store || K > xchg::kMaxH || (K & 3) || (((uintptr_t)pull_resid | (uintptr_t)pull_store) & 15)))
    return fail(c, NFAI_ERR_ARG, "pull needs a 16-byte aligned residual and store, K a multiple of 4 and K <= 16384");
  if (push_epoch && N > xchg::kMaxH) return fail(c, NFAI_ERR_ARG, "push needs N <= 16384");
  GemvParams p;
  p.W = W; p.N = N; p.K = K; p.x = x; p.gain = gain; p.eps = eps; p.y = y;
  p.err = c->dev_err;
  rc = op_xchg_hooks(c, areas, world, rank, wait_ns, &p.tp);
  if (rc) return rc;
  if (pull_epoch) {
    p.tp.pull = 1;
    p.tp.pull_index = pull_epoch - 1;
    p.tp.pull_resid = pull_resid;
    p.tp.pull_store = pull_store;
  }
  if (push_epoch) {
    p.tp.push = 1;
    p.tp.push_index = push_epoch - 1;
  }
  GemvTune t;
  read_tune("OP", t, 2, 4);
  return op_end_xchg(c, launch_gemv(c->stream, dtype, NFAI_F32, EPI_STORE, p, t, false));
}

int nfai_op_lm_head_xchg(nfai_ctx* c, const void* W, int dtype, const float* x, const float* gain, float eps, uint32_t H,
                         uint32_t Vl, uint32_t v_lo, float* logits, void* const* areas, int world, int rank, uint32_t epoch,
                         int push, int pull, uint32_t* argmax_out, uint64_t wait_ns) {
  int rc = op_begin(c);
  if (rc) return rc;
  if (!epoch || (push && (!W || !x || !logits || bad_dtype(dtype) || !H || !Vl)) || (pull && !argmax_out) || (!push && !pull))
    return fail(c, NFAI_ERR_ARG, "bad argument");
  XchgHooks h;
  rc = op_xchg_hooks(c, areas, world, rank, wait_ns, &h);
  if (rc) return rc;
  cudaError_t e = cudaSuccess;
  float* pv = nullptr;
  if (push) {
    GemvParams p;
    p.W = W; p.N = Vl; p.K = H; p.x = x; p.gain = gain; p.eps = eps; p.y = logits;
    p.err = c->dev_err;
    p.v_lo = v_lo;
    p.tp = h;
    p.tp.push = 1;
    p.tp.push_index = epoch - 1;
    p.tp_ticket = c->dev_err + 18;
    GemvTune t;
    read_tune("OP", t, 2, 4);
    const uint32_t nparts = gemv_grid(dtype, EPI_LOGITS, p, t);
    CU(c, cudaMallocAsync((void**)&pv, (size_t)nparts * 8, c->stream));
    p.part_val = pv;
    p.part_idx = (uint32_t*)(pv + nparts);
    e = launch_gemv(c->stream, dtype, NFAI_F32, EPI_LOGITS, p, t, false);
  }
  if (pull && e == cudaSuccess) {
    h.pull = 1;
    h.pull_index = epoch - 1;
    // the state-less form reports a time-out through the step state only; give it one for the duration of the call
    StepState* st = reinterpret_cast<StepState*>(c->dev_err + 32);
    CU(c, cudaMemsetAsync(st, 0, sizeof(StepState), c->stream));
    e = launch_argmax_final(c->stream, nullptr, nullptr, (uint32_t)world, st, argmax_out, nullptr, 0, PrefetchPlan(), nullptr, 0, h, false);
    if (e == cudaSuccess) e = cudaMemcpyAsync(c->dev_err, &st->err, 4, cudaMemcpyDeviceToDevice, c->stream);
  }
  if (pv) cudaFreeAsync(pv, c->stream);
  return op_end_xchg(c, e);
}

int nfai_ctx_set_wait_ns(nfai_ctx* c, uint64_t ns) {
  if (!c) return fail(nullptr, NFAI_ERR_ARG, "ctx is null");
  if (!ns) return fail(c, NFAI_ERR_ARG, "the wait budget must be positive");
  c->wait_ns = ns;
  if (c->tp) tp_set_wait_ns(c->tp, ns);
  return NFAI_OK;
}

int nfai_op_sample_top_p(nfai_ctx* c, const float* logits, uint32_t V, float temperature, float top_p, int top_k, float u,
                         uint32_t* token_out) {
  int rc = op_begin(c);
  if (rc) return rc;
  if (!logits || !token_out || !V || !(temperature > 0.f) || !(top_p > 0.f) || top_k < 1 || top_k > 64 || !(u >= 0.f && u < 1.f))
    return fail(c, NFAI_ERR_ARG, "bad argument");
  void* scratch = nullptr;
  CU(c, cudaMallocAsync(&scratch, sample_scratch_bytes(V, nullptr), c->stream));
  cudaError_t e = launch_sample_top_p(c->stream, logits, V, nullptr, nullptr, temperature, top_p, top_k, u, scratch, token_out);
  cudaFreeAsync(scratch, c->stream);
  return op_end(c, e);
}

}  // extern "C"
