// The decode step as one persistent kernel whose weight stream never stops: every warp pulls the rows it owns --
// of ALL matrices of the step, in consumption order -- through a private shared-memory ring filled by 1-D bulk
// asynchronous copies (TMA). Weights do not depend on activations, so the ring keeps filling across the grid
// barriers that separate the phases (QKV, attention, O, gate/up, down, LM head): while the grid synchronises and
// the new input vector is normalised, ~160 KB per SM (24 MB on the GPU, ~3.5 microseconds of HBM time) of the next
// matrices are already on their way. HBM idles only while attention runs longer than the ring can absorb.
//
// One CTA per SM, 16 warps. A ring stage is one 2 KB chunk of one weight row; a warp's items are
// (phase, row block, row, chunk) in order; lane 0 arms the stage's mbarrier and issues the copy, all lanes wait on
// the parity, FMA the chunk against x (float32 in shared memory) and the stage is refilled with the item S ahead,
// which may belong to a later phase. Epilogues, arithmetic order and results are those of the per-kernel path.
// Every wait is bounded (mbarrier polls and grid barrier: one second); a time-out raises the abort flag, every CTA
// leaves at its next barrier and the host reports NFAI_ERR_TIMEOUT.
#include "attn_core.cuh"
#include "gemv_common.cuh"
#include "megastep.h"

namespace nfai {

using namespace gemv_detail;
using namespace attn_detail;

namespace {

constexpr int kFT = 512;             // threads per CTA
constexpr int kFW = kFT / 32;        // warps per CTA
constexpr uint32_t kFChunk = 2048;   // bytes of one ring stage
constexpr unsigned long long kFWaitNs = 1000000000ull;

__device__ __forceinline__ unsigned long long f_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t f_s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t f_ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool f_bar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

struct FSync {
  uint32_t* counter;
  uint32_t* abort_flag;
  uint32_t epoch;
  unsigned long long* trace;  // diagnostics: CTA 0 / thread 0 appends time stamps (null in normal runs)
  uint32_t trace_n;
};

__device__ __forceinline__ void f_stamp(FSync& sy) {
  if (sy.trace && blockIdx.x == 0 && threadIdx.x == 0 && sy.trace_n < (uint32_t)kTraceSlots - 1) {
    sy.trace[1 + sy.trace_n] = f_ns();
    sy.trace_n += 1;
    sy.trace[0] = sy.trace_n;
  }
}

__device__ __forceinline__ bool f_grid_barrier(FSync& sy, uint32_t* s_flag) {
  f_stamp(sy);  // warp 0 of this CTA has finished the phase
  __syncthreads();
  f_stamp(sy);  // the CTA has
  if (threadIdx.x == 0) {
    sy.epoch += 1;
    const uint32_t target = sy.epoch * gridDim.x;
    __threadfence();
    atomicAdd(sy.counter, 1u);
    uint32_t ok = 1;
    if (f_ld_acquire(sy.counter) < target) {
      const unsigned long long t0 = f_ns();
      uint32_t polls = 0;
      while (f_ld_acquire(sy.counter) < target) {
        if ((++polls & 255u) == 0) {
          if (f_ld_acquire(sy.abort_flag) != 0) { ok = 0; break; }
          if (f_ns() - t0 > kFWaitNs) {
            atomicExch(sy.abort_flag, 1u);
            ok = 0;
            break;
          }
        }
      }
    }
    if (ok && f_ld_acquire(sy.abort_flag) != 0) ok = 0;  // a warp somewhere gave up on its ring
    __threadfence();
    *s_flag = ok;
  }
  __syncthreads();
  f_stamp(sy);  // the grid has
  return *s_flag != 0;
}

// One GEMV phase of the step as the streamer sees it.
struct FPhase {
  const unsigned char* W;  // [N][K] rows of row_bytes
  uint32_t N, row_bytes, nchunks, R;  // R = rows per row block (1, or 2 where the epilogue pairs rows)
};

// Position of a warp in its item list: (phase, row block, row in block, chunk).
struct FCursor {
  uint32_t ph, rb, r, c;
};

__device__ __forceinline__ FPhase f_phase(const StepDesc& d, uint32_t ph, uint32_t elem_bytes) {
  FPhase p;
  const uint32_t qDim = d.qH * d.d, kvDim = d.kvH * d.d;
  if (ph >= 4 * d.L) {  // LM head
    p.W = (const unsigned char*)d.head;
    p.N = d.V;
    p.row_bytes = d.H * elem_bytes;
    p.R = 1;
  } else {
    const LayerDesc& L = d.layers[ph >> 2];
    switch (ph & 3u) {
      case 0: p.W = (const unsigned char*)L.qkv; p.N = qDim + 2 * kvDim; p.row_bytes = d.H * elem_bytes; p.R = 2; break;
      case 1: p.W = (const unsigned char*)L.o; p.N = d.H; p.row_bytes = qDim * elem_bytes; p.R = 1; break;
      case 2: p.W = (const unsigned char*)L.gateup; p.N = 2 * d.F; p.row_bytes = d.H * elem_bytes; p.R = 2; break;
      default: p.W = (const unsigned char*)L.down; p.N = d.H; p.row_bytes = d.F * elem_bytes; p.R = 1; break;
    }
  }
  p.nchunks = (p.row_bytes + kFChunk - 1) / kFChunk;
  return p;
}

// The streaming state of one warp: the ring, the cursor of the next item to issue and how many were consumed.
struct FStream {
  uint32_t ring_s, bar_s;  // shared-memory addresses of this warp's stages and mbarriers
  unsigned char* ring;
  int S;
  uint32_t gw, TW, P, elem_bytes;
  FCursor ic;        // next item to issue (ic.ph == P: nothing left)
  FPhase ip;         // phase descriptor of ic.ph
  uint32_t slot, parity;  // stage of the next item to consume and the mbarrier parity it completes with
  bool dead;         // a bounded wait gave up: stop streaming, keep walking the barriers
};

__device__ __forceinline__ void f_enter_phase(const StepDesc& d, FStream& st, FCursor& c) {
  // first row block of this warp in phase c.ph, skipping phases where it has none
  while (c.ph < st.P) {
    FPhase p = f_phase(d, c.ph, st.elem_bytes);
    const uint32_t nrb = (p.N + p.R - 1) / p.R;
    if (st.gw < nrb) {
      c.rb = st.gw;
      c.r = 0;
      c.c = 0;
      return;
    }
    c.ph += 1;
  }
}

// Advance a cursor by one item inside phase `p`; moves on to the next phase that has rows for this warp.
__device__ __forceinline__ void f_advance(const StepDesc& d, FStream& st, FCursor& c, FPhase& p) {
  if (++c.c < p.nchunks) return;
  c.c = 0;
  if (++c.r < p.R && c.rb * p.R + c.r < p.N) return;
  c.r = 0;
  c.rb += st.TW;
  if (c.rb < (p.N + p.R - 1) / p.R) return;
  c.ph += 1;
  f_enter_phase(d, st, c);
  if (c.ph < st.P) p = f_phase(d, c.ph, st.elem_bytes);
}

// Arm stage `slot` and copy the item at the issue cursor into it (lane 0 issues; every lane advances its copy of
// the cursor, so the warp stays uniform).
__device__ __forceinline__ void f_issue(const StepDesc& d, FStream& st, uint32_t slot) {
  if (st.ic.ph >= st.P) return;
  const FPhase& p = st.ip;
  const uint32_t off = st.ic.c * kFChunk;
  const uint32_t bytes = p.row_bytes - off < kFChunk ? p.row_bytes - off : kFChunk;
  const unsigned char* src = p.W + (size_t)(st.ic.rb * p.R + st.ic.r) * p.row_bytes + off;
  const uint32_t bar = st.bar_s + 8 * slot;
  if ((threadIdx.x & 31) == 0) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     st.ring_s + slot * kFChunk),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
  }
  f_advance(d, st, st.ic, st.ip);
}

// Consume this warp's items of phase `ph` (R rows per block, epilogue EPI). cc is the consume cursor.
// Inlined on purpose: the stream state (cursors, slot, parity) must live in registers -- behind a call it would sit
// in local memory, and with nearly all of the L1 carved out as shared memory every access would go to L2.
template <typename WT, typename KVT, int R, int EPI>
__device__ __forceinline__ void f_consume_phase(const StepDesc& d, FStream& st, FCursor& cc, const uint32_t ph, const GemvParams p,
                                             const float* xs, float& best_v, uint32_t& best_i) {
  constexpr int VE = WeightVec<WT>::kElems;
  const int lane = threadIdx.x & 31;
  const uint32_t row_bytes = p.K * sizeof(WT);
  const uint32_t nchunks = (row_bytes + kFChunk - 1) / kFChunk;
  float acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.f;
  while (!st.dead && cc.ph == ph) {
    const uint32_t slot = st.slot, parity = st.parity;
    const uint32_t bar = st.bar_s + 8 * slot;
    bool ok = __all_sync(0xffffffffu, f_bar_try(bar, parity));
    if (!ok) {
      const unsigned long long t0 = f_ns();
      uint32_t polls = 0;
      while (!ok) {
        ok = __all_sync(0xffffffffu, f_bar_try(bar, parity));
        if (!ok && (++polls & 63u) == 0) {
          const bool late = f_ns() - t0 > kFWaitNs;
          if (__any_sync(0xffffffffu, late)) break;
        }
      }
    }
    if (!ok) {
      st.dead = true;
      if (lane == 0) {
        atomicExch(d.abort_flag, 1u);
        atomicOr(&d.state->err, 4u);
      }
      break;
    }
    const uint32_t off = cc.c * kFChunk;
    const uint32_t bytes = row_bytes - off < kFChunk ? row_bytes - off : kFChunk;
    const unsigned char* stg = st.ring + (size_t)slot * kFChunk;
    float a = 0.f;
#pragma unroll
    for (int v = 0; v < (int)(kFChunk / 512); ++v) {
      const uint32_t vb = (lane + 32 * v) * 16;
      if (vb < bytes) {
        const uint4 w = *reinterpret_cast<const uint4*>(stg + vb);
        float wf[VE];
        WeightVec<WT>::unpack(w, wf);
        const float4* xp = reinterpret_cast<const float4*>(xs + (off + vb) / sizeof(WT));
#pragma unroll
        for (int k = 0; k < VE / 4; ++k) {
          const float4 t = xp[k];
          a = fmaf(wf[4 * k], t.x, a);
          a = fmaf(wf[4 * k + 1], t.y, a);
          a = fmaf(wf[4 * k + 2], t.z, a);
          a = fmaf(wf[4 * k + 3], t.w, a);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
      if ((int)cc.r == r) acc[r] += a;
    __syncwarp();  // every lane has read the stage before it is refilled
    f_issue(d, st, slot);
    if (++st.slot == (uint32_t)st.S) {
      st.slot = 0;
      st.parity ^= 1u;
    }
    const bool row_done = cc.c + 1 == nchunks;
    const bool block_done = row_done && (cc.r + 1 == (uint32_t)R || cc.rb * R + cc.r + 1 >= p.N);
    const uint32_t rb_now = cc.rb;
    // advance the consume cursor (same rules as the issue cursor)
    if (!row_done) {
      cc.c += 1;
    } else if (!block_done) {
      cc.c = 0;
      cc.r += 1;
    } else {
#pragma unroll
      for (int r = 0; r < R; ++r) acc[r] = warp_sum(acc[r]);
      row_epilogue<KVT, R, EPI>(p, rb_now * R, acc, best_v, best_i);
#pragma unroll
      for (int r = 0; r < R; ++r) acc[r] = 0.f;
      cc.c = 0;
      cc.r = 0;
      cc.rb += st.TW;
      if (cc.rb >= (p.N + R - 1) / R) {
        cc.ph += 1;
        f_enter_phase(d, st, cc);
      }
    }
  }
}

// x into shared memory with L2-only loads, RMS-normalised when the phase has a gain (512 threads).
template <typename WT>
__device__ __forceinline__ void f_load_x(const GemvParams& p, const float* x, const void* embd_row, float* x_copy, float* xs,
                                         const float* gs, float* red) {
  const uint32_t K = p.K;
  const int tid = threadIdx.x;
  float ss = 0.f;
  if (embd_row) {
    for (uint32_t i = tid; i < K; i += kFT) {
      const float v = to_float(reinterpret_cast<const WT*>(embd_row)[i]);  // TokenEmbedShader.cs:139-158
      if (x_copy && blockIdx.x == 0) x_copy[i] = v;
      xs[i] = v;
      ss = fmaf(v, v, ss);
    }
  } else if ((K & 3u) == 0) {
    const float4* x4 = reinterpret_cast<const float4*>(x);
    float4* xs4 = reinterpret_cast<float4*>(xs);
    const uint32_t n4 = K >> 2;
    for (uint32_t base = 0; base < n4; base += 4 * kFT) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t i = base + u * kFT + tid;
        v[u] = i < n4 ? __ldcg(x4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t i = base + u * kFT + tid;
        if (i < n4) {
          xs4[i] = v[u];
          ss = fmaf(v[u].x, v[u].x, ss);
          ss = fmaf(v[u].y, v[u].y, ss);
          ss = fmaf(v[u].z, v[u].z, ss);
          ss = fmaf(v[u].w, v[u].w, ss);
        }
      }
    }
  } else {
    for (uint32_t i = tid; i < K; i += kFT) {
      const float v = __ldcg(x + i);
      xs[i] = v;
      ss = fmaf(v, v, ss);
    }
  }
  if (p.gain == nullptr) {
    __syncthreads();
    return;
  }
  ss = warp_sum(ss);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < kFW; ++w) tot += red[w];
  const float rms = sqrtf(__fdiv_rn(tot, (float)K) + p.eps);
  for (uint32_t i = tid; i < K; i += kFT) xs[i] = __fmul_rn(__fdiv_rn(xs[i], rms), gs[i]);
  __syncthreads();
}

template <typename KVT, int D, int GH>
__device__ __noinline__ void f_attn_phase(const AttnParams a, uint32_t bx, uint32_t s, uint32_t seq, uint32_t min_chunk) {
  attn_core<KVT, D, kFW, true, GH, (GH == 1 ? 2 * KV8<KVT>::kUnroll : 0)>(a, bx, s, seq, min_chunk);
}

template <typename WT, typename KVT, int D>
__global__ void __launch_bounds__(kFT, 1) fused_ring_step_kernel(const StepDesc* __restrict__ dp, const int S) {
  extern __shared__ __align__(128) unsigned char fsm[];
  __shared__ uint32_t s_flag;
  const StepDesc& d = *dp;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t H = d.H, qDim = d.qH * D, kvDim = d.kvH * D;
  uint32_t kmax = H > d.F ? H : d.F;
  kmax = kmax > qDim ? kmax : qDim;
  // layout: [rings: 16 warps x S x 2 KB][mbarriers: 16 x S x 8 B, padded to 128][red: 32 floats][x: kmax][gain: H]
  unsigned char* rings = fsm;
  uint64_t* bars = reinterpret_cast<uint64_t*>(fsm + (size_t)kFW * S * kFChunk);
  float* red = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(bars) + 128 * ((kFW * S * 8 + 127) / 128));
  float* xs = red + 32;
  float* gs = xs + kmax;

  FSync sy{d.sync_counter, d.abort_flag, 0, d.trace, 0};
  const uint32_t pos = d.state->pos;
  uint32_t tok = d.prompt ? d.prompt[d.state->prompt_idx] : d.state->cur_token;
  if (pos >= d.ctx) {
    if (blockIdx.x == 0 && tid == 0) atomicOr(&d.state->err, 2u);
    return;
  }
  if (tok >= d.embd_rows) {
    if (blockIdx.x == 0 && tid == 0) atomicOr(&d.state->err, 1u);
    tok = 0;
  }

  FStream st;
  st.ring = rings + (size_t)warp * S * kFChunk;
  st.ring_s = f_s32(st.ring);
  st.bar_s = f_s32(bars + warp * S);
  st.S = S;
  st.gw = blockIdx.x * kFW + warp;
  st.TW = gridDim.x * kFW;
  st.P = 4 * d.L + (d.with_head ? 1u : 0u);
  st.elem_bytes = sizeof(WT);
  st.slot = 0;
  st.parity = 0;
  st.dead = false;
  if (lane == 0) {
    for (int s = 0; s < S; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(st.bar_s + 8 * s), "r"(1) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  st.ic.ph = 0;
  st.ic.rb = st.ic.r = st.ic.c = 0;
  f_enter_phase(d, st, st.ic);
  if (st.ic.ph < st.P) st.ip = f_phase(d, st.ic.ph, st.elem_bytes);
  FCursor cc = st.ic;  // the consume cursor starts where the issue cursor starts
  for (int s = 0; s < S; ++s) f_issue(d, st, (uint32_t)s);  // fill the ring: weights depend on nothing

  float best_v = -INFINITY;
  uint32_t best_i = 0xffffffffu;
  bool ok = true;
  for (uint32_t l = 0; l < d.L && ok; ++l) {
    const LayerDesc& L = d.layers[l];
    float* x_in = d.xbuf + (size_t)(2 * l) * H;
    float* x_mid = x_in + H;
    float* x_out = x_mid + H;
    char* kcl = (char*)d.kc + (size_t)l * d.kv_layer_bytes;
    char* vcl = (char*)d.vc + (size_t)l * d.kv_layer_bytes;
    {  // RMSNorm + QKV + RoPE + cache row
      GemvParams p;
      p.W = L.qkv; p.N = qDim + 2 * kvDim; p.K = H; p.gain = L.attn_norm; p.eps = d.eps;
      p.q_out = d.q; p.kcache = kcl; p.vcache = vcl; p.qDim = qDim; p.kvDim = kvDim; p.d = D; p.ropeDim = d.ropeDim;
      p.ctx = d.ctx; p.rope_cs = d.rope_cs; p.pos_imm = pos;
      for (uint32_t i = tid; i < H; i += kFT) gs[i] = p.gain[i];
      if (l != 0) {
        ok = f_grid_barrier(sy, &s_flag);
        if (!ok) break;
      }
      f_load_x<WT>(p, x_in, l == 0 ? (const char*)d.embd + (size_t)tok * H * sizeof(WT) : nullptr, l == 0 ? x_in : nullptr, xs,
                   gs, red);
      f_stamp(sy);
      f_consume_phase<WT, KVT, 2, EPI_QKV_ROPE>(d, st, cc, 4 * l + 0, p, xs, best_v, best_i);
    }
    {  // attention over positions 0..pos
      ok = f_grid_barrier(sy, &s_flag);
      if (!ok) break;
      AttnParams a;
      a.q = d.q; a.kcache = kcl; a.vcache = vcl; a.qH = d.qH; a.kvH = d.kvH; a.d = D; a.out = d.attn_out;
      a.part = d.attn_part; a.tickets = d.tickets; a.S_max = d.S_max;
      const uint32_t G = d.qH / d.kvH;
      if (d.attn_heads == 1) {
        const uint32_t nx = d.qH;
        if (blockIdx.x < nx * d.S_max) f_attn_phase<KVT, D, 1>(a, blockIdx.x % nx, blockIdx.x / nx, pos + 1, d.attn_min_chunk);
      } else {
        const uint32_t nx = d.kvH * ((G + 3) / 4);
        if (blockIdx.x < nx * d.S_max) f_attn_phase<KVT, D, 4>(a, blockIdx.x % nx, blockIdx.x / nx, pos + 1, d.attn_min_chunk);
      }
    }
    {  // O projection + residual
      GemvParams p;
      p.W = L.o; p.N = H; p.K = qDim; p.resid = x_in; p.y = x_mid;
      ok = f_grid_barrier(sy, &s_flag);
      if (!ok) break;
      f_load_x<WT>(p, d.attn_out, nullptr, nullptr, xs, gs, red);
      f_stamp(sy);
      f_consume_phase<WT, KVT, 1, EPI_STORE>(d, st, cc, 4 * l + 1, p, xs, best_v, best_i);
    }
    {  // RMSNorm + gate/up + SiLU*up
      GemvParams p;
      p.W = L.gateup; p.N = 2 * d.F; p.K = H; p.gain = L.ffn_norm; p.eps = d.eps; p.y = d.hbuf;
      for (uint32_t i = tid; i < H; i += kFT) gs[i] = p.gain[i];
      ok = f_grid_barrier(sy, &s_flag);
      if (!ok) break;
      f_load_x<WT>(p, x_mid, nullptr, nullptr, xs, gs, red);
      f_stamp(sy);
      f_consume_phase<WT, KVT, 2, EPI_SILU_MUL>(d, st, cc, 4 * l + 2, p, xs, best_v, best_i);
    }
    {  // down projection + residual
      GemvParams p;
      p.W = L.down; p.N = H; p.K = d.F; p.resid = x_mid; p.y = x_out;
      ok = f_grid_barrier(sy, &s_flag);
      if (!ok) break;
      f_load_x<WT>(p, d.hbuf, nullptr, nullptr, xs, gs, red);
      f_stamp(sy);
      f_consume_phase<WT, KVT, 1, EPI_STORE>(d, st, cc, 4 * l + 3, p, xs, best_v, best_i);
    }
  }
  if (ok && d.with_head) {
    GemvParams p;
    p.W = d.head; p.N = d.V; p.K = H; p.gain = d.out_norm; p.eps = d.eps; p.y = d.logits;
    for (uint32_t i = tid; i < H; i += kFT) gs[i] = p.gain[i];
    ok = f_grid_barrier(sy, &s_flag);
    if (ok) {
      f_load_x<WT>(p, d.xbuf + (size_t)(2 * d.L) * H, nullptr, nullptr, xs, gs, red);
      f_consume_phase<WT, KVT, 1, EPI_LOGITS>(d, st, cc, 4 * d.L, p, xs, best_v, best_i);
      // one (max, lowest index) partial per CTA
      uint32_t* redi = reinterpret_cast<uint32_t*>(red);
      __syncthreads();
      if (lane == 0) {
        red[warp] = best_v;
        redi[kFW + warp] = best_i;
      }
      __syncthreads();
      if (tid == 0) {
        float v = red[0];
        uint32_t ix = redi[kFW];
        for (int w = 1; w < kFW; ++w) {
          const float wv = red[w];
          const uint32_t wi = redi[kFW + w];
          if (wi != 0xffffffffu && (ix == 0xffffffffu || wv > v || (wv == v && wi < ix))) {
            v = wv;
            ix = wi;
          }
        }
        d.part_val[blockIdx.x] = v;
        d.part_idx[blockIdx.x] = ix;
      }
      ok = f_grid_barrier(sy, &s_flag);
    }
  }
  if (!ok || st.dead) {
    if (tid == 0) atomicOr(&d.state->err, 4u);
    // copies of this CTA may still be landing: give them a bounded time before the shared memory is released
    for (volatile uint32_t spin = 0; spin < (1u << 20); ++spin) {
    }
    return;
  }
  if (blockIdx.x != 0) return;
  if (d.with_head) {
    // lowest index among the maxima (SamplingUtils.cs:55-56) over the per-CTA partials
    __shared__ float sv[kFT];
    __shared__ uint32_t si[kFT];
    float bv = -INFINITY;
    uint32_t bi = 0xffffffffu;
    for (uint32_t i = tid; i < gridDim.x; i += kFT) {
      const float v = __ldcg(d.part_val + i);
      const uint32_t ix = __ldcg(d.part_idx + i);
      if (ix != 0xffffffffu && (bi == 0xffffffffu || v > bv || (v == bv && ix < bi))) {
        bv = v;
        bi = ix;
      }
    }
    sv[tid] = bv;
    si[tid] = bi;
    __syncthreads();
    for (int o = kFT / 2; o > 0; o >>= 1) {
      if (tid < o) {
        const float v = sv[tid + o], cv = sv[tid];
        const uint32_t ix = si[tid + o], ci = si[tid];
        if (ix != 0xffffffffu && (ci == 0xffffffffu || v > cv || (v == cv && ix < ci))) {
          sv[tid] = v;
          si[tid] = ix;
        }
      }
      __syncthreads();
    }
    if (tid == 0) {
      const uint32_t best = si[0] == 0xffffffffu ? 0u : si[0];
      StepState* sst = d.state;
      if (d.history && sst->steps < d.history_cap) d.history[sst->steps] = best;
      sst->last_argmax = best;
      sst->cur_token = best;
      sst->pos = pos + 1;
      sst->steps += 1;
    }
  } else if (tid == 0) {
    d.state->pos = pos + 1;
    d.state->prompt_idx += 1;
  }
}

template <typename WT, typename KVT>
cudaError_t f_pick_d(uint32_t d, const void** fn) {
  switch (d) {
    case 32: *fn = (const void*)fused_ring_step_kernel<WT, KVT, 32>; return cudaSuccess;
    case 64: *fn = (const void*)fused_ring_step_kernel<WT, KVT, 64>; return cudaSuccess;
    case 128: *fn = (const void*)fused_ring_step_kernel<WT, KVT, 128>; return cudaSuccess;
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t f_pick(int wdtype, int kvdtype, uint32_t d, const void** fn) {
  if (wdtype == 1) return kvdtype == 1 ? f_pick_d<__half, __half>(d, fn) : f_pick_d<__half, float>(d, fn);
  return kvdtype == 1 ? f_pick_d<float, __half>(d, fn) : f_pick_d<float, float>(d, fn);
}

size_t f_fixed_smem(uint32_t H, uint32_t F, uint32_t qDim) {
  uint32_t kmax = H > F ? H : F;
  kmax = kmax > qDim ? kmax : qDim;
  return (32 + (size_t)kmax + H) * sizeof(float);
}

}  // namespace

// Ring depth (2..6 stages per warp) that fits beside x, the gain and the kernel's static shared memory in 227 KB;
// sets the function attributes and reports the grid (one CTA per SM). stages_out = 0 when nothing fits.
cudaError_t fused_ring_prepare(int wdtype, int kvdtype, uint32_t d, uint32_t H, uint32_t F, uint32_t qDim, int* grid_out,
                               int* stages_out, size_t* smem_out) {
  *stages_out = 0;
  const void* fn = nullptr;
  cudaError_t e = f_pick(wdtype, kvdtype, d, &fn);
  if (e != cudaSuccess) return e;
  cudaFuncAttributes fa;
  e = cudaFuncGetAttributes(&fa, fn);
  if (e != cudaSuccess) return e;
  const size_t fixed = f_fixed_smem(H, F, qDim);
  const size_t budget = 227 * 1024 - fa.sharedSizeBytes - 1024;
  int best = 0;
  size_t best_bytes = 0;
  for (int S = 2; S <= 6; ++S) {
    const size_t total = (size_t)kFW * S * kFChunk + 128 * (((size_t)kFW * S * 8 + 127) / 128) + fixed;
    if (total <= budget) {
      best = S;
      best_bytes = total;
    }
  }
  if (best == 0) return cudaSuccess;
  e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)best_bytes);
  if (e != cudaSuccess) return e;
  e = prefer_max_shared(fn);
  if (e != cudaSuccess) return e;
  int per_sm = 0, dev = 0, sms = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kFT, best_bytes);
  if (e != cudaSuccess) return e;
  e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return e;
  if (per_sm < 1) return cudaSuccess;
  *grid_out = sms;  // one CTA per SM
  *stages_out = best;
  *smem_out = best_bytes;
  return cudaSuccess;
}

cudaError_t launch_fused_ring(cudaStream_t s, int wdtype, int kvdtype, uint32_t d, const StepDesc* desc_dev, int grid,
                              size_t smem, int stages) {
  const void* fn = nullptr;
  cudaError_t e = f_pick(wdtype, kvdtype, d, &fn);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kFT);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  void* args[] = {(void*)&desc_dev, (void*)&stages};
  return cudaLaunchKernelExC(&cfg, fn, args);
}

}  // namespace nfai
