// The whole decode step as ONE persistent kernel: embed, L x (QKV+RoPE, attention, O+residual, gate/up+SiLU,
// down+residual), LM head, arg-max -- the same arithmetic as the per-kernel path (gemv.cu, attn.cu), phase by
// phase, with a grid barrier where the per-kernel path has a kernel boundary.
//
// Why: at batch 1 a layer's matrices are 1-10 microsecond streams and a kernel boundary costs ~4 microseconds of
// idle HBM (drain, launch, x prologue, ramp). Inside one kernel every warp requests the first weights of the NEXT
// phase before it arrives at the barrier, so ~10 MB are in flight across the barrier and HBM keeps streaming while
// the grid synchronises and the new x is normalised.
//
// The barrier is a counter in global memory (one atomic per CTA, thread 0 polls with acquire loads). The launch is
// cooperative, so all CTAs are resident; the poll is bounded all the same (one second), after which the CTA raises
// the abort flag, every CTA leaves at its next barrier and the host reports NFAI_ERR_TIMEOUT.
// Activations written earlier in the same kernel are read with L2-only loads (ld.global.cg): the L1 is not
// coherent between SMs. Weights, gains and tables are immutable and use the streaming / default paths.
#include "attn_core.cuh"
#include "gemv_common.cuh"
#include "megastep.h"

namespace nfai {

using namespace gemv_detail;
using namespace attn_detail;

namespace {

constexpr unsigned long long kBarrierLimitNs = 1000000000ull;
// launch shape of the phases: rows per warp / 16-byte loads per row per lane
constexpr int kFusedCtasPerSm = 2;
constexpr int kWideR = 2, kWideU = 4;    // QKV, gate/up, LM head
constexpr int kNarrowR = 2, kNarrowU = 4;  // O and down projections
constexpr int kMegaHeads = 2;  // query heads per attention CTA inside the fused step (register budget: 128 per thread)

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct Sync {
  uint32_t* counter;
  uint32_t* abort_flag;
  uint32_t epoch;
  unsigned long long* trace;
  uint32_t trace_n;
};

// CTA 0 / thread 0 appends a time stamp (diagnostics; trace == nullptr in normal runs).
__device__ __forceinline__ void stamp(Sync& sy) {
  if (sy.trace && blockIdx.x == 0 && threadIdx.x == 0 && sy.trace_n < (uint32_t)kTraceSlots - 1) {
    sy.trace[1 + sy.trace_n] = global_ns();
    sy.trace_n += 1;
    sy.trace[0] = sy.trace_n;
  }
}

// Returns false (in every thread of the CTA) once any CTA has given up.
__device__ __forceinline__ bool grid_barrier(Sync& sy, uint32_t* s_flag) {
  stamp(sy);  // this thread's work of the phase is done
  __syncthreads();
  stamp(sy);  // the whole CTA is done
  if (threadIdx.x == 0) {
    sy.epoch += 1;
    const uint32_t target = sy.epoch * gridDim.x;
    __threadfence();
    atomicAdd(sy.counter, 1u);
    uint32_t ok = 1;
    if (ld_acquire(sy.counter) < target) {
      const unsigned long long t0 = global_ns();
      uint32_t polls = 0;
      while (ld_acquire(sy.counter) < target) {
        if ((++polls & 255u) == 0) {
          if (ld_acquire(sy.abort_flag) != 0) { ok = 0; break; }
          if (global_ns() - t0 > kBarrierLimitNs) {
            atomicExch(sy.abort_flag, 1u);
            ok = 0;
            break;
          }
        }
      }
    }
    __threadfence();
    *s_flag = ok;
  }
  __syncthreads();
  stamp(sy);  // the whole grid is done
  return *s_flag != 0;
}

// Where a phase's input vector comes from.
struct XSource {
  const float* x = nullptr;      // plain float32 vector (written earlier in this kernel)
  const void* embd_row = nullptr;  // or: row of the embedding matrix (weight type), first phase only
  float* x_copy = nullptr;       // CTA 0 also stores the widened embedding row here (the residual needs it)
};

// The gain of the NEXT phase is staged before the barrier, while slower warps of this CTA may still read the
// current phase's x: it therefore has its own region (gs), never a tail of the x region.
__device__ __forceinline__ void stage_gain(const GemvParams& p, float* gs) {
  if (p.gain == nullptr) return;
  for (uint32_t i = threadIdx.x; i < p.K; i += kThreads) gs[i] = p.gain[i];
}

// x into shared memory (and RMS-normalised when the phase has a gain). The vector is read with L2-only 16-byte
// loads, eight of them in flight per thread, so the prologue costs about one L2 round trip whatever K is.
template <typename WT>
__device__ __forceinline__ void load_x_cg(const GemvParams& p, const XSource& src, float* xs, const float* gs,
                                          float* red) {
  const uint32_t K = p.K;
  const int tid = threadIdx.x;
  float ss = 0.f;
  if (src.embd_row) {
    for (uint32_t i = tid; i < K; i += kThreads) {
      const float v = to_float(reinterpret_cast<const WT*>(src.embd_row)[i]);  // TokenEmbedShader.cs:139-158
      if (src.x_copy && blockIdx.x == 0) src.x_copy[i] = v;
      xs[i] = v;
      ss = fmaf(v, v, ss);
    }
  } else if ((K & 3u) == 0) {
    const float4* x4 = reinterpret_cast<const float4*>(src.x);
    float4* xs4 = reinterpret_cast<float4*>(xs);
    const uint32_t n4 = K >> 2;
    for (uint32_t base = 0; base < n4; base += 8 * kThreads) {
      float4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const uint32_t i = base + u * kThreads + tid;
        v[u] = i < n4 ? __ldcg(x4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const uint32_t i = base + u * kThreads + tid;
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
    for (uint32_t i = tid; i < K; i += kThreads) {
      const float v = __ldcg(src.x + i);
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
  for (int w = 0; w < kWarps; ++w) tot += red[w];
  const float rms = sqrtf(__fdiv_rn(tot, (float)K) + p.eps);
  for (uint32_t i = tid; i < K; i += kThreads) xs[i] = __fmul_rn(__fdiv_rn(xs[i], rms), gs[i]);
  __syncthreads();
}

// One GEMV phase: request the first weights, synchronise the grid (unless this is the first phase of the step),
// bring x in, stream. Same streamer as gemv_kernel (gemv.cu).
template <typename WT, typename KVT, int R, int U, int EPI>
__device__ __noinline__ bool gemv_phase(const GemvParams p, const XSource src, Sync& sy, bool barrier_first,
                                           float* smem, float* gs, uint32_t* s_flag) {
  float* red = smem;
  float* xs = smem + 32;
  constexpr int VE = WeightVec<WT>::kElems;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t nvec = p.K / VE;
  const uint32_t nkb = (nvec + 32 * U - 1) / (32 * U);
  const uint32_t nrb = (p.N + R - 1) / R;
  const uint32_t TW = gridDim.x * kWarps;
  const WT* const Wbase = reinterpret_cast<const WT*>(p.W);
  const uint4 zero = make_uint4(0, 0, 0, 0);

  auto load_batch = [&](uint4(&buf)[U][R], uint32_t rb, uint32_t kb) {
    if (rb >= nrb) return;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      uint32_t n = rb * R + r;
      n = n < p.N ? n : p.N - 1;
      const uint4* wrow = reinterpret_cast<const uint4*>(Wbase + (size_t)n * p.K);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        uint32_t v = kb * (32 * U) + lane + 32 * u;
        buf[u][r] = v < nvec ? ld_stream16(wrow + v) : zero;
      }
    }
  };

  uint32_t rb = blockIdx.x * kWarps + warp, kb = 0;
  uint4 cur[U][R];
  load_batch(cur, rb, 0);
  stage_gain(p, gs);
  if (barrier_first) {
    if (!grid_barrier(sy, s_flag)) return false;
  }
  load_x_cg<WT>(p, src, xs, gs, red);
  stamp(sy);  // x is in shared memory

  float best_v = -INFINITY;
  uint32_t best_i = 0xffffffffu;
  float acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.f;

  while (rb < nrb) {
    uint32_t nrb_next = rb, nkb_next = kb + 1;
    if (nkb_next == nkb) {
      nkb_next = 0;
      nrb_next = rb + TW;
    }
    uint4 nxt[U][R];
    load_batch(nxt, nrb_next, nkb_next);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      uint32_t v = kb * (32 * U) + lane + 32 * u;
      if (v < nvec) {
        float xv[VE];
        const float4* xp = reinterpret_cast<const float4*>(xs + (size_t)v * VE);
#pragma unroll
        for (int i = 0; i < VE / 4; ++i) {
          float4 t = xp[i];
          xv[4 * i] = t.x;
          xv[4 * i + 1] = t.y;
          xv[4 * i + 2] = t.z;
          xv[4 * i + 3] = t.w;
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
          float wf[VE];
          WeightVec<WT>::unpack(cur[u][r], wf);
#pragma unroll
          for (int i = 0; i < VE; ++i) acc[r] = fmaf(wf[i], xv[i], acc[r]);
        }
      }
    }
    if (nkb_next == 0) {
#pragma unroll
      for (int r = 0; r < R; ++r) acc[r] = warp_sum(acc[r]);
      row_epilogue<KVT, R, EPI>(p, rb * R, acc, best_v, best_i);
#pragma unroll
      for (int r = 0; r < R; ++r) acc[r] = 0.f;
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int r = 0; r < R; ++r) cur[u][r] = nxt[u][r];
    rb = nrb_next;
    kb = nkb_next;
  }
  if constexpr (EPI == EPI_LOGITS) cta_argmax_partial(p, best_v, best_i, red);
  return true;
}

// Not inlined: each phase gets its own register allocation instead of one allocation for the union of all phases.
template <typename KVT, int D>
__device__ __noinline__ void attn_phase(const AttnParams a, uint32_t bx, uint32_t s, uint32_t seq) {
  attn_core<KVT, D, kWarps, true, kMegaHeads>(a, bx, s, seq, kMegaMinChunk);
}

template <typename WT, typename KVT, int D>
__global__ void __launch_bounds__(kThreads, kFusedCtasPerSm) decode_step_kernel(const StepDesc* __restrict__ dp) {
  extern __shared__ __align__(16) float smem[];
  __shared__ uint32_t s_flag;
  const StepDesc& d = *dp;
  Sync sy{d.sync_counter, d.abort_flag, 0, d.trace, 0};
  const uint32_t H = d.H, qDim = d.qH * D, kvDim = d.kvH * D;
  uint32_t kmax = H > d.F ? H : d.F;
  kmax = kmax > qDim ? kmax : qDim;
  float* gs = smem + 32 + kmax;  // gain region behind the longest x (layout of megastep_smem)
  const uint32_t pos = d.state->pos;
  uint32_t tok = d.prompt ? d.prompt[d.state->prompt_idx] : d.state->cur_token;
  if (pos >= d.ctx) {  // same value in every CTA: all leave
    if (blockIdx.x == 0 && threadIdx.x == 0) atomicOr(&d.state->err, 2u);
    return;
  }
  if (tok >= d.embd_rows) {
    if (blockIdx.x == 0 && threadIdx.x == 0) atomicOr(&d.state->err, 1u);
    tok = 0;
  }
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
      XSource src;
      if (l == 0) {
        src.embd_row = (const char*)d.embd + (size_t)tok * H * sizeof(WT);
        src.x_copy = x_in;
      } else {
        src.x = x_in;
      }
      ok = gemv_phase<WT, KVT, kWideR, kWideU, EPI_QKV_ROPE>(p, src, sy, l != 0, smem, gs, &s_flag);
      if (!ok) break;
    }
    {  // attention over positions 0..pos
      ok = grid_barrier(sy, &s_flag);
      if (!ok) break;
      AttnParams a;
      a.q = d.q; a.kcache = kcl; a.vcache = vcl; a.qH = d.qH; a.kvH = d.kvH; a.d = D; a.out = d.attn_out;
      a.part = d.attn_part; a.tickets = d.tickets; a.S_max = d.S_max;
      const uint32_t nx = d.kvH * ((d.qH / d.kvH + kMegaHeads - 1) / kMegaHeads);
      if (blockIdx.x < nx * d.S_max)
        attn_phase<KVT, D>(a, blockIdx.x % nx, blockIdx.x / nx, pos + 1);
    }
    {  // O projection + residual
      GemvParams p;
      p.W = L.o; p.N = H; p.K = qDim; p.resid = x_in; p.y = x_mid;
      XSource src;
      src.x = d.attn_out;
      ok = gemv_phase<WT, KVT, kNarrowR, kNarrowU, EPI_STORE>(p, src, sy, true, smem, gs, &s_flag);
      if (!ok) break;
    }
    {  // RMSNorm + gate/up + SiLU*up
      GemvParams p;
      p.W = L.gateup; p.N = 2 * d.F; p.K = H; p.gain = L.ffn_norm; p.eps = d.eps; p.y = d.hbuf;
      XSource src;
      src.x = x_mid;
      ok = gemv_phase<WT, KVT, kWideR, kWideU, EPI_SILU_MUL>(p, src, sy, true, smem, gs, &s_flag);
      if (!ok) break;
    }
    {  // down projection + residual
      GemvParams p;
      p.W = L.down; p.N = H; p.K = d.F; p.resid = x_mid; p.y = x_out;
      XSource src;
      src.x = d.hbuf;
      ok = gemv_phase<WT, KVT, kNarrowR, kNarrowU, EPI_STORE>(p, src, sy, true, smem, gs, &s_flag);
      if (!ok) break;
    }
  }
  if (!ok) {
    if (threadIdx.x == 0) atomicOr(&d.state->err, 4u);
    return;
  }
  if (d.with_head) {
    GemvParams p;
    p.W = d.head; p.N = d.V; p.K = H; p.gain = d.out_norm; p.eps = d.eps; p.y = d.logits;
    p.part_val = d.part_val; p.part_idx = d.part_idx;
    XSource src;
    src.x = d.xbuf + (size_t)(2 * d.L) * H;
    ok = gemv_phase<WT, KVT, kWideR, kWideU, EPI_LOGITS>(p, src, sy, true, smem, gs, &s_flag);
    if (ok) ok = grid_barrier(sy, &s_flag);
    if (!ok) {
      if (threadIdx.x == 0) atomicOr(&d.state->err, 4u);
      return;
    }
    if (blockIdx.x != 0) return;
    // lowest index among the maxima (SamplingUtils.cs:55-56) over the per-CTA partials
    float* sv = smem;
    uint32_t* si = reinterpret_cast<uint32_t*>(smem) + kThreads;
    float bv = -INFINITY;
    uint32_t bi = 0xffffffffu;
    for (uint32_t i = threadIdx.x; i < gridDim.x; i += kThreads) {
      const float v = __ldcg(d.part_val + i);
      const uint32_t ix = __ldcg(d.part_idx + i);
      if (ix != 0xffffffffu && (bi == 0xffffffffu || v > bv || (v == bv && ix < bi))) {
        bv = v;
        bi = ix;
      }
    }
    sv[threadIdx.x] = bv;
    si[threadIdx.x] = bi;
    __syncthreads();
    for (int o = kThreads / 2; o > 0; o >>= 1) {
      if ((int)threadIdx.x < o) {
        const float v = sv[threadIdx.x + o], cv = sv[threadIdx.x];
        const uint32_t ix = si[threadIdx.x + o], ci = si[threadIdx.x];
        if (ix != 0xffffffffu && (ci == 0xffffffffu || v > cv || (v == cv && ix < ci))) {
          sv[threadIdx.x] = v;
          si[threadIdx.x] = ix;
        }
      }
      __syncthreads();
    }
    if (threadIdx.x == 0) {
      const uint32_t best = si[0] == 0xffffffffu ? 0u : si[0];
      StepState* st = d.state;
      if (d.history && st->steps < d.history_cap) d.history[st->steps] = best;
      st->last_argmax = best;
      st->cur_token = best;
      st->pos = pos + 1;
      st->steps += 1;
    }
  } else {
    // head-less prompt step: the position may only advance once every CTA has read it -- all did, at entry,
    // before their first barrier, and this CTA has passed 5L barriers since
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      d.state->pos = pos + 1;
      d.state->prompt_idx += 1;
    }
  }
}

template <typename WT, typename KVT>
cudaError_t pick_d(uint32_t d, const void** fn) {
  switch (d) {
    case 32: *fn = (const void*)decode_step_kernel<WT, KVT, 32>; return cudaSuccess;
    case 64: *fn = (const void*)decode_step_kernel<WT, KVT, 64>; return cudaSuccess;
    case 128: *fn = (const void*)decode_step_kernel<WT, KVT, 128>; return cudaSuccess;
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t pick(int wdtype, int kvdtype, uint32_t d, const void** fn) {
  if (wdtype == 1) return kvdtype == 1 ? pick_d<__half, __half>(d, fn) : pick_d<__half, float>(d, fn);
  return kvdtype == 1 ? pick_d<float, __half>(d, fn) : pick_d<float, float>(d, fn);
}

}  // namespace

size_t megastep_smem(uint32_t H, uint32_t F, uint32_t qDim) {
  uint32_t kmax = H > F ? H : F;
  kmax = kmax > qDim ? kmax : qDim;
  size_t floats = 32 + (size_t)kmax + H;  // reduction scratch, x (longest input), gain (only for K = H phases)
  if (floats < 2 * kThreads) floats = 2 * kThreads;  // the final arg-max reduction reuses the buffer
  return floats * sizeof(float);
}

cudaError_t megastep_max_grid(int wdtype, int kvdtype, uint32_t d, size_t smem, int* grid_out) {
  const void* fn = nullptr;
  cudaError_t e = pick(wdtype, kvdtype, d, &fn);
  if (e != cudaSuccess) return e;
  if (smem > 48 * 1024) {
    e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  int per_sm = 0, dev = 0, sms = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kThreads, smem);
  if (e != cudaSuccess) return e;
  e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return e;
  if (per_sm < 1) return cudaErrorLaunchOutOfResources;
  if (per_sm > kFusedCtasPerSm) per_sm = kFusedCtasPerSm;
  *grid_out = per_sm * sms;
  return cudaSuccess;
}

cudaError_t launch_megastep(cudaStream_t s, int wdtype, int kvdtype, uint32_t d, const StepDesc* desc_dev, int grid,
                            size_t smem) {
  const void* fn = nullptr;
  cudaError_t e = pick(wdtype, kvdtype, d, &fn);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs resident, or the launch fails
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  void* args[] = {(void*)&desc_dev};
  return cudaLaunchKernelExC(&cfg, fn, args);
}

}  // namespace nfai
