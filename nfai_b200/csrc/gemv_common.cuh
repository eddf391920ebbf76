// Prologue (x, optional RMSNorm) and epilogues shared by the GEMV kernels of the decode step.
#pragma once
#include "common.cuh"
#include "kernels.h"

namespace nfai {
namespace gemv_detail {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

// ---- prologue: x (optionally RMS-normalised) into shared memory ----------------------------------------------
// The gain is a weight: it can be staged in shared memory before the programmatic-dependency wait.
__device__ __forceinline__ void load_gain(const GemvParams& p, float* xs, float* gs_at = nullptr) {
  if (p.gain == nullptr) return;
  float* gs = gs_at ? gs_at : xs + p.K;
  for (uint32_t i = threadIdx.x; i < p.K; i += kThreads) gs[i] = p.gain[i];
}

// Tensor-parallel input: x = residual + the partial vectors of all ranks, which the previous row-parallel GEMV of
// every rank stored into this rank's exchange area as (value, epoch) words. Four consecutive elements per call: the
// words of all ranks are requested together (each is an L2 round trip), re-read (bounded) until every one carries the
// epoch, then added from zero in rank order -- the arithmetic of xchg::sum_slots, the same on every rank. CTA 0 keeps
// the summed vector as the residual stream. Returns false when the budget ran out (x is then zero).
__device__ __forceinline__ bool pull_value4(const GemvParams& p, uint32_t epoch, uint32_t i4, float4* out) {
  const XchgHooks& t = p.tp;
  const uint4* mine = reinterpret_cast<const uint4*>(t.view.slots[t.view.rank]);  // one uint4 = two (value, epoch) words
  const float4 resid = __ldcg(reinterpret_cast<const float4*>(t.pull_resid) + i4);
  uint4 w[xchg::kMaxWorld][2];
  auto request = [&](int src) {
    const uint4* q = mine + (xchg::slot_offset(epoch, src) + 4 * (size_t)i4) / 2;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[src][0].x), "=r"(w[src][0].y), "=r"(w[src][0].z), "=r"(w[src][0].w) : "l"(q) : "memory");
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[src][1].x), "=r"(w[src][1].y), "=r"(w[src][1].z), "=r"(w[src][1].w) : "l"(q + 1) : "memory");
  };
  auto arrived = [&](int src) {
    return w[src][0].y == epoch && w[src][0].w == epoch && w[src][1].y == epoch && w[src][1].w == epoch;
  };
#pragma unroll
  for (int src = 0; src < xchg::kMaxWorld; ++src)
    if (src < t.view.world) request(src);
  bool ok = true;
  unsigned long long t0 = 0;
  uint32_t polls = 0;
#pragma unroll
  for (int src = 0; src < xchg::kMaxWorld; ++src) {
    if (src < t.view.world) {
      while (ok && !arrived(src)) {
        if (t0 == 0) t0 = global_timer_ns();
        request(src);
        if ((++polls & 15u) == 0 && global_timer_ns() - t0 > t.wait_ns) ok = false;
      }
    }
  }
  float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int src = 0; src < xchg::kMaxWorld; ++src) {
    if (src < t.view.world) {
      sum.x += __uint_as_float(w[src][0].x);
      sum.y += __uint_as_float(w[src][0].z);
      sum.z += __uint_as_float(w[src][1].x);
      sum.w += __uint_as_float(w[src][1].z);
    }
  }
  *out = ok ? make_float4(resid.x + sum.x, resid.y + sum.y, resid.z + sum.z, resid.w + sum.w) : make_float4(0.f, 0.f, 0.f, 0.f);
  if (blockIdx.x == 0 && ok) reinterpret_cast<float4*>(t.pull_store)[i4] = *out;
  return ok;
}

// Where element k of x sits in shared memory. Natural order for kernels whose lanes read 16 bytes of x per step
// (float32 weights, and the register streamer). With float16 weights a lane needs 32 bytes per step (elements
// 8*lane .. 8*lane+7 of a 256-element block); read as two 16-byte loads from the natural order those loads hit every
// bank twice, and the stream from shared memory is bandwidth-bound on exactly these loads. The permuted order keeps,
// per 256-element block, the first halves of all lanes together and then the second halves: both loads of a warp
// cover 512 contiguous bytes.
template <bool PERM>
__device__ __forceinline__ uint32_t x_slot4(uint32_t i4) {  // index of the float4 that holds elements 4*i4 .. 4*i4+3
  if constexpr (!PERM) return i4;
  const uint32_t r = i4 & 63u;
  return (i4 & ~63u) + ((r & 1u) << 5) + (r >> 1);
}
template <bool PERM>
__device__ __forceinline__ uint32_t x_slot(uint32_t k) { return 4u * x_slot4<PERM>(k >> 2) + (k & 3u); }

// ss = sum x^2 ; rms = sqrt(ss/K + eps) ; xs = (x / rms) * gain   (RMSNormShader.cs:136-148)
// With PERM the shared-memory area of x must be a whole number of 256-element blocks.
template <bool PERM = false>
__device__ __forceinline__ void load_x(const GemvParams& p, float* xs, float* red, const float* gs_in = nullptr) {
  const uint32_t K = p.K;
  const int tid = threadIdx.x;
  const bool pull = p.tp.pull != 0;
  // x sits in L2 (another kernel, or under tensor parallelism other GPUs, wrote it): the loads of one thread are
  // issued together, four elements each, before any of them is used.
  const float* gs = gs_in ? gs_in : xs + K;  // staged by load_gain() before the dependency wait
  const bool norm = p.gain != nullptr;
  float ss = 0.f;
  if (pull) {  // the host guarantees K % 4 == 0 and 16-byte aligned vectors for a pulling kernel
    const uint32_t pull_epoch = *p.tp.epoch_base + p.tp.pull_index + 1;
    bool pull_ok = true;
    for (uint32_t i = tid; i < (K >> 2); i += kThreads) {
      float4 v;
      if (pull_ok) pull_ok = pull_value4(p, pull_epoch, i, &v);
      else v = make_float4(0.f, 0.f, 0.f, 0.f);
      reinterpret_cast<float4*>(xs)[x_slot4<PERM>(i)] = v;
      ss = fmaf(v.x, v.x, ss);
      ss = fmaf(v.y, v.y, ss);
      ss = fmaf(v.z, v.z, ss);
      ss = fmaf(v.w, v.w, ss);
    }
    if (!pull_ok) {  // a rank did not deliver in time: report, the kernel still runs to its end
      if (p.state) atomicOr(&p.state->err, 4u);
      if (p.err) atomicOr(p.err, 4u);
    }
  } else if ((K & 3u) == 0 && (reinterpret_cast<uintptr_t>(p.x) & 15) == 0) {
    const float4* x4 = reinterpret_cast<const float4*>(p.x);
    const uint32_t n4 = K >> 2;
    constexpr int B = 4;
    for (uint32_t base = 0; base < n4; base += B * kThreads) {
      float4 v[B];
#pragma unroll
      for (int j = 0; j < B; ++j) {
        const uint32_t i = base + j * kThreads + tid;
        v[j] = i < n4 ? x4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int j = 0; j < B; ++j) {
        const uint32_t i = base + j * kThreads + tid;
        if (i < n4) {
          reinterpret_cast<float4*>(xs)[x_slot4<PERM>(i)] = v[j];
          ss = fmaf(v[j].x, v[j].x, ss);
          ss = fmaf(v[j].y, v[j].y, ss);
          ss = fmaf(v[j].z, v[j].z, ss);
          ss = fmaf(v[j].w, v[j].w, ss);
        }
      }
    }
  } else {
    for (uint32_t i = tid; i < K; i += kThreads) {
      const float v = p.x[i];
      xs[x_slot<PERM>(i)] = v;
      ss = fmaf(v, v, ss);
    }
  }
  if (!norm) {
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
  for (uint32_t i = tid; i < K; i += kThreads) {
    const uint32_t j = x_slot<PERM>(i);
    xs[j] = __fmul_rn(__fdiv_rn(xs[j], rms), gs[i]);
  }
  __syncthreads();
}

// ---- tensor-parallel push: the finished row sums of this rank go into its slot on every rank ----------------------
// Each value travels with the exchange's epoch in one 8-byte word; two neighbouring rows go out as one 16-byte store
// (two independent words: a reader checks the epoch of each). Nothing else is needed to publish them.
template <int R>
__device__ __forceinline__ void push_rows(const GemvParams& p, uint32_t row0, const float (&acc)[R]) {
  const xchg::View& v = p.tp.view;
  const uint32_t epoch = *p.tp.epoch_base + p.tp.push_index + 1;
  const size_t base = xchg::slot_offset(epoch, v.rank);
#pragma unroll
  for (int r = 0; r < R; r += 2) {
    const uint32_t n = row0 + r;
    if (n >= p.N) break;
    if (r + 1 < R && n + 1 < p.N && (n & 1u) == 0) {
      for (int dst = 0; dst < v.world; ++dst) {
        unsigned long long* q = v.slots[dst] + base + n;
        asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(q), "r"(__float_as_uint(acc[r])), "r"(epoch),
                     "r"(__float_as_uint(acc[r + 1])), "r"(epoch)
                     : "memory");
      }
    } else {
      DeviceXchgMem mem;
      xchg::push_value(mem, v, epoch, n, acc[r]);
      if (r + 1 < R && n + 1 < p.N) xchg::push_value(mem, v, epoch, n + 1, acc[r + 1]);
    }
  }
}

// ---- epilogues (lane 0 of the warp holds the R finished row sums of one row block) --------------------------------
template <typename KVT, int R, int EPI>
__device__ __forceinline__ void row_epilogue(const GemvParams& p, uint32_t row0, const float (&acc)[R], float& best_v,
                                             uint32_t& best_i) {
  if ((threadIdx.x & 31) != 0) return;
  if constexpr (EPI == EPI_STORE) {
    if (p.tp.push) {
      push_rows<R>(p, row0, acc);
      return;
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      uint32_t n = row0 + r;
      if (n < p.N) p.y[n] = p.resid ? __ldcg(p.resid + n) + acc[r] : acc[r];
    }
  } else if constexpr (EPI == EPI_QKV_ROPE) {
    static_assert(R % 2 == 0, "RoPE pairs adjacent rows");
    const uint32_t pos = p.state ? p.state->pos : p.pos_imm;
    if (pos >= p.ctx) {
      if (p.state) atomicOr(&p.state->err, 2u);
      return;
    }
#pragma unroll
    for (int r = 0; r < R; r += 2) {
      uint32_t n = row0 + r;
      if (n >= p.N) break;
      float a = acc[r], b = acc[r + 1];
      if (n < p.qDim + p.kvDim) {  // Q or K: rotate the pair (2m, 2m+1) of its head
        uint32_t local = n < p.qDim ? n : n - p.qDim;
        uint32_t i = local % p.d;
        if (i < p.ropeDim) {
          float2 cs = p.rope_cs[(size_t)pos * (p.ropeDim / 2) + (i >> 1)];
          // value1 = cos*a - sin*b ; value2 = sin*a + cos*b (RoPEShader.cs:256-257), products rounded separately
          float v1 = __fsub_rn(__fmul_rn(cs.x, a), __fmul_rn(cs.y, b));
          float v2 = __fadd_rn(__fmul_rn(cs.y, a), __fmul_rn(cs.x, b));
          a = v1;
          b = v2;
        }
        if (n < p.qDim) {
          p.q_out[n] = a;
          p.q_out[n + 1] = b;
        } else {
          KVT* kc = reinterpret_cast<KVT*>(p.kcache) + (size_t)pos * p.kvDim + local;
          store_as(kc, a);
          store_as(kc + 1, b);
        }
      } else {
        KVT* vc = reinterpret_cast<KVT*>(p.vcache) + (size_t)pos * p.kvDim + (n - p.qDim - p.kvDim);
        store_as(vc, a);
        store_as(vc + 1, b);
      }
    }
  } else if constexpr (EPI == EPI_SILU_MUL) {
    static_assert(R % 2 == 0, "gate and up rows are interleaved");
#pragma unroll
    for (int r = 0; r < R; r += 2) {
      uint32_t n = row0 + r;
      if (n >= p.N) break;
      float gate = acc[r], up = acc[r + 1];
      // sigmoid = 1/(1+exp(-x)); silu = x*sigmoid; h = up*silu (SiLUShader.cs:121-123, ElementWiseMul A=up,B=silu)
      float sig = __fdiv_rn(1.0f, 1.0f + expf(-gate));
      p.y[n >> 1] = __fmul_rn(up, __fmul_rn(gate, sig));
    }
  } else {  // EPI_LOGITS: store and keep the warp's best (lowest index among equal maxima)
#pragma unroll
    for (int r = 0; r < R; ++r) {
      uint32_t n = row0 + r;
      if (n < p.N) {
        p.y[n] = acc[r];
        if (best_i == 0xffffffffu || acc[r] > best_v || (acc[r] == best_v && n < best_i)) {
          best_v = acc[r];
          best_i = n;
        }
      }
    }
  }
}

// ---- the same epilogues with their inputs fetched ahead of time ------------------------------------------------
// What an epilogue reads besides the row sums (the residual, the position's cos/sin pair) sits in L2; fetched at
// the moment the row sum is complete it would add a full L2 round trip to the tail of every row block. The
// streamer asks for it one item ahead and hands it over here. Every lane runs the preload (same address: one
// broadcast load).
template <int R, int EPI>
__device__ __forceinline__ void epi_preload(const GemvParams& p, uint32_t row0, uint32_t pos, float (&pre)[R]) {
  if constexpr (EPI == EPI_STORE) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const uint32_t n = row0 + r < p.N ? row0 + r : p.N - 1;
      pre[r] = p.resid ? __ldcg(p.resid + n) : 0.f;
    }
  } else if constexpr (EPI == EPI_QKV_ROPE) {
#pragma unroll
    for (int r = 0; r < R; r += 2) {
      const uint32_t n = row0 + r;
      float2 cs = make_float2(1.f, 0.f);
      if (n < p.qDim + p.kvDim && n < p.N && pos < p.ctx) {
        const uint32_t local = n < p.qDim ? n : n - p.qDim;
        const uint32_t i = local % p.d;
        if (i < p.ropeDim) cs = __ldg(p.rope_cs + (size_t)pos * (p.ropeDim / 2) + (i >> 1));
      }
      pre[r] = cs.x;
      pre[r + 1] = cs.y;
    }
  } else {
#pragma unroll
    for (int r = 0; r < R; ++r) pre[r] = 0.f;
  }
}

template <typename KVT, int R, int EPI>
__device__ __forceinline__ void row_epilogue_pre(const GemvParams& p, uint32_t row0, const float (&acc)[R],
                                                 const float (&pre)[R], uint32_t pos, float& best_v, uint32_t& best_i) {
  if ((threadIdx.x & 31) != 0) return;
  if constexpr (EPI == EPI_STORE) {
    if (p.tp.push) {
      push_rows<R>(p, row0, acc);
      return;
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      uint32_t n = row0 + r;
      if (n < p.N) p.y[n] = p.resid ? pre[r] + acc[r] : acc[r];
    }
  } else if constexpr (EPI == EPI_QKV_ROPE) {
    static_assert(R % 2 == 0, "RoPE pairs adjacent rows");
    if (pos >= p.ctx) {
      if (p.state) atomicOr(&p.state->err, 2u);
      return;
    }
#pragma unroll
    for (int r = 0; r < R; r += 2) {
      uint32_t n = row0 + r;
      if (n >= p.N) break;
      float a = acc[r], b = acc[r + 1];
      if (n < p.qDim + p.kvDim) {
        uint32_t local = n < p.qDim ? n : n - p.qDim;
        uint32_t i = local % p.d;
        if (i < p.ropeDim) {
          const float c = pre[r], sn = pre[r + 1];
          float v1 = __fsub_rn(__fmul_rn(c, a), __fmul_rn(sn, b));
          float v2 = __fadd_rn(__fmul_rn(sn, a), __fmul_rn(c, b));
          a = v1;
          b = v2;
        }
        if (n < p.qDim) {
          p.q_out[n] = a;
          p.q_out[n + 1] = b;
        } else {
          KVT* kc = reinterpret_cast<KVT*>(p.kcache) + (size_t)pos * p.kvDim + local;
          store_as(kc, a);
          store_as(kc + 1, b);
        }
      } else {
        KVT* vc = reinterpret_cast<KVT*>(p.vcache) + (size_t)pos * p.kvDim + (n - p.qDim - p.kvDim);
        store_as(vc, a);
        store_as(vc + 1, b);
      }
    }
  } else {
    row_epilogue<KVT, R, EPI>(p, row0, acc, best_v, best_i);
  }
}

// EPI_LOGITS: one (max, lowest index) partial per CTA. Under tensor parallelism the CTA that finishes last also
// reduces all partials of this rank and pushes (value, global index) to every rank: the arg-max exchange needs no
// kernel of its own.
__device__ __forceinline__ void cta_argmax_partial(const GemvParams& p, float best_v, uint32_t best_i, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t* redi = reinterpret_cast<uint32_t*>(red);
  auto better = [](float v, uint32_t i, float bv, uint32_t bi) {
    return i != 0xffffffffu && (bi == 0xffffffffu || v > bv || (v == bv && i < bi));
  };
  __syncthreads();  // red[] may still be read by the prologue of a slower warp
  if (lane == 0) {
    red[warp] = best_v;
    redi[kWarps + warp] = best_i;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float v = red[0];
    uint32_t ix = redi[kWarps];
    for (int w = 1; w < kWarps; ++w)
      if (better(red[w], redi[kWarps + w], v, ix)) {
        v = red[w];
        ix = redi[kWarps + w];
      }
    p.part_val[blockIdx.x] = v;
    p.part_idx[blockIdx.x] = ix;
  }
  if (!p.tp.push) return;
  uint32_t* s_last = redi + 30;
  uint32_t* ticket = p.tp_ticket;
  if (threadIdx.x == 0) {
    __threadfence();
    *s_last = atomicAdd(ticket, 1u) == gridDim.x - 1 ? 1u : 0u;
  }
  __syncthreads();
  if (!*s_last) return;
  __threadfence();
  float bv = 0.f;
  uint32_t bi = 0xffffffffu;
  for (uint32_t i = threadIdx.x; i < gridDim.x; i += kThreads) {
    const float v = __ldcg(p.part_val + i);
    const uint32_t ix = __ldcg(p.part_idx + i);
    if (better(v, ix, bv, bi)) {
      bv = v;
      bi = ix;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, bv, bi)) {
      bv = ov;
      bi = oi;
    }
  }
  __syncthreads();
  if (lane == 0) {
    red[warp] = bv;
    redi[kWarps + warp] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 0; w < kWarps; ++w)
      if (w == 0 || better(red[w], redi[kWarps + w], bv, bi)) {
        bv = red[w];
        bi = redi[kWarps + w];
      }
    *ticket = 0;
    DeviceXchgMem mem;
    xchg::push_pair(mem, p.tp.view, *p.tp.epoch_base + p.tp.push_index + 1, bv, bi == 0xffffffffu ? bi : bi + p.v_lo);
  }
}

}  // namespace gemv_detail
}  // namespace nfai
