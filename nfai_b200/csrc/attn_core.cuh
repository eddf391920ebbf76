// The body of the split-KV decode attention, shared by the stand-alone kernel (attn.cu) and the fused decode step.
#pragma once
#include <math.h>

#include "common.cuh"
#include "kernels.h"

namespace nfai {
namespace attn_detail {

constexpr float kNegBig = -1.0e38f;  // AttentionSoftmaxShader.cs:156: maxScore = -1.0e38

// Eight consecutive cache elements: fetched raw (so that several steps can be in flight in few registers) and
// widened to float32 when used.
template <typename KVT>
struct KV8;
template <>
struct KV8<float> {
  static constexpr int kUnroll = 2;
  struct Raw { float4 a, b; };
  template <bool CG>
  __device__ __forceinline__ static Raw ld(const float* p) {
    Raw r;
    r.a = CG ? __ldcg(reinterpret_cast<const float4*>(p)) : *reinterpret_cast<const float4*>(p);
    r.b = CG ? __ldcg(reinterpret_cast<const float4*>(p + 4)) : *reinterpret_cast<const float4*>(p + 4);
    return r;
  }
  __device__ __forceinline__ static Raw zero() {
    Raw r;
    r.a = r.b = make_float4(0.f, 0.f, 0.f, 0.f);
    return r;
  }
  __device__ __forceinline__ static void unpack(const Raw& r, float (&f)[8]) {
    f[0] = r.a.x; f[1] = r.a.y; f[2] = r.a.z; f[3] = r.a.w;
    f[4] = r.b.x; f[5] = r.b.y; f[6] = r.b.z; f[7] = r.b.w;
  }
};
template <>
struct KV8<__half> {
  static constexpr int kUnroll = 4;
  struct Raw { uint4 v; };
  template <bool CG>
  __device__ __forceinline__ static Raw ld(const __half* p) {
    Raw r;
    r.v = CG ? __ldcg(reinterpret_cast<const uint4*>(p)) : *reinterpret_cast<const uint4*>(p);
    return r;
  }
  __device__ __forceinline__ static Raw zero() {
    Raw r;
    r.v = make_uint4(0, 0, 0, 0);
    return r;
  }
  __device__ __forceinline__ static void unpack(const Raw& r, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&r.v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __half22float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
};

// Last step of a split sequence, run by the CTA that drew the last ticket of its (KV head, head group): the partials
// (unnormalised sums, m, l) of the S_eff splits of heads h0 .. h0 + nh - 1 are merged and the output is written.
// A warp per head turns the m's into weights (lanes along the splits: one round trip to L2 for any S_eff <= 32), then
// every thread adds one output element over the splits with eight loads in flight -- a loop of dependent loads here
// costs a round trip per split, microseconds at 18 splits. Every thread of the CTA calls it (one block barrier).
constexpr int kAttnMergeCap = 256;  // upper bound on S_max (attn_splits never returns more)
template <int D, int NT>
__device__ __forceinline__ void attn_merge_splits(const AttnParams& p, const uint32_t h0, const uint32_t nh, const uint32_t S_eff) {
  constexpr int STR = D + 2;
  __shared__ float mw[4][kAttnMergeCap];
  __shared__ float mlinv[4];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (uint32_t j = warp; j < nh; j += NT / 32) {
    const float* bp = p.part + (size_t)(h0 + j) * p.S_max * STR;
    float mk[kAttnMergeCap / 32];
    float M = kNegBig;
#pragma unroll
    for (int u = 0; u < kAttnMergeCap / 32; ++u) {
      const uint32_t k = lane + 32 * u;
      mk[u] = k < S_eff ? __ldcg(bp + k * STR + D) : kNegBig;
      M = fmaxf(M, mk[u]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    float ls = 0.f;
#pragma unroll
    for (int u = 0; u < kAttnMergeCap / 32; ++u) {
      const uint32_t k = lane + 32 * u;
      if (k < S_eff) {
        const float w = __expf(mk[u] - M);
        mw[j][k] = w;
        ls = fmaf(__ldcg(bp + k * STR + D + 1), w, ls);
      }
    }
    ls = warp_sum(ls);
    if (lane == 0) mlinv[j] = 1.0f / ls;
  }
  __syncthreads();
  for (int idx = tid; idx < (int)nh * D; idx += NT) {
    const int j = idx / D, i = idx % D;
    const float* bp = p.part + (size_t)(h0 + j) * p.S_max * STR + i;
    float O = 0.f;
    uint32_t k = 0;
    for (; k + 8 <= S_eff; k += 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = __ldcg(bp + (size_t)(k + u) * STR);
#pragma unroll
      for (int u = 0; u < 8; ++u) O = fmaf(v[u], mw[j][k + u], O);
    }
    for (; k < S_eff; ++k) O = fmaf(__ldcg(bp + (size_t)k * STR), mw[j][k], O);
    p.out[(h0 + j) * D + i] = O * mlinv[j];
  }
}

// Second half of the attention of one CTA: every lane holds an online-softmax state (m, l, acc) over its own
// positions for up to kG query heads; merge lanes -> warps -> (if the sequence was split) CTAs, and write the output.
// Every thread of the CTA must call it (block barriers).
template <int D, int NW, int kG>
__device__ __forceinline__ void attn_finish(const AttnParams& p, const uint32_t bx, const uint32_t s, const uint32_t S_eff,
                                            const uint32_t h0, const uint32_t nh, float (&m)[kG], float (&l)[kG],
                                            float (&acc)[kG][8]) {
  constexpr int kAT = NW * 32;
  constexpr int kAW = NW;
  constexpr int LPP = D / 8;    // lanes per position
  constexpr int STR = D + 2;    // one partial in scratch: D accumulators, m, l
  constexpr int SSTR = D + 4;   // the same in shared memory, padded so that every row stays 16-byte aligned
  __shared__ __align__(16) float wpart[kAW][kG][SSTR];  // per-warp partials
  __shared__ float fin_scale[kAW][kG];
  __shared__ float fin_ML[kG][2];
  __shared__ uint32_t is_last;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int grp = lane / LPP, sub = lane % LPP;

  // ---- merge the lane groups of the warp (same dims, different positions)
#pragma unroll
  for (int o = LPP; o < 32; o <<= 1) {
#pragma unroll
    for (int j = 0; j < kG; ++j) {
      const float m_o = __shfl_xor_sync(0xffffffffu, m[j], o);
      const float l_o = __shfl_xor_sync(0xffffffffu, l[j], o);
      const float m_new = fmaxf(m[j], m_o);
      const float a = __expf(m[j] - m_new), b = __expf(m_o - m_new);
      l[j] = l[j] * a + l_o * b;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float acc_o = __shfl_xor_sync(0xffffffffu, acc[j][e], o);
        acc[j][e] = acc[j][e] * a + acc_o * b;
      }
      m[j] = m_new;
    }
  }
  if (grp == 0) {
#pragma unroll
    for (int j = 0; j < kG; ++j) {
      float* w = &wpart[warp][j][sub * 8];
      *reinterpret_cast<float4*>(w) = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
      *reinterpret_cast<float4*>(w + 4) = make_float4(acc[j][4], acc[j][5], acc[j][6], acc[j][7]);
      if (sub == 0) {
        wpart[warp][j][D] = m[j];
        wpart[warp][j][D + 1] = l[j];
      }
    }
  }
  __syncthreads();
  // ---- merge the warps of the CTA
  if (tid < kG) {
    float M = kNegBig;
    for (int w = 0; w < kAW; ++w) M = fmaxf(M, wpart[w][tid][D]);
    float L = 0.f;
    for (int w = 0; w < kAW; ++w) {
      const float sc = __expf(wpart[w][tid][D] - M);
      fin_scale[w][tid] = sc;
      L = fmaf(wpart[w][tid][D + 1], sc, L);
    }
    fin_ML[tid][0] = M;
    fin_ML[tid][1] = L;
  }
  __syncthreads();
  const uint32_t pstride = STR;
  for (int idx = tid; idx < (int)nh * D; idx += kAT) {
    const int j = idx / D, i = idx % D;
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < kAW; ++w) o = fmaf(wpart[w][j][i], fin_scale[w][j], o);
    if (S_eff == 1) {
      const float r = o * (1.0f / fin_ML[j][1]);
      if (p.out_half)
        p.out_half[(h0 + j) * D + i] = __float2half_rn(r);
      else
        p.out[(h0 + j) * D + i] = r;
    }
    else
      p.part[((size_t)(h0 + j) * p.S_max + s) * pstride + i] = o;
  }
  if (S_eff == 1) return;

  // ---- several splits: publish the partial, the last CTA of this (kv head, head group) merges
  if (tid < (int)nh) {
    float* pp = p.part + ((size_t)(h0 + tid) * p.S_max + s) * pstride;
    pp[D] = fin_ML[tid][0];
    pp[D + 1] = fin_ML[tid][1];
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const uint32_t ticket = atomicAdd(&p.tickets[bx], 1u);
    is_last = ticket == S_eff - 1 ? 1u : 0u;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  attn_merge_splits<D, kAT>(p, h0, nh, S_eff);
  if (tid == 0) p.tickets[bx] = 0;  // ready for the next launch
}

// One CTA of NW warps: KV head / head group `bx`, split `s` of a sequence of `seq` positions. Every thread of the
// CTA must call it (it uses block barriers); it returns early, uniformly, when the split is not active.
// CG = true reads q, K and V with L2-only loads (needed when the caller wrote them earlier in the same kernel, or
// when the kernel may have started before its producer stored them).
// kG = query heads that share one pass over K and V (fewer heads, fewer registers).
// The CTA itself waits for the kernel that produced q and the newest K/V row (programmatic dependency wait): the K
// and V rows of all EARLIER positions were written by earlier steps, so the first batch of them is requested before
// that wait and is in registers when q arrives.
template <typename KVT, int D, int NW, bool CG, int kG, int UNR_ = 0>
__device__ __forceinline__ void attn_core(const AttnParams& p, const uint32_t bx, const uint32_t s, const uint32_t seq,
                                          const uint32_t min_chunk) {
  constexpr int kAT = NW * 32;
  constexpr int kAW = NW;
  constexpr int LPP = D / 8;    // lanes per position
  constexpr int PPW = 32 / LPP; // positions per warp step
  constexpr int UNR = UNR_ > 0 ? UNR_ : KV8<KVT>::kUnroll;  // steps whose K and V are requested together

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int grp = lane / LPP, sub = lane % LPP;
  const uint32_t G = p.qH / p.kvH;
  const uint32_t hgroups = (G + kG - 1) / kG;
  const uint32_t g = bx / hgroups;
  const uint32_t hg = bx % hgroups;
  const uint32_t h0 = g * G + hg * kG;
  const uint32_t nh = min((uint32_t)kG, G - hg * kG);
  const uint32_t kvDim = p.kvH * D;
  uint32_t chunk = (seq + p.S_max - 1) / p.S_max;
  chunk = chunk < min_chunk ? min_chunk : chunk;
  chunk = (chunk + 63) / 64 * 64;
  const uint32_t S_eff = (seq + chunk - 1) / chunk;
  if (s >= S_eff) return;
  const uint32_t t0 = s * chunk;
  const uint32_t t1 = min(seq, t0 + chunk);
  // the row the producing kernel of this step writes; with p.early == 0 the wait comes first and no row is special
  if (!p.early) pdl_wait();
  const uint32_t newest = p.early ? seq - 1 : 0xffffffffu;

  const KVT* kc = reinterpret_cast<const KVT*>(p.kcache) + g * D + sub * 8;
  const KVT* vc = reinterpret_cast<const KVT*>(p.vcache) + g * D + sub * 8;

  // ---- first batch, requested ahead of the dependency
  uint32_t base = t0 + warp * PPW;
  typename KV8<KVT>::Raw kr[UNR], vr[UNR];
  bool valid[UNR];
#pragma unroll
  for (int u = 0; u < UNR; ++u) {
    const uint32_t t = base + u * (kAW * PPW) + grp;
    valid[u] = t < t1;
    const bool early = valid[u] && t != newest;
    kr[u] = early ? KV8<KVT>::template ld<CG>(kc + (size_t)t * kvDim) : KV8<KVT>::zero();
    vr[u] = early ? KV8<KVT>::template ld<CG>(vc + (size_t)t * kvDim) : KV8<KVT>::zero();
  }
  if (p.early) pdl_wait();
#pragma unroll
  for (int u = 0; u < UNR; ++u) {
    const uint32_t t = base + u * (kAW * PPW) + grp;
    if (valid[u] && t == newest) {
      kr[u] = KV8<KVT>::template ld<CG>(kc + (size_t)t * kvDim);
      vr[u] = KV8<KVT>::template ld<CG>(vc + (size_t)t * kvDim);
    }
  }

  // this lane's eight dims of the (up to) four query heads
  float q[kG][8];
#pragma unroll
  for (int j = 0; j < kG; ++j) {
    if (j < (int)nh) {
      const float* qp = p.q + (h0 + j) * D + sub * 8;
      float4 a = CG ? __ldcg(reinterpret_cast<const float4*>(qp)) : *reinterpret_cast<const float4*>(qp);
      float4 b = CG ? __ldcg(reinterpret_cast<const float4*>(qp + 4)) : *reinterpret_cast<const float4*>(qp + 4);
      q[j][0] = a.x; q[j][1] = a.y; q[j][2] = a.z; q[j][3] = a.w;
      q[j][4] = b.x; q[j][5] = b.y; q[j][6] = b.z; q[j][7] = b.w;
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) q[j][e] = 0.f;
    }
  }
  const float scale = 1.0f / sqrtf((float)D);  // AttentionScoreCalculationShader.cs:112
  float m[kG], l[kG], acc[kG][8];
#pragma unroll
  for (int j = 0; j < kG; ++j) {
    m[j] = kNegBig;
    l[j] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[j][e] = 0.f;
  }

  while (base < t1) {
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      if (base + u * (kAW * PPW) >= t1) break;  // warp-uniform
      float kf[8], vf[8];
      KV8<KVT>::unpack(kr[u], kf);
      KV8<KVT>::unpack(vr[u], vf);
#pragma unroll
      for (int j = 0; j < kG; ++j) {
        float dot = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) dot = fmaf(q[j][e], kf[e], dot);
#pragma unroll
        for (int o = 1; o < LPP; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (valid[u]) {
          const float sc = dot * scale;
          const float m_new = fmaxf(m[j], sc);
          const float alpha = __expf(m[j] - m_new);
          const float pr = __expf(sc - m_new);
          l[j] = fmaf(l[j], alpha, pr);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[j][e] = fmaf(acc[j][e], alpha, pr * vf[e]);
          m[j] = m_new;
        }
      }
    }
    base += kAW * PPW * UNR;
    if (base >= t1) break;
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const uint32_t t = base + u * (kAW * PPW) + grp;
      valid[u] = t < t1;
      kr[u] = valid[u] ? KV8<KVT>::template ld<CG>(kc + (size_t)t * kvDim) : KV8<KVT>::zero();
      vr[u] = valid[u] ? KV8<KVT>::template ld<CG>(vc + (size_t)t * kvDim) : KV8<KVT>::zero();
    }
  }

  attn_finish<D, NW, kG>(p, bx, s, S_eff, h0, nh, m, l, acc);
}

}  // namespace attn_detail
}  // namespace nfai
