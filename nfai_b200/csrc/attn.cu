// Split-KV flash-decoding attention for one new token (batch 1) over a position-major KV cache.
//
// One kernel does what the reference does in three dispatches (scores, softmax, weighted value sum:
// NFAI.Vulkan.Shaders/AttentionScoreCalculationShader.cs:170-205, AttentionSoftmaxShader.cs:145-177,
// AttentionWeightedValueSumShader.cs:181-215) with single-thread workgroups:
//  * grid = (kvH * head_groups, S_max); a CTA of 16 warps owns one KV head, up to four of the query heads that
//    share it (GQA: kvHead = qHead / (qH/kvH)) and one contiguous range of positions, so K and V are read once
//    for all of those query heads;
//  * there is no shared-memory staging and no block barrier in the main loop: d/8 lanes own one position (eight
//    head dims each: one 16-byte load of a float16 row slice, two of a float32 one), so a warp covers 256/d
//    positions per step and the 16 warps of the CTA stride over the range; K and V of several steps are
//    requested before the first is used;
//  * every lane keeps an online softmax (running max m, sum l, accumulators rescaled by exp(m_old - m_new)) for
//    its own positions; lane groups are merged with shuffles, warps through shared memory;
//  * with more than one active split every CTA writes (unnormalised o, m, l) to scratch and takes a ticket;
//    the CTA that draws the last ticket of its KV head merges the splits and writes the output. No CTA waits
//    for another one, so nothing can hang.
// The number of active splits is derived on the device from the current position (512 positions per CTA at
// least), so one captured launch shape serves every position.
//
// Softmax equivalence: the reference computes exp(clamp(s - max, -80, 80)) / sum; s - max <= 0 so the upper clamp
// never acts, the lower clamp only replaces weights below e^-80 by e^-80 (a relative change below 1e-34), and
// sum >= 1 (the maximum contributes exp(0)) so the "sum > eps" guard always passes.
#include <math.h>

#include "common.cuh"
#include "kernels.h"

namespace nfai {

namespace {

constexpr int kAT = 512;            // threads per CTA
constexpr int kAW = kAT / 32;       // warps per CTA
constexpr int kG = (int)kAttnHeadsPerCta;
constexpr float kNegBig = -1.0e38f;  // AttentionSoftmaxShader.cs:156: maxScore = -1.0e38

// Eight consecutive cache elements: fetched raw (so that several steps can be in flight in few registers) and
// widened to float32 when used.
template <typename KVT>
struct KV8;
template <>
struct KV8<float> {
  static constexpr int kUnroll = 2;
  struct Raw { float4 a, b; };
  __device__ __forceinline__ static Raw ld(const float* p) {
    Raw r;
    r.a = *reinterpret_cast<const float4*>(p);
    r.b = *reinterpret_cast<const float4*>(p + 4);
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
  __device__ __forceinline__ static Raw ld(const __half* p) {
    Raw r;
    r.v = *reinterpret_cast<const uint4*>(p);
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

template <typename KVT, int D>
__global__ void __launch_bounds__(kAT, 1) attn_decode_kernel(const AttnParams p) {
  constexpr int LPP = D / 8;    // lanes per position
  constexpr int PPW = 32 / LPP; // positions per warp step
  constexpr int UNR = KV8<KVT>::kUnroll;
  constexpr int STR = D + 2;    // one partial in scratch: D accumulators, m, l
  constexpr int SSTR = D + 4;   // the same in shared memory, padded so that every row stays 16-byte aligned

  __shared__ __align__(16) float wpart[kAW][kG][SSTR];  // per-warp partials
  __shared__ float fin_scale[kAW][kG];
  __shared__ float fin_ML[kG][2];
  __shared__ uint32_t is_last;

  prefetch_plan(p.pf, kPrefetchChunk);
  pdl_launch_dependents();
  pdl_wait();  // q, K and V of this position come from the previous kernel

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int grp = lane / LPP, sub = lane % LPP;
  const uint32_t G = p.qH / p.kvH;
  const uint32_t hgroups = (G + kG - 1) / kG;
  const uint32_t g = blockIdx.x / hgroups;
  const uint32_t hg = blockIdx.x % hgroups;
  const uint32_t h0 = g * G + hg * kG;
  const uint32_t nh = min((uint32_t)kG, G - hg * kG);
  const uint32_t kvDim = p.kvH * D;
  const uint32_t seq = p.state ? p.state->pos + 1 : p.seq_imm;
  uint32_t chunk = (seq + p.S_max - 1) / p.S_max;
  chunk = chunk < kAttnMinChunk ? kAttnMinChunk : chunk;
  chunk = (chunk + 63) / 64 * 64;
  const uint32_t S_eff = (seq + chunk - 1) / chunk;
  const uint32_t s = blockIdx.y;
  if (s >= S_eff) return;
  const uint32_t t0 = s * chunk;
  const uint32_t t1 = min(seq, t0 + chunk);

  // this lane's eight dims of the (up to) four query heads
  float q[kG][8];
#pragma unroll
  for (int j = 0; j < kG; ++j) {
    if (j < (int)nh) {
      const float* qp = p.q + (h0 + j) * D + sub * 8;
      float4 a = *reinterpret_cast<const float4*>(qp);
      float4 b = *reinterpret_cast<const float4*>(qp + 4);
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
  const KVT* kc = reinterpret_cast<const KVT*>(p.kcache) + g * D + sub * 8;
  const KVT* vc = reinterpret_cast<const KVT*>(p.vcache) + g * D + sub * 8;

  for (uint32_t base = t0 + warp * PPW; base < t1; base += kAW * PPW * UNR) {
    typename KV8<KVT>::Raw kr[UNR], vr[UNR];
    bool valid[UNR];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const uint32_t t = base + u * (kAW * PPW) + grp;
      valid[u] = t < t1;
      kr[u] = valid[u] ? KV8<KVT>::ld(kc + (size_t)t * kvDim) : KV8<KVT>::zero();
      vr[u] = valid[u] ? KV8<KVT>::ld(vc + (size_t)t * kvDim) : KV8<KVT>::zero();
    }
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
  }

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
    if (S_eff == 1)
      p.out[(h0 + j) * D + i] = o * (1.0f / fin_ML[j][1]);
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
    const uint32_t ticket = atomicAdd(&p.tickets[blockIdx.x], 1u);
    is_last = ticket == S_eff - 1 ? 1u : 0u;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int idx = tid; idx < (int)nh * D; idx += kAT) {
    const int j = idx / D, i = idx % D;
    const float* bp = p.part + (size_t)(h0 + j) * p.S_max * pstride;
    float M = kNegBig;
    for (uint32_t k = 0; k < S_eff; ++k) M = fmaxf(M, __ldcg(bp + k * pstride + D));
    float Lsum = 0.f, O = 0.f;
    for (uint32_t k = 0; k < S_eff; ++k) {
      const float w = __expf(__ldcg(bp + k * pstride + D) - M);
      Lsum = fmaf(__ldcg(bp + k * pstride + D + 1), w, Lsum);
      O = fmaf(__ldcg(bp + k * pstride + i), w, O);
    }
    p.out[(h0 + j) * D + i] = O * (1.0f / Lsum);
  }
  if (tid == 0) p.tickets[blockIdx.x] = 0;  // ready for the next launch
}

template <typename KVT>
cudaError_t launch_d(cudaStream_t s, const AttnParams& p, bool pdl) {
  const uint32_t hgroups = attn_head_groups(p.qH, p.kvH);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.kvH * hgroups, p.S_max);
  cfg.blockDim = dim3(kAT);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  switch (p.d) {
    case 32: return cudaLaunchKernelEx(&cfg, attn_decode_kernel<KVT, 32>, p);
    case 64: return cudaLaunchKernelEx(&cfg, attn_decode_kernel<KVT, 64>, p);
    case 128: return cudaLaunchKernelEx(&cfg, attn_decode_kernel<KVT, 128>, p);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

uint32_t attn_head_groups(uint32_t qH, uint32_t kvH) {
  uint32_t G = qH / kvH;
  return (G + kAttnHeadsPerCta - 1) / kAttnHeadsPerCta;
}

// Upper bound on the number of splits for a cache of max_seq positions: at least kAttnMinChunk positions per
// split, and no more CTAs than the 148 SMs hold at once (one 512-thread CTA each), so there is no second wave.
uint32_t attn_splits(uint32_t qH, uint32_t kvH, uint32_t max_seq) {
  uint32_t ctas_x = kvH * attn_head_groups(qH, kvH);
  uint32_t by_len = (max_seq + kAttnMinChunk - 1) / kAttnMinChunk;
  uint32_t by_sm = 148u / ctas_x;
  if (by_sm < 1) by_sm = 1;
  uint32_t s = by_len < by_sm ? by_len : by_sm;
  return s < 1 ? 1 : s;
}

size_t attn_part_floats(uint32_t qH, uint32_t d, uint32_t S_max) { return (size_t)qH * S_max * (d + 2); }

cudaError_t launch_attn_decode(cudaStream_t s, int kvdtype, const AttnParams& p, bool pdl) {
  if (p.qH == 0 || p.kvH == 0 || p.qH % p.kvH != 0 || p.S_max == 0) return cudaErrorInvalidValue;
  if (!p.state && p.seq_imm == 0) return cudaErrorInvalidValue;
  return kvdtype == 1 ? launch_d<__half>(s, p, pdl) : launch_d<float>(s, p, pdl);
}

}  // namespace nfai
