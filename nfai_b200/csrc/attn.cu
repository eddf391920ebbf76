// Split-KV flash-decoding attention for one new token (batch 1) over a position-major KV cache.
//
// One kernel does what the reference does in three dispatches (scores, softmax, weighted value sum:
// NFAI.Vulkan.Shaders/AttentionScoreCalculationShader.cs:170-205, AttentionSoftmaxShader.cs:145-177,
// AttentionWeightedValueSumShader.cs:181-215) with single-thread workgroups:
//  * grid = (kvH * head_groups, S_max); a CTA owns one KV head, up to four of the query heads that share it
//    (GQA: kvHead = qHead / (qH/kvH)) and one contiguous range of positions, so K and V are read once for all
//    of those query heads;
//  * positions are walked in tiles of 32: scores (16-byte loads, four lanes per K row), an online-softmax
//    update per head (running max m and sum l, accumulators rescaled by exp(m_old - m_new)), then the weighted
//    sum of the V tile with each thread owning four consecutive head dims;
//  * with more than one active split every CTA writes (unnormalised o, m, l) to scratch and takes a ticket;
//    the CTA that draws the last ticket of its KV head merges the splits and writes the output. No CTA waits
//    for another one, so nothing can hang.
// The number of active splits is derived on the device from the current position, so one captured launch shape
// serves every position.
//
// Softmax equivalence: the reference computes exp(clamp(s - max, -80, 80)) / sum; s - max <= 0 so the upper clamp
// never acts, the lower clamp only replaces weights below e^-80 by e^-80 (a relative change below 1e-34), and
// sum >= 1 (the maximum contributes exp(0)) so the "sum > eps" guard always passes.
#include <math.h>

#include "common.cuh"
#include "kernels.h"

namespace nfai {

namespace {

constexpr int kAT = 128;  // threads per CTA
constexpr int kG = (int)kAttnHeadsPerCta;
constexpr int kTile = (int)kAttnTile;

template <typename KVT>
struct KVLoad;
template <>
struct KVLoad<float> {
  // 4 consecutive elements
  __device__ __forceinline__ static float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
};
template <>
struct KVLoad<__half> {
  __device__ __forceinline__ static float4 ld4(const __half* p) {
    uint2 raw = *reinterpret_cast<const uint2*>(p);
    float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
    float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
};

template <typename KVT, int D>
__global__ void __launch_bounds__(kAT) attn_decode_kernel(const AttnParams p) {
  constexpr int EPT = D / 4;       // phase 1: elements of a K row per thread (4 threads per row)
  constexpr int VPR = D / 4;       // phase 2: 4-element vectors per V row
  constexpr int NPG = kAT / VPR;   // phase 2: position groups
  static_assert(kTile % NPG == 0 || NPG > kTile, "tile must split evenly over the position groups");

  __shared__ __align__(16) float qs[kG][D];
  __shared__ float s_s[kG][kTile];   // scores, then weights of the current tile
  __shared__ float alpha_s[kG];      // rescale factor of the running accumulators for this tile
  __shared__ float m_s[kG], l_s[kG];
  __shared__ __align__(16) float red[NPG][kG][D];
  __shared__ uint32_t is_last;

  pdl_launch_dependents();
  pdl_wait();  // q, K and V of this position come from the previous kernel

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t G = p.qH / p.kvH;
  const uint32_t hgroups = (G + kG - 1) / kG;
  const uint32_t g = blockIdx.x / hgroups;
  const uint32_t hg = blockIdx.x % hgroups;
  const uint32_t h0 = g * G + hg * kG;
  const uint32_t nh = min((uint32_t)kG, G - hg * kG);
  const uint32_t kvDim = p.kvH * D;
  const uint32_t seq = p.state ? p.state->pos + 1 : p.seq_imm;
  uint32_t chunk = (seq + p.S_max - 1) / p.S_max;
  chunk = ((chunk + kTile - 1) / kTile) * kTile;
  const uint32_t S_eff = (seq + chunk - 1) / chunk;
  const uint32_t s = blockIdx.y;
  if (s >= S_eff) return;
  const uint32_t t0 = s * chunk;
  const uint32_t t1 = min(seq, t0 + chunk);

  for (int i = tid; i < kG * D; i += kAT) {
    int j = i / D, e = i % D;
    qs[j][e] = j < (int)nh ? p.q[(h0 + j) * D + e] : 0.f;
  }
  float m_run = -1.0e38f, l_run = 0.f;  // live in warp j == head j (AttentionSoftmaxShader.cs:156: maxScore = -1e38)
  float acc[kG][4];
#pragma unroll
  for (int j = 0; j < kG; ++j)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[j][c] = 0.f;
  const float scale = 1.0f / sqrtf((float)D);  // AttentionScoreCalculationShader.cs:112
  const KVT* kc = reinterpret_cast<const KVT*>(p.kcache) + g * D;
  const KVT* vc = reinterpret_cast<const KVT*>(p.vcache) + g * D;
  __syncthreads();

  const int p1_pos = tid >> 2, p1_part = tid & 3;
  const int iv = tid % VPR, pg = tid / VPR;

  for (uint32_t tile0 = t0; tile0 < t1; tile0 += kTile) {
    // ---- phase 1: scores of 32 positions x kG heads
    {
      const uint32_t t = tile0 + p1_pos;
      float dot[kG];
#pragma unroll
      for (int j = 0; j < kG; ++j) dot[j] = 0.f;
      if (t < t1) {
        const KVT* kr = kc + (size_t)t * kvDim + p1_part * EPT;
#pragma unroll
        for (int e = 0; e < EPT; e += 4) {
          float4 kv = KVLoad<KVT>::ld4(kr + e);
#pragma unroll
          for (int j = 0; j < kG; ++j) {
            float4 qv = *reinterpret_cast<const float4*>(&qs[j][p1_part * EPT + e]);
            dot[j] = fmaf(qv.x, kv.x, dot[j]);
            dot[j] = fmaf(qv.y, kv.y, dot[j]);
            dot[j] = fmaf(qv.z, kv.z, dot[j]);
            dot[j] = fmaf(qv.w, kv.w, dot[j]);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < kG; ++j) {
        dot[j] += __shfl_xor_sync(0xffffffffu, dot[j], 1);
        dot[j] += __shfl_xor_sync(0xffffffffu, dot[j], 2);
      }
      if (p1_part == 0) {
#pragma unroll
        for (int j = 0; j < kG; ++j) s_s[j][p1_pos] = t < t1 ? dot[j] * scale : -INFINITY;
      }
    }
    __syncthreads();
    // ---- online softmax: warp j owns head j, lane = position in tile
    if (warp < kG) {
      float sc = s_s[warp][lane];
      float mt = warp_max(sc);
      float m_new = fmaxf(m_run, mt);
      float pr = sc == -INFINITY ? 0.f : expf(sc - m_new);
      float alpha = expf(m_run - m_new);
      l_run = l_run * alpha + warp_sum(pr);
      m_run = m_new;
      s_s[warp][lane] = pr;
      if (lane == 0) alpha_s[warp] = alpha;
    }
    __syncthreads();
    // ---- phase 2: acc[j][:] = acc[j][:]*alpha_j + sum_t w[j][t] * V[t][4*iv .. 4*iv+3]
#pragma unroll
    for (int j = 0; j < kG; ++j) {
      float a = alpha_s[j];
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[j][c] *= a;
    }
#pragma unroll
    for (int tt = pg; tt < kTile; tt += NPG) {
      const uint32_t t = tile0 + tt;
      if (t < t1) {
        float4 vv = KVLoad<KVT>::ld4(vc + (size_t)t * kvDim + iv * 4);
#pragma unroll
        for (int j = 0; j < kG; ++j) {
          float w = s_s[j][tt];
          acc[j][0] = fmaf(w, vv.x, acc[j][0]);
          acc[j][1] = fmaf(w, vv.y, acc[j][1]);
          acc[j][2] = fmaf(w, vv.z, acc[j][2]);
          acc[j][3] = fmaf(w, vv.w, acc[j][3]);
        }
      }
    }
    __syncthreads();
  }

  // ---- merge the position groups of this CTA
#pragma unroll
  for (int j = 0; j < kG; ++j)
    *reinterpret_cast<float4*>(&red[pg][j][iv * 4]) = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
  if (warp < kG && lane == 0) {
    m_s[warp] = m_run;
    l_s[warp] = l_run;
  }
  __syncthreads();

  if (S_eff == 1) {
    for (int idx = tid; idx < (int)nh * D; idx += kAT) {
      int j = idx / D, i = idx % D;
      float o = 0.f;
#pragma unroll
      for (int g2 = 0; g2 < NPG; ++g2) o += red[g2][j][i];
      p.out[(h0 + j) * D + i] = o * (1.0f / l_s[j]);
    }
    return;
  }

  // ---- several splits: publish the partial, the last CTA of this (kv head, head group) merges
  const uint32_t stride = D + 2;
  for (int idx = tid; idx < (int)nh * D; idx += kAT) {
    int j = idx / D, i = idx % D;
    float o = 0.f;
#pragma unroll
    for (int g2 = 0; g2 < NPG; ++g2) o += red[g2][j][i];
    p.part[((size_t)(h0 + j) * p.S_max + s) * stride + i] = o;
  }
  if (tid < (int)nh) {
    float* pp = p.part + ((size_t)(h0 + tid) * p.S_max + s) * stride;
    pp[D] = m_s[tid];
    pp[D + 1] = l_s[tid];
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    uint32_t ticket = atomicAdd(&p.tickets[blockIdx.x], 1u);
    is_last = ticket == S_eff - 1 ? 1u : 0u;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int idx = tid; idx < (int)nh * D; idx += kAT) {
    int j = idx / D, i = idx % D;
    const float* base = p.part + (size_t)(h0 + j) * p.S_max * stride;
    float M = -1.0e38f;
    for (uint32_t k = 0; k < S_eff; ++k) M = fmaxf(M, __ldcg(base + k * stride + D));
    float Lsum = 0.f, O = 0.f;
    for (uint32_t k = 0; k < S_eff; ++k) {
      float w = expf(__ldcg(base + k * stride + D) - M);
      Lsum = fmaf(__ldcg(base + k * stride + D + 1), w, Lsum);
      O = fmaf(__ldcg(base + k * stride + i), w, O);
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

// Upper bound on the number of splits for a cache of max_seq positions: one tile per split at most, and about
// eight 128-thread CTAs per SM across the 148 SMs.
uint32_t attn_splits(uint32_t qH, uint32_t kvH, uint32_t max_seq) {
  uint32_t ctas_x = kvH * attn_head_groups(qH, kvH);
  uint32_t by_len = (max_seq + kAttnTile - 1) / kAttnTile;
  uint32_t by_sm = (148u * 8u + ctas_x - 1) / ctas_x;
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
