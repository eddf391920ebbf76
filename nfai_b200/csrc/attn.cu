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
#include "attn_core.cuh"

namespace nfai {

using namespace attn_detail;

namespace {

constexpr int kAT = 512;       // threads per CTA
constexpr int kAW = kAT / 32;  // warps per CTA

template <typename KVT, int D, int GH>
__global__ void __launch_bounds__(kAT, 1) attn_decode_kernel(const AttnParams p) {
  prefetch_plan(p.pf, kPrefetchChunk);
  pdl_launch_dependents();
  // q and the newest K/V row come from the previous kernel of this step: the wait for it is inside attn_core, after
  // the earlier rows (written by earlier steps) have been requested. The position was advanced by the previous
  // STEP's last kernel, which has completed. K and V are read with L2 loads: a line fetched before the wait must not
  // serve a later read of the newest row from L1.
  const uint32_t seq = p.state ? p.state->pos + 1 : p.seq_imm;
  // one head per CTA leaves registers for eight steps of K and V in flight
  attn_core<KVT, D, kAW, true, GH, (GH == 1 ? 2 * KV8<KVT>::kUnroll : 0)>(p, blockIdx.x, blockIdx.y, seq, p.min_chunk);
}

// Prompt path: blockIdx.y is the token of the chunk; its sequence is one longer than the previous token's.
template <typename KVT, int D>
__global__ void __launch_bounds__(kAT, 1) attn_prefill_kernel(const AttnParams p) {
  const uint32_t t = blockIdx.y;
  AttnParams pp = p;
  pp.q = p.q + (size_t)t * p.qH * D;
  pp.out_half = p.out_half + (size_t)t * p.qH * D;
  pp.S_max = 1;
  attn_core<KVT, D, kAW, false, (int)kAttnHeadsPerCta>(pp, blockIdx.x, 0, p.seq_imm + t, 1u << 30);
}

template <typename KVT>
cudaError_t launch_p(cudaStream_t s, const AttnParams& p, uint32_t T) {
  dim3 grid(p.kvH * attn_head_groups(p.qH, p.kvH), T);
  switch (p.d) {
    case 32: attn_prefill_kernel<KVT, 32><<<grid, kAT, 0, s>>>(p); break;
    case 64: attn_prefill_kernel<KVT, 64><<<grid, kAT, 0, s>>>(p); break;
    case 128: attn_prefill_kernel<KVT, 128><<<grid, kAT, 0, s>>>(p); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

template <typename Kern>
cudaError_t launch_cfg(const cudaLaunchConfig_t& cfg, Kern kernel, const AttnParams& p) {
  return cudaLaunchKernelEx(&cfg, kernel, p);
}

template <typename KVT>
cudaError_t launch_d(cudaStream_t s, const AttnParams& p, bool pdl) {
  const uint32_t hgroups = attn_head_groups(p.qH, p.kvH, p.heads_per_cta);
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
  if (p.heads_per_cta == 1) {
    switch (p.d) {
      case 32: return launch_cfg(cfg, attn_decode_kernel<KVT, 32, 1>, p);
      case 64: return launch_cfg(cfg, attn_decode_kernel<KVT, 64, 1>, p);
      case 128: return launch_cfg(cfg, attn_decode_kernel<KVT, 128, 1>, p);
      default: return cudaErrorInvalidValue;
    }
  }
  if (p.heads_per_cta == 2) {
    switch (p.d) {
      case 32: return launch_cfg(cfg, attn_decode_kernel<KVT, 32, 2>, p);
      case 64: return launch_cfg(cfg, attn_decode_kernel<KVT, 64, 2>, p);
      case 128: return launch_cfg(cfg, attn_decode_kernel<KVT, 128, 2>, p);
      default: return cudaErrorInvalidValue;
    }
  }
  switch (p.d) {
    case 32: return launch_cfg(cfg, attn_decode_kernel<KVT, 32, 4>, p);
    case 64: return launch_cfg(cfg, attn_decode_kernel<KVT, 64, 4>, p);
    case 128: return launch_cfg(cfg, attn_decode_kernel<KVT, 128, 4>, p);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

uint32_t attn_head_groups(uint32_t qH, uint32_t kvH, uint32_t heads_per_cta) {
  uint32_t G = qH / kvH;
  return (G + heads_per_cta - 1) / heads_per_cta;
}

// Upper bound on the number of splits for a cache of max_seq positions: at least kAttnMinChunk positions per
// split, and no more CTAs than the SMs hold at once (one 512-thread CTA each), so there is no second wave.
uint32_t attn_splits(uint32_t qH, uint32_t kvH, uint32_t max_seq, uint32_t heads_per_cta, uint32_t min_chunk) {
  uint32_t ctas_x = kvH * attn_head_groups(qH, kvH, heads_per_cta);
  uint32_t by_len = (max_seq + min_chunk - 1) / min_chunk;
  uint32_t by_sm = sm_count() / ctas_x;
  if (by_sm < 1) by_sm = 1;
  uint32_t s = by_len < by_sm ? by_len : by_sm;
  if (s > (uint32_t)attn_detail::kAttnMergeCap) s = attn_detail::kAttnMergeCap;  // the merge keeps one weight per split in shared memory
  return s < 1 ? 1 : s;
}

size_t attn_part_floats(uint32_t qH, uint32_t d, uint32_t S_max) { return (size_t)qH * S_max * (d + 2); }

cudaError_t launch_attn_prefill(cudaStream_t s, int kvdtype, const AttnParams& p, uint32_t T) {
  if (p.qH == 0 || p.kvH == 0 || p.qH % p.kvH != 0 || !p.out_half || !p.seq_imm || !T || T > 65535) return cudaErrorInvalidValue;
  return kvdtype == 1 ? launch_p<__half>(s, p, T) : launch_p<float>(s, p, T);
}

cudaError_t launch_attn_decode(cudaStream_t s, int kvdtype, const AttnParams& p, bool pdl) {
  if (p.qH == 0 || p.kvH == 0 || p.qH % p.kvH != 0 || p.S_max == 0 || p.S_max > (uint32_t)attn_detail::kAttnMergeCap) return cudaErrorInvalidValue;
  if (!p.state && p.seq_imm == 0) return cudaErrorInvalidValue;
  if (p.heads_per_cta != 1 && p.heads_per_cta != 2 && p.heads_per_cta != 4) return cudaErrorInvalidValue;
  return kvdtype == 1 ? launch_d<__half>(s, p, pdl) : launch_d<float>(s, p, pdl);
}

}  // namespace nfai
