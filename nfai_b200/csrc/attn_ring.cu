// Long-context decode attention: K and V of a float16 cache staged through per-warp shared-memory rings by 2-D
// TMA tiles, so that the stream keeps flowing while the warps do the softmax arithmetic.
//
// Why a second kernel: at tens of thousands of positions the register-streaming kernel (attn.cu) alternates
// between waiting for a batch of 16-byte loads and ~1.5 us of arithmetic on it (four query heads share every K
// and V row), so HBM idles half of the time (measured 1.9 TB/s at 32 768 positions). Here the copies are
// asynchronous and two (optionally three) stages deep per warp (128 KB per SM in flight), and the arithmetic is blocked:
// the scores of a whole stage are computed first, the running maximum and the rescale of the accumulators are
// paid once per stage instead of once per position.
//
// Shape: grid (kvH * head_groups, S_max) as in attn.cu, 16 warps per CTA, four query heads per CTA. A stage is
// one K tile and one V tile of 2 KB each (2048 / (2 d) positions x d dims of one KV head: the cache is
// position-major, the tile is a box of a 2-D tensor map over [ctx][kvDim]). Warp w of the CTA takes the stages
// w, w + 16, ... of the CTA's position range; lane 0 arms the stage's mbarrier and issues the two tile copies,
// all lanes wait on the parity, d/8 lanes own one position and 8 dims each (conflict-free 16-byte shared loads),
// and after a __syncwarp() lane 0 refills the stage. No barrier is shared between warps until the final merge
// (attn_finish in attn_core.cuh, the same code as the register-streaming kernel).
// Rows of a tile beyond the sequence hold stale cache contents: their scores are replaced by -inf and their V
// bits by zero before use. Rows beyond the cache are zero-filled by the copy engine.
// Every mbarrier wait is bounded (one second); a warp that gives up sets error bit 4 and goes on to the merge.
//
// Reference arithmetic: AttentionScoreCalculationShader.cs:170-205, AttentionSoftmaxShader.cs:145-177,
// AttentionWeightedValueSumShader.cs:181-215 (see attn.cu for the softmax equivalence argument).
#include <cuda.h>
#include <stdlib.h>

#include "attn_core.cuh"

namespace nfai {

using namespace attn_detail;

namespace {

constexpr int kRT = 512;                 // threads per CTA
constexpr int kRW = kRT / 32;            // warps per CTA
constexpr int kRMaxStages = 3;           // stages per warp: 2 or 3
constexpr uint32_t kTileBytes = 2048;    // one K (or V) tile
constexpr uint32_t kStageBytes = 2 * kTileBytes;
constexpr unsigned long long kRingWaitNs = 1000000000ull;

__device__ __forceinline__ unsigned long long ring_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void rbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void rbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool rbar_try(uint32_t bar, uint32_t parity) {
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
__device__ __forceinline__ void tile_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D, int kRStages>
__global__ void __launch_bounds__(kRT, 1) attn_ring_kernel(const AttnParams p, const __grid_constant__ CUtensorMap kmap,
                                                          const __grid_constant__ CUtensorMap vmap) {
  extern __shared__ unsigned char ring_raw[];
  constexpr int kG = 4;
  constexpr int LPP = D / 8;                     // lanes per position
  constexpr int PPW = 32 / LPP;                  // positions per warp step
  constexpr int PPS = kTileBytes / (D * 2);      // positions per stage
  constexpr int SPS = PPS / PPW;                 // warp steps per stage
  static_assert(SPS >= 1 && PPS % PPW == 0, "a stage is a whole number of warp steps");
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int grp = lane / LPP, sub = lane % LPP;

  // shared-memory layout: [ring: kRW x kRStages x 4 KB, 128-byte aligned][mbarriers: kRW x kRStages]
  const uint32_t raw_s = (uint32_t)__cvta_generic_to_shared(ring_raw);
  const uint32_t ring_s = (raw_s + 127u) & ~127u;
  unsigned char* ring = ring_raw + (ring_s - raw_s);
  const uint32_t bars_s = ring_s + kRW * kRStages * kStageBytes;
  const uint32_t my_ring_s = ring_s + warp * kRStages * kStageBytes;
  const unsigned char* my_ring = ring + (size_t)warp * kRStages * kStageBytes;
  const uint32_t my_bar_s = bars_s + warp * kRStages * 8;
  if (lane == 0) {
#pragma unroll
    for (int st = 0; st < kRStages; ++st) rbar_init(my_bar_s + 8 * st, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  prefetch_plan(p.pf, kPrefetchChunk);
  pdl_launch_dependents();
  pdl_wait();  // q, K and V of this position come from the previous kernel
  const uint32_t seq = p.state ? p.state->pos + 1 : p.seq_imm;
  const uint32_t bx = blockIdx.x, s = blockIdx.y;
  const uint32_t G = p.qH / p.kvH;
  const uint32_t hgroups = (G + kG - 1) / kG;
  const uint32_t g = bx / hgroups;
  const uint32_t hg = bx % hgroups;
  const uint32_t h0 = g * G + hg * kG;
  const uint32_t nh = min((uint32_t)kG, G - hg * kG);
  uint32_t chunk = (seq + p.S_max - 1) / p.S_max;
  chunk = chunk < p.min_chunk ? p.min_chunk : chunk;
  chunk = (chunk + 63) / 64 * 64;
  const uint32_t S_eff = (seq + chunk - 1) / chunk;
  if (s >= S_eff) return;  // the whole CTA: nothing is in flight yet
  const uint32_t t0 = s * chunk;
  const uint32_t t1 = min(seq, t0 + chunk);
  const uint32_t nblk = (t1 - t0 + PPS - 1) / PPS;
  const uint32_t nbw = (uint32_t)warp < nblk ? (nblk - warp + kRW - 1) / kRW : 0;  // stages of this warp

  auto issue = [&](uint32_t i) {
    const uint32_t tb = t0 + (warp + i * kRW) * PPS;
    const uint32_t st = i % kRStages;
    const uint32_t bar = my_bar_s + 8 * st;
    rbar_expect_tx(bar, kStageBytes);
    tile_load_2d(my_ring_s + st * kStageBytes, &kmap, (int)(g * D), (int)tb, bar);
    tile_load_2d(my_ring_s + st * kStageBytes + kTileBytes, &vmap, (int)(g * D), (int)tb, bar);
  };
  if (lane == 0) {
    const uint32_t first = nbw < (uint32_t)kRStages ? nbw : (uint32_t)kRStages;
    for (uint32_t i = 0; i < first; ++i) issue(i);
  }

  // this lane's eight dims of the four query heads, pre-multiplied by (1/sqrt(d)) * log2(e): scores live in the
  // base-2 domain, every exponential is one ex2
  const float qscale = (1.0f / sqrtf((float)D)) * 1.4426950408889634f;
  float q[kG][8];
#pragma unroll
  for (int j = 0; j < kG; ++j) {
    if (j < (int)nh) {
      const float* qp = p.q + (h0 + j) * D + sub * 8;
      const float4 a = *reinterpret_cast<const float4*>(qp);
      const float4 b = *reinterpret_cast<const float4*>(qp + 4);
      q[j][0] = a.x * qscale; q[j][1] = a.y * qscale; q[j][2] = a.z * qscale; q[j][3] = a.w * qscale;
      q[j][4] = b.x * qscale; q[j][5] = b.y * qscale; q[j][6] = b.z * qscale; q[j][7] = b.w * qscale;
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) q[j][e] = 0.f;
    }
  }
  float m[kG], l[kG], acc[kG][8];
#pragma unroll
  for (int j = 0; j < kG; ++j) {
    m[j] = kNegBig;
    l[j] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[j][e] = 0.f;
  }

  bool gave_up = false;
  for (uint32_t i = 0; i < nbw; ++i) {
    const uint32_t st = i % kRStages;
    const uint32_t bar = my_bar_s + 8 * st;
    const uint32_t parity = (i / kRStages) & 1;
    bool ok = __all_sync(0xffffffffu, rbar_try(bar, parity));
    if (!ok) {
      const unsigned long long t_start = ring_ns();
      uint32_t polls = 0;
      while (!ok) {
        ok = __all_sync(0xffffffffu, rbar_try(bar, parity));
        if (!ok && (++polls & 63u) == 0) {
          const bool late = ring_ns() - t_start > kRingWaitNs;
          if (__any_sync(0xffffffffu, late)) break;
        }
      }
    }
    if (!ok) {
      gave_up = true;  // same value in every lane
      break;
    }
    const uint32_t tb = t0 + (warp + i * kRW) * PPS;
    const unsigned char* kst = my_ring + (size_t)st * kStageBytes + (size_t)sub * 16;
    const unsigned char* vst = kst + kTileBytes;

    // pass 1: the scores of the stage
    float sc[kG][SPS];
#pragma unroll
    for (int u = 0; u < SPS; ++u) {
      const int row = u * PPW + grp;
      typename KV8<__half>::Raw kr;
      kr.v = *reinterpret_cast<const uint4*>(kst + (size_t)row * (D * 2));
      float kf[8];
      KV8<__half>::unpack(kr, kf);
      const bool valid = tb + row < t1;
#pragma unroll
      for (int j = 0; j < kG; ++j) {
        float dot = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) dot = fmaf(q[j][e], kf[e], dot);
#pragma unroll
        for (int o = 1; o < LPP; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        sc[j][u] = valid ? dot : -INFINITY;
      }
    }
    // one new maximum and one rescale per stage
#pragma unroll
    for (int j = 0; j < kG; ++j) {
      float mb = sc[j][0];
#pragma unroll
      for (int u = 1; u < SPS; ++u) mb = fmaxf(mb, sc[j][u]);
      const float m_new = fmaxf(m[j], mb);  // m starts finite, so m_new is finite even when every score is -inf
      const float alpha = ex2(m[j] - m_new);
      m[j] = m_new;
      l[j] *= alpha;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[j][e] *= alpha;
    }
    // pass 2: weights and the weighted V sum
#pragma unroll
    for (int u = 0; u < SPS; ++u) {
      const int row = u * PPW + grp;
      typename KV8<__half>::Raw vr;
      vr.v = *reinterpret_cast<const uint4*>(vst + (size_t)row * (D * 2));
      if (!(tb + row < t1)) vr.v = make_uint4(0, 0, 0, 0);  // stale cache rows may hold anything
      float vf[8];
      KV8<__half>::unpack(vr, vf);
#pragma unroll
      for (int j = 0; j < kG; ++j) {
        const float pr = ex2(sc[j][u] - m[j]);
        l[j] += pr;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[j][e] = fmaf(pr, vf[e], acc[j][e]);
      }
    }
    __syncwarp();  // every lane has read the stage before it is refilled
    if (lane == 0 && i + kRStages < nbw) issue(i + kRStages);
  }
  if (gave_up) {
    if (lane == 0 && p.state) atomicOr(&p.state->err, 4u);
    // copies of this warp may still be in flight: give them a bounded time to land before shared memory is released
    for (volatile uint32_t spin = 0; spin < (1u << 20); ++spin) {
    }
  }
  // back to the natural-log domain the merge works in
#pragma unroll
  for (int j = 0; j < kG; ++j) m[j] *= 0.6931471805599453f;
  attn_finish<D, kRW, kG>(p, bx, s, S_eff, h0, nh, m, l, acc);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn ring_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess || !ptr) return nullptr;
  fn = (EncodeTiledFn)ptr;
  return fn;
}

template <int D, int STAGES>
cudaError_t launch_ring_d(cudaStream_t s, const AttnParams& p, const AttnTileMaps& maps, bool pdl) {
  auto kern = attn_ring_kernel<D, STAGES>;
  const size_t smem = attn_ring_smem(STAGES);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.kvH * attn_head_groups(p.qH, p.kvH, 4), p.S_max);
  cfg.blockDim = dim3(kRT);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const CUtensorMap* km = reinterpret_cast<const CUtensorMap*>(maps.k);
  const CUtensorMap* vm = reinterpret_cast<const CUtensorMap*>(maps.v);
  return cudaLaunchKernelEx(&cfg, kern, p, *km, *vm);
}

}  // namespace

size_t attn_ring_smem(int stages) { return (size_t)kRW * stages * kStageBytes + kRW * stages * 8 + 128; }

// Stages per warp: 2 (128 KB of ring per SM) unless NFAI_ATTN_RING_STAGES=3 (192 KB). Two measured faster for the
// whole step (924 vs 1040 us per token at 32 768 positions): with three, the kernel needs the SM's largest
// shared-memory partition and every neighbouring kernel pays for the re-partitioning.
static int ring_stages() {
  static int st = 0;
  if (st == 0) {
    const char* v = getenv("NFAI_ATTN_RING_STAGES");
    st = (v && atoi(v) == 3) ? 3 : 2;
  }
  return st;
}

bool attn_ring_supported(int kvdtype, uint32_t d) { return kvdtype == 1 && (d == 64 || d == 128); }

cudaError_t attn_ring_make_maps(const void* kcache, const void* vcache, uint32_t ctx, uint32_t kvDim, uint32_t d,
                                AttnTileMaps* out) {
  static_assert(sizeof(CUtensorMap) == sizeof(out->k), "tensor map storage");
  EncodeTiledFn fn = ring_encode_fn();
  if (!fn || !attn_ring_supported(1, d) || kvDim % d != 0) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(kcache) & 15) || (reinterpret_cast<uintptr_t>(vcache) & 15) || (kvDim * 2) % 16) return cudaErrorInvalidValue;
  cuuint64_t dims[2] = {kvDim, ctx};
  cuuint64_t strides[1] = {(cuuint64_t)kvDim * 2};
  cuuint32_t box[2] = {d, kTileBytes / (d * 2)};
  cuuint32_t estr[2] = {1, 1};
  const void* base[2] = {kcache, vcache};
  void* dst[2] = {out->k, out->v};
  for (int i = 0; i < 2; ++i) {
    CUresult r = fn(reinterpret_cast<CUtensorMap*>(dst[i]), CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base[i]), dims,
                    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  }
  return cudaSuccess;
}

cudaError_t launch_attn_ring(cudaStream_t s, const AttnParams& p, const AttnTileMaps& maps, bool pdl) {
  if (p.qH == 0 || p.kvH == 0 || p.qH % p.kvH != 0 || p.S_max == 0 || p.S_max > (uint32_t)attn_detail::kAttnMergeCap || p.out_half) return cudaErrorInvalidValue;
  if (!p.state && p.seq_imm == 0) return cudaErrorInvalidValue;
  const bool two = ring_stages() == 2;
  switch (p.d) {
    case 64: return two ? launch_ring_d<64, 2>(s, p, maps, pdl) : launch_ring_d<64, 3>(s, p, maps, pdl);
    case 128: return two ? launch_ring_d<128, 2>(s, p, maps, pdl) : launch_ring_d<128, 3>(s, p, maps, pdl);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace nfai
