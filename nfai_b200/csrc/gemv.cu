// Batch-1 decode GEMV family: y = W * f(x) with fused prologue (RMSNorm) and epilogues (residual add,
// RoPE + KV-cache write, SiLU*up, logits + arg-max partials).
//
// The work is HBM-bound (one FMA per 2 or 4 weight bytes), so the kernel is a weight streamer:
//  * the grid is persistent: at most a few CTAs per SM, and every warp walks row blocks gw, gw + TW, gw + 2 TW ...
//    (R consecutive rows each) as ONE continuous stream, so the prologue is paid once per CTA and the loads of
//    the next row block are already in flight while the current one is reduced and stored;
//  * the lanes walk a row in 16-byte vectors (8 halves / 4 floats), 512 contiguous bytes per warp per row per
//    step; U steps are issued back to back and the next batch is requested before the current one is consumed,
//    so every lane keeps 2*U*R 16-byte loads in flight;
//  * the first batch is requested BEFORE the programmatic-dependency wait: the weights do not depend on the
//    previous kernel, so they stream while it drains and while this CTA normalises x;
//  * x (float32) sits in shared memory and is reused by all R rows of all warps; accumulation is float32;
//  * the row sum is finished with warp shuffles; lane 0 applies the epilogue.
// No tensor cores: with one right-hand side there is nothing for them to reuse.
//
// Reference arithmetic this replaces: NFAI.Vulkan.Shaders/MatrixMultiplyShader.cs:266-288 (one thread per
// output, serial k loop), RMSNormShader.cs:129-150, RoPEShader.cs:238-271, SiLUShader.cs:112-127,
// ElementWiseMultiplicationShader.cs:127-138, host residual adds at TransformerBlock.cs:151-161,174-181.
#include "gemv_common.cuh"

namespace nfai {

using namespace gemv_detail;

namespace {

constexpr int kSmemHeader = 96;  // floats ahead of x in shared memory: reduction scratch and split-row partials

// ---- the streamer ---------------------------------------------------------------------------------------------
template <typename WT, typename KVT, int R, int U, int EPI>
__global__ void __launch_bounds__(kThreads, 2) gemv_kernel(const GemvParams p) {
  extern __shared__ __align__(16) float smem[];
  float* red = smem;                  // 2*kWarps words of reduction scratch
  float* part = smem + 32;            // [2][kWarps][R] partial row sums of a split row block (two parities)
  float* xs = smem + kSmemHeader;     // K floats of x, then K floats of gain
  constexpr int VE = WeightVec<WT>::kElems;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t nvec = p.K / VE;  // host guarantees K % VE == 0 and 16-byte aligned rows
  // A work item is (row block, K chunk): R rows x cv vectors. With split = 1 the chunk is the whole row.
  const uint32_t sl = p.split_log2, S = 1u << sl;
  const uint32_t cv = (((nvec + S - 1) >> sl) + 31u) & ~31u;  // vectors per chunk, a whole number of warp strides
  const uint32_t nkb = (cv + 32 * U - 1) / (32 * U);          // batches per item
  const uint32_t nrb = (p.N + R - 1) / R;                     // row blocks
  const uint32_t nitems = nrb << sl;
  const uint32_t TW = gridDim.x * kWarps;
  const uint32_t nrounds = (nitems + TW - 1) / TW;  // the same for every warp of the grid: barriers stay uniform
  const WT* const Wbase = reinterpret_cast<const WT*>(p.W);
  const uint4 zero = make_uint4(0, 0, 0, 0);

  auto load_batch = [&](uint4(&buf)[U][R], uint32_t t, uint32_t kb) {
    if (t >= nitems) return;
    const uint32_t rb = t >> sl, c = t & (S - 1);
    const uint32_t v0 = c * cv + kb * (32 * U) + lane;
    const uint32_t vend = min((c + 1) * cv, nvec);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      uint32_t n = rb * R + r;
      n = n < p.N ? n : p.N - 1;  // a ragged last block re-reads the last row, never out of bounds
      const uint4* wrow = reinterpret_cast<const uint4*>(Wbase + (size_t)n * p.K);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint32_t v = v0 + 32 * u;
        buf[u][r] = v < vend ? ld_stream16(wrow + v) : zero;
      }
    }
  };

  uint32_t t = blockIdx.x * kWarps + warp;
  uint32_t lt = t, lkb = 0;  // load cursor: the batch the next request asks for
  auto advance = [&]() {
    if (++lkb == nkb) {
      lkb = 0;
      lt += TW;
    }
  };
  // Weights do not depend on the previous kernel: the first batch is requested before the dependency wait.
  // (Requesting the first two there, in either loop order, measured 10-30% slower in the steady state.)
  uint4 cur[U][R], nxt[U][R];
  load_batch(cur, lt, lkb);
  advance();
  load_gain(p, xs);
  prefetch_plan(p.pf, kPrefetchChunk);
  pdl_launch_dependents();
  pdl_wait();
  // what the epilogue of the first item reads (residual / cos, sin of this position) travels with x
  uint32_t pos = 0;
  if constexpr (EPI == EPI_QKV_ROPE) pos = p.state ? p.state->pos : p.pos_imm;
  float pre[R];
  epi_preload<R, EPI>(p, (min(t, nitems - 1) >> sl) * R, pos, pre);
  load_x(p, xs, red);

  float best_v = -INFINITY;
  uint32_t best_i = 0xffffffffu;
  float acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.f;
  for (uint32_t round = 0; round < nrounds; ++round, t += TW) {
    const uint32_t c = t & (S - 1);
    float pre_next[R];
    epi_preload<R, EPI>(p, (min(t + TW, nitems - 1) >> sl) * R, pos, pre_next);
    const uint32_t vend = min((c + 1) * cv, nvec);
    for (uint32_t kb = 0; kb < nkb; ++kb) {
      load_batch(nxt, lt, lkb);
      advance();
      if (t < nitems) {
        const uint32_t v0 = c * cv + kb * (32 * U) + lane;
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const uint32_t v = v0 + 32 * u;
          if (v < vend) {
            float xv[VE];
            const float4* xp = reinterpret_cast<const float4*>(xs + (size_t)v * VE);
#pragma unroll
            for (int i = 0; i < VE / 4; ++i) {
              float4 q = xp[i];
              xv[4 * i] = q.x;
              xv[4 * i + 1] = q.y;
              xv[4 * i + 2] = q.z;
              xv[4 * i + 3] = q.w;
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
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int r = 0; r < R; ++r) cur[u][r] = nxt[u][r];
    }
    // the item is complete
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = warp_sum(acc[r]);
    if (S == 1) {
      if (t < nitems) row_epilogue_pre<KVT, R, EPI>(p, t * R, acc, pre, pos, best_v, best_i);
    } else {
      // the S chunks of a row block sit in S consecutive warps of this CTA: add them up in warp order
      float* pr = part + (round & 1) * (kWarps * R);
      if (lane == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r) pr[warp * R + r] = acc[r];
      }
      __syncthreads();
      if (c == 0 && t < nitems) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
          float a = pr[warp * R + r];
          for (uint32_t j = 1; j < S; ++j) a += pr[(warp + j) * R + r];
          acc[r] = a;
        }
        row_epilogue_pre<KVT, R, EPI>(p, (t >> sl) * R, acc, pre, pos, best_v, best_i);
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      acc[r] = 0.f;
      pre[r] = pre_next[r];
    }
  }
  if constexpr (EPI == EPI_LOGITS) cta_argmax_partial(p, best_v, best_i, red);
}

// Same contract for any K and any alignment (element loads); used when K is not a multiple of the vector width.
template <typename WT, typename KVT, int EPI>
__global__ void __launch_bounds__(kThreads) gemv_scalar_kernel(const GemvParams p) {
  extern __shared__ __align__(16) float smem[];
  float* red = smem;
  float* xs = smem + kSmemHeader;
  constexpr int R = 2;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t nrb = (p.N + R - 1) / R;
  load_gain(p, xs);
  prefetch_plan(p.pf, kPrefetchChunk);
  pdl_launch_dependents();
  pdl_wait();
  load_x(p, xs, red);
  float best_v = -INFINITY;
  uint32_t best_i = 0xffffffffu;
  for (uint32_t rb = blockIdx.x * kWarps + warp; rb < nrb; rb += gridDim.x * kWarps) {
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      uint32_t n = rb * R + r < p.N ? rb * R + r : p.N - 1;
      const WT* w = reinterpret_cast<const WT*>(p.W) + (size_t)n * p.K;
      float a = 0.f;
      for (uint32_t k = lane; k < p.K; k += 32) a = fmaf(to_float(w[k]), xs[k], a);
      acc[r] = warp_sum(a);
    }
    row_epilogue<KVT, R, EPI>(p, rb * R, acc, best_v, best_i);
  }
  if constexpr (EPI == EPI_LOGITS) cta_argmax_partial(p, best_v, best_i, red);
}

template <typename K>
cudaError_t launch_k(K kernel, dim3 grid, size_t smem, cudaStream_t s, bool pdl, const GemvParams& p) {
  cudaError_t e = cudaSuccess;
  if (smem > 48 * 1024) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, p);
}

template <typename WT, typename KVT, int R, int EPI>
cudaError_t launch_u(int U, dim3 grid, size_t smem, cudaStream_t s, bool pdl, const GemvParams& p) {
  switch (U) {
    case 2: return launch_k(gemv_kernel<WT, KVT, R, 2, EPI>, grid, smem, s, pdl, p);
    case 4: return launch_k(gemv_kernel<WT, KVT, R, 4, EPI>, grid, smem, s, pdl, p);
    case 8:
      if constexpr (R <= 2) return launch_k(gemv_kernel<WT, KVT, R, 8, EPI>, grid, smem, s, pdl, p);
      return cudaErrorInvalidValue;  // 4 rows x 8 steps x 2 buffers would not fit the register file
    default: return cudaErrorInvalidValue;
  }
}

template <typename WT, typename KVT, int EPI>
cudaError_t launch_r(int R, int U, dim3 grid, size_t smem, cudaStream_t s, bool pdl, const GemvParams& p) {
  if constexpr (EPI == EPI_STORE || EPI == EPI_LOGITS) {
    if (R == 1) return launch_u<WT, KVT, 1, EPI>(U, grid, smem, s, pdl, p);
  }
  if (R == 2) return launch_u<WT, KVT, 2, EPI>(U, grid, smem, s, pdl, p);
  if (R == 4) return launch_u<WT, KVT, 4, EPI>(U, grid, smem, s, pdl, p);
  return cudaErrorInvalidValue;
}

template <typename WT, typename KVT>
cudaError_t launch_e(GemvEpilogue epi, bool vec, int R, int U, dim3 grid, size_t smem, cudaStream_t s, bool pdl,
                     const GemvParams& p) {
  if (!vec) {
    switch (epi) {
      case EPI_STORE: return launch_k(gemv_scalar_kernel<WT, float, EPI_STORE>, grid, smem, s, pdl, p);
      case EPI_QKV_ROPE: return launch_k(gemv_scalar_kernel<WT, KVT, EPI_QKV_ROPE>, grid, smem, s, pdl, p);
      case EPI_SILU_MUL: return launch_k(gemv_scalar_kernel<WT, float, EPI_SILU_MUL>, grid, smem, s, pdl, p);
      case EPI_LOGITS: return launch_k(gemv_scalar_kernel<WT, float, EPI_LOGITS>, grid, smem, s, pdl, p);
    }
    return cudaErrorInvalidValue;
  }
  switch (epi) {
    case EPI_STORE: return launch_r<WT, float, EPI_STORE>(R, U, grid, smem, s, pdl, p);
    case EPI_QKV_ROPE: return launch_r<WT, KVT, EPI_QKV_ROPE>(R, U, grid, smem, s, pdl, p);
    case EPI_SILU_MUL: return launch_r<WT, float, EPI_SILU_MUL>(R, U, grid, smem, s, pdl, p);
    case EPI_LOGITS: return launch_r<WT, float, EPI_LOGITS>(R, U, grid, smem, s, pdl, p);
  }
  return cudaErrorInvalidValue;
}

bool vector_ok(int wdtype, const GemvParams& p) {
  const uint32_t ve = wdtype == 1 ? 8 : 4;
  return p.K % ve == 0 && (reinterpret_cast<uintptr_t>(p.W) & 15) == 0;
}

int rows_per_warp(GemvEpilogue epi, bool vec, const GemvTune& t) {
  if (!vec) return 2;
  int R = t.rows_per_warp;
  if ((epi == EPI_QKV_ROPE || epi == EPI_SILU_MUL) && R < 2) R = 2;
  return R;
}

}  // namespace

static bool use_ring(int wdtype, const GemvParams& p, const GemvTune& t) {
  if (t.mode != 1 || !vector_ok(wdtype, p)) return false;
  return t.unroll >= 1 && t.unroll <= 4 && gemv_ring_smem(p, t.unroll) <= 227 * 1024;
}

// How many warps share one row block (1, 2, 4 or 8; returned as log2). A matrix with fewer row blocks than the
// persistent grid has warps (the down projections: 2 048-4 096 rows of 16-28 KB) leaves warps without work and the
// others with long serial rows; splitting K gives every warp the same amount and puts the whole matrix in flight at
// once. It is used only where it measured faster (the 1B model's down projection: 10.3 -> 9.0 us): rows of at least
// four batches, chunks of whole batches, at most half of the warps busy without it, and no more chunks than needed to
// cover the grid. Short rows and matrices with more rows stream best unsplit (3B down projection: 12.2 vs 13.4 us).
static uint32_t gemv_split_log2(int wdtype, bool vec, int R, const GemvParams& p, const GemvTune& t) {
  if (!vec) return 0;
  if (t.split == 1 || t.split == 2 || t.split == 4 || t.split == 8) return t.split == 1 ? 0 : t.split == 2 ? 1 : t.split == 4 ? 2 : 3;
  const uint32_t ve = wdtype == 1 ? 8 : 4;
  const uint32_t U = (uint32_t)t.unroll;
  const uint32_t per_lane = p.K / ve / 32;  // 16-byte vectors per lane per row
  const uint32_t nrb = (p.N + R - 1) / R;
  const uint32_t warps = (t.grid > 0 ? (uint32_t)t.grid : sm_count() * (uint32_t)(t.ctas_per_sm < 1 ? 1 : t.ctas_per_sm)) * kWarps;
  if (p.K % (ve * 32) != 0) return 0;
  if (2 * nrb > warps) {
    // Plenty of rows: a split does not add parallelism, but it can even out the last round. 8 192 row pairs on 2 368
    // warps are 3.46 rounds, i.e. four with 13.5 % of the warp slots idle; as 16 384 half rows they are 6.9 rounds
    // (1.4 % idle): 14.1 -> 13.8 us for the gate/up product of the 1B model, 605 -> 597 us per step.
    auto idle = [&](uint32_t tasks) {
      const uint32_t rounds = (tasks + warps - 1) / warps;
      return (float)(rounds * warps - tasks) / (float)(rounds * warps);
    };
    if (per_lane % (2 * U) == 0 && idle(nrb) > 0.08f && idle(2 * nrb) + 0.04f < idle(nrb)) return 1;  // halves of whole batches
    return 0;
  }
  if (per_lane < 4 * U) return 0;
  for (uint32_t sl = 1; sl <= 3; ++sl) {
    if ((per_lane % (U << sl)) != 0) break;  // chunks must stay whole batches
    if ((nrb << sl) >= warps) return sl;
  }
  return 0;
}

uint32_t gemv_grid(int wdtype, GemvEpilogue epi, const GemvParams& p, const GemvTune& t) {
  if (use_ring(wdtype, p, t)) return gemv_ring_grid(p, t.ctas_per_sm);
  const bool vec = vector_ok(wdtype, p);
  const int R = rows_per_warp(epi, vec, t);
  const uint32_t nitems = ((p.N + R - 1) / R) << gemv_split_log2(wdtype, vec, R, p, t);
  const uint32_t want = (nitems + kWarps - 1) / kWarps;
  uint32_t cap = sm_count() * (uint32_t)(t.ctas_per_sm < 1 ? 1 : t.ctas_per_sm);  // persistent: warps loop over items
  if (t.grid > 0) cap = (uint32_t)t.grid;
  return want < cap ? want : cap;
}

cudaError_t launch_gemv(cudaStream_t s, int wdtype, int kvdtype, GemvEpilogue epi, const GemvParams& p_in,
                        const GemvTune& t, bool pdl) {
  GemvParams p = p_in;
  if (p.N == 0 || p.K == 0) return cudaErrorInvalidValue;
  if ((epi == EPI_QKV_ROPE || epi == EPI_SILU_MUL) && (p.N % 2) != 0) return cudaErrorInvalidValue;
  if (use_ring(wdtype, p, t)) {
    p.l2_ahead = (uint32_t)(t.l2_ahead < 0 ? 0 : t.l2_ahead);
    return launch_gemv_ring(s, wdtype, kvdtype, epi, p, t.unroll, t.ctas_per_sm, pdl);
  }
  const bool vec = vector_ok(wdtype, p);
  const int R = rows_per_warp(epi, vec, t);
  dim3 grid(gemv_grid(wdtype, epi, p, t));
  p.split_log2 = gemv_split_log2(wdtype, vec, R, p, t);
  size_t smem = (kSmemHeader + (size_t)p.K * (p.gain ? 2 : 1)) * sizeof(float);
  if (smem > 227 * 1024) return cudaErrorInvalidValue;
  if (wdtype == 1) {
    if (kvdtype == 1) return launch_e<__half, __half>(epi, vec, R, t.unroll, grid, smem, s, pdl, p);
    return launch_e<__half, float>(epi, vec, R, t.unroll, grid, smem, s, pdl, p);
  }
  if (kvdtype == 1) return launch_e<float, __half>(epi, vec, R, t.unroll, grid, smem, s, pdl, p);
  return launch_e<float, float>(epi, vec, R, t.unroll, grid, smem, s, pdl, p);
}

}  // namespace nfai
