// Small kernels around the GEMV/attention pair: token embedding, arg-max finish + state advance, and the
// upload-side convert/scatter.
#include "common.cuh"
#include "kernels.h"

namespace nfai {

uint32_t sm_count() {
  // per device: contexts on different GPUs may live in one process
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return (uint32_t)cached[dev];
}

namespace {

cudaLaunchConfig_t make_cfg(dim3 grid, dim3 block, cudaStream_t s, cudaLaunchAttribute* attr, bool pdl) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = 0;
  cfg.stream = s;
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cfg;
}

// out[i] = E[H*token + i], widened exactly (NFAI.Vulkan.Shaders/TokenEmbedShader.cs:139-158).
// Token source: the prompt buffer at state->prompt_idx, else state->cur_token, else the immediate.
template <typename WT>
__global__ void embed_kernel(const WT* __restrict__ E, uint32_t H, uint32_t V, StepState* state,
                             const uint32_t* __restrict__ prompt, uint32_t token_imm, float* __restrict__ x_out,
                             const PrefetchPlan pf) {
  prefetch_plan(pf, kPrefetchChunk);
  pdl_launch_dependents();
  pdl_wait();
  uint32_t tok = token_imm;
  if (state) tok = prompt ? prompt[state->prompt_idx] : state->cur_token;
  if (tok >= V) {
    if (state && threadIdx.x == 0 && blockIdx.x == 0) atomicOr(&state->err, 1u);
    tok = 0;
  }
  const WT* row = E + (size_t)tok * H;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < H; i += gridDim.x * blockDim.x)
    x_out[i] = to_float(row[i]);
}

// Lowest index among the maxima (values.ToList().IndexOf(values.Max()), NFAI.Models.Llama3/SamplingUtils.cs:55-56),
// from per-CTA partials that already hold the lowest index of their own maximum.
__global__ void __launch_bounds__(256) argmax_final_kernel(const float* __restrict__ part_val,
                                                          const uint32_t* __restrict__ part_idx, uint32_t nparts,
                                                          StepState* state, uint32_t* argmax_out, uint32_t* history,
                                                          uint32_t history_cap, const PrefetchPlan pf,
                                                          uint32_t* xchg_epoch, uint32_t xchg_per_step,
                                                          const XchgHooks tp) {
  __shared__ float sv[256];
  __shared__ uint32_t si[256];
  __shared__ uint32_t s_ok;
  prefetch_plan(pf, kPrefetchChunk);
  pdl_launch_dependents();
  pdl_wait();
  float bv = -INFINITY;
  uint32_t bi = 0xffffffffu;
  if (tp.pull) {
    // tensor parallel: every rank's LM-head kernel pushed its best (value, global index) into this rank's area
    if (threadIdx.x == 0) {
      DeviceXchgMem mem;
      const uint32_t epoch = *tp.epoch_base + tp.pull_index + 1;
      float v = 0.f;
      uint32_t ix = 0xffffffffu;
      s_ok = xchg::best_pair(mem, tp.view, epoch, tp.wait_ns, &v, &ix) ? 1u : 0u;
      if (s_ok) {
        bv = v;
        bi = ix;
      } else if (state) {
        atomicOr(&state->err, 4u);
      }
    }
  } else {
    for (uint32_t i = threadIdx.x; i < nparts; i += blockDim.x) {
      float v = part_val[i];
      uint32_t ix = part_idx[i];
      if (ix != 0xffffffffu && (bi == 0xffffffffu || v > bv || (v == bv && ix < bi))) {
        bv = v;
        bi = ix;
      }
    }
  }
  sv[threadIdx.x] = bv;
  si[threadIdx.x] = bi;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) {
      float v = sv[threadIdx.x + o];
      uint32_t ix = si[threadIdx.x + o];
      float cv = sv[threadIdx.x];
      uint32_t ci = si[threadIdx.x];
      if (ix != 0xffffffffu && (ci == 0xffffffffu || v > cv || (v == cv && ix < ci))) {
        sv[threadIdx.x] = v;
        si[threadIdx.x] = ix;
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    uint32_t best = si[0] == 0xffffffffu ? 0u : si[0];
    if (argmax_out) *argmax_out = best;
    if (state) {
      if (history && state->steps < history_cap) history[state->steps] = best;
      state->last_argmax = best;
      state->cur_token = best;  // greedy feedback: the next step embeds this token unless the host overwrites it
      state->pos += 1;
      state->steps += 1;
      if (xchg_epoch) *xchg_epoch += xchg_per_step;
    }
  }
}

__global__ void advance_kernel(StepState* state, uint32_t* xchg_epoch, uint32_t xchg_per_step) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    state->pos += 1;
    state->prompt_idx += 1;
    if (xchg_epoch) *xchg_epoch += xchg_per_step;
  }
}

template <typename ST, typename DT>
__global__ void ingest_kernel(const IngestParams p) {
  const ST* src = reinterpret_cast<const ST*>(p.src);
  DT* dst = reinterpret_cast<DT*>(p.dst);
  for (uint64_t e = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; e < p.n; e += (uint64_t)gridDim.x * blockDim.x) {
    uint64_t g = p.elem_off + e;
    uint64_t row = g / p.K, col = g - row * p.K;
    if (row < p.row_lo || row >= p.row_hi || col < p.col_lo || col >= p.col_hi) continue;
    uint64_t drow = (row - p.row_lo) * p.row_mul + p.row_off;
    store_as(dst + drow * p.ldd + (col - p.col_lo), to_float(src[e]));
  }
}

}  // namespace

cudaError_t launch_embed(cudaStream_t s, int wdtype, const void* E, uint32_t H, uint32_t V, StepState* state,
                         const uint32_t* prompt, uint32_t token_imm, float* x_out, const PrefetchPlan& pf, bool pdl) {
  cudaLaunchAttribute attr[1];
  uint32_t blocks = (H + 255) / 256;
  cudaLaunchConfig_t cfg = make_cfg(dim3(blocks), dim3(256), s, attr, pdl);
  if (wdtype == 1)
    return cudaLaunchKernelEx(&cfg, embed_kernel<__half>, reinterpret_cast<const __half*>(E), H, V, state, prompt,
                              token_imm, x_out, pf);
  return cudaLaunchKernelEx(&cfg, embed_kernel<float>, reinterpret_cast<const float*>(E), H, V, state, prompt,
                            token_imm, x_out, pf);
}

cudaError_t launch_argmax_final(cudaStream_t s, const float* part_val, const uint32_t* part_idx, uint32_t nparts,
                                StepState* state, uint32_t* argmax_out, uint32_t* history, uint32_t history_cap,
                                const PrefetchPlan& pf, uint32_t* xchg_epoch, uint32_t xchg_per_step, const XchgHooks& tp,
                                bool pdl) {
  cudaLaunchAttribute attr[1];
  cudaLaunchConfig_t cfg = make_cfg(dim3(1), dim3(256), s, attr, pdl);
  return cudaLaunchKernelEx(&cfg, argmax_final_kernel, part_val, part_idx, nparts, state, argmax_out, history,
                            history_cap, pf, xchg_epoch, xchg_per_step, tp);
}

cudaError_t launch_advance(cudaStream_t s, StepState* state, uint32_t* xchg_epoch, uint32_t xchg_per_step, bool pdl) {
  cudaLaunchAttribute attr[1];
  cudaLaunchConfig_t cfg = make_cfg(dim3(1), dim3(32), s, attr, pdl);
  return cudaLaunchKernelEx(&cfg, advance_kernel, state, xchg_epoch, xchg_per_step);
}

cudaError_t launch_ingest(cudaStream_t s, int src_dtype, int dst_dtype, const IngestParams& p) {
  if (p.n == 0) return cudaSuccess;
  uint64_t want = (p.n + 255) / 256;
  const uint64_t cap = (uint64_t)sm_count() * 16;
  dim3 grid((unsigned)(want < cap ? want : cap)), block(256);
  if (src_dtype == 0 && dst_dtype == 0) ingest_kernel<float, float><<<grid, block, 0, s>>>(p);
  else if (src_dtype == 0 && dst_dtype == 1) ingest_kernel<float, __half><<<grid, block, 0, s>>>(p);
  else if (src_dtype == 1 && dst_dtype == 0) ingest_kernel<__half, float><<<grid, block, 0, s>>>(p);
  else if (src_dtype == 1 && dst_dtype == 1) ingest_kernel<__half, __half><<<grid, block, 0, s>>>(p);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

}  // namespace nfai
