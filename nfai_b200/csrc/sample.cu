// On-device temperature / top-k / top-p sampling of the last step's logits, so that only the chosen token id
// crosses PCIe (the reference reads 513 KB of logits back and sorts them with LINQ for every token:
// NFAI.Models.Llama3/LlamaModel.cs:128-130,165, SamplingUtils.cs:5-33). The uniform random number comes from the
// caller (the reference uses Random.Shared), which also makes the result reproducible.
//
// Arithmetic follows SamplingUtils.TopP: scaled = logit / T; p = exp(scaled - max) / sum (sum accumulated in
// double, as LINQ's Sum does); the top_k largest p in stable order (ties: lower index first); accumulate until the
// cumulative probability reaches top_p; renormalise; first index whose running sum exceeds u, else the last.
//
// Two kernels: every CTA takes a slice of the vocabulary, sums exp(scaled - max) in double and selects its own
// top_k by repeated block arg-max; one CTA then merges the slices' candidates the same way and samples.
#include <stdlib.h>

#include "common.cuh"
#include "kernels.h"

namespace nfai {

namespace {

constexpr int kST = 256;         // threads per CTA
constexpr int kSPer = 8;         // logits per thread in the slice kernel
constexpr int kSliceMax = kST * kSPer;
constexpr int kMaxTopK = 64;

struct Pick {
  float v;
  uint32_t i;
};
// a precedes b: larger value first, then lower index
__device__ __forceinline__ bool before(float av, uint32_t ai, float bv, uint32_t bi) { return av > bv || (av == bv && ai < bi); }

// Block-wide best of one (value, index) per thread; index 0xffffffff = nothing.
__device__ __forceinline__ Pick block_best(float v, uint32_t i, Pick* sm /*[kST/32]*/, Pick* bcast) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const uint32_t oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (oi != 0xffffffffu && (i == 0xffffffffu || before(ov, oi, v, i))) {
      v = ov;
      i = oi;
    }
  }
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = Pick{v, i};
  __syncthreads();
  if (threadIdx.x < 32) {
    Pick p = threadIdx.x < kST / 32 ? sm[threadIdx.x] : Pick{0.f, 0xffffffffu};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, p.v, o);
      const uint32_t oi = __shfl_xor_sync(0xffffffffu, p.i, o);
      if (oi != 0xffffffffu && (p.i == 0xffffffffu || before(ov, oi, p.v, p.i))) {
        p.v = ov;
        p.i = oi;
      }
    }
    if (threadIdx.x == 0) *bcast = p;
  }
  __syncthreads();
  return *bcast;
}

// Slice kernel: CTA c owns logits [c*slice, (c+1)*slice).
__global__ void __launch_bounds__(kST) sample_slice_kernel(const float* __restrict__ logits, uint32_t V, uint32_t slice,
                                                          const uint32_t* __restrict__ argmax, float temperature, int top_k,
                                                          double* __restrict__ part_sum, float* __restrict__ cand_val,
                                                          uint32_t* __restrict__ cand_idx) {
  __shared__ Pick sm[kST / 32];
  __shared__ Pick bcast;
  __shared__ double dsum[kST / 32];
  const uint32_t lo = blockIdx.x * slice;
  const uint32_t am = *argmax;
  const float mx = logits[am < V ? am : 0] / temperature;  // max of the scaled logits
  float v[kSPer];
  uint32_t idx[kSPer];
  double s = 0.0;
#pragma unroll
  for (int k = 0; k < kSPer; ++k) {
    const uint32_t i = lo + k * kST + threadIdx.x;
    if (k * kST + threadIdx.x < slice && i < V) {
      v[k] = logits[i] / temperature;
      idx[k] = i;
      s += (double)expf(v[k] - mx);
    } else {
      v[k] = 0.f;
      idx[k] = 0xffffffffu;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) dsum[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < kST / 32; ++w) t += dsum[w];
    part_sum[blockIdx.x] = t;
  }
  for (int r = 0; r < top_k; ++r) {
    float bv = 0.f;
    uint32_t bi = 0xffffffffu;
#pragma unroll
    for (int k = 0; k < kSPer; ++k)
      if (idx[k] != 0xffffffffu && (bi == 0xffffffffu || before(v[k], idx[k], bv, bi))) {
        bv = v[k];
        bi = idx[k];
      }
    const Pick w = block_best(bv, bi, sm, &bcast);
    if (threadIdx.x == 0) {
      cand_val[blockIdx.x * kMaxTopK + r] = w.v;
      cand_idx[blockIdx.x * kMaxTopK + r] = w.i;
    }
#pragma unroll
    for (int k = 0; k < kSPer; ++k)
      if (idx[k] == w.i) idx[k] = 0xffffffffu;  // taken
  }
}

// Final kernel: merge the slices' candidates, then the cumulative / renormalise / draw of SamplingUtils.TopP.
__global__ void __launch_bounds__(kST) sample_final_kernel(const float* __restrict__ logits, uint32_t V,
                                                          const uint32_t* __restrict__ argmax, uint32_t* cur_token,
                                                          float temperature, float top_p, int top_k, float u, int nslices,
                                                          const double* __restrict__ part_sum, const float* __restrict__ cand_val,
                                                          const uint32_t* __restrict__ cand_idx, uint32_t* __restrict__ token_out) {
  __shared__ Pick sm[kST / 32];
  __shared__ Pick bcast;
  __shared__ Pick chosen[kMaxTopK];
  const int ncand = nslices * top_k;
  for (int r = 0; r < top_k; ++r) {
    float bv = 0.f;
    uint32_t bi = 0xffffffffu;
    for (int c = threadIdx.x; c < ncand; c += kST) {
      const int sl = c / top_k, k = c - sl * top_k;
      const float v = cand_val[sl * kMaxTopK + k];
      const uint32_t i = cand_idx[sl * kMaxTopK + k];
      if (i == 0xffffffffu) continue;
      // skip what earlier rounds already took: everything that precedes or equals the last pick
      if (r > 0) {
        const Pick last = chosen[r - 1];
        if (!before(last.v, last.i, v, i)) continue;
      }
      if (bi == 0xffffffffu || before(v, i, bv, bi)) {
        bv = v;
        bi = i;
      }
    }
    const Pick w = block_best(bv, bi, sm, &bcast);
    if (threadIdx.x == 0) chosen[r] = w;
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    double tot = 0.0;
    for (int c = 0; c < nslices; ++c) tot += part_sum[c];
    const float sumf = (float)tot;
    const uint32_t am = *argmax;
    const float mx = logits[am < V ? am : 0] / temperature;
    if (am >= V || chosen[0].i == 0xffffffffu || chosen[0].v != mx) {  // the arg-max does not belong to these logits
      *token_out = 0xffffffffu;
      return;
    }
    float pr[kMaxTopK];
    int n = 0;
    float cumulative = 0.f;
    for (int r = 0; r < top_k; ++r) {
      if (chosen[r].i == 0xffffffffu) break;
      const float p = __fdiv_rn(expf(chosen[r].v - mx), sumf);
      cumulative += p;
      pr[n++] = p;
      if (cumulative >= top_p) break;
    }
    double t2 = 0.0;
    for (int r = 0; r < n; ++r) t2 += (double)pr[r];
    const float total = (float)t2;
    uint32_t tok = chosen[n > 0 ? n - 1 : 0].i;
    float running = 0.f;
    for (int r = 0; r < n; ++r) {
      running += __fdiv_rn(pr[r], total);
      if (u < running) {
        tok = chosen[r].i;
        break;
      }
    }
    *token_out = tok;
    if (cur_token) *cur_token = tok;  // a following device-side step continues with the sampled token
  }
}

// Arg-max (lowest index among equals) of a logits vector that did not come out of a model step.
__global__ void __launch_bounds__(1024) sample_argmax_kernel(const float* __restrict__ logits, uint32_t V, uint32_t* __restrict__ out) {
  __shared__ Pick sm[32];
  float v = 0.f;
  uint32_t i = 0xffffffffu;
  for (uint32_t k = threadIdx.x; k < V; k += 1024) {
    const float x = logits[k];
    if (i == 0xffffffffu || before(x, k, v, i)) {
      v = x;
      i = k;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const uint32_t oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (oi != 0xffffffffu && (i == 0xffffffffu || before(ov, oi, v, i))) {
      v = ov;
      i = oi;
    }
  }
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = Pick{v, i};
  __syncthreads();
  if (threadIdx.x < 32) {
    Pick p = sm[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, p.v, o);
      const uint32_t oi = __shfl_xor_sync(0xffffffffu, p.i, o);
      if (oi != 0xffffffffu && (p.i == 0xffffffffu || before(ov, oi, p.v, p.i))) {
        p.v = ov;
        p.i = oi;
      }
    }
    if (threadIdx.x == 0) *out = p.i;
  }
}

// ---- fast path for large vocabularies: histogram cut instead of 2 x top_k rounds of block arg-max ---------------
// Pass 1 sums exp(scaled - max) per CTA (as above) and counts the scaled logits in 128 bins of width 1/4 below the
// maximum. The bin in which the count from the top reaches top_k bounds the top_k-th largest value from below, so
// pass 2 keeps every element of that bin and the bins above it (typically a few dozen to a few hundred of 128 256).
// Pass 3 (one CTA) ranks the kept elements by counting, in the reference's order (value descending, index ascending;
// the order in which pass 2 appended them does not matter), and runs the same cumulative / renormalise / draw code.
// More than kMaxCand kept elements (a nearly flat distribution) falls back, inside pass 3, to block arg-max rounds
// over the whole vector.
constexpr int kHistBins = 128;
constexpr float kBinsPerUnit = 4.0f;
constexpr int kMaxCand = 1024;

__device__ __forceinline__ int hist_bin(float scaled, float mx) {
  const float d = (mx - scaled) * kBinsPerUnit;  // >= 0 up to rounding
  const int b = d <= 0.f ? 0 : (d >= (float)(kHistBins - 1) ? kHistBins - 1 : (int)d);
  return b;
}

__global__ void __launch_bounds__(kST) sample_hist_kernel(const float* __restrict__ logits, uint32_t V, uint32_t slice,
                                                         const uint32_t* __restrict__ argmax, float temperature,
                                                         double* __restrict__ part_sum, uint32_t* __restrict__ ghist) {
  __shared__ double dsum[kST / 32];
  __shared__ uint32_t hist[kHistBins];
  if (threadIdx.x < kHistBins) hist[threadIdx.x] = 0;
  __syncthreads();
  const uint32_t lo = blockIdx.x * slice;
  const uint32_t am = *argmax;
  const float mx = logits[am < V ? am : 0] / temperature;
  double s = 0.0;
#pragma unroll
  for (int k = 0; k < kSPer; ++k) {
    const uint32_t i = lo + k * kST + threadIdx.x;
    if (k * kST + threadIdx.x < slice && i < V) {
      const float v = logits[i] / temperature;
      s += (double)expf(v - mx);
      atomicAdd(&hist[hist_bin(v, mx)], 1u);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) dsum[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < kST / 32; ++w) t += dsum[w];
    part_sum[blockIdx.x] = t;
  }
  if (threadIdx.x < kHistBins && hist[threadIdx.x]) atomicAdd(&ghist[threadIdx.x], hist[threadIdx.x]);
}

__global__ void __launch_bounds__(kST) sample_collect_kernel(const float* __restrict__ logits, uint32_t V, uint32_t slice,
                                                            const uint32_t* __restrict__ argmax, float temperature, int top_k,
                                                            const uint32_t* __restrict__ ghist, uint32_t* __restrict__ count,
                                                            float* __restrict__ cand_val, uint32_t* __restrict__ cand_idx) {
  __shared__ int cut;
  if (threadIdx.x == 0) {
    uint32_t c = 0;
    int b = 0;
    for (; b < kHistBins - 1; ++b) {
      c += ghist[b];
      if (c >= (uint32_t)top_k) break;
    }
    cut = b;  // every bin up to and including this one is kept
  }
  __syncthreads();
  const int cutb = cut;
  const uint32_t lo = blockIdx.x * slice;
  const uint32_t am = *argmax;
  const float mx = logits[am < V ? am : 0] / temperature;
#pragma unroll
  for (int k = 0; k < kSPer; ++k) {
    const uint32_t i = lo + k * kST + threadIdx.x;
    if (k * kST + threadIdx.x < slice && i < V) {
      const float v = logits[i] / temperature;
      if (hist_bin(v, mx) <= cutb) {
        const uint32_t slot = atomicAdd(count, 1u);
        if (slot < (uint32_t)kMaxCand) {
          cand_val[slot] = v;
          cand_idx[slot] = i;
        }
      }
    }
  }
}

__global__ void __launch_bounds__(1024) sample_pick_kernel(const float* __restrict__ logits, uint32_t V,
                                                           const uint32_t* __restrict__ argmax, uint32_t* cur_token,
                                                           float temperature, float top_p, int top_k, float u, int nslices,
                                                           const double* __restrict__ part_sum, uint32_t* __restrict__ ghist,
                                                           uint32_t* __restrict__ count, const float* __restrict__ cand_val,
                                                           const uint32_t* __restrict__ cand_idx, uint32_t* __restrict__ token_out) {
  __shared__ float sv[kMaxCand];
  __shared__ uint32_t si[kMaxCand];
  __shared__ Pick chosen[kMaxTopK];
  __shared__ Pick sm[32];
  __shared__ Pick bcast;
  const uint32_t total = *count;
  const int tid = threadIdx.x;
  if (tid < kMaxTopK) chosen[tid] = Pick{0.f, 0xffffffffu};
  __syncthreads();
  if (total <= (uint32_t)kMaxCand) {
    const int n = (int)total;
    if (tid < n) {
      sv[tid] = cand_val[tid];
      si[tid] = cand_idx[tid];
    }
    __syncthreads();
    if (tid < n) {
      const float v = sv[tid];
      const uint32_t i = si[tid];
      int rank = 0;
      for (int c = 0; c < n; ++c) rank += before(sv[c], si[c], v, i) ? 1 : 0;
      if (rank < top_k) chosen[rank] = Pick{v, i};
    }
  } else {
    // nearly flat distribution: top_k rounds of block arg-max over the whole vector
    for (int r = 0; r < top_k; ++r) {
      float bv = 0.f;
      uint32_t bi = 0xffffffffu;
      for (uint32_t c = tid; c < V; c += 1024) {
        const float v = logits[c] / temperature;
        if (r > 0) {
          const Pick last = chosen[r - 1];
          if (!before(last.v, last.i, v, c)) continue;
        }
        if (bi == 0xffffffffu || before(v, c, bv, bi)) {
          bv = v;
          bi = c;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi != 0xffffffffu && (bi == 0xffffffffu || before(ov, oi, bv, bi))) {
          bv = ov;
          bi = oi;
        }
      }
      if ((tid & 31) == 0) sm[tid >> 5] = Pick{bv, bi};
      __syncthreads();
      if (tid < 32) {
        Pick q = sm[tid];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, q.v, o);
          const uint32_t oi = __shfl_xor_sync(0xffffffffu, q.i, o);
          if (oi != 0xffffffffu && (q.i == 0xffffffffu || before(ov, oi, q.v, q.i))) {
            q.v = ov;
            q.i = oi;
          }
        }
        if (tid == 0) bcast = q;
      }
      __syncthreads();
      if (tid == 0) chosen[r] = bcast;
      __syncthreads();
    }
  }
  __syncthreads();
  // the scratch counters go back to zero for the next call
  if (tid < kHistBins) ghist[tid] = 0;
  if (tid == 0) *count = 0;
  if (tid == 0) {
    double tot = 0.0;
    for (int c = 0; c < nslices; ++c) tot += part_sum[c];
    const float sumf = (float)tot;
    const uint32_t am = *argmax;
    const float mx = logits[am < V ? am : 0] / temperature;
    if (am >= V || chosen[0].i == 0xffffffffu || chosen[0].v != mx) {  // the arg-max does not belong to these logits
      *token_out = 0xffffffffu;
      return;
    }
    float pr[kMaxTopK];
    int n = 0;
    float cumulative = 0.f;
    for (int r = 0; r < top_k; ++r) {
      if (chosen[r].i == 0xffffffffu) break;
      const float p = __fdiv_rn(expf(chosen[r].v - mx), sumf);
      cumulative += p;
      pr[n++] = p;
      if (cumulative >= top_p) break;
    }
    double t2 = 0.0;
    for (int r = 0; r < n; ++r) t2 += (double)pr[r];
    const float totalp = (float)t2;
    uint32_t tok = chosen[n > 0 ? n - 1 : 0].i;
    float running = 0.f;
    for (int r = 0; r < n; ++r) {
      running += __fdiv_rn(pr[r], totalp);
      if (u < running) {
        tok = chosen[r].i;
        break;
      }
    }
    *token_out = tok;
    if (cur_token) *cur_token = tok;
  }
}

}  // namespace

size_t sample_scratch_bytes(uint32_t V, int* nslices_out) {
  int n = (int)((V + kSliceMax - 1) / kSliceMax);
  if (n < 148 && V >= 148u * 64u) n = 148;  // spread a mid-sized vocabulary over every SM
  if (nslices_out) *nslices_out = n;
  return (size_t)n * (8 + kMaxTopK * 8) + 256;
}

cudaError_t launch_sample_top_p(cudaStream_t s, const float* logits, uint32_t V, const uint32_t* argmax, uint32_t* cur_token,
                                float temperature, float top_p, int top_k, float u, void* scratch, uint32_t* token_out) {
  if (top_k < 1 || top_k > kMaxTopK || !(temperature > 0.f)) return cudaErrorInvalidValue;
  int nslices = 0;
  sample_scratch_bytes(V, &nslices);
  const uint32_t slice = (V + nslices - 1) / nslices;
  if (slice > (uint32_t)kSliceMax) return cudaErrorInvalidValue;
  double* part_sum = reinterpret_cast<double*>(scratch);
  static const bool fast_ok = [] { const char* v = getenv("NFAI_SAMPLE_FAST"); return !(v && atoi(v) == 0); }();
  if (fast_ok && nslices >= 148) {  // the scratch of >= 148 slices holds the histogram path's buffers
    uint32_t* ghist = reinterpret_cast<uint32_t*>(part_sum + nslices);
    uint32_t* count = ghist + kHistBins;
    float* fval = reinterpret_cast<float*>(count + 4);
    uint32_t* fidx = reinterpret_cast<uint32_t*>(fval + kMaxCand);
    cudaError_t e = cudaMemsetAsync(ghist, 0, (kHistBins + 4) * sizeof(uint32_t), s);
    if (e != cudaSuccess) return e;
    if (!argmax) {
      uint32_t* am = fidx + kMaxCand;
      sample_argmax_kernel<<<1, 1024, 0, s>>>(logits, V, am);
      argmax = am;
    }
    sample_hist_kernel<<<nslices, kST, 0, s>>>(logits, V, slice, argmax, temperature, part_sum, ghist);
    sample_collect_kernel<<<nslices, kST, 0, s>>>(logits, V, slice, argmax, temperature, top_k, ghist, count, fval, fidx);
    sample_pick_kernel<<<1, 1024, 0, s>>>(logits, V, argmax, cur_token, temperature, top_p, top_k, u, nslices, part_sum, ghist,
                                          count, fval, fidx, token_out);
    return cudaGetLastError();
  }
  float* cand_val = reinterpret_cast<float*>(part_sum + nslices);
  uint32_t* cand_idx = reinterpret_cast<uint32_t*>(cand_val + (size_t)nslices * kMaxTopK);
  if (!argmax) {
    uint32_t* am = cand_idx + (size_t)nslices * kMaxTopK;
    sample_argmax_kernel<<<1, 1024, 0, s>>>(logits, V, am);
    argmax = am;
  }
  sample_slice_kernel<<<nslices, kST, 0, s>>>(logits, V, slice, argmax, temperature, top_k, part_sum, cand_val, cand_idx);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  sample_final_kernel<<<1, kST, 0, s>>>(logits, V, argmax, cur_token, temperature, top_p, top_k, u, nslices, part_sum, cand_val,
                                        cand_idx, token_out);
  return cudaGetLastError();
}

}  // namespace nfai
