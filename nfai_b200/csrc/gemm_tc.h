// Tensor-core GEMM for prompt ingestion (internal interface).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nfai {

enum GemmEpilogueKind { GEMM_EPI_STORE = 0, GEMM_EPI_SILU_MUL = 1, GEMM_EPI_QKV_ROPE = 2 };

struct GemmEpilogue {
  int kind = GEMM_EPI_STORE;
  float* out_f32 = nullptr;      // STORE: [M][N]; QKV_ROPE: q rows [M][qDim]
  const float* resid = nullptr;  // STORE: optional [M][N] addend
  __half* out_f16 = nullptr;     // SILU_MUL: [M][N/2]
  // QKV_ROPE
  void* kcache = nullptr;
  void* vcache = nullptr;
  int kv_f16 = 0;
  uint32_t qDim = 0, kvDim = 0, d = 0, ropeDim = 0, pos0 = 0;
  const float2* rope_cs = nullptr;
  // Optional scratch for split-K: when the tile grid alone would leave most SMs idle (a short prompt chunk), the K
  // range is divided over several CTAs, each stores its float32 partial tile here ([split][M][N]) and a second
  // kernel adds the partials in split order and applies the epilogue. Without scratch the GEMM never splits.
  float* scratch = nullptr;
  size_t scratch_floats = 0;
};

// Number of K splits launch_gemm_tc would use for this shape given enough scratch (1 = no split).
uint32_t gemm_tc_splits(uint32_t M, uint32_t N, uint32_t K);

// C = A[M][K] * W[N][K]^T with the epilogue applied; A and W are float16, K contiguous, K % 8 == 0, 16-byte aligned.
// err (optional device word) gets bit 4 when a bounded wait inside the kernel gave up.
cudaError_t launch_gemm_tc(cudaStream_t s, const __half* A, const __half* W, uint32_t M, uint32_t N, uint32_t K,
                           const GemmEpilogue& ep, uint32_t* err);

// x[M][H] float32 -> RMS-normalised, gain-scaled float16 rows (the A operand of the QKV and gate/up GEMMs).
// after_collective: x was produced by a library collective enqueued just before; the kernel is then launched with
// plain stream order (no programmatic dependent launch across the library's kernels).
cudaError_t launch_rmsnorm_to_half(cudaStream_t s, const float* x, const float* gain, float eps, uint32_t M, uint32_t H,
                                   __half* out, bool after_collective = false);
// rows of the embedding matrix (float16) widened to float32: x[t] = E[tokens[t]].
cudaError_t launch_embed_rows(cudaStream_t s, const __half* E, const uint32_t* tokens, uint32_t M, uint32_t H, float* x);
cudaError_t launch_float_to_half(cudaStream_t s, const float* in, __half* out, size_t n);

}  // namespace nfai
