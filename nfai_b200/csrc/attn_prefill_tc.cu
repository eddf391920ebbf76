// Causal attention over a chunk of prompt tokens on the tensor cores (flash-attention forward, one pass over K/V).
//
// The token-at-a-time prompt kernel (attn_prefill_kernel in attn.cu) re-reads the whole prefix of K and V for every
// token: at 2 048 prompt tokens that is 80 % of the prompt time. Here a CTA owns 128 consecutive tokens of one
// query head (8 warps x 16 rows) and walks the prefix once in tiles of 64 positions:
//   S = Q K^T   (mma.sync m16n8k16, float16 operands, float32 accumulators; Q fragments stay in registers,
//                pre-multiplied by 1/sqrt(d) * log2(e) so every exponential is one ex2)
//   online softmax on the accumulator fragments (running max and sum per token row, quad shuffles)
//   O += P V    (the S accumulators are re-packed as the A operand; V is read transposed with ldmatrix.trans)
// K and V tiles are staged in shared memory (rows padded by 16 bytes: conflict-free ldmatrix) in three buffers: tiles
// i + 1 and i + 2 are being copied with cp.async (16 bytes per copy, zero-filled past the range) while tile i is
// multiplied, and one block barrier per tile suffices; a float32 cache is converted to float16 on the way in with
// plain loads instead.
// Token t of the chunk sits at position p0 + t and attends to positions 0 .. p0 + t (causal); rows past the
// chunk and positions past the last token are masked with -inf, and V rows past the range are zero-filled so that
// a zero weight never meets a non-finite stale value.
//
// Precision: q, the softmax weights and (for a float32 cache) K and V are rounded to float16 for the products,
// accumulation is float32 -- the arithmetic of every tensor-core attention; the path is only taken for float16
// models, whose tolerance (logits within 2e-2 absolute) it meets with two orders of magnitude to spare.
//
// Reference arithmetic replaced: AttentionScoreCalculationShader.cs:170-205, AttentionSoftmaxShader.cs:145-177,
// AttentionWeightedValueSumShader.cs:181-215, applied once per prompt token by LlamaModel.cs:103-126.
#include "attn_core.cuh"

namespace nfai {

namespace {

constexpr int kPM = 128;      // tokens per CTA
constexpr int kPN = 64;       // positions per K/V tile
constexpr int kPThreads = 256;
constexpr int kBufs = 3;      // K/V tile buffers

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

__device__ __forceinline__ float p_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

// eight consecutive float32 cache elements of one row -> eight halves (a float16 cache is copied with cp.async)
__device__ __forceinline__ uint4 load8_as_half(const __half* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ uint4 load8_as_half(const float* p) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  uint4 r;
  r.x = pack_half2(a.x, a.y);
  r.y = pack_half2(a.z, a.w);
  r.z = pack_half2(b.x, b.y);
  r.w = pack_half2(b.z, b.w);
  return r;
}

template <typename KVT, int D>
__global__ void __launch_bounds__(kPThreads, D == 64 ? 2 : 1) attn_prefill_tc_kernel(const AttnParams p, const uint32_t T) {
  constexpr int LD = D + 8;  // shared-memory row stride in halves (16 bytes of padding)
  constexpr int kTile = kPN * LD;  // halves of one K (or V) tile
  extern __shared__ __align__(16) unsigned char ptc_smem[];
  __half* const Ks = reinterpret_cast<__half*>(ptc_smem);  // [kBufs][kTile]
  __half* const Vs = Ks + kBufs * kTile;                    // [kBufs][kTile]
  pdl_launch_dependents();
  pdl_wait();  // q and the chunk's cache rows come from the QKV GEMM launched just before
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qr = lane >> 2, qc = (lane & 3) * 2;
  // Causal work grows with the token tile: CTAs are numbered so that the last (longest) tiles of all heads start
  // first and the short ones fill the gaps at the end.
  const uint32_t h = blockIdx.x % p.qH;
  const uint32_t tile_x = gridDim.x / p.qH - 1 - blockIdx.x / p.qH;
  const uint32_t g = h / (p.qH / p.kvH);
  const uint32_t kvDim = p.kvH * D, qDim = p.qH * D;
  const uint32_t p0 = p.seq_imm - 1;  // position of the chunk's first token
  const uint32_t row_a = tile_x * kPM + warp * 16 + qr, row_b = row_a + 8;  // this thread's two token rows
  const uint32_t rows_end = min(T, (tile_x + 1) * (uint32_t)kPM);           // tokens of this CTA end here
  const uint32_t kv_end = p0 + rows_end;                                         // positions [0, kv_end) are needed

  // Q fragments (A operand, 16 x 16 per k step), scaled into the base-2 domain
  const float qscale = (1.0f / sqrtf((float)D)) * 1.4426950408889634f;
  uint32_t qf[D / 16][4];
  {
    const float* qa = p.q + (size_t)row_a * qDim + h * D;
    const float* qb = p.q + (size_t)row_b * qDim + h * D;
    const bool va = row_a < T, vb = row_b < T;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const int c = kk * 16 + qc;
      const float2 a0 = va ? *reinterpret_cast<const float2*>(qa + c) : make_float2(0.f, 0.f);
      const float2 b0 = vb ? *reinterpret_cast<const float2*>(qb + c) : make_float2(0.f, 0.f);
      const float2 a1 = va ? *reinterpret_cast<const float2*>(qa + c + 8) : make_float2(0.f, 0.f);
      const float2 b1 = vb ? *reinterpret_cast<const float2*>(qb + c + 8) : make_float2(0.f, 0.f);
      qf[kk][0] = pack_half2(a0.x * qscale, a0.y * qscale);
      qf[kk][1] = pack_half2(b0.x * qscale, b0.y * qscale);
      qf[kk][2] = pack_half2(a1.x * qscale, a1.y * qscale);
      qf[kk][3] = pack_half2(b1.x * qscale, b1.y * qscale);
    }
  }
  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m_a = attn_detail::kNegBig, m_b = attn_detail::kNegBig, l_a = 0.f, l_b = 0.f;

  const KVT* kbase = reinterpret_cast<const KVT*>(p.kcache) + (size_t)g * D;
  const KVT* vbase = reinterpret_cast<const KVT*>(p.vcache) + (size_t)g * D;
  const uint32_t ks_base = (uint32_t)__cvta_generic_to_shared(Ks), vs_base = (uint32_t)__cvta_generic_to_shared(Vs);
  // ldmatrix row addresses of this lane (see the operand layouts in the file header)
  const int lm = lane >> 3, lr = lane & 7;
  const uint32_t k_lane_off = (uint32_t)(((lm >> 1) * 8 + lr) * LD + (lm & 1) * 8) * 2;   // K: pair of position tiles
  const uint32_t v_lane_off = (uint32_t)(((lm & 1) * 8 + lr) * LD + (lm >> 1) * 8) * 2;   // V: pair of dim tiles

  // copy (or convert) the K and V rows of tile `tile` into buffer `buf`
  constexpr int CPR = D / 8;  // 16-byte chunks per row
  auto issue = [&](int buf, uint32_t tile) {
    const uint32_t n0 = tile * kPN;
#pragma unroll
    for (int i = 0; i < kPN * CPR / kPThreads; ++i) {
      const int c = tid + i * kPThreads;
      const int r = c / CPR, c8 = (c % CPR) * 8;
      const uint32_t pos = n0 + r;
      const bool in = pos < kv_end;
      const size_t row = (size_t)(in ? pos : 0u) * kvDim + c8;  // a valid address even when nothing is copied
      __half* kd = Ks + buf * kTile + r * LD + c8;
      __half* vd = Vs + buf * kTile + r * LD + c8;
      if constexpr (sizeof(KVT) == 2) {
        cp_async16((uint32_t)__cvta_generic_to_shared(kd), kbase + row, in ? 16u : 0u);
        cp_async16((uint32_t)__cvta_generic_to_shared(vd), vbase + row, in ? 16u : 0u);
      } else {
        uint4 kv = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
        if (in) {
          kv = load8_as_half(kbase + row);
          vv = load8_as_half(vbase + row);
        }
        *reinterpret_cast<uint4*>(kd) = kv;
        *reinterpret_cast<uint4*>(vd) = vv;
      }
    }
  };
  const uint32_t ntiles = (kv_end + kPN - 1) / kPN;
  // Three buffers: tile it + 2 is requested into the buffer that tile it - 1 was multiplied from, right after the one
  // block barrier of the iteration (which says both that tile it has landed everywhere and that every warp is done
  // with tile it - 1); two tiles are in flight while one is multiplied.
  issue(0, 0);
  cp_async_commit();
  if (ntiles > 1) issue(1, 1);
  cp_async_commit();  // (an empty group keeps the count uniform)
  for (uint32_t it = 0; it < ntiles; ++it) {
    const uint32_t n0 = it * kPN;
    cp_async_wait_all_but_one();  // this thread's copies of tile it have landed
    __syncthreads();              // ... and everybody else's; every warp has left tile it - 1
    if (it + 2 < ntiles) issue((int)((it + 2) % kBufs), it + 2);
    cp_async_commit();
    const uint32_t ks_s = ks_base + (it % kBufs) * (uint32_t)(kTile * 2), vs_s = vs_base + (it % kBufs) * (uint32_t)(kTile * 2);
    // a warp whose rows all lie before this tile's first position has nothing to add (causal), but it keeps
    // taking part in the block barriers
    const uint32_t warp_last_pos = p0 + tile_x * kPM + warp * 16 + 15;
    if (n0 <= warp_last_pos) {
    // ---- S = Q K^T : 16 rows x 64 positions per warp
    float s[kPN / 8][4];
#pragma unroll
    for (int j = 0; j < kPN / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
      for (int j = 0; j < kPN / 8; j += 2) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(ks_s + (uint32_t)(j * 8 * LD + kk * 16) * 2 + k_lane_off, b0, b1, b2, b3);
        mma_16816(s[j], qf[kk], b0, b1);
        mma_16816(s[j + 1], qf[kk], b2, b3);
      }
    }
    // ---- causal mask (only tiles that reach past the warp's first row need it)
    if (n0 + kPN - 1 > p0 + tile_x * kPM + warp * 16) {
      const uint32_t lim_a = row_a < T ? p0 + row_a : 0u, lim_b = row_b < T ? p0 + row_b : 0u;  // last visible position
      const bool va = row_a < T, vb = row_b < T;
#pragma unroll
      for (int j = 0; j < kPN / 8; ++j) {
        const uint32_t c = n0 + j * 8 + qc;
        if (!va || c > lim_a) s[j][0] = -INFINITY;
        if (!va || c + 1 > lim_a) s[j][1] = -INFINITY;
        if (!vb || c > lim_b) s[j][2] = -INFINITY;
        if (!vb || c + 1 > lim_b) s[j][3] = -INFINITY;
      }
    }
    // ---- online softmax: one new maximum and one rescale per tile
    float mx_a = s[0][0], mx_b = s[0][2];
#pragma unroll
    for (int j = 0; j < kPN / 8; ++j) {
      mx_a = fmaxf(mx_a, fmaxf(s[j][0], s[j][1]));
      mx_b = fmaxf(mx_b, fmaxf(s[j][2], s[j][3]));
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);  // finite: the running maxima start finite
    const float al_a = p_ex2(m_a - mn_a), al_b = p_ex2(m_b - mn_b);
    m_a = mn_a;
    m_b = mn_b;
    float sum_a = 0.f, sum_b = 0.f;
    uint32_t pf[kPN / 16][4];
#pragma unroll
    for (int j = 0; j < kPN / 8; ++j) {
      const float e0 = p_ex2(s[j][0] - mn_a), e1 = p_ex2(s[j][1] - mn_a);
      const float e2 = p_ex2(s[j][2] - mn_b), e3 = p_ex2(s[j][3] - mn_b);
      sum_a += e0 + e1;
      sum_b += e2 + e3;
      // accumulator layout of two neighbouring position tiles = A-operand layout of one 16-position k step
      pf[j >> 1][(j & 1) * 2 + 0] = pack_half2(e0, e1);
      pf[j >> 1][(j & 1) * 2 + 1] = pack_half2(e2, e3);
    }
    l_a = l_a * al_a + sum_a;
    l_b = l_b * al_b + sum_b;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      o[j][0] *= al_a;
      o[j][1] *= al_a;
      o[j][2] *= al_b;
      o[j][3] *= al_b;
    }
    // ---- O += P V
#pragma unroll
    for (int kk = 0; kk < kPN / 16; ++kk) {
#pragma unroll
      for (int j = 0; j < D / 8; j += 2) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_trans(vs_s + (uint32_t)(kk * 16 * LD + j * 8) * 2 + v_lane_off, b0, b1, b2, b3);
        mma_16816(o[j], pf[kk], b0, b1);
        mma_16816(o[j + 1], pf[kk], b2, b3);
      }
    }
    }  // tile visible to this warp
  }
  // ---- normalise and store (float16: the A operand of the output projection)
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  if (row_a < T) {
    const float inv = 1.0f / l_a;
    __half* out = p.out_half + (size_t)row_a * qDim + h * D + qc;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) *reinterpret_cast<__half2*>(out + j * 8) = __floats2half2_rn(o[j][0] * inv, o[j][1] * inv);
  }
  if (row_b < T) {
    const float inv = 1.0f / l_b;
    __half* out = p.out_half + (size_t)row_b * qDim + h * D + qc;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) *reinterpret_cast<__half2*>(out + j * 8) = __floats2half2_rn(o[j][2] * inv, o[j][3] * inv);
  }
}

template <typename KVT, int D>
cudaError_t launch_ptc_d(cudaStream_t s, const AttnParams& p, uint32_t T) {
  constexpr size_t smem = (size_t)2 * kBufs * kPN * (D + 8) * 2;  // kBufs buffers of a K and a V tile
  static thread_local int attr_device = -1;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (attr_device != dev) {
    e = cudaFuncSetAttribute(attn_prefill_tc_kernel<KVT, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    attr_device = dev;
  }
  dim3 grid(((T + kPM - 1) / kPM) * p.qH);
  return launch_pdl(attn_prefill_tc_kernel<KVT, D>, grid, dim3(kPThreads), smem, s, prefill_pdl(), p, T);
}

template <typename KVT>
cudaError_t launch_ptc(cudaStream_t s, const AttnParams& p, uint32_t T) {
  switch (p.d) {
    case 64: return launch_ptc_d<KVT, 64>(s, p, T);
    case 128: return launch_ptc_d<KVT, 128>(s, p, T);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

bool attn_prefill_tc_supported(uint32_t d) { return d == 64 || d == 128; }

cudaError_t launch_attn_prefill_tc(cudaStream_t s, int kvdtype, const AttnParams& p, uint32_t T) {
  if (p.qH == 0 || p.kvH == 0 || p.qH % p.kvH != 0 || !p.out_half || !p.seq_imm || !T || p.qH > 65535) return cudaErrorInvalidValue;
  return kvdtype == 1 ? launch_ptc<__half>(s, p, T) : launch_ptc<float>(s, p, T);
}

}  // namespace nfai
