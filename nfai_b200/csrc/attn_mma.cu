// Long-context decode attention on the tensor cores (float16 cache, head dimension 64 or 128).
//
// At 32 768 positions the attention of one decode step streams 67 MB of K and V per layer. With the four query
// heads of a KV group multiplied on the CUDA cores the kernel is bound by instruction issue (about 260 FMAs plus
// shuffles per position), not by HBM: 3.0 TB/s. Here the query heads of a KV group are the rows of a 16-row tile
// (rows beyond the group are zero) and both products run as warp-level MMAs:
//   S = Q K^T   mma.sync m16n8k16, float16 operands, float32 accumulators
//   online softmax on the accumulator fragments (running max and sum per row, quad shuffles, base-2 exponentials)
//   O += P V    the S accumulators re-packed as the A operand, V read transposed with ldmatrix.trans
// which is 16 times fewer instructions per position, so the kernel streams at the rate HBM delivers.
// q and the softmax weights are float32 values: each is split into a float16 head and a float16 remainder and both
// parts are multiplied (two MMAs into the same accumulator), which keeps the products exact to ~2^-22; K and V are
// float16 in the cache already. Accumulation is float32.
//
// Shape: grid = (KV heads x head groups, S_max splits); a CTA of 8 warps owns one KV head, up to 4 of its query
// heads and one contiguous range of positions. The range is dealt to the warps in slices of 16 positions (slice i of
// the range goes to warp i mod 8, so that the CTA reads contiguous memory at every step). Every warp is its own
// pipeline: it copies its slices of K and V rows into private, padded shared-memory stages with 16-byte cp.async
// (zero-filled past the range), keeps up to three slices in flight (one for head dimension 128) and multiplies the
// oldest; nothing but a warp barrier separates copy and use, so the warps drift apart freely and HBM always has
// requests queued. Every warp keeps its own online-softmax state; at the end the warps are merged through shared
// memory, and -- when the sequence was split -- the CTAs through scratch partials and a ticket: the CTA that
// draws the last ticket of its head group merges. No CTA waits for another one.
//
// Reference arithmetic replaced: AttentionScoreCalculationShader.cs:170-205, AttentionSoftmaxShader.cs:145-177,
// AttentionWeightedValueSumShader.cs:181-215 (softmax equivalence as argued in attn.cu).
#include "attn_core.cuh"

namespace nfai {

namespace {

using attn_detail::kNegBig;

constexpr int kMW = 8;             // warps per CTA
constexpr int kMThreads = kMW * 32;
constexpr int kMG = 4;             // query heads per CTA

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ float m_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// (head, remainder) of two float32 values as two float16 pairs: a = hi + lo to ~2^-22
__device__ __forceinline__ void split_half2(float a, float b, uint32_t& hi, uint32_t& lo) {
  const __half2 h = __floats2half2_rn(a, b);
  const float2 hf = __half22float2(h);
  const __half2 l = __floats2half2_rn(a - hf.x, b - hf.y);
  hi = *reinterpret_cast<const uint32_t*>(&h);
  lo = *reinterpret_cast<const uint32_t*>(&l);
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

template <int N>
__device__ __forceinline__ void cp_async_wait_all_but() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int D>
__global__ void __launch_bounds__(kMThreads, 1) attn_mma_kernel(const AttnParams p) {
  constexpr int PW = 16;                  // positions per slice (one k step of the second product)
  constexpr int NST = D == 64 ? 4 : 2;    // stages per warp
  constexpr int LD = D + 8;               // shared-memory row stride in halves (16 bytes of padding: conflict-free ldmatrix)
  constexpr int kSlice = PW * LD;         // halves of one K (or V) slice
  constexpr int STR = D + 2;              // one partial in scratch: D accumulators, m, l
  extern __shared__ __align__(16) unsigned char mma_smem[];
  constexpr int kRowsMax = 64;                                // rows of partials merged per pass
  constexpr int kRegion = ((kRowsMax + 2) * STR + 4 + 3) / 4 * 4;  // floats per head in the merge buffer
  static_assert(kRowsMax >= kMW, "the warps' rows are the first pass");
  __shared__ float fin_scale[kRowsMax + 1][kMG];
  __shared__ float fin_ML[kMG][2];
  __shared__ uint32_t is_last;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qr = lane >> 2, qc = (lane & 3) * 2;
  __half* const Ks = reinterpret_cast<__half*>(mma_smem) + (size_t)warp * NST * 2 * kSlice;  // this warp: [NST][K slice, V slice]
  prefetch_plan(p.pf, kPrefetchChunk);
  pdl_launch_dependents();
  const uint32_t seq = p.state ? p.state->pos + 1 : p.seq_imm;  // advanced by the previous step, which has completed
  const uint32_t bx = blockIdx.x, s = blockIdx.y;
  const uint32_t G = p.qH / p.kvH;
  const uint32_t hgroups = (G + kMG - 1) / kMG;
  const uint32_t g = bx / hgroups, hg = bx % hgroups;
  const uint32_t h0 = g * G + hg * kMG;
  const uint32_t nh = min((uint32_t)kMG, G - hg * kMG);
  const uint32_t kvDim = p.kvH * D;
  uint32_t chunk = (seq + p.S_max - 1) / p.S_max;
  chunk = chunk < p.min_chunk ? p.min_chunk : chunk;
  chunk = (chunk + 63) / 64 * 64;
  const uint32_t S_eff = (seq + chunk - 1) / chunk;
  if (s >= S_eff) return;  // the whole CTA; nothing is in flight
  const uint32_t t0 = s * chunk;
  const uint32_t t1 = min(seq, t0 + chunk);
  const uint32_t nslices = (t1 - t0 + PW - 1) / PW;
  const uint32_t my_n = (uint32_t)warp < nslices ? (nslices - warp + kMW - 1) / kMW : 0;  // slices of this warp

  const __half* kbase = reinterpret_cast<const __half*>(p.kcache) + (size_t)g * D;
  const __half* vbase = reinterpret_cast<const __half*>(p.vcache) + (size_t)g * D;
  const uint32_t ks_base = (uint32_t)__cvta_generic_to_shared(Ks);
  const int lm = lane >> 3, lr = lane & 7;
  const uint32_t k_lane_off = (uint32_t)(((lm >> 1) * 8 + lr) * LD + (lm & 1) * 8) * 2;  // K: pair of position tiles
  const uint32_t v_lane_off = (uint32_t)(((lm & 1) * 8 + lr) * LD + (lm >> 1) * 8) * 2;  // V: pair of dim tiles

  constexpr int CPR = D / 8;  // 16-byte chunks per row
  auto slice_pos = [&](uint32_t i) { return t0 + (i * kMW + warp) * PW; };
  // the rows of this warp's slice i into stage i % NST; positions at or beyond t1 are zero-filled
  auto issue = [&](uint32_t i) {
    const uint32_t n0 = slice_pos(i);
    __half* kd = Ks + (size_t)(i % NST) * 2 * kSlice;
    __half* vd = kd + kSlice;
#pragma unroll
    for (int k = 0; k < PW * CPR / 32; ++k) {
      const int c = lane + k * 32;
      const int r = c / CPR, c8 = (c % CPR) * 8;
      const uint32_t pos = n0 + r;
      const bool in = pos < t1;
      const size_t row = (size_t)(in ? pos : 0u) * kvDim + c8;  // a valid address even when nothing is copied
      cp_async16((uint32_t)__cvta_generic_to_shared(kd + r * LD + c8), kbase + row, in ? 16u : 0u);
      cp_async16((uint32_t)__cvta_generic_to_shared(vd + r * LD + c8), vbase + row, in ? 16u : 0u);
    }
  };
  // The newest row (seq - 1) is written by the previous kernel of this step; every other row by earlier steps. The
  // slices that lie wholly before it are requested ahead of the dependency wait. One commit group per slice, in order.
  uint32_t issued = 0;
  for (; issued < NST - 1; ++issued) {
    if (issued < my_n && slice_pos(issued) + PW < seq) issue(issued);
    else break;
    cp_async_commit();
  }
  pdl_wait();  // q and the newest K/V row come from the previous kernel
  for (; issued < NST - 1; ++issued) {
    if (issued < my_n) issue(issued);
    cp_async_commit();  // (an empty group keeps the count uniform)
  }

  // Q fragments (A operand: 16 rows x 16 dims per k step; rows >= nh are zero), scaled into the base-2 domain and
  // split into head + remainder. Row qr of the tile is query head h0 + qr; rows 8..15 are always padding.
  const float qscale = (1.0f / sqrtf((float)D)) * 1.4426950408889634f;
  uint32_t qh[D / 16][4], ql[D / 16][4];
  {
    const bool real = (uint32_t)qr < nh;
    const float* qa = p.q + (size_t)(h0 + (real ? qr : 0)) * D;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const int c = kk * 16 + qc;
      const float2 a0 = real ? __ldcg(reinterpret_cast<const float2*>(qa + c)) : make_float2(0.f, 0.f);
      const float2 a1 = real ? __ldcg(reinterpret_cast<const float2*>(qa + c + 8)) : make_float2(0.f, 0.f);
      split_half2(a0.x * qscale, a0.y * qscale, qh[kk][0], ql[kk][0]);
      split_half2(a1.x * qscale, a1.y * qscale, qh[kk][2], ql[kk][2]);
      qh[kk][1] = ql[kk][1] = qh[kk][3] = ql[kk][3] = 0u;  // rows 8..15
    }
  }
  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m_a = kNegBig, l_a = 0.f;  // row qr (base-2 domain); rows 8..15 carry no state

  for (uint32_t i = 0; i < my_n; ++i) {
    // stage (i + NST - 1) % NST was read in iteration i - 1; every lane is past that read
    __syncwarp();
    if (i + NST - 1 < my_n) issue(i + NST - 1);
    cp_async_commit();
    cp_async_wait_all_but<NST - 1>();  // this lane's copies of slice i have landed
    __syncwarp();                      // ... and the other lanes'
    const uint32_t n0 = slice_pos(i);
    const uint32_t ks_s = ks_base + (uint32_t)((i % NST) * 2 * kSlice) * 2;
    const uint32_t vs_s = ks_s + (uint32_t)kSlice * 2;
    // ---- S = Q K^T : 16 rows x 16 positions
    float sc[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4(ks_s + (uint32_t)(kk * 16) * 2 + k_lane_off, b0, b1, b2, b3);
      mma_16816(sc[0], qh[kk], b0, b1);
      mma_16816(sc[0], ql[kk], b0, b1);
      mma_16816(sc[1], qh[kk], b2, b3);
      mma_16816(sc[1], ql[kk], b2, b3);
    }
    // ---- mask positions past the range (their K and V rows are zero-filled)
    if (n0 + PW > t1) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const uint32_t c = n0 + j * 8 + qc;
        if (c >= t1) sc[j][0] = -INFINITY;
        if (c + 1 >= t1) sc[j][1] = -INFINITY;
      }
    }
    // ---- online softmax of row qr (the slice's first position is inside the range: the maximum is finite)
    float mx = fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float mn = fmaxf(m_a, mx);
    const float al = m_ex2(m_a - mn);
    m_a = mn;
    uint32_t ph[4], pl[4];
    const float e0 = m_ex2(sc[0][0] - mn), e1 = m_ex2(sc[0][1] - mn), e2 = m_ex2(sc[1][0] - mn), e3 = m_ex2(sc[1][1] - mn);
    // accumulator layout of two neighbouring position tiles = A-operand layout of one 16-position k step
    split_half2(e0, e1, ph[0], pl[0]);
    split_half2(e2, e3, ph[2], pl[2]);
    ph[1] = pl[1] = ph[3] = pl[3] = 0u;  // rows 8..15
    l_a = l_a * al + (e0 + e1) + (e2 + e3);
    if (al != 1.0f) {  // the running maximum moved (rare once the range is under way)
#pragma unroll
      for (int j = 0; j < D / 8; ++j) {
        o[j][0] *= al;
        o[j][1] *= al;
      }
    }
    // ---- O += P V
#pragma unroll
    for (int j = 0; j < D / 8; j += 2) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4_trans(vs_s + (uint32_t)(j * 8) * 2 + v_lane_off, b0, b1, b2, b3);
      mma_16816(o[j], ph, b0, b1);
      mma_16816(o[j], pl, b0, b1);
      mma_16816(o[j + 1], ph, b2, b3);
      mma_16816(o[j + 1], pl, b2, b3);
    }
  }
  cp_async_wait_all_but<0>();

  // ---- merge. One routine adds rows of (unnormalised sums, m, l): first the rows of the eight warps, then -- in the
  // CTA that drew the last ticket of its (KV head, head group) -- the rows of all splits, copied from scratch into the
  // shared memory the stages occupied (L2-only 16-byte copies, all in flight at once). The routine is one piece of
  // code run by every CTA, so the last CTA finds it in the instruction caches; what only the last CTA runs (the copy
  // loop) is a few instructions. (Code run once per launch is fetched from HBM behind 67 MB of K and V: a merge that
  // unrolled its loads per split cost more in instruction fetch than it saved in round trips.)
  // Rows of head j lie STR floats apart from mrow0 + j * kRegion + (misalignment of the scratch rows, 0 or 2 floats);
  // two more rows per head carry the running result when the splits do not fit one pass.
  __syncthreads();  // every warp is past its last read of its stages
  float* const mbuf = reinterpret_cast<float*>(mma_smem);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  if ((uint32_t)qr < nh) {  // natural-log domain for the merge
    float* row = mbuf + qr * kRegion + warp * STR;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) *reinterpret_cast<float2*>(row + j * 8 + qc) = make_float2(o[j][0], o[j][1]);
    if ((lane & 3) == 0) {
      row[D] = m_a * 0.6931471805599453f;
      row[D + 1] = l_a;
    }
  }
  uint32_t cnt = kMW, k0 = 0, k_next = 0, carry_rd = 0;
  bool global_phase = false, has_carry = false;
#pragma unroll 1
  for (;;) {
    __syncthreads();  // the rows of this pass are in place
    const uint32_t n = cnt + (has_carry ? 1u : 0u);
    auto rowp = [&](uint32_t j, uint32_t r) -> const float* {
      const float* base = mbuf + j * kRegion;
      if (r >= cnt) return base + 4 + (kRowsMax + carry_rd) * STR;
      const uint32_t mis = global_phase ? (uint32_t)((((size_t)(h0 + j) * p.S_max + k0) * STR) & 3) : 0u;
      return base + mis + r * STR;
    };
    // (a warp, or a split, that saw no position holds m = kNegBig, l = 0: weight exp(-inf) = 0)
    if (warp < (int)nh) {  // warp j turns the m's of head j into weights, lanes along the rows
      static_assert(kRowsMax + 1 <= 96, "three rows per lane");
      float mr[3], M = kNegBig;
#pragma unroll
      for (int u = 0; u < 3; ++u) {
        const uint32_t r = lane + 32 * u;
        mr[u] = r < n ? rowp(warp, r)[D] : kNegBig;
        M = fmaxf(M, mr[u]);
      }
#pragma unroll
      for (int o2 = 16; o2 > 0; o2 >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o2));
      float Lsum = 0.f;
#pragma unroll
      for (int u = 0; u < 3; ++u) {
        const uint32_t r = lane + 32 * u;
        if (r < n) {
          const float scw = __expf(mr[u] - M);
          fin_scale[r][warp] = scw;
          Lsum = fmaf(rowp(warp, r)[D + 1], scw, Lsum);
        }
      }
      Lsum = warp_sum(Lsum);
      if (lane == 0) {
        fin_ML[warp][0] = M;
        fin_ML[warp][1] = Lsum;
      }
    }
    __syncthreads();
    const bool final_pass = global_phase ? k_next >= S_eff : S_eff == 1;
    const uint32_t carry_wr = has_carry ? carry_rd ^ 1u : 0u;
    for (int idx = tid; idx < (int)nh * D; idx += kMThreads) {
      const int j = idx / D, i = idx % D;
      float acc = 0.f;
#pragma unroll 4
      for (uint32_t r = 0; r < n; ++r) acc = fmaf(rowp(j, r)[i], fin_scale[r][j], acc);
      if (final_pass) p.out[(h0 + j) * D + i] = acc * (1.0f / fin_ML[j][1]);
      else if (!global_phase) p.part[((size_t)(h0 + j) * p.S_max + s) * STR + i] = acc;
      else mbuf[j * kRegion + 4 + (kRowsMax + carry_wr) * STR + i] = acc;
    }
    if (final_pass) break;
    if (!global_phase) {
      // several splits: publish the partial, the last CTA of this (kv head, head group) goes on
      if (tid < (int)nh) {
        float* pp = p.part + ((size_t)(h0 + tid) * p.S_max + s) * STR;
        pp[D] = fin_ML[tid][0];
        pp[D + 1] = fin_ML[tid][1];
      }
      __threadfence();
      __syncthreads();
      if (tid == 0) is_last = atomicAdd(&p.tickets[bx], 1u) == S_eff - 1 ? 1u : 0u;
      __syncthreads();
      if (!is_last) return;
      __threadfence();
      global_phase = true;
    } else {
      if (tid < (int)nh) {
        float* cr = mbuf + tid * kRegion + 4 + (kRowsMax + carry_wr) * STR;
        cr[D] = fin_ML[tid][0];
        cr[D + 1] = fin_ML[tid][1];
      }
      carry_rd = carry_wr;
      has_carry = true;
      __syncthreads();  // every thread is past its reads of this pass's rows
    }
    // the next rows of every head: whole 16-byte pieces around them (scratch rows are 8-byte aligned)
    k0 = k_next;
    cnt = min(S_eff - k_next, (uint32_t)kRowsMax);
    k_next += cnt;
    for (uint32_t j = 0; j < nh; ++j) {
      const size_t first = ((size_t)(h0 + j) * p.S_max + k0) * STR;
      const uint32_t mis = (uint32_t)(first & 3);
      const uint32_t pieces = (mis + cnt * STR + 3) / 4;
      const float* src = p.part + (first - mis);
      float* dst = mbuf + j * kRegion;
      for (uint32_t c = tid; c < pieces; c += kMThreads) cp_async16((uint32_t)__cvta_generic_to_shared(dst + 4 * c), src + 4 * c, 16u);
    }
    cp_async_commit();
    cp_async_wait_all_but<0>();
  }
  if (global_phase && tid == 0) p.tickets[bx] = 0;  // ready for the next launch
}

template <int D>
cudaError_t launch_mma_d(cudaStream_t s, const AttnParams& p, bool pdl) {
  constexpr int NST = D == 64 ? 4 : 2;
  constexpr size_t smem = (size_t)kMW * NST * 2 * 16 * (D + 8) * 2;  // per warp: NST stages of a K and a V slice
  static_assert(smem >= (size_t)kMG * (((64 + 2) * (D + 2) + 4 + 3) / 4 * 4) * 4, "the merge buffer reuses the stages");
  cudaError_t e = cudaFuncSetAttribute(attn_mma_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  return launch_pdl(attn_mma_kernel<D>, dim3(p.kvH * attn_head_groups(p.qH, p.kvH, kMG), p.S_max), dim3(kMThreads), smem, s,
                    pdl, p);
}

}  // namespace

bool attn_mma_supported(int kvdtype, uint32_t d) { return kvdtype == 1 && (d == 64 || d == 128); }

cudaError_t launch_attn_mma(cudaStream_t s, const AttnParams& p, bool pdl) {
  if (p.qH == 0 || p.kvH == 0 || p.qH % p.kvH != 0 || p.S_max == 0 || p.S_max > (uint32_t)attn_detail::kAttnMergeCap || p.out_half) return cudaErrorInvalidValue;
  if (!p.state && p.seq_imm == 0) return cudaErrorInvalidValue;
  if (((uintptr_t)p.kcache | (uintptr_t)p.vcache | (uintptr_t)p.part) & 15) return cudaErrorInvalidValue;
  switch (p.d) {
    case 64: return launch_mma_d<64>(s, p, pdl);
    case 128: return launch_mma_d<128>(s, p, pdl);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace nfai
