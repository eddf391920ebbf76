// Prompt-ingestion GEMM on the 5th-generation tensor cores: C[M][N] = A[M][K] * W[N][K]^T, A and W float16 with K
// contiguous, float32 accumulation in tensor memory. M = prompt tokens of a chunk, N = output features.
//
// The reference has no batched prompt path (it pushes prompt tokens through the single-token shaders one by one:
// NFAI.Models.Llama3/LlamaModel.cs:103-126); results must equal that token-by-token evaluation within the FP16
// tolerance, so the fused epilogues below are the same ones the decode GEMVs use (RoPE + cache write, SiLU*up,
// residual add) applied row by row.
//
// Shape of one CTA (192 threads, one 128 x BN output tile):
//   warp 0      producer: one lane issues TMA tile loads (A 128x64, W BNx64 halves, 128-byte swizzle) into a ring of
//               shared-memory stages, completion counted on the stage's "full" mbarrier;
//   warp 1      MMA: allocates BN tensor-memory columns; one lane waits for a full stage, issues four
//               tcgen05.mma (K = 16 each) from shared-memory descriptors, and commits to the stage's "empty"
//               mbarrier so that the producer may refill it; after the last stage it commits to "accumulator ready";
//   warps 2-5   epilogue: each reads its 32 accumulator rows with tcgen05.ld and applies the epilogue.
// No cluster-wide delivery is used anywhere. Every mbarrier wait is bounded (one second): on a time-out the role
// records an error bit and leaves; the tensor memory is released on every path.
#include <cuda.h>

#include "common.cuh"
#include "gemm_tc.h"
#include "kernels.h"

#include <stdlib.h>

#include <functional>
#include <type_traits>
#include <unordered_map>

namespace nfai {

namespace {

constexpr int kBM = 128;
constexpr int kBK = 64;  // halves per stage row = 128 bytes = one swizzle span
constexpr int kGemmThreads = 192;
constexpr unsigned long long kGemmWaitNs = 1000000000ull;

__device__ __forceinline__ unsigned long long g_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t s_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_try(uint32_t bar, uint32_t parity) {
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
// Bounded wait; false after one second.
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity) {
  if (bar_try(bar, parity)) return true;
  const unsigned long long t0 = g_ns();
  uint32_t polls = 0;
  while (!bar_try(bar, parity)) {
    if ((++polls & 63u) == 0 && g_ns() - t0 > kGemmWaitNs) return false;
  }
  return true;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);   // start address, 16-byte units
  d |= (uint64_t)1 << 16;                     // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;           // stride byte offset: next 8-row group
  d |= (uint64_t)1 << 46;                     // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                     // layout: 128-byte swizzle
  return d;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,"
      "%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// ---- epilogues: two adjacent output columns (n, n+1) of row m; n is even -----------------------------------------
// What the epilogue of a pair reads from memory: the residual pair of a plain store, the (cos, sin) of a rotated Q/K
// pair. The callers fetch it for a whole block of pairs before they touch the accumulators: a loop of load -> add ->
// store per pair runs at one memory round trip per pair (the store may alias the next load as far as the compiler
// knows), which cost more than the tile's MMAs.
// KIND >= 0 fixes the epilogue at compile time (the persistent kernel dispatches once per tile); -1 reads ep.kind.
template <int KIND = -1>
__device__ __forceinline__ float2 epilogue_aux(const GemmEpilogue& ep, uint32_t m, uint32_t n, uint32_t N) {
  switch (KIND >= 0 ? KIND : (int)ep.kind) {
    case GEMM_EPI_STORE: {
      if (!ep.resid) break;
      const float* res = ep.resid + (size_t)m * N;
      if ((N & 1u) == 0) return __ldcg(reinterpret_cast<const float2*>(res + n));
      return make_float2(__ldcg(res + n), n + 1 < N ? __ldcg(res + n + 1) : 0.f);
    }
    case GEMM_EPI_QKV_ROPE: {
      if (n < ep.qDim + ep.kvDim) {
        const uint32_t local = n < ep.qDim ? n : n - ep.qDim;
        const uint32_t e = local % ep.d;
        if (e < ep.ropeDim) return ep.rope_cs[(size_t)(ep.pos0 + m) * (ep.ropeDim / 2) + (e >> 1)];
      }
      break;
    }
    default: break;
  }
  return make_float2(0.f, 0.f);
}

template <int KIND = -1>
__device__ __forceinline__ void epilogue_pair(const GemmEpilogue& ep, uint32_t m, uint32_t n, uint32_t N, float a, float b,
                                              const float2 aux) {
  switch (KIND >= 0 ? KIND : (int)ep.kind) {
    case GEMM_EPI_STORE: {
      float* out = ep.out_f32 + (size_t)m * N;
      if ((N & 1u) == 0) {  // rows start on an 8-byte boundary: one store per pair
        float2 r = make_float2(a, b);
        if (ep.resid) {
          r.x += aux.x;
          r.y += aux.y;
        }
        *reinterpret_cast<float2*>(out + n) = r;
      } else {
        out[n] = ep.resid ? aux.x + a : a;
        if (n + 1 < N) out[n + 1] = ep.resid ? aux.y + b : b;
      }
      break;
    }
    case GEMM_EPI_SILU_MUL: {  // columns (2j, 2j+1) = (gate_j, up_j); h_j = up * silu(gate), stored as float16
      if (n + 1 < N) {
        const float sig = __fdiv_rn(1.0f, 1.0f + expf(-a));
        ep.out_f16[(size_t)m * (N / 2) + (n >> 1)] = __float2half_rn(__fmul_rn(b, __fmul_rn(a, sig)));
      }
      break;
    }
    case GEMM_EPI_QKV_ROPE: {  // columns [Q | K | V]; RoPE on adjacent pairs at position pos0 + m
      const uint32_t pos = ep.pos0 + m;
      if (n < ep.qDim + ep.kvDim) {
        const uint32_t local = n < ep.qDim ? n : n - ep.qDim;
        const uint32_t e = local % ep.d;
        if (e < ep.ropeDim) {
          const float2 cs = aux;
          const float v1 = __fsub_rn(__fmul_rn(cs.x, a), __fmul_rn(cs.y, b));
          const float v2 = __fadd_rn(__fmul_rn(cs.y, a), __fmul_rn(cs.x, b));
          a = v1;
          b = v2;
        }
        if (n < ep.qDim) {
          // (n, local and the row lengths are even: pairs are naturally aligned)
          *reinterpret_cast<float2*>(ep.out_f32 + (size_t)m * ep.qDim + n) = make_float2(a, b);
        } else if (ep.kv_f16) {
          __half* kc = reinterpret_cast<__half*>(ep.kcache) + (size_t)pos * ep.kvDim + local;
          *reinterpret_cast<__half2*>(kc) = __floats2half2_rn(a, b);
        } else {
          float* kc = reinterpret_cast<float*>(ep.kcache) + (size_t)pos * ep.kvDim + local;
          kc[0] = a;
          kc[1] = b;
        }
      } else {
        const uint32_t local = n - ep.qDim - ep.kvDim;
        if (ep.kv_f16) {
          __half* vc = reinterpret_cast<__half*>(ep.vcache) + (size_t)pos * ep.kvDim + local;
          *reinterpret_cast<__half2*>(vc) = __floats2half2_rn(a, b);
        } else {
          float* vc = reinterpret_cast<float*>(ep.vcache) + (size_t)pos * ep.kvDim + local;
          vc[0] = a;
          vc[1] = b;
        }
      }
      break;
    }
  }
}

// 32 consecutive output columns [n0, n0+32) of row m (n0 is a multiple of 32)
__device__ __forceinline__ void epilogue_cols(const GemmEpilogue& ep, uint32_t m, uint32_t n0, uint32_t N, const float (&v)[32]) {
  float2 aux[16];
#pragma unroll
  for (int i = 0; i < 32; i += 2) aux[i >> 1] = n0 + i < N ? epilogue_aux(ep, m, n0 + i, N) : make_float2(0.f, 0.f);
#pragma unroll
  for (int i = 0; i < 32; i += 2)
    if (n0 + i < N) epilogue_pair(ep, m, n0 + i, N, v[i], v[i + 1], aux[i >> 1]);
}

// Split-K: raw partial sums of the same 32 columns into [split][M][N]
__device__ __forceinline__ void partial_cols(float* part, uint32_t m, uint32_t n0, uint32_t N, const float (&v)[32]) {
  float* out = part + (size_t)m * N + n0;
#pragma unroll
  for (int i = 0; i < 32; ++i)
    if (n0 + i < N) out[i] = v[i];
}

// Second kernel of a split GEMM: one thread per column pair adds the partials in split order and applies the epilogue.
__global__ void __launch_bounds__(256) gemm_finish_kernel(const float* __restrict__ part, uint32_t M, uint32_t N, uint32_t Z,
                                                          const GemmEpilogue ep) {
  pdl_launch_dependents();
  pdl_wait();  // the partial tiles come from the GEMM launched just before
  const uint32_t pairs = (N + 1) / 2;
  const size_t total = (size_t)M * pairs;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const uint32_t m = (uint32_t)(idx / pairs), n = (uint32_t)(idx % pairs) * 2;
    float a = 0.f, b = 0.f;
    for (uint32_t z = 0; z < Z; ++z) {
      const float* p = part + ((size_t)z * M + m) * N + n;
      a += p[0];
      if (n + 1 < N) b += p[1];
    }
    epilogue_pair(ep, m, n, N, a, b, epilogue_aux(ep, m, n, N));
  }
}

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr uint32_t kABytes = kBM * kBK * 2;
  static constexpr uint32_t kBBytes = BN * kBK * 2;
  static constexpr uint32_t kStage = kABytes + kBBytes;
  static constexpr uint32_t kBarOff = STAGES * kStage;
  static constexpr uint32_t kTotal = kBarOff + 256 + 1024;  // barriers + slack for the 1024-byte alignment
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(kGemmThreads) gemm_tc_kernel(const __grid_constant__ CUtensorMap mapA,
                                                               const __grid_constant__ CUtensorMap mapW, uint32_t M,
                                                               uint32_t N, uint32_t K, const GemmEpilogue ep,
                                                               uint32_t* err) {
  using SM = GemmSmem<BN, STAGES>;
  extern __shared__ unsigned char gsm_raw[];
  unsigned char* gsm = reinterpret_cast<unsigned char*>(((uintptr_t)gsm_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(gsm + SM::kBarOff);
  // bars[0..STAGES) full, [STAGES..2*STAGES) empty, [2*STAGES] accumulator ready; then the TMEM base address word
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
  const uint32_t full0 = s_u32(bars), empty0 = s_u32(bars + STAGES), accbar = s_u32(bars + 2 * STAGES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t m0 = blockIdx.y * kBM, n0 = blockIdx.x * BN;
  // this CTA's share of the K tiles (split-K: blockIdx.z of gridDim.z; every share holds at least one tile)
  const uint32_t KT_all = (K + kBK - 1) / kBK;
  const uint32_t kt0 = (uint32_t)((uint64_t)KT_all * blockIdx.z / gridDim.z);
  const uint32_t KT = (uint32_t)((uint64_t)KT_all * (blockIdx.z + 1) / gridDim.z) - kt0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      bar_init(full0 + 8 * s, 1);
      bar_init(empty0 + 8 * s, 1);
    }
    bar_init(accbar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // the MMA warp owns the tensor-memory allocation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_u32(tmem_slot)), "r"((uint32_t)BN)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;
  // barriers and tensor memory are set up; the operands (and the residual) come from the previous kernel
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      for (uint32_t kt = 0; kt < KT; ++kt) {
        const uint32_t s = kt % STAGES;
        if (kt >= (uint32_t)STAGES) {
          if (!bar_wait(empty0 + 8 * s, ((kt / STAGES) - 1) & 1)) { ok = false; break; }
        }
        const uint32_t a_dst = s_u32(gsm + s * SM::kStage), b_dst = a_dst + SM::kABytes;
        bar_expect_tx(full0 + 8 * s, SM::kABytes + SM::kBBytes);
        tma_load_2d(a_dst, &mapA, (int)((kt0 + kt) * kBK), (int)m0, full0 + 8 * s);
        tma_load_2d(b_dst, &mapW, (int)((kt0 + kt) * kBK), (int)n0, full0 + 8 * s);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // instruction descriptor: D float32, A and B float16, both K-major, N = BN, M = 128
      const uint32_t idesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
      for (uint32_t kt = 0; kt < KT; ++kt) {
        const uint32_t s = kt % STAGES;
        if (!bar_wait(full0 + 8 * s, (kt / STAGES) & 1)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_s = s_u32(gsm + s * SM::kStage), b_s = a_s + SM::kABytes;
#pragma unroll
        for (int k = 0; k < kBK / 16; ++k) {
          umma_f16(tmem_base, smem_desc_sw128(a_s + k * 32), smem_desc_sw128(b_s + k * 32), idesc, (kt | (uint32_t)k) != 0);
        }
        umma_commit(empty0 + 8 * s);  // arrives when the MMAs above have finished reading the stage
      }
      if (ok) umma_commit(accbar);
    }
  } else {
    // epilogue warps 2..5: warp w may touch tensor-memory lanes 32*(w%4) .. +31
    const uint32_t lane_grp = (uint32_t)(warp & 3);
    ok = bar_wait(accbar, 0);
    ok = __all_sync(0xffffffffu, ok);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
      const uint32_t m = m0 + lane_grp * 32 + lane;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        float v[32];
        tmem_ld32(tmem_base + ((lane_grp * 32u) << 16) + (uint32_t)c * 32u, v);
        if (m < M && n0 + c * 32 < N) {
          if (gridDim.z > 1) partial_cols(ep.scratch + (size_t)blockIdx.z * M * N, m, n0 + c * 32, N, v);
          else epilogue_cols(ep, m, n0 + c * 32, N, v);
        }
      }
    }
  }
  if (!ok) {
    if (lane == 0 && err) atomicOr(err, 4u);
    // tile copies of this CTA may still be in flight: give them a bounded time to land before shared memory and
    // tensor memory are released
    for (volatile uint32_t spin = 0; spin < (1u << 20); ++spin) {
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)BN) : "memory");
  }
}

// ---- persistent variant: 128 x 256 tiles, two accumulators in tensor memory ------------------------------------
// A 128 x 128 tile needs 32 KB of operands per 262 tensor-pipe cycles (125 B/clk per SM, about what L2 delivers), so
// the kernel above is fed at half speed; a 128 x 256 tile needs 48 KB per 524 cycles. One CTA per SM walks tiles
// blockIdx.x, + gridDim.x, ... (token tiles fastest, so that CTAs running together share one weight tile); the
// accumulator alternates between two 256-column halves of tensor memory, so the epilogue of tile i (tcgen05.ld,
// fused epilogue, global stores) runs while the tensor pipe is already on tile i + 1.
constexpr int kPBN = 256;
constexpr int kPStages = 4;
struct PSmem {
  static constexpr uint32_t kABytes = kBM * kBK * 2;
  static constexpr uint32_t kBBytes = kPBN * kBK * 2;
  static constexpr uint32_t kStage = kABytes + kBBytes;
  static constexpr uint32_t kBarOff = kPStages * kStage;
  static constexpr uint32_t kEpiOff = kBarOff + 256;             // 8 warps x 32 x 33 floats: accumulator block turned
  static constexpr uint32_t kEpiBytes = 8 * 32 * 33 * 4;         // so that lanes run along a row of the output
  static constexpr uint32_t kTotal = kEpiOff + kEpiBytes + 1024;
};

__device__ __forceinline__ void bar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Eight epilogue warps, two per quarter of the tensor-memory lanes (a warp may only read the lanes of its index modulo 4),
// each pair sharing the column blocks of its rows: with one warp per scheduler the SiLU epilogue (an exponential and
// an IEEE division per output) ran at the latency of its dependent instructions and took longer than the tile's MMAs.
constexpr int kPThreadsGemm = 64 + 8 * 32;
static_assert(PSmem::kTotal <= 227 * 1024, "shared memory of the persistent kernel");
__global__ void __launch_bounds__(kPThreadsGemm) gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap mapA,
                                                                          const __grid_constant__ CUtensorMap mapW, uint32_t M,
                                                                          uint32_t N, uint32_t K, const GemmEpilogue ep,
                                                                          uint32_t* err) {
  using SM = PSmem;
  constexpr int STAGES = kPStages;
  extern __shared__ unsigned char gsm_raw[];
  unsigned char* gsm = reinterpret_cast<unsigned char*>(((uintptr_t)gsm_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(gsm + SM::kBarOff);
  // bars: [0, S) full, [S, 2S) empty, [2S, 2S+2) accumulator full, [2S+2, 2S+4) accumulator empty; then the TMEM base word
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  const uint32_t full0 = s_u32(bars), empty0 = s_u32(bars + STAGES), tfull0 = s_u32(bars + 2 * STAGES),
                 tempty0 = s_u32(bars + 2 * STAGES + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t KT = (K + kBK - 1) / kBK;
  const uint32_t mtiles = (M + kBM - 1) / kBM, ntiles = (N + kPBN - 1) / kPBN, tiles = mtiles * ntiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      bar_init(full0 + 8 * s, 1);
      bar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      bar_init(tfull0 + 8 * a, 1);
      bar_init(tempty0 + 8 * a, 8);  // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;
  // barriers and tensor memory are set up; the operands (and the residual) come from the previous kernel
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      for (uint32_t tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        const uint32_t m0 = (tile % mtiles) * kBM, n0 = (tile / mtiles) * kPBN;
        for (uint32_t kt = 0; kt < KT; ++kt, ++it) {
          const uint32_t s = it % STAGES;
          if (it >= (uint32_t)STAGES) {
            if (!bar_wait(empty0 + 8 * s, ((it / STAGES) - 1) & 1)) { ok = false; break; }
          }
          const uint32_t a_dst = s_u32(gsm + s * SM::kStage), b_dst = a_dst + SM::kABytes;
          bar_expect_tx(full0 + 8 * s, SM::kABytes + SM::kBBytes);
          tma_load_2d(a_dst, &mapA, (int)(kt * kBK), (int)m0, full0 + 8 * s);
          tma_load_2d(b_dst, &mapW, (int)(kt * kBK), (int)n0, full0 + 8 * s);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | ((uint32_t)(kPBN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
      uint32_t it = 0, i = 0;
      for (uint32_t tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++i) {
        const uint32_t acc = i & 1;
        if (i >= 2) {  // the epilogue must have drained this half of tensor memory (tile i - 2)
          if (!bar_wait(tempty0 + 8 * acc, ((i >> 1) - 1) & 1)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        const uint32_t d = tmem_base + acc * (uint32_t)kPBN;
        for (uint32_t kt = 0; kt < KT; ++kt, ++it) {
          const uint32_t s = it % STAGES;
          if (!bar_wait(full0 + 8 * s, (it / STAGES) & 1)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_s = s_u32(gsm + s * SM::kStage), b_s = a_s + SM::kABytes;
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            umma_f16(d, smem_desc_sw128(a_s + k * 32), smem_desc_sw128(b_s + k * 32), idesc, (kt | (uint32_t)k) != 0);
          }
          umma_commit(empty0 + 8 * s);
        }
        if (ok) umma_commit(tfull0 + 8 * acc);
      }
    }
  } else {
    const uint32_t lane_grp = (uint32_t)(warp & 3);
    uint32_t i = 0;
    for (uint32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++i) {
      const uint32_t acc = i & 1;
      const uint32_t m0 = (tile % mtiles) * kBM, n0 = (tile / mtiles) * kPBN;
      // this lane's 16 pairs of a 32 x 32 block: lanes 0-15 along the column pairs of one row, lanes 16-31 on the next
      const uint32_t col = 2u * (lane & 15);
      float* eb = reinterpret_cast<float*>(gsm + SM::kEpiOff) + (warp - 2) * (32 * 33);
      // One instance per epilogue kind, chosen once per tile: the loops below are straight-line code for that kind.
      auto tile_epilogue = [&](auto kind_c) -> bool {
        constexpr int KIND = decltype(kind_c)::value;
        constexpr bool kAux = KIND != GEMM_EPI_SILU_MUL;  // residual pairs / (cos, sin) pairs come from memory
        float2 aux[16];
        // Q/K/V columns: everything that depends on the column only (which of Q, K, V; the position inside the head;
        // whether the pair is rotated) is the same for the 16 pairs of a lane in one block and is worked out once.
        struct ColInfo {
          uint32_t seg, local, half_e;  // 0 = Q, 1 = K, 2 = V; column inside the segment; index into a (cos, sin) row
          bool rot, live;
        };
        auto col_info = [&](int c) {
          ColInfo ci;
          const uint32_t n = n0 + c * 32 + col;
          ci.live = n < N;
          ci.seg = n < ep.qDim ? 0u : n < ep.qDim + ep.kvDim ? 1u : 2u;
          ci.local = n - (ci.seg == 0 ? 0u : ci.seg == 1 ? ep.qDim : ep.qDim + ep.kvDim);
          const uint32_t e = ci.local & (ep.d - 1);  // head dimensions are powers of two (32, 64, 128)
          ci.rot = ci.seg < 2 && e < ep.ropeDim;
          ci.half_e = e >> 1;
          return ci;
        };
        auto load_aux = [&](int c) {
          if constexpr (KIND == GEMM_EPI_QKV_ROPE) {
            const ColInfo ci = col_info(c);
            const float2* cs = ep.rope_cs + (size_t)(ep.pos0 + m0 + lane_grp * 32 + (lane >> 4)) * (ep.ropeDim / 2) + ci.half_e;
#pragma unroll
            for (int rr = 0; rr < 16; ++rr) {
              const uint32_t m = m0 + lane_grp * 32 + 2u * rr + (lane >> 4);
              aux[rr] = ci.rot && ci.live && m < M ? cs[(size_t)(2 * rr) * (ep.ropeDim / 2)] : make_float2(1.f, 0.f);
            }
          } else if constexpr (kAux) {
#pragma unroll
            for (int rr = 0; rr < 16; ++rr) {
              const uint32_t m = m0 + lane_grp * 32 + 2u * rr + (lane >> 4), n = n0 + c * 32 + col;
              aux[rr] = m < M && n < N ? epilogue_aux<KIND>(ep, m, n, N) : make_float2(0.f, 0.f);
            }
          }
        };
        const int c_first = (warp - 2) >> 2;  // this warp's column blocks: c_first, c_first + 2, ...
        load_aux(c_first);  // on its way while the tensor pipe still works on this tile
        bool good = bar_wait(tfull0 + 8 * acc, (i >> 1) & 1);
        good = __all_sync(0xffffffffu, good);
        if (!good) return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // tcgen05.ld hands every lane one accumulator row; stores along a row would touch 32 different rows per
        // instruction. The 32 x 32 block goes through shared memory (row stride 33: conflict-free both ways) and comes
        // back with lanes 0-15 on the column pairs of one row and lanes 16-31 on the next row: 128-byte coalesced rows.
#pragma unroll 1
        for (int c = c_first; c < kPBN / 32; c += 2) {
          float v[32];
          tmem_ld32(tmem_base + ((lane_grp * 32u) << 16) + acc * (uint32_t)kPBN + (uint32_t)c * 32u, v);
          const bool live = m0 + lane_grp * 32 < M && n0 + c * 32 < N;  // warp-uniform
          if (live) {
#pragma unroll
            for (int e = 0; e < 32; ++e) eb[lane * 33 + e] = v[e];
            __syncwarp();
          }
          float2 cur[16];
          if constexpr (kAux) {
#pragma unroll
            for (int rr = 0; rr < 16; ++rr) cur[rr] = aux[rr];
            if (c + 2 < kPBN / 32) load_aux(c + 2);  // the next block's reads are in flight during this block's stores
          }
          if constexpr (KIND == GEMM_EPI_QKV_ROPE) {
            if (live) {
              const ColInfo ci = col_info(c);
              const uint32_t mrow = m0 + lane_grp * 32 + (lane >> 4);  // rows mrow, mrow + 2, ...
              if (ci.live) {
                // destination of row mrow; the next pair of this lane lies two rows (positions) further on
                float* qd = ep.out_f32 + (size_t)mrow * ep.qDim + ci.local;
                const size_t kvoff = (size_t)(ep.pos0 + mrow) * ep.kvDim + ci.local;
                void* const cache = ci.seg == 1 ? ep.kcache : ep.vcache;
#pragma unroll
                for (int rr = 0; rr < 16; ++rr) {
                  const uint32_t row = 2u * rr + (lane >> 4);
                  if (mrow + 2u * rr >= M) break;
                  float a = eb[row * 33 + col], b = eb[row * 33 + col + 1];
                  if (ci.rot) {  // value1 = cos*a - sin*b ; value2 = sin*a + cos*b, products rounded separately
                    const float2 cs = cur[rr];
                    const float v1 = __fsub_rn(__fmul_rn(cs.x, a), __fmul_rn(cs.y, b));
                    const float v2 = __fadd_rn(__fmul_rn(cs.y, a), __fmul_rn(cs.x, b));
                    a = v1;
                    b = v2;
                  }
                  if (ci.seg == 0) {
                    *reinterpret_cast<float2*>(qd + (size_t)(2 * rr) * ep.qDim) = make_float2(a, b);
                  } else if (ep.kv_f16) {
                    *reinterpret_cast<__half2*>(reinterpret_cast<__half*>(cache) + kvoff + (size_t)(2 * rr) * ep.kvDim) =
                        __floats2half2_rn(a, b);
                  } else {
                    *reinterpret_cast<float2*>(reinterpret_cast<float*>(cache) + kvoff + (size_t)(2 * rr) * ep.kvDim) =
                        make_float2(a, b);
                  }
                }
              }
              __syncwarp();
            }
          } else if (live) {
#pragma unroll
            for (int rr = 0; rr < 16; ++rr) {
              const uint32_t row = 2u * rr + (lane >> 4);
              const uint32_t m = m0 + lane_grp * 32 + row, n = n0 + c * 32 + col;
              if (m < M && n < N)
                epilogue_pair<KIND>(ep, m, n, N, eb[row * 33 + col], eb[row * 33 + col + 1], kAux ? cur[rr] : make_float2(0.f, 0.f));
            }
            __syncwarp();
          }
        }
        return true;
      };
      switch (ep.kind) {
        case GEMM_EPI_STORE: ok = tile_epilogue(std::integral_constant<int, (int)GEMM_EPI_STORE>{}); break;
        case GEMM_EPI_SILU_MUL: ok = tile_epilogue(std::integral_constant<int, (int)GEMM_EPI_SILU_MUL>{}); break;
        default: ok = tile_epilogue(std::integral_constant<int, (int)GEMM_EPI_QKV_ROPE>{}); break;
      }
      if (!ok) break;
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) bar_arrive(tempty0 + 8 * acc);
    }
  }
  if (!ok) {
    if (lane == 0 && err) atomicOr(err, 4u);
    // tile copies of this CTA may still be in flight: give them a bounded time to land before shared memory and
    // tensor memory are released
    for (volatile uint32_t spin = 0; spin < (1u << 20); ++spin) {
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ---- small producers of the float16 A operands ----------------------------------------------------------------
__global__ void __launch_bounds__(256) rmsnorm_to_half_kernel(const float* __restrict__ x, const float* __restrict__ gain,
                                                              float eps, uint32_t H, __half* __restrict__ out) {
  __shared__ float red[8];
  pdl_launch_dependents();
  pdl_wait();
  const float* xr = x + (size_t)blockIdx.x * H;
  float ss = 0.f;
  for (uint32_t i = threadIdx.x; i < H; i += 256) ss = fmaf(xr[i], xr[i], ss);
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) tot += red[w];
  const float rms = sqrtf(__fdiv_rn(tot, (float)H) + eps);
  __half* o = out + (size_t)blockIdx.x * H;
  for (uint32_t i = threadIdx.x; i < H; i += 256) o[i] = __float2half_rn(__fmul_rn(__fdiv_rn(xr[i], rms), gain[i]));
}

__global__ void embed_rows_kernel(const __half* __restrict__ E, const uint32_t* __restrict__ tokens, uint32_t H,
                                  float* __restrict__ x) {
  pdl_launch_dependents();
  pdl_wait();
  const __half* row = E + (size_t)tokens[blockIdx.x] * H;
  float* o = x + (size_t)blockIdx.x * H;
  for (uint32_t i = threadIdx.x; i < H; i += blockDim.x) o[i] = __half2float(row[i]);
}

__global__ void float_to_half_kernel(const float* __restrict__ in, __half* __restrict__ out, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = __float2half_rn(in[i]);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || !p) return nullptr;
  fn = (EncodeTiledFn)p;
  return fn;
}

// [rows][K] float16, K contiguous; box = 64 halves x box_rows rows, 128-byte swizzle, zero fill outside.
// A descriptor depends only on (address, rows, K, box rows); a prompt re-uses the same few hundred of them for every
// chunk, so they are kept per host thread instead of being encoded again at each of ~130 launches per chunk.
struct MapKey {
  const void* base;
  uint64_t rows, K;
  uint32_t box_rows;
  bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows && K == o.K && box_rows == o.box_rows; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<uint64_t>()((uint64_t)(uintptr_t)k.base ^ (k.rows * 0x9E3779B97F4A7C15ull) ^ (k.K << 20) ^ k.box_rows);
  }
};

bool make_map(CUtensorMap* map, const __half* base, uint64_t rows, uint64_t K, uint32_t box_rows) {
  static thread_local std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{base, rows, K, box_rows};
  auto it = cache.find(key);
  if (it != cache.end()) {
    *map = it->second;
    return true;
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {K * 2};
  cuuint32_t box[2] = {(cuuint32_t)kBK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  if (fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *map);
  return true;
}

template <int BN, int STAGES>
cudaError_t launch_bn(cudaStream_t s, const __half* A, const __half* W, uint32_t M, uint32_t N, uint32_t K,
                      const GemmEpilogue& ep, uint32_t* err, uint32_t Z = 1) {
  CUtensorMap mapA, mapW;
  if (!make_map(&mapA, A, M, K, kBM) || !make_map(&mapW, W, N, K, BN)) return cudaErrorInvalidValue;
  auto kern = gemm_tc_kernel<BN, STAGES>;
  const size_t smem = GemmSmem<BN, STAGES>::kTotal;
  static thread_local int attr_device = -1;  // the attribute is per device: set it once per (thread, device)
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (attr_device != dev) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    attr_device = dev;
  }
  dim3 grid((N + BN - 1) / BN, (M + kBM - 1) / kBM, Z);
  e = launch_pdl(kern, grid, dim3(kGemmThreads), smem, s, prefill_pdl(), mapA, mapW, M, N, K, ep, err);
  if (e != cudaSuccess || Z == 1) return e;
  const size_t pairs = (size_t)M * ((N + 1) / 2);
  const size_t want = (pairs + 255) / 256;
  return launch_pdl(gemm_finish_kernel, dim3((unsigned)(want < 1184 ? want : 1184)), dim3(256), 0, s, prefill_pdl(),
                    (const float*)ep.scratch, M, N, Z, ep);
}

cudaError_t launch_persistent(cudaStream_t s, const __half* A, const __half* W, uint32_t M, uint32_t N, uint32_t K,
                              const GemmEpilogue& ep, uint32_t* err) {
  CUtensorMap mapA, mapW;
  if (!make_map(&mapA, A, M, K, kBM) || !make_map(&mapW, W, N, K, kPBN)) return cudaErrorInvalidValue;
  static thread_local int attr_device = -1;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (attr_device != dev) {
    e = cudaFuncSetAttribute(gemm_tc_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PSmem::kTotal);
    if (e != cudaSuccess) return e;
    attr_device = dev;
  }
  const uint32_t tiles = ((M + kBM - 1) / kBM) * ((N + kPBN - 1) / kPBN);
  return launch_pdl(gemm_tc_persistent_kernel, dim3(tiles < sm_count() ? tiles : sm_count()), dim3(kPThreadsGemm), PSmem::kTotal, s,
                    prefill_pdl(), mapA, mapW, M, N, K, ep, err);
}

}  // namespace

// A tile grid of fewer than 120 CTAs of 128 x 128 leaves SMs without work (a chunk of <= 128 prompt tokens times a
// 2048-column matrix is 16 tiles): divide K so that about one CTA per SM streams weights, at least two K tiles each.
uint32_t gemm_tc_splits(uint32_t M, uint32_t N, uint32_t K) {
  const uint32_t tiles = ((M + kBM - 1) / kBM) * ((N + 127) / 128);
  const uint32_t KT = (K + kBK - 1) / kBK;
  if (tiles >= 120) return 1;
  uint32_t z = sm_count() / tiles;
  if (z > KT / 2) z = KT / 2;
  if (z > 16) z = 16;
  return z < 1 ? 1 : z;
}

cudaError_t launch_gemm_tc(cudaStream_t s, const __half* A, const __half* W, uint32_t M, uint32_t N, uint32_t K,
                           const GemmEpilogue& ep, uint32_t* err) {
  if (!A || !W || !M || !N || !K || (K & 7u) || (((uintptr_t)A | (uintptr_t)W) & 15)) return cudaErrorInvalidValue;
  if ((ep.kind == GEMM_EPI_SILU_MUL || ep.kind == GEMM_EPI_QKV_ROPE) && (N & 1u)) return cudaErrorInvalidValue;
  // enough CTAs to pull weights with every SM when the chunk is a single row of tiles
  const uint32_t mtiles = (M + kBM - 1) / kBM;
  // enough 128 x 256 tiles to occupy most SMs: the persistent kernel (NFAI_GEMM_PERSISTENT=0 keeps the tile-per-CTA one)
  static const bool persistent_ok = [] { const char* v = getenv("NFAI_GEMM_PERSISTENT"); return !(v && atoi(v) == 0); }();
  if (persistent_ok && mtiles * ((N + 255) / 256) >= 96) return launch_persistent(s, A, W, M, N, K, ep, err);
  if (ep.scratch) {
    uint32_t Z = gemm_tc_splits(M, N, K);
    while (Z > 1 && (size_t)Z * M * N > ep.scratch_floats) --Z;
    if (Z > 1) return launch_bn<128, 4>(s, A, W, M, N, K, ep, err, Z);
  }
  if (mtiles * ((N + 127) / 128) >= 120) return launch_bn<128, 4>(s, A, W, M, N, K, ep, err);
  if (mtiles * ((N + 63) / 64) >= 120) return launch_bn<64, 6>(s, A, W, M, N, K, ep, err);
  return launch_bn<32, 8>(s, A, W, M, N, K, ep, err);
}

bool prefill_pdl() {
  static const bool on = [] { const char* v = getenv("NFAI_PREFILL_PDL"); return !(v && atoi(v) == 0); }();
  return on;
}

cudaError_t launch_rmsnorm_to_half(cudaStream_t s, const float* x, const float* gain, float eps, uint32_t M, uint32_t H,
                                   __half* out, bool after_collective) {
  return launch_pdl(rmsnorm_to_half_kernel, dim3(M), dim3(256), 0, s, prefill_pdl() && !after_collective, x, gain, eps, H, out);
}

cudaError_t launch_embed_rows(cudaStream_t s, const __half* E, const uint32_t* tokens, uint32_t M, uint32_t H, float* x) {
  return launch_pdl(embed_rows_kernel, dim3(M), dim3(256), 0, s, prefill_pdl(), E, tokens, H, x);
}

cudaError_t launch_float_to_half(cudaStream_t s, const float* in, __half* out, size_t n) {
  size_t want = (n + 255) / 256;
  float_to_half_kernel<<<(unsigned)(want < 2368 ? want : 2368), 256, 0, s>>>(in, out, n);
  return cudaGetLastError();
}

}  // namespace nfai
