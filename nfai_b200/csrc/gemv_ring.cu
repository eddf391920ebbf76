// Decode GEMV with the weight stream staged through shared-memory rings by bulk asynchronous copies (TMA, 1-D).
//
// Why: at batch 1 every matrix of a layer is a 1-10 microsecond stream, so what decides the step time is whether
// HBM keeps streaming across kernel boundaries. Bulk copies hold the bytes in flight in shared memory, not in
// registers and not in L1 lines, so a CTA of 256 threads with ~100 KB of ring takes under half of an SM and the
// kernels of the step overlap in pairs: while kernel k computes, the CTAs of kernel k+1 (started early by
// programmatic dependent launch) are already resident, have asked for their first ~100 KB of weights per SM and only
// then wait for kernel k's output. A short matrix (the O projection: 57 KB per SM) is on chip in full before its
// input exists.
//
// Shape: the row blocks (R = 2 rows) are dealt to the CTAs in contiguous, equal shares; inside a CTA the blocks go
// round-robin to eight warps. Each warp owns a private ring of S stages of 2 rows x 2 KB: lane 0 arms the stage's
// mbarrier with the byte count and issues one bulk copy per row; all lanes wait on the mbarrier phase, read the
// stage with 16-byte shared loads, FMA against x (float32) and lane 0 refills the stage. No barrier is shared
// between warps. The stream out of shared memory is bound by shared-memory bandwidth (measured: 43 bytes of weights
// per clock per SM when x is read beside the weights with bank conflicts, 64 without), so x is kept out of it: in
// registers when a row is exactly two chunks of float16, else in a conflict-free order.
// Every mbarrier wait is bounded: when it gives up it records error bit 4 and the warp stops streaming.
//
// Arithmetic it replaces: NFAI.Vulkan.Shaders/MatrixMultiplyShader.cs:266-288 (and the prologue / epilogue shaders
// listed in gemv.cu); same FP32 accumulation, summation order differs (per-lane partial sums, then a shuffle tree).
#include "gemv_common.cuh"

namespace nfai {

using namespace gemv_detail;

namespace {

constexpr unsigned long long kCopyWaitNs = 1000000000ull;  // one second: a stage normally lands in microseconds

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
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
// Bulk copy global -> this CTA's shared memory; completion is counted in bytes on the mbarrier.
// (An evict-first L2 hint on these copies measured 12 % slower in the steady state: 5.8 against 6.6 TB/s.)
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

constexpr int kRingSmemHeader = 128;  // bytes: 32 words of reduction scratch
constexpr int kChunk = 2048;          // bytes of one row in one stage
constexpr int kRows = 2;              // rows per stage

// One stage of kRows x kChunk bytes against the lane's x values. XV: 16-byte steps per lane per chunk (4).
template <typename WT, int VE>
__device__ __forceinline__ void fma_vec(const uint4& w, const float (&xv)[VE], float& acc) {
  float wf[VE];
  WeightVec<WT>::unpack(w, wf);
#pragma unroll
  for (int k = 0; k < VE; ++k) acc = fmaf(wf[k], xv[k], acc);
}

// XREG = true: float16 weights and K = 2 048 exactly. A lane always meets the same 64 elements of x (columns
// 8*lane + 256*v + e), so it keeps them in registers and the stream from shared memory is the weights alone.
// XREG = false: x is read from shared memory next to the weights (conflict-free order for float16 weights).
template <typename WT, typename KVT, int S, int EPI, bool XREG>
__global__ void __launch_bounds__(kThreads, 2) gemv_ring_kernel(const GemvParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  // layout: [ring: kWarps x S x kRows x kChunk][mbarriers: kWarps x S x 8 B, padded to 128][red: 32 words]
  //         [x: K rounded up to 256][gain: K]
  constexpr int R = kRows;
  constexpr int CHUNK = kChunk;
  constexpr uint32_t kStageBytes = R * CHUNK;
  constexpr uint32_t kBarBytes = 128 * ((kWarps * S * 8 + 127) / 128);
  constexpr int VE = WeightVec<WT>::kElems;
  constexpr uint32_t kElemBytes = sizeof(WT);
  constexpr bool kPerm = VE == 8;
  unsigned char* ring = smem_raw;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + (size_t)kWarps * S * kStageBytes);
  float* red = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(bars) + kBarBytes);
  float* xs = red + 32;
  float* gs = xs + ((p.K + 255u) & ~255u);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t row_bytes = p.K * kElemBytes;  // host guarantees a multiple of 16
  const uint32_t nch = (row_bytes + CHUNK - 1) / CHUNK;
  const uint32_t nrb = (p.N + R - 1) / R;
  // contiguous share of this CTA, then round-robin over its warps
  const uint32_t rb_lo = (uint32_t)((unsigned long long)blockIdx.x * nrb / gridDim.x);
  const uint32_t rb_hi = (uint32_t)((unsigned long long)(blockIdx.x + 1) * nrb / gridDim.x);
  const uint32_t first = rb_lo + warp;
  const uint32_t my_rb = first < rb_hi ? (rb_hi - first + kWarps - 1) / kWarps : 0;
  const uint32_t n_items = my_rb * nch;
  const unsigned char* Wb = reinterpret_cast<const unsigned char*>(p.W);
  unsigned char* my_ring = ring + (size_t)warp * S * kStageBytes;
  const uint32_t my_ring_s = smem_u32(my_ring);
  const uint32_t my_bar_s = smem_u32(bars + warp * S);

  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < S; ++s) mbar_init(my_bar_s + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  // item i = (row block first + (i / nch) * kWarps, chunk i % nch) lands in stage s = i % S
  auto item_rows = [&](uint32_t i, uint32_t& rb, uint32_t& off, uint32_t& bytes) {
    const uint32_t rbi = i / nch, c = i - rbi * nch;
    rb = first + rbi * kWarps;
    off = c * CHUNK;
    bytes = row_bytes - off < (uint32_t)CHUNK ? row_bytes - off : (uint32_t)CHUNK;
    const uint32_t rows = p.N - rb * R;
    return rows < (uint32_t)R ? rows : (uint32_t)R;
  };
  auto issue = [&](uint32_t i, uint32_t s) {
    uint32_t rb, off, bytes;
    const uint32_t rows = item_rows(i, rb, off, bytes);
    const uint32_t bar = my_bar_s + 8 * s;
    mbar_expect_tx(bar, bytes * rows);
    for (uint32_t r = 0; r < rows; ++r)
      bulk_g2s(my_ring_s + s * kStageBytes + r * CHUNK, Wb + (size_t)(rb * R + r) * row_bytes + off, bytes, bar);
  };

  if (lane == 0) {
    const uint32_t ahead = n_items < (uint32_t)S ? n_items : (uint32_t)S;
    for (uint32_t i = 0; i < ahead; ++i) issue(i, i);  // weights do not depend on the previous kernel
    // While this kernel waits for its input HBM would idle once the ring is full: ask the L2 for the next stages of
    // this warp, so that the stream continues and the first refills of the ring are L2 hits.
    const uint32_t pf_end = n_items < ahead + p.l2_ahead ? n_items : ahead + p.l2_ahead;
    for (uint32_t i = ahead; i < pf_end; ++i) {
      uint32_t rb, off, bytes;
      const uint32_t rows = item_rows(i, rb, off, bytes);
      for (uint32_t r = 0; r < rows; ++r)
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(Wb + (size_t)(rb * R + r) * row_bytes + off), "r"(bytes)
                     : "memory");
    }
  }
  load_gain(p, xs, gs);
  pdl_launch_dependents();
  pdl_wait();
  uint32_t pos = 0;
  if constexpr (EPI == EPI_QKV_ROPE) pos = p.state ? p.state->pos : p.pos_imm;
  load_x<kPerm>(p, xs, red, gs);

  // this lane's x: 4 steps of 8 elements per chunk, two chunks (K = 2 048)
  constexpr int kVecPerChunk = CHUNK / 512;
  constexpr int kXChunks = XREG ? 2 : 1;
  float xr[kXChunks][kVecPerChunk][XREG ? VE : 1];
  if constexpr (XREG) {
#pragma unroll
    for (int c = 0; c < kXChunks; ++c)
#pragma unroll
      for (int v = 0; v < kVecPerChunk; ++v) {
        const float4* xb = reinterpret_cast<const float4*>(xs) + (c * kVecPerChunk + v) * 64;
        const float4 a = xb[lane], b = xb[32 + lane];
        xr[c][v][0] = a.x; xr[c][v][1] = a.y; xr[c][v][2] = a.z; xr[c][v][3] = a.w;
        xr[c][v][4] = b.x; xr[c][v][5] = b.y; xr[c][v][6] = b.z; xr[c][v][7] = b.w;
      }
  }

  float best_v = -INFINITY;
  uint32_t best_i = 0xffffffffu;
  float acc[R], pre[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = pre[r] = 0.f;
  bool gave_up = false;
  uint32_t s = 0, phase = 0, rb = first, i = 0;

  // wait for stage s (bounded); false when the copy did not land in time
  auto stage_ready = [&]() {
    const uint32_t bar = my_bar_s + 8 * s;
    bool ok = mbar_try_wait(bar, phase);
    if (!ok) {
      const unsigned long long t_start = global_timer_ns();
      uint32_t polls = 0;
      while (!(ok = mbar_try_wait(bar, phase))) {
        if ((++polls & 63u) == 0 && global_timer_ns() - t_start > kCopyWaitNs) break;
      }
    }
    return __all_sync(0xffffffffu, ok);  // all lanes are back together here
  };
  auto stage_release = [&]() {
    __syncwarp();  // every lane has read the stage before it is refilled
    if (lane == 0 && i + S < n_items) issue(i + S, s);
    ++i;
    if (++s == S) {
      s = 0;
      phase ^= 1u;
    }
  };
  auto finish_block = [&]() {
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = warp_sum(acc[r]);
    // a ragged last block holds stale bytes for the rows beyond N: the epilogues never store those rows
    row_epilogue_pre<KVT, R, EPI>(p, rb * R, acc, pre, pos, best_v, best_i);
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.f;
    rb += kWarps;
  };

  if constexpr (XREG) {
    // nch == 2: the two chunks of a row block are two consecutive stages; x comes from registers
    for (uint32_t b = 0; b < my_rb && !gave_up; ++b) {
      // what the epilogue reads besides the sums (residual, cos/sin pair) is requested when the row block begins
      epi_preload<R, EPI>(p, rb * R, pos, pre);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        if (!stage_ready()) {
          gave_up = true;
          break;
        }
        const unsigned char* st = my_ring + (size_t)s * kStageBytes;
        uint4 w[kVecPerChunk][R];
#pragma unroll
        for (int v = 0; v < kVecPerChunk; ++v)
#pragma unroll
          for (int r = 0; r < R; ++r) w[v][r] = *reinterpret_cast<const uint4*>(st + r * CHUNK + (lane + 32 * v) * 16);
#pragma unroll
        for (int v = 0; v < kVecPerChunk; ++v)
#pragma unroll
          for (int r = 0; r < R; ++r) fma_vec<WT, VE>(w[v][r], xr[c][v], acc[r]);
        stage_release();
      }
      if (!gave_up) finish_block();
    }
  } else {
    uint32_t c = 0;
    while (i < n_items) {
      if (c == 0) epi_preload<R, EPI>(p, rb * R, pos, pre);
      if (!stage_ready()) {
        gave_up = true;
        break;
      }
      const uint32_t off = c * CHUNK;
      const uint32_t bytes = row_bytes - off < (uint32_t)CHUNK ? row_bytes - off : (uint32_t)CHUNK;
      const unsigned char* st = my_ring + (size_t)s * kStageBytes;
      // 16-byte steps of this chunk; x for step v of chunk c: elements (off + (lane + 32 v) * 16) / elem size ...
      const uint32_t nvec = (bytes + 511) / 512;
      for (uint32_t v = 0; v < nvec; ++v) {
        const uint32_t vb = (lane + 32 * v) * 16;  // byte offset of this lane's vector inside the chunk
        if (vb < bytes) {
          float xv[VE];
          if constexpr (kPerm) {
            const float4* xb = reinterpret_cast<const float4*>(xs) + ((off + 512 * v) / kElemBytes / 256) * 64;
            const float4 a = xb[lane], b4 = xb[32 + lane];
            xv[0] = a.x; xv[1] = a.y; xv[2] = a.z; xv[3] = a.w;
            xv[4] = b4.x; xv[5] = b4.y; xv[6] = b4.z; xv[7] = b4.w;
          } else {
            const float4 a = *reinterpret_cast<const float4*>(xs + (off + vb) / kElemBytes);
            xv[0] = a.x; xv[1] = a.y; xv[2] = a.z; xv[3] = a.w;
          }
#pragma unroll
          for (int r = 0; r < R; ++r) fma_vec<WT, VE>(*reinterpret_cast<const uint4*>(st + r * CHUNK + vb), xv, acc[r]);
        }
      }
      stage_release();
      if (++c == nch) {
        finish_block();
        c = 0;
      }
    }
  }
  if (gave_up) {
    // Copies of this warp may still be in flight: give them a bounded time to land before the CTA's shared
    // memory is released, and report.
    if (lane == 0 && p.state) atomicOr(&p.state->err, 4u);
    if (lane == 0 && p.err) atomicOr(p.err, 4u);
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 2000000ull) {
    }
  }
  if constexpr (EPI == EPI_LOGITS) cta_argmax_partial(p, best_v, best_i, red);
}

template <typename Kern>
cudaError_t launch_ring(Kern kernel, dim3 grid, size_t smem, cudaStream_t s, bool pdl, const GemvParams& p) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  e = prefer_max_shared(kernel);
  if (e != cudaSuccess) return e;
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

template <typename WT, typename KVT, int EPI, bool XREG>
cudaError_t launch_s(int S, dim3 grid, size_t smem, cudaStream_t s, bool pdl, const GemvParams& p) {
  switch (S) {
    case 1: return launch_ring(gemv_ring_kernel<WT, KVT, 1, EPI, XREG>, grid, smem, s, pdl, p);
    case 2: return launch_ring(gemv_ring_kernel<WT, KVT, 2, EPI, XREG>, grid, smem, s, pdl, p);
    case 3: return launch_ring(gemv_ring_kernel<WT, KVT, 3, EPI, XREG>, grid, smem, s, pdl, p);
    case 4: return launch_ring(gemv_ring_kernel<WT, KVT, 4, EPI, XREG>, grid, smem, s, pdl, p);
    default: return cudaErrorInvalidValue;
  }
}

template <typename WT, typename KVT, int EPI>
cudaError_t launch_x(int S, dim3 grid, size_t smem, cudaStream_t s, bool pdl, const GemvParams& p) {
  // x in registers: float16 weights and rows of exactly two chunks
  if constexpr (sizeof(WT) == 2) {
    if (p.K * 2u == 2u * kChunk) return launch_s<WT, KVT, EPI, true>(S, grid, smem, s, pdl, p);
  }
  return launch_s<WT, KVT, EPI, false>(S, grid, smem, s, pdl, p);
}

template <typename WT, typename KVT>
cudaError_t launch_re(GemvEpilogue epi, int S, dim3 grid, size_t smem, cudaStream_t s, bool pdl, const GemvParams& p) {
  switch (epi) {
    case EPI_STORE: return launch_x<WT, float, EPI_STORE>(S, grid, smem, s, pdl, p);
    case EPI_QKV_ROPE: return launch_x<WT, KVT, EPI_QKV_ROPE>(S, grid, smem, s, pdl, p);
    case EPI_SILU_MUL: return launch_x<WT, float, EPI_SILU_MUL>(S, grid, smem, s, pdl, p);
    case EPI_LOGITS: return launch_x<WT, float, EPI_LOGITS>(S, grid, smem, s, pdl, p);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

size_t gemv_ring_smem(const GemvParams& p, int S) {
  const size_t ring = (size_t)kWarps * S * kRows * kChunk;
  const size_t bars = 128 * (((size_t)kWarps * S * 8 + 127) / 128);
  const size_t xfloats = ((size_t)p.K + 255) / 256 * 256 + (p.gain ? (size_t)p.K : 0);
  return ring + bars + kRingSmemHeader + xfloats * sizeof(float);
}

uint32_t gemv_ring_grid(const GemvParams& p, int ctas_per_sm) {
  const uint32_t nrb = (p.N + 1) / 2;
  const uint32_t cap = sm_count() * (uint32_t)(ctas_per_sm < 1 ? 1 : ctas_per_sm);
  return nrb < cap ? nrb : cap;
}

cudaError_t launch_gemv_ring(cudaStream_t s, int wdtype, int kvdtype, GemvEpilogue epi, const GemvParams& p, int S,
                             int ctas_per_sm, bool pdl) {
  if ((epi == EPI_QKV_ROPE || epi == EPI_SILU_MUL) && (p.N % 2) != 0) return cudaErrorInvalidValue;
  const size_t smem = gemv_ring_smem(p, S);
  if (smem > 227 * 1024) return cudaErrorInvalidValue;
  dim3 grid(gemv_ring_grid(p, ctas_per_sm));
  if (wdtype == 1) {
    if (kvdtype == 1) return launch_re<__half, __half>(epi, S, grid, smem, s, pdl, p);
    return launch_re<__half, float>(epi, S, grid, smem, s, pdl, p);
  }
  if (kvdtype == 1) return launch_re<float, __half>(epi, S, grid, smem, s, pdl, p);
  return launch_re<float, float>(epi, S, grid, smem, s, pdl, p);
}

}  // namespace nfai
