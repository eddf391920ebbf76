// Decode GEMV with the weight stream staged through a shared-memory ring by bulk asynchronous copies (TMA, 1-D).
//
// Why: at batch 1 every matrix of a layer is a 1-10 microsecond stream, so what decides the step time is how
// much of the next kernel's stream is already under way when the previous kernel ends. Bulk copies keep ~100 KB
// per SM in flight without holding registers, and a CTA needs under half of an SM (256 threads, ~105 KB of
// shared memory). Two consecutive kernels of the step therefore sit on the SM together: while kernel k computes,
// kernel k+1 (started early by programmatic dependent launch) has already filled its ring with its first
// ~15 MB of weights and only then waits for kernel k's output.
//
// Shape: one CTA per SM, eight warps; each warp owns a private ring of S stages and walks its row blocks
// (R rows x the whole K, in chunks of 2 KB per row). Lane 0 arms the stage's mbarrier with the byte count and
// issues one bulk copy per row; all lanes wait on the mbarrier parity, read the stage with 16-byte shared loads,
// FMA against x (float32, shared memory) and refill the stage. No barrier is shared between warps.
// Every mbarrier wait is bounded: when it gives up it records an error bit and the warp stops streaming.
#include "gemv_common.cuh"

namespace nfai {

using namespace gemv_detail;

namespace {

constexpr uint32_t kChunkBytes = 2048;     // bytes of one row in one stage
constexpr unsigned long long kWaitLimitNs = 1000000000ull;  // one second: a stage normally lands in microseconds

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

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
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

template <typename WT, typename KVT, int R, int S, int EPI>
__global__ void __launch_bounds__(kThreads, 2) gemv_ring_kernel(const GemvParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  // layout: [ring: kWarps x S x R x 2 KB][mbarriers: kWarps x S x 8 B, padded][red: 32 floats][x: K][gain: K]
  constexpr uint32_t kStageBytes = R * kChunkBytes;
  unsigned char* ring = smem_raw;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + (size_t)kWarps * S * kStageBytes);
  float* red = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(bars) + 128 * ((kWarps * S * 8 + 127) / 128));
  float* xs = red + 32;
  constexpr int VE = WeightVec<WT>::kElems;
  constexpr uint32_t kElemBytes = sizeof(WT);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t row_bytes = p.K * kElemBytes;  // host guarantees a multiple of 16
  const uint32_t nchunks = (row_bytes + kChunkBytes - 1) / kChunkBytes;
  const uint32_t nrb = (p.N + R - 1) / R;
  const uint32_t TW = gridDim.x * kWarps;
  const uint32_t gw = blockIdx.x * kWarps + warp;
  const uint32_t my_rb = gw < nrb ? (nrb - gw + TW - 1) / TW : 0;  // row blocks of this warp
  const uint32_t n_items = my_rb * nchunks;
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

  // item i = (row block gw + (i / nchunks) * TW, chunk i % nchunks) lands in stage i % S
  auto issue = [&](uint32_t i) {
    const uint32_t rb = gw + (i / nchunks) * TW, c = i % nchunks, s = i % S;
    const uint32_t off = c * kChunkBytes;
    const uint32_t bytes = row_bytes - off < kChunkBytes ? row_bytes - off : kChunkBytes;
    uint32_t rows = p.N - rb * R;
    rows = rows < (uint32_t)R ? rows : (uint32_t)R;
    const uint32_t bar = my_bar_s + 8 * s;
    mbar_expect_tx(bar, bytes * rows);
    for (uint32_t r = 0; r < rows; ++r)
      bulk_g2s(my_ring_s + s * kStageBytes + r * kChunkBytes, Wb + (size_t)(rb * R + r) * row_bytes + off, bytes, bar);
  };

  if (lane == 0) {
    const uint32_t first = n_items < (uint32_t)S ? n_items : (uint32_t)S;
    for (uint32_t i = 0; i < first; ++i) issue(i);  // weights do not depend on the previous kernel
  }
  load_gain(p, xs);
  pdl_launch_dependents();
  pdl_wait();
  load_x(p, xs, red);

  float best_v = -INFINITY;
  uint32_t best_i = 0xffffffffu;
  float acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.f;
  bool gave_up = false;
  for (uint32_t i = 0; i < n_items; ++i) {
    const uint32_t rbi = i / nchunks, c = i - rbi * nchunks, s = i % S;
    const uint32_t rb = gw + rbi * TW;
    const uint32_t bar = my_bar_s + 8 * s;
    const uint32_t parity = (i / S) & 1;
    // warp-uniform bounded wait: every lane polls until all lanes have seen the phase complete
    bool ok = __all_sync(0xffffffffu, mbar_try_wait(bar, parity));
    if (!ok) {
      const unsigned long long t_start = global_ns();
      uint32_t polls = 0;
      while (!ok) {
        ok = __all_sync(0xffffffffu, mbar_try_wait(bar, parity));
        if (!ok && (++polls & 63u) == 0) {
          const bool late = global_ns() - t_start > kWaitLimitNs;
          if (__any_sync(0xffffffffu, late)) break;
        }
      }
    }
    if (!ok) {
      gave_up = true;  // same value in every lane
      break;
    }
    const uint32_t off = c * kChunkBytes;
    const uint32_t bytes = row_bytes - off < kChunkBytes ? row_bytes - off : kChunkBytes;
    const unsigned char* st = my_ring + (size_t)s * kStageBytes;
#pragma unroll
    for (int v = 0; v < (int)(kChunkBytes / 512); ++v) {
      const uint32_t vb = (lane + 32 * v) * 16;  // byte offset of this lane's vector inside the chunk
      if (vb < bytes) {
        float xv[VE];
        const float4* xp = reinterpret_cast<const float4*>(xs + (off + vb) / kElemBytes);
#pragma unroll
        for (int k = 0; k < VE / 4; ++k) {
          float4 t = xp[k];
          xv[4 * k] = t.x;
          xv[4 * k + 1] = t.y;
          xv[4 * k + 2] = t.z;
          xv[4 * k + 3] = t.w;
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const uint4 w = *reinterpret_cast<const uint4*>(st + r * kChunkBytes + vb);
          float wf[VE];
          WeightVec<WT>::unpack(w, wf);
#pragma unroll
          for (int k = 0; k < VE; ++k) acc[r] = fmaf(wf[k], xv[k], acc[r]);
        }
      }
    }
    __syncwarp();  // every lane has read the stage before it is refilled
    if (lane == 0 && i + S < n_items) issue(i + S);
    if (c == nchunks - 1) {
#pragma unroll
      for (int r = 0; r < R; ++r) acc[r] = warp_sum(acc[r]);
      row_epilogue<KVT, R, EPI>(p, rb * R, acc, best_v, best_i);
#pragma unroll
      for (int r = 0; r < R; ++r) acc[r] = 0.f;
    }
  }
  if (gave_up) {
    // Copies of this warp may still be in flight: give them a bounded time to land before the CTA's shared
    // memory is released, and report.
    if (lane == 0 && p.state) atomicOr(&p.state->err, 4u);
    if (lane == 0 && p.err) atomicOr(p.err, 4u);
    for (volatile uint32_t spin = 0; spin < (1u << 20); ++spin) {
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

template <typename WT, typename KVT, int R, int EPI>
cudaError_t launch_s(int S, dim3 grid, size_t smem, cudaStream_t s, bool pdl, const GemvParams& p) {
  switch (S) {
    case 2: return launch_ring(gemv_ring_kernel<WT, KVT, R, 2, EPI>, grid, smem, s, pdl, p);
    case 3: return launch_ring(gemv_ring_kernel<WT, KVT, R, 3, EPI>, grid, smem, s, pdl, p);
    case 4: return launch_ring(gemv_ring_kernel<WT, KVT, R, 4, EPI>, grid, smem, s, pdl, p);
    case 6: return launch_ring(gemv_ring_kernel<WT, KVT, R, 6, EPI>, grid, smem, s, pdl, p);
    default: return cudaErrorInvalidValue;
  }
}

template <typename WT, typename KVT>
cudaError_t launch_re(GemvEpilogue epi, int R, int S, dim3 grid, size_t smem, cudaStream_t s, bool pdl,
                      const GemvParams& p) {
  switch (epi) {
    case EPI_STORE:
      return R == 1 ? launch_s<WT, float, 1, EPI_STORE>(S, grid, smem, s, pdl, p)
                    : launch_s<WT, float, 2, EPI_STORE>(S, grid, smem, s, pdl, p);
    case EPI_QKV_ROPE: return launch_s<WT, KVT, 2, EPI_QKV_ROPE>(S, grid, smem, s, pdl, p);
    case EPI_SILU_MUL: return launch_s<WT, float, 2, EPI_SILU_MUL>(S, grid, smem, s, pdl, p);
    case EPI_LOGITS:
      return R == 1 ? launch_s<WT, float, 1, EPI_LOGITS>(S, grid, smem, s, pdl, p)
                    : launch_s<WT, float, 2, EPI_LOGITS>(S, grid, smem, s, pdl, p);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

size_t gemv_ring_smem(const GemvParams& p, int R, int S) {
  size_t ring = (size_t)kWarps * S * R * kChunkBytes;
  size_t bars = 128 * (((size_t)kWarps * S * 8 + 127) / 128);
  return ring + bars + (32 + (size_t)p.K * (p.gain ? 2 : 1)) * sizeof(float);
}

uint32_t gemv_ring_grid(const GemvParams& p, int R, int ctas_per_sm) {
  const uint32_t nrb = (p.N + R - 1) / R;
  const uint32_t want = (nrb + kWarps - 1) / kWarps;
  const uint32_t cap = kNumSMs * (uint32_t)(ctas_per_sm < 1 ? 1 : ctas_per_sm);
  return want < cap ? want : cap;
}

cudaError_t launch_gemv_ring(cudaStream_t s, int wdtype, int kvdtype, GemvEpilogue epi, const GemvParams& p, int R,
                             int S, int ctas_per_sm, bool pdl) {
  if (R != 1 && R != 2) return cudaErrorInvalidValue;
  if ((epi == EPI_QKV_ROPE || epi == EPI_SILU_MUL) && R != 2) return cudaErrorInvalidValue;
  const size_t smem = gemv_ring_smem(p, R, S);
  if (smem > 227 * 1024) return cudaErrorInvalidValue;
  dim3 grid(gemv_ring_grid(p, R, ctas_per_sm));
  if (wdtype == 1) {
    if (kvdtype == 1) return launch_re<__half, __half>(epi, R, S, grid, smem, s, pdl, p);
    return launch_re<__half, float>(epi, R, S, grid, smem, s, pdl, p);
  }
  if (kvdtype == 1) return launch_re<float, __half>(epi, R, S, grid, smem, s, pdl, p);
  return launch_re<float, float>(epi, R, S, grid, smem, s, pdl, p);
}

}  // namespace nfai
