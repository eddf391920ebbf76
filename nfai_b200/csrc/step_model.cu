// A model of the batch-1 decode step for finding out where its time goes.
//
//   python -m nfai_b200.build --step-model && nfai_b200/build/step_model
//
// The step of the Llama-3.2-1B architecture is replayed as its chain of dependent launches in one CUDA graph with
// programmatic dependent launch: per layer QKV (3072 x 2048) -> attention stand-in (32 CTAs) -> O (2048 x 2048) ->
// gate/up (16384 x 2048) -> down (2048 x 8192), 16 layers, then the LM head (128256 x 2048); float16 weights in
// distinct buffers (2.47 GB: nothing stays in L2), every kernel reads what its predecessor wrote. The kernels are
// reduced forms of the library's GEMVs (same streaming structure, no epilogue fusion), in two shapes:
//   reg   two CTAs of 8 warps per SM, weights double-buffered in registers (the library's default shape);
//   ring  one CTA per SM, per-warp shared-memory rings of 3 stages x 2 rows x 2 KB fed by 1-D bulk copies, so that
//         two consecutive kernels are resident on an SM together and kernel k+1 fills its ring while kernel k runs.
// Printed: microseconds per step for each shape, and for one layer in steady state a time line from %globaltimer:
// for every kernel the first and last CTA's time of entry, of release from the dependency wait, of "x is normalised
// in shared memory", and of its last store. The gaps between one kernel's last end and the next kernel's release,
// and between release and x-ready, are the per-hand-over costs that a 1-10 microsecond kernel cannot hide.
// Last, the rate at which one CTA of 8 warps turns float16 weights that already sit in shared memory into float32 dot
// products (bytes of weights per clock per SM), with x read beside the weights in natural order (two-way bank
// conflicts on the 32-byte-per-lane reads), in the conflict-free order, and held in registers: what a kernel that has
// its weights on chip before its input arrives can make of them.
// Every wait in here is bounded.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

#define CK(x)                                                                              \
  do {                                                                                     \
    cudaError_t e_ = (x);                                                                  \
    if (e_ != cudaSuccess) {                                                               \
      printf("CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__);      \
      exit(1);                                                                             \
    }                                                                                      \
  } while (0)

namespace {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t c) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(c) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t b) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(b) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
               "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ float warp_sum(float v) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// event ev of this kernel: earliest and latest CTA
__device__ __forceinline__ void stamp(unsigned long long* ts, int ev) {
  if (ts && threadIdx.x == 0) {
    const unsigned long long t = now_ns();
    atomicMin(ts + 2 * ev, t);
    atomicMax(ts + 2 * ev + 1, t);
  }
}

struct P {
  const __half* W;
  const float* x;
  float* y;
  uint32_t N, K;
  int norm;
  unsigned long long* ts;
};

__device__ __forceinline__ void load_x_norm(const P& p, float* xs, float* red, int nthreads) {
  float ss = 0.f;
  for (uint32_t i = threadIdx.x; i < p.K; i += nthreads) {
    const float v = p.x[i % 2048];
    xs[i] = v;
    ss = fmaf(v, v, ss);
  }
  if (p.norm) {
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0;
    for (int w = 0; w < nthreads / 32; ++w) tot += red[w];
    const float r = rsqrtf(tot / p.K + 1e-5f);
    for (uint32_t i = threadIdx.x; i < p.K; i += nthreads) xs[i] *= r;
  }
  __syncthreads();
}

__device__ __forceinline__ float dot8(const uint4& w, const float4& x0, const float4& x1, float t) {
  const __half2* h = reinterpret_cast<const __half2*>(&w);
  const float2 a = __half22float2(h[0]), b = __half22float2(h[1]), c = __half22float2(h[2]), d = __half22float2(h[3]);
  t = fmaf(a.x, x0.x, t); t = fmaf(a.y, x0.y, t); t = fmaf(b.x, x0.z, t); t = fmaf(b.y, x0.w, t);
  t = fmaf(c.x, x1.x, t); t = fmaf(c.y, x1.y, t); t = fmaf(d.x, x1.z, t); t = fmaf(d.y, x1.w, t);
  return t;
}

constexpr int kR = 2, kChunk = 2048, kNW = 8;

template <int S>
__global__ void __launch_bounds__(kNW * 32) ring_kernel(const P p) {
  extern __shared__ __align__(128) unsigned char sm[];
  stamp(p.ts, 0);
  constexpr uint32_t STB = kR * kChunk;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + (size_t)kNW * S * STB);
  float* red = reinterpret_cast<float*>(bars + kNW * S);
  float* xs = red + 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t row_bytes = p.K * 2, nch = row_bytes / kChunk, nrb = p.N / kR;
  const uint32_t rb_lo = (uint32_t)((uint64_t)blockIdx.x * nrb / gridDim.x), rb_hi = (uint32_t)((uint64_t)(blockIdx.x + 1) * nrb / gridDim.x);
  const uint32_t first = rb_lo + warp;
  const uint32_t my_rb = first < rb_hi ? (rb_hi - first + kNW - 1) / kNW : 0, n_items = my_rb * nch;
  unsigned char* my_ring = sm + (size_t)warp * S * STB;
  const uint32_t my_ring_s = smem_u32(my_ring), my_bar = smem_u32(bars + warp * S);
  if (lane == 0) {
    for (int s = 0; s < S; ++s) mbar_init(my_bar + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  auto issue = [&](uint32_t i) {
    const uint32_t rb = first + (i / nch) * kNW, c = i % nch, s = i % S, bar = my_bar + 8 * s;
    mbar_expect_tx(bar, STB);
    for (int r = 0; r < kR; ++r)
      bulk_g2s(my_ring_s + s * STB + r * kChunk, reinterpret_cast<const unsigned char*>(p.W) + (size_t)(rb * kR + r) * row_bytes + c * kChunk,
               kChunk, bar);
  };
  if (lane == 0)
    for (uint32_t i = 0; i < (n_items < (uint32_t)S ? n_items : (uint32_t)S); ++i) issue(i);
  pdl_launch();
  pdl_wait();
  stamp(p.ts, 1);
  load_x_norm(p, xs, red, kNW * 32);
  stamp(p.ts, 2);
  float acc[kR] = {0.f, 0.f};
  for (uint32_t i = 0; i < n_items; ++i) {
    const uint32_t rbi = i / nch, c = i - rbi * nch, s = i % S, bar = my_bar + 8 * s, parity = (i / S) & 1;
    uint32_t polls = 0;
    while (!mbar_try_wait(bar, parity))
      if (++polls > (1u << 24)) return;  // bounded: a copy that never lands ends the warp
    const unsigned char* st = my_ring + (size_t)s * STB;
#pragma unroll
    for (int v = 0; v < kChunk / 512; ++v) {
      const uint32_t vb = (lane + 32 * v) * 16;
      const float4* xp = reinterpret_cast<const float4*>(xs + (c * kChunk + vb) / 2);
      const float4 x0 = xp[0], x1 = xp[1];
#pragma unroll
      for (int r = 0; r < kR; ++r) acc[r] = dot8(*reinterpret_cast<const uint4*>(st + r * kChunk + vb), x0, x1, acc[r]);
    }
    __syncwarp();
    if (lane == 0 && i + S < n_items) issue(i + S);
    if (c == nch - 1) {
      const uint32_t rb = first + rbi * kNW;
#pragma unroll
      for (int r = 0; r < kR; ++r) {
        const float t = warp_sum(acc[r]);
        if (lane == 0) p.y[rb * kR + r] = t * 1e-3f;
        acc[r] = 0.f;
      }
    }
  }
  __syncthreads();
  stamp(p.ts, 3);
}

template <int U>
__global__ void __launch_bounds__(256, 2) reg_kernel(const P p) {
  extern __shared__ __align__(16) float sm2[];
  stamp(p.ts, 0);
  float* red = sm2;
  float* xs = sm2 + 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t nkb = p.K / 8 / (32 * U), nrb = p.N / kR, TW = gridDim.x * 8;
  uint32_t rb = blockIdx.x * 8 + warp;
  uint4 buf[U][kR];
  auto ld = [&](uint32_t rbx, uint32_t kb) {
    if (rbx >= nrb) return;
#pragma unroll
    for (int r = 0; r < kR; ++r) {
      const uint4* wr = reinterpret_cast<const uint4*>(p.W + (size_t)(rbx * kR + r) * p.K);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        uint4 v;
        const uint4* q = wr + kb * 32 * U + 32 * u + lane;
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(q));
        buf[u][r] = v;
      }
    }
  };
  ld(rb, 0);
  pdl_launch();
  pdl_wait();
  stamp(p.ts, 1);
  load_x_norm(p, xs, red, 256);
  stamp(p.ts, 2);
  for (; rb < nrb; rb += TW) {
    float acc[kR] = {0.f, 0.f};
    for (uint32_t kb = 0; kb < nkb; ++kb) {
      uint4 cur[U][kR];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int r = 0; r < kR; ++r) cur[u][r] = buf[u][r];
      if (kb + 1 < nkb) ld(rb, kb + 1);
      else ld(rb + TW, 0);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const float4* xp = reinterpret_cast<const float4*>(xs + (size_t)(kb * 32 * U + 32 * u + lane) * 8);
        const float4 x0 = xp[0], x1 = xp[1];
#pragma unroll
        for (int r = 0; r < kR; ++r) acc[r] = dot8(cur[u][r], x0, x1, acc[r]);
      }
    }
#pragma unroll
    for (int r = 0; r < kR; ++r) {
      const float t = warp_sum(acc[r]);
      if (lane == 0) p.y[rb * kR + r] = t * 1e-3f;
    }
  }
  __syncthreads();
  stamp(p.ts, 3);
}

// attention stand-in: 32 CTAs x 512 threads, reads q (the dependency) and 25 KB each of a "cache" in three dependent rounds
__global__ void __launch_bounds__(512) attn_like(const float* q, const uint4* cache, float* out, unsigned long long* ts) {
  stamp(ts, 0);
  pdl_launch();
  pdl_wait();
  stamp(ts, 1);
  const float qq = q[threadIdx.x];
  float acc = 0;
  for (int it = 0; it < 3; ++it) acc += __uint_as_float(cache[(size_t)blockIdx.x * 1536 + it * 512 + threadIdx.x].x) * (qq + acc);
  __shared__ float s[16];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 64) out[blockIdx.x * 64 + threadIdx.x] = s[threadIdx.x & 15] * 1e-6f;
  __syncthreads();
  stamp(ts, 3);
}

template <typename Kern, typename... A>
void launch(Kern k, dim3 g, dim3 b, size_t smem, cudaStream_t s, bool pdl, A... a) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = g;
  cfg.blockDim = b;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  CK(cudaLaunchKernelEx(&cfg, k, a...));
}

struct Mat {
  __half* W;
  uint32_t N, K;
};
constexpr int L = 16;
Mat qkv[L], o[L], gu[L], dn[L], head;
float *xa, *xb, *qbuf, *abuf, *hbuf, *lg;
uint4* cache;
unsigned long long* g_ts = nullptr;
int g_tk = 0;
bool g_trace = false;
unsigned long long* next_ts() { return g_trace ? g_ts + 8 * (g_tk++) : nullptr; }

void gemv(bool ring, cudaStream_t s, bool pdl, const Mat& m, const float* x, float* y, int norm) {
  P p{m.W, x, y, m.N, m.K, norm, next_ts()};
  if (!ring) {
    launch(reg_kernel<4>, dim3(296), dim3(256), 128 + (size_t)m.K * 4, s, pdl, p);
  } else if (m.K == 8192) {  // 32 KB of x: two stages keep the CTA under half of an SM
    launch(ring_kernel<2>, dim3(148), dim3(kNW * 32), (size_t)kNW * 2 * kR * kChunk + kNW * 2 * 8 + 128 + (size_t)m.K * 4, s, pdl, p);
  } else {
    launch(ring_kernel<3>, dim3(148), dim3(kNW * 32), (size_t)kNW * 3 * kR * kChunk + kNW * 3 * 8 + 128 + (size_t)m.K * 4, s, pdl, p);
  }
}

void record(bool ring, cudaStream_t s, bool pdl) {
  g_tk = 0;
  for (int l = 0; l < L; ++l) {
    gemv(ring, s, pdl && l > 0, qkv[l], xa, qbuf, 1);
    launch(attn_like, dim3(32), dim3(512), 0, s, pdl, (const float*)qbuf, (const uint4*)cache, abuf, next_ts());
    gemv(ring, s, pdl, o[l], abuf, xb, 0);
    gemv(ring, s, pdl, gu[l], xb, hbuf, 1);
    gemv(ring, s, pdl, dn[l], hbuf, xa, 0);
  }
  gemv(ring, s, pdl, head, xa, lg, 1);
}

void run(const char* tag, bool ring, bool pdl, bool trace) {
  cudaStream_t s;
  CK(cudaStreamCreate(&s));
  cudaGraph_t g;
  cudaGraphExec_t ge;
  g_trace = trace;
  CK(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
  record(ring, s, pdl);
  CK(cudaStreamEndCapture(s, &g));
  CK(cudaGraphInstantiate(&ge, g, 0));
  g_trace = false;
  for (int i = 0; i < 5; ++i) CK(cudaGraphLaunch(ge, s));
  CK(cudaStreamSynchronize(s));
  if (!trace) {
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaEventRecord(e0, s);
    for (int i = 0; i < 50; ++i) CK(cudaGraphLaunch(ge, s));
    cudaEventRecord(e1, s);
    CK(cudaStreamSynchronize(s));
    float ms;
    cudaEventElapsedTime(&ms, e0, e1);
    printf("%-34s dependent launch %d : %.1f us per step\n", tag, (int)pdl, ms / 50 * 1e3);
  } else {
    const int nk = g_tk;
    std::vector<unsigned long long> h(8 * nk);
    for (int i = 0; i < nk; ++i)
      for (int e = 0; e < 4; ++e) {
        h[8 * i + 2 * e] = ~0ull;
        h[8 * i + 2 * e + 1] = 0;
      }
    CK(cudaMemcpy(g_ts, h.data(), 8 * nk * 8, cudaMemcpyHostToDevice));
    CK(cudaGraphLaunch(ge, s));
    CK(cudaStreamSynchronize(s));
    CK(cudaMemcpy(h.data(), g_ts, 8 * nk * 8, cudaMemcpyDeviceToHost));
    const char* names[5] = {"QKV", "attn", "O", "gate/up", "down"};
    const int l0 = 8 * 5;
    const unsigned long long t0 = h[8 * l0];
    printf("time line, %s, layer 8 and the next QKV (ns after the layer's first CTA entered; first / last CTA):\n", tag);
    printf("  %-8s %15s %15s %15s %15s\n", "kernel", "entry", "released", "x ready", "end");
    for (int i = l0; i < l0 + 6 && i < nk; ++i) {
      printf("  %-8s", names[(i - l0) % 5]);
      for (int e = 0; e < 4; ++e) {
        if (h[8 * i + 2 * e + 1] == 0) printf(" %15s", "-");
        else printf(" %7lld/%7lld", (long long)(h[8 * i + 2 * e] - t0), (long long)(h[8 * i + 2 * e + 1] - t0));
      }
      printf("\n");
    }
  }
  fflush(stdout);
  cudaGraphExecDestroy(ge);
  cudaGraphDestroy(g);
  cudaStreamDestroy(s);
}

// MODE 0: x from shared memory, natural order; 1: conflict-free order; 2: x in registers (K = 2 048)
template <int MODE>
__global__ void __launch_bounds__(256) consume_rate(const uint4* fill, float* y, unsigned long long* cyc, int rep) {
  extern __shared__ __align__(128) unsigned char sm[];
  constexpr int kStages = 3;                              // per warp: 3 stages x 2 rows x 2 KB, as the ring kernel
  constexpr uint32_t kWeights = 8 * kStages * kR * kChunk;  // 96 KB
  float* xs = reinterpret_cast<float*>(sm + kWeights);    // 2 048 floats
  for (uint32_t i = threadIdx.x; i < kWeights / 16; i += 256) reinterpret_cast<uint4*>(sm)[i] = fill[i & 4095];
  for (uint32_t i = threadIdx.x; i < 2048; i += 256) xs[i] = 1e-3f * (float)(i & 63);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned char* my = sm + (size_t)warp * kStages * kR * kChunk;
  float xr[8][8];
  if (MODE == 2)
    for (int v = 0; v < 8; ++v)
      for (int e = 0; e < 8; ++e) xr[v][e] = xs[v * 256 + lane * 8 + e];
  float total = 0.f;
  asm volatile("" ::: "memory");
  const long long t0 = clock64();
  for (int it = 0; it < rep; ++it) {
    float acc[kR] = {0.f, 0.f};
    for (int s = 0; s < kStages; ++s) {
      const unsigned char* st = my + (size_t)s * kR * kChunk;
#pragma unroll
      for (int v = 0; v < kChunk / 512; ++v) {
        // the same bytes every repetition, rotated by 16 bytes per repetition (same bank pattern): the address depends
        // on the repetition, so no load can be kept from one repetition to the next
        const uint32_t vb = ((lane + 32 * v + it) * 16) & (kChunk - 1);
        float4 x0, x1;
        if (MODE == 0) {
          const float4* xp = reinterpret_cast<const float4*>(xs + ((s & 1) * kChunk + vb) / 2);
          x0 = xp[0];
          x1 = xp[1];
        } else if (MODE == 1) {
          const float4* xb = reinterpret_cast<const float4*>(xs) + ((s & 1) * 4 + v) * 64;
          x0 = xb[lane];
          x1 = xb[32 + lane];
        } else {
          const int b = (s & 1) * 4 + v;
          x0 = make_float4(xr[b][0], xr[b][1], xr[b][2], xr[b][3]);
          x1 = make_float4(xr[b][4], xr[b][5], xr[b][6], xr[b][7]);
        }
#pragma unroll
        for (int r = 0; r < kR; ++r) acc[r] = dot8(*reinterpret_cast<const uint4*>(st + r * kChunk + vb), x0, x1, acc[r]);
      }
    }
    total += acc[0] + acc[1];
    asm volatile("" : "+f"(total) : : "memory");  // the next repetition reads shared memory again
  }
  asm volatile("" : "+f"(total) : : "memory");    // the sums exist before the clock is read
  const long long t1 = clock64();
  total = warp_sum(total);
  if (lane == 0) y[blockIdx.x * 8 + warp] = total;
  if (threadIdx.x == 0) cyc[blockIdx.x] = (unsigned long long)(t1 - t0);
}

template <int MODE>
void run_consume(const char* tag) {
  const size_t smem = 8 * 3 * kR * kChunk + 2048 * 4;
  CK(cudaFuncSetAttribute(consume_rate<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  uint4* fill;
  float* y;
  unsigned long long* cyc;
  CK(cudaMalloc(&fill, 4096 * 16));
  CK(cudaMemset(fill, 0x11, 4096 * 16));
  CK(cudaMalloc(&y, 148 * 8 * 4));
  CK(cudaMalloc(&cyc, 148 * 8));
  const int rep = 2000;
  cudaEvent_t e0, e1;
  CK(cudaEventCreate(&e0));
  CK(cudaEventCreate(&e1));
  consume_rate<MODE><<<148, 256, smem>>>(fill, y, cyc, rep);
  CK(cudaGetLastError());
  CK(cudaEventRecord(e0));
  consume_rate<MODE><<<148, 256, smem>>>(fill, y, cyc, rep);
  CK(cudaEventRecord(e1));
  CK(cudaGetLastError());
  CK(cudaDeviceSynchronize());
  float ms = 0.f;
  CK(cudaEventElapsedTime(&ms, e0, e1));
  std::vector<unsigned long long> h(148);
  CK(cudaMemcpy(h.data(), cyc, 148 * 8, cudaMemcpyDeviceToHost));
  double avg = 0;
  for (auto c : h) avg += (double)c;
  avg /= 148;
  const double bytes = 8.0 * 3 * kR * kChunk * rep;
  printf("consume from shared memory, %-36s: %.1f bytes of weights per clock per SM (%.0f GB/s per SM by the event clock; HBM delivers ~23 B/clk)\n",
         tag, bytes / avg, bytes / (ms * 1e-3) * 1e-9);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(fill);
  cudaFree(y);
  cudaFree(cyc);
}

Mat mk(uint32_t N, uint32_t K) {
  Mat m;
  m.N = N;
  m.K = K;
  CK(cudaMalloc(&m.W, (size_t)N * K * 2));
  CK(cudaMemset(m.W, 0x11, (size_t)N * K * 2));
  return m;
}

}  // namespace

int main() {
  for (int l = 0; l < L; ++l) {
    qkv[l] = mk(3072, 2048);
    o[l] = mk(2048, 2048);
    gu[l] = mk(16384, 2048);
    dn[l] = mk(2048, 8192);
  }
  head = mk(128256, 2048);
  CK(cudaMalloc(&xa, 8192 * 4)); CK(cudaMalloc(&xb, 8192 * 4)); CK(cudaMalloc(&qbuf, 8192 * 4)); CK(cudaMalloc(&abuf, 8192 * 4));
  CK(cudaMalloc(&hbuf, 16384 * 4)); CK(cudaMalloc(&lg, 128256 * 4)); CK(cudaMalloc(&cache, 32 * 1536 * 16));
  CK(cudaMalloc(&g_ts, 8 * 8 * 128));
  CK(cudaMemset(xa, 0, 8192 * 4)); CK(cudaMemset(xb, 0, 8192 * 4)); CK(cudaMemset(qbuf, 0, 8192 * 4)); CK(cudaMemset(abuf, 0, 8192 * 4));
  CK(cudaMemset(hbuf, 0, 16384 * 4)); CK(cudaMemset(cache, 0, 32 * 1536 * 16));
  CK(cudaFuncSetAttribute(ring_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  CK(cudaFuncSetAttribute(ring_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  printf("weights per step 2.4715 GB: %.1f us at 6.55 TB/s\n", 2.4715e9 / 6.55e12 * 1e6);
  run("register streamer, 2 CTAs/SM", false, true, false);
  run("register streamer, 2 CTAs/SM", false, false, false);
  run("shared-memory rings, 1 CTA/SM", true, true, false);
  run("shared-memory rings, 1 CTA/SM", true, false, false);
  run("register streamer, 2 CTAs/SM", false, true, true);
  run("shared-memory rings, 1 CTA/SM", true, true, true);
  run_consume<0>("x beside the weights, natural order");
  run_consume<1>("x beside the weights, no conflicts");
  run_consume<2>("x in registers");
  return 0;
}
