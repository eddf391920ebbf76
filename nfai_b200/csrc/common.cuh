// Shared device helpers for the sm_100a kernels of libnfai_cuda.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nfai {

constexpr int kWarp = 32;

// 16-byte streaming load of weights that are read exactly once per token: bypass L1 allocation so the
// activations and the KV cache keep their lines.
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Programmatic dependent launch: a kernel may start while its predecessor in the stream drains. Everything
// that reads the predecessor's output (or overwrites what it reads) must come after pdl_wait(); reads of
// weights and constant tables may come before it.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Memory operations of the tensor-parallel exchange protocol (xchg_protocol.h) on the device: one 8-byte store per
// word into peer memory over NVLink (delivered whole), volatile 8-byte loads of this GPU's own area (never served
// from L1: another GPU writes the lines).
struct DeviceXchgMem {
  __device__ __forceinline__ void store_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
  }
  __device__ __forceinline__ unsigned long long load_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
  }
  __device__ __forceinline__ unsigned long long now_ns() { return global_timer_ns(); }
};

// Ask the L2 for [ptr, ptr+bytes) of both ranges of a plan, the work split over every thread of the grid.
// Nothing waits for the data: it is a hint that keeps HBM busy for the kernels that follow.
template <typename Plan>
__device__ __forceinline__ void prefetch_plan(const Plan& pf, uint32_t chunk) {
  const unsigned long long nthreads = (unsigned long long)gridDim.x * gridDim.y * blockDim.x;
  const unsigned long long gtid =
      ((unsigned long long)blockIdx.y * gridDim.x + blockIdx.x) * blockDim.x + threadIdx.x;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const char* base = pf.ptr[r];
    const unsigned long long bytes = pf.bytes[r];
    if (bytes == 0) continue;
    if (pf.mode == 0) {
      for (unsigned long long off = gtid * 128ull; off < bytes; off += nthreads * 128ull)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(base + off));
    } else {
      // one lane per warp issues bulk prefetches; sizes are multiples of 16 bytes (the plan is 256-byte aligned)
      if ((threadIdx.x & 31) == 0) {
        const unsigned long long nwarps = nthreads >> 5, gw = gtid >> 5;
        for (unsigned long long off = gw * chunk; off < bytes; off += nwarps * chunk) {
          unsigned long long n = bytes - off < chunk ? bytes - off : chunk;
          n &= ~15ull;
          if (n) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base + off), "r"((uint32_t)n) : "memory");
        }
      }
    }
  }
}

// Unpack a 16-byte vector of weights into float32 (exact widening).
template <typename WT>
struct WeightVec;

template <>
struct WeightVec<__half> {
  static constexpr int kElems = 8;
  __device__ __forceinline__ static void unpack(const uint4& v, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __half22float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
};

template <>
struct WeightVec<float> {
  static constexpr int kElems = 4;
  __device__ __forceinline__ static void unpack(const uint4& v, float (&f)[4]) {
    f[0] = __uint_as_float(v.x);
    f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z);
    f[3] = __uint_as_float(v.w);
  }
};

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
__device__ __forceinline__ void store_as(float* p, float v) { *p = v; }
__device__ __forceinline__ void store_as(__half* p, float v) { *p = __float2half_rn(v); }

}  // namespace nfai
