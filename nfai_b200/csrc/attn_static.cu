// nfai_op_attn_decode_static: the split-KV attention kernel with its scratch in a fixed device array, so that the
// call performs no device allocation and needs no scratch pointer from the caller.
//
// Who needs this: hosts that may not allocate device memory at the point where they run attention -- an engine that
// was handed a fixed device-memory budget by an embedding application and has spent it, or a serving loop that must
// not pay cudaMalloc's device-wide synchronisation between tokens. nfai_op_attn_decode makes such a caller size and
// own a scratch buffer; this variant carries its own.
//
// The array below is part of the library image: every GPU on which the library is loaded holds kStaticScratchBytes
// of it from load until the process exits, whether or not this entry point is ever called.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/nfai_cuda.h"
#include "kernels.h"

struct nfai_ctx;

namespace nfai {
int ctx_device(const nfai_ctx* c);
cudaStream_t ctx_stream(const nfai_ctx* c);
int ctx_fail(nfai_ctx* c, int code, const char* message);
}  // namespace nfai

namespace {

constexpr size_t kStaticScratchBytes = 256u << 10;  // 256 KiB: 24 query heads x 18 splits x head dim 128 needs 220 KiB
constexpr int kMaxDevices = 64;

// Split partials followed by the ticket counters. In host code this name is only a stand-in for the device
// object: its device address comes from cudaGetSymbolAddress, once per device.
static __device__ __align__(256) unsigned char g_attn_scratch[kStaticScratchBytes];

std::mutex g_setup_mutex;
void* g_scratch_ptr[kMaxDevices] = {};

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

}  // namespace

extern "C" int nfai_op_attn_decode_static(nfai_ctx* c, const float* q, const void* kcache, const void* vcache,
                                          int kv_dtype, uint32_t seq, uint32_t qH, uint32_t kvH, uint32_t d,
                                          float* out) {
  using namespace nfai;
  if (!c) return NFAI_ERR_ARG;
  if (!q || !kcache || !vcache || !out || (kv_dtype != NFAI_F32 && kv_dtype != NFAI_F16) || !seq || !qH || !kvH ||
      qH % kvH || (d != 32 && d != 64 && d != 128))
    return ctx_fail(c, NFAI_ERR_ARG, "bad argument");
  if (((uintptr_t)kcache | (uintptr_t)vcache | (uintptr_t)q) & 15)
    return ctx_fail(c, NFAI_ERR_ARG, "pointers must be 16-byte aligned");
  const size_t need = nfai_op_attn_scratch_bytes(qH, kvH, d, seq);
  if (need == 0 || need > kStaticScratchBytes)
    return ctx_fail(c, NFAI_ERR_ARG,
                    "this geometry needs more split scratch than the 256 KiB built into the library; use "
                    "nfai_op_attn_decode with a caller-owned scratch buffer");
  const int dev = ctx_device(c);
  if (dev < 0 || dev >= kMaxDevices) return ctx_fail(c, NFAI_ERR_ARG, "device ordinal beyond the static scratch table");
  cudaError_t e = cudaSetDevice(dev);
  if (e != cudaSuccess) return ctx_fail(c, NFAI_ERR_CUDA, cudaGetErrorString(e));
  void* scratch = nullptr;
  {
    // set-up, once per device, with that device current: resolve the array's device address
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_ptr[dev]) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_attn_scratch);
      if (e != cudaSuccess) return ctx_fail(c, NFAI_ERR_CUDA, cudaGetErrorString(e));
      if (!p) return ctx_fail(c, NFAI_ERR_CUDA, "cudaGetSymbolAddress gave a null address for the built-in scratch array");
      g_scratch_ptr[dev] = p;
    }
    scratch = g_scratch_ptr[dev];
  }
  cudaStream_t s = ctx_stream(c);
  AttnParams a;
  a.q = q;
  a.kcache = kcache;
  a.vcache = vcache;
  a.qH = qH;
  a.kvH = kvH;
  a.d = d;
  a.seq_imm = seq;
  a.out = out;
  a.S_max = attn_splits(qH, kvH, seq);
  a.part = (float*)scratch;
  const size_t tick_off = align256(attn_part_floats(qH, d, a.S_max) * 4);
  a.tickets = (uint32_t*)((char*)scratch + tick_off);
  // the array keeps whatever the previous call left: the ticket counters must start at zero (the partials are
  // fully written before they are read)
  e = cudaMemsetAsync(a.tickets, 0, (size_t)kvH * attn_head_groups(qH, kvH) * 4, s);
  if (e == cudaSuccess) e = launch_attn_decode(s, kv_dtype, a, false);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return ctx_fail(c, e == cudaErrorInvalidValue ? NFAI_ERR_ARG : NFAI_ERR_CUDA, cudaGetErrorString(e));
  return NFAI_OK;
}
