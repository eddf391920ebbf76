// Tensor-parallel exchange: NCCL all-reduce after the O and down projections, arg-max pair gather after the
// vocabulary-sharded LM head. The reference has no counterpart (single device).
#include "tp.h"

#include <dlfcn.h>
#include <nccl.h>
#include <string.h>
#include <unistd.h>

#include "../../include/nfai_cuda.h"
#include "common.cuh"

namespace nfai {

namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

NcclApi g_nccl;

bool load_nccl(std::string& err) {
  if (g_nccl.handle) return true;
  const char* names[] = {"libnccl.so.2", "libnccl.so"};
  void* h = nullptr;
  for (const char* n : names) {
    h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (h) break;
  }
  if (!h) {
    err = std::string("cannot load NCCL: ") + dlerror();
    return false;
  }
  NcclApi a;
  a.handle = h;
#define SYM(field, name)                                      \
  a.field = (decltype(a.field))dlsym(h, name);                \
  if (!a.field) {                                             \
    err = std::string("NCCL symbol missing: ") + name;        \
    return false;                                             \
  }
  SYM(GetUniqueId, "ncclGetUniqueId");
  SYM(CommInitRank, "ncclCommInitRank");
  SYM(CommDestroy, "ncclCommDestroy");
  SYM(AllReduce, "ncclAllReduce");
  SYM(AllGather, "ncclAllGather");
  SYM(GetErrorString, "ncclGetErrorString");
#undef SYM
  g_nccl = a;
  return true;
}

__global__ void add_residual_kernel(const float* __restrict__ sum, const float* __restrict__ resid,
                                    float* __restrict__ out, uint32_t n) {
  uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = resid[i] + sum[i];
}

// One CTA: this rank's partials -> (max, lowest global index) at pairs[rank].
__global__ void __launch_bounds__(256) local_argmax_kernel(const float* __restrict__ part_val,
                                                          const uint32_t* __restrict__ part_idx, uint32_t nparts,
                                                          uint32_t v_lo, uint2* pairs, int rank) {
  __shared__ float sv[256];
  __shared__ uint32_t si[256];
  float bv = -INFINITY;
  uint32_t bi = 0xffffffffu;
  for (uint32_t i = threadIdx.x; i < nparts; i += blockDim.x) {
    float v = part_val[i];
    uint32_t ix = part_idx[i];
    if (ix != 0xffffffffu && (bi == 0xffffffffu || v > bv || (v == bv && ix < bi))) {
      bv = v;
      bi = ix;
    }
  }
  sv[threadIdx.x] = bv;
  si[threadIdx.x] = bi;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) {
      float v = sv[threadIdx.x + o], cv = sv[threadIdx.x];
      uint32_t ix = si[threadIdx.x + o], ci = si[threadIdx.x];
      if (ix != 0xffffffffu && (ci == 0xffffffffu || v > cv || (v == cv && ix < ci))) {
        sv[threadIdx.x] = v;
        si[threadIdx.x] = ix;
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) pairs[rank] = make_uint2(__float_as_uint(sv[0]), si[0] == 0xffffffffu ? 0xffffffffu : si[0] + v_lo);
}

__global__ void unpack_pairs_kernel(const uint2* __restrict__ pairs, int world, float* part_val, uint32_t* part_idx) {
  int i = threadIdx.x;
  if (i < world) {
    part_val[i] = __uint_as_float(pairs[i].x);
    part_idx[i] = pairs[i].y;
  }
}

}  // namespace

// Peer-memory exchange area of one rank, written by every rank (this one included) over NVLink; layout and
// protocol in xchg_protocol.h.
struct PeerDesc {  // 128 bytes on the wire
  int32_t pid;
  int32_t device;
  uint64_t ptr;
  cudaIpcMemHandle_t handle;  // 64 bytes
  char pad[kTpPeerDescBytes - 16 - sizeof(cudaIpcMemHandle_t)];
};
static_assert(sizeof(PeerDesc) == kTpPeerDescBytes, "descriptor layout");

struct TpComm {
  int device = 0, rank = 0, world = 1;
  ncclComm_t comm = nullptr;
  uint2* pairs = nullptr;       // [world]
  float* full_logits = nullptr; // [world * Vl], allocated on first use
  size_t full_logits_elems = 0;
  char* push_local = nullptr;   // this rank's exchange area (its own cudaMalloc: it is exported whole)
  void* push_opened[xchg::kMaxWorld] = {};  // IPC mappings to close
  xchg::View view{};
  bool push_ready = false;
  unsigned long long wait_ns = 1000000000ull;
};

int tp_unique_id(void* out, size_t out_bytes, std::string& err) {
  if (!out || out_bytes < sizeof(ncclUniqueId)) {
    err = "unique id buffer must hold 128 bytes";
    return NFAI_ERR_ARG;
  }
  if (!load_nccl(err)) return NFAI_ERR_NCCL;
  ncclUniqueId id;
  ncclResult_t r = g_nccl.GetUniqueId(&id);
  if (r != ncclSuccess) {
    err = std::string("ncclGetUniqueId: ") + g_nccl.GetErrorString(r);
    return NFAI_ERR_NCCL;
  }
  memcpy(out, &id, sizeof id);
  return NFAI_OK;
}

int tp_create(TpComm** out, int device, int rank, int world, const void* uid, size_t uid_bytes, cudaStream_t s,
              std::string& err) {
  (void)s;
  if (!uid || uid_bytes < sizeof(ncclUniqueId)) {
    err = "nccl unique id missing";
    return NFAI_ERR_ARG;
  }
  if (!load_nccl(err)) return NFAI_ERR_NCCL;
  TpComm* tp = new TpComm();
  tp->device = device;
  tp->rank = rank;
  tp->world = world;
  ncclUniqueId id;
  memcpy(&id, uid, sizeof id);
  ncclResult_t r = g_nccl.CommInitRank(&tp->comm, world, id, rank);
  if (r != ncclSuccess) {
    err = std::string("ncclCommInitRank: ") + g_nccl.GetErrorString(r);
    delete tp;
    return NFAI_ERR_NCCL;
  }
  cudaError_t e = cudaMalloc((void**)&tp->push_local, xchg::kAreaBytes);  // own allocation: it is exported whole
  if (e == cudaSuccess) e = cudaMemset(tp->push_local, 0, xchg::kAreaBytes);
  if (e == cudaSuccess) e = cudaMalloc((void**)&tp->pairs, sizeof(uint2) * 8);
  if (e != cudaSuccess) {
    err = std::string("cudaMalloc: ") + cudaGetErrorString(e);
    g_nccl.CommDestroy(tp->comm);
    delete tp;
    return NFAI_ERR_OOM;
  }
  *out = tp;
  return NFAI_OK;
}

void tp_destroy(TpComm* tp) {
  if (!tp) return;
  for (int i = 0; i < xchg::kMaxWorld; ++i)
    if (tp->push_opened[i]) cudaIpcCloseMemHandle(tp->push_opened[i]);
  if (tp->push_local) cudaFree(tp->push_local);
  if (tp->comm) g_nccl.CommDestroy(tp->comm);
  if (tp->pairs) cudaFree(tp->pairs);
  if (tp->full_logits) cudaFree(tp->full_logits);
  delete tp;
}

// Baseline exchange (kept for comparison and for peers without mutual memory access): NCCL all-reduce of the
// partial vector, then one kernel that adds the residual.
cudaError_t tp_allreduce_residual(TpComm* tp, cudaStream_t s, float* buf, const float* resid, float* x_out, uint32_t H,
                                  int* launches) {
  ncclResult_t r = g_nccl.AllReduce(buf, buf, H, ncclFloat, ncclSum, tp->comm, s);
  if (r != ncclSuccess) return cudaErrorUnknown;
  add_residual_kernel<<<(H + 255) / 256, 256, 0, s>>>(buf, resid, x_out, H);
  if (launches) *launches += 1;
  return cudaGetLastError();
}

// Sum of buf[0..n) over the ranks, in place (prompt passes: [tokens][H] floats, megabytes, where NCCL over NVLink
// is the right tool). The result is bit-identical on every rank.
cudaError_t tp_allreduce(TpComm* tp, cudaStream_t s, float* buf, size_t n) {
  ncclResult_t r = g_nccl.AllReduce(buf, buf, n, ncclFloat, ncclSum, tp->comm, s);
  return r == ncclSuccess ? cudaSuccess : cudaErrorUnknown;
}

bool tp_push_ready(const TpComm* tp) { return tp->push_ready; }

// Hooks for the kernels of one step; the caller fills in pull / push and the exchange indices.
XchgHooks tp_hooks(TpComm* tp) {
  XchgHooks h;
  h.view = tp->view;
  h.epoch_base = tp_epoch_ptr(tp);
  h.wait_ns = tp->wait_ns;
  return h;
}

uint32_t* tp_ticket_ptr(TpComm* tp) { return tp_epoch_ptr(tp) + 2; }

void tp_set_wait_ns(TpComm* tp, unsigned long long ns) { tp->wait_ns = ns ? ns : 1; }

cudaError_t tp_gather_argmax(TpComm* tp, cudaStream_t s, float* part_val, uint32_t* part_idx, uint32_t nparts,
                             uint32_t v_lo, int* launches) {
  local_argmax_kernel<<<1, 256, 0, s>>>(part_val, part_idx, nparts, v_lo, tp->pairs, tp->rank);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  ncclResult_t r = g_nccl.AllGather(tp->pairs + tp->rank, tp->pairs, sizeof(uint2), ncclUint8, tp->comm, s);
  if (r != ncclSuccess) return cudaErrorUnknown;
  unpack_pairs_kernel<<<1, 32, 0, s>>>(tp->pairs, tp->world, part_val, part_idx);
  if (launches) *launches += 2;
  return cudaGetLastError();
}

uint32_t* tp_epoch_ptr(TpComm* tp) { return reinterpret_cast<uint32_t*>(tp->push_local + xchg::kLocalOffset); }

int tp_export_peer_desc(TpComm* tp, void* out, size_t out_bytes, std::string& err) {
  if (!out || out_bytes < kTpPeerDescBytes) {
    err = "peer descriptor buffer must hold 128 bytes";
    return NFAI_ERR_ARG;
  }
  PeerDesc d;
  memset(&d, 0, sizeof d);
  d.pid = (int32_t)getpid();
  d.device = tp->device;
  d.ptr = (uint64_t)(uintptr_t)tp->push_local;
  cudaError_t e = cudaIpcGetMemHandle(&d.handle, tp->push_local);
  if (e != cudaSuccess) {
    err = std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e);
    return NFAI_ERR_CUDA;
  }
  memcpy(out, &d, sizeof d);
  return NFAI_OK;
}

int tp_import_peer_descs(TpComm* tp, const void* descs, int n, std::string& err) {
  if (!descs || n != tp->world) {
    err = "one peer descriptor per rank is needed";
    return NFAI_ERR_ARG;
  }
  const PeerDesc* d = reinterpret_cast<const PeerDesc*>(descs);
  char* bases[xchg::kMaxWorld] = {};
  for (int r = 0; r < n; ++r) {
    char* base = nullptr;
    if (r == tp->rank) {
      base = tp->push_local;
    } else if (d[r].pid == (int32_t)getpid()) {
      // same process, another device: plain peer access to the other context's allocation
      int can = 0;
      cudaDeviceCanAccessPeer(&can, tp->device, d[r].device);
      if (!can) {
        err = "no peer access between the devices";
        return NFAI_ERR_CUDA;
      }
      cudaError_t e = cudaDeviceEnablePeerAccess(d[r].device, 0);
      if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
        err = std::string("cudaDeviceEnablePeerAccess: ") + cudaGetErrorString(e);
        return NFAI_ERR_CUDA;
      }
      cudaGetLastError();
      base = (char*)(uintptr_t)d[r].ptr;
    } else {
      void* p = nullptr;
      cudaError_t e = cudaIpcOpenMemHandle(&p, d[r].handle, cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess) {
        err = std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e);
        return NFAI_ERR_CUDA;
      }
      tp->push_opened[r] = p;
      base = (char*)p;
    }
    bases[r] = base;
  }
  tp->view = xchg::make_view(bases, tp->rank, tp->world);
  tp->push_ready = true;
  return NFAI_OK;
}

int tp_allgather_logits(TpComm* tp, cudaStream_t s, const float* logits_local, uint32_t Vl, float* host_out,
                        std::string& err) {
  size_t need = (size_t)Vl * tp->world;
  if (tp->full_logits_elems < need) {
    if (tp->full_logits) cudaFree(tp->full_logits);
    tp->full_logits = nullptr;
    cudaError_t e = cudaMalloc((void**)&tp->full_logits, need * 4);
    if (e != cudaSuccess) {
      err = std::string("cudaMalloc: ") + cudaGetErrorString(e);
      return NFAI_ERR_OOM;
    }
    tp->full_logits_elems = need;
  }
  ncclResult_t r = g_nccl.AllGather(logits_local, tp->full_logits, Vl, ncclFloat, tp->comm, s);
  if (r != ncclSuccess) {
    err = std::string("ncclAllGather: ") + g_nccl.GetErrorString(r);
    return NFAI_ERR_NCCL;
  }
  cudaError_t e = cudaMemcpyAsync(host_out, tp->full_logits, need * 4, cudaMemcpyDeviceToHost, s);
  if (e != cudaSuccess) {
    err = std::string("cudaMemcpyAsync: ") + cudaGetErrorString(e);
    return NFAI_ERR_CUDA;
  }
  return NFAI_OK;
}

}  // namespace nfai
