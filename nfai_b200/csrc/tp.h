// Tensor-parallel exchange steps of the decode path (internal). NCCL is loaded at run time with dlopen so that
// single-GPU use needs no NCCL at all.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <string>

#include "kernels.h"

namespace nfai {

struct TpComm;

int tp_unique_id(void* out, size_t out_bytes, std::string& err);
int tp_create(TpComm** out, int device, int rank, int world, const void* uid, size_t uid_bytes, cudaStream_t s,
              std::string& err);
void tp_destroy(TpComm* tp);

// buf[0..H) holds this rank's partial sums; afterwards x_out = resid + sum over ranks (identical on every rank).
// *launches is advanced by the number of kernels of this library that were enqueued.
// Device word counting the exchanges completed on this context (advanced by the last kernel of every step).
uint32_t* tp_epoch_ptr(TpComm* tp);

// Baseline: NCCL all-reduce of buf[0..H) plus a residual-add kernel: x_out = resid + sum over ranks.
cudaError_t tp_allreduce_residual(TpComm* tp, cudaStream_t s, float* buf, const float* resid, float* x_out, uint32_t H,
                                  int* launches);

// In-place sum of buf[0..n) over the ranks with NCCL (the prompt path's [tokens][H] exchanges).
cudaError_t tp_allreduce(TpComm* tp, cudaStream_t s, float* buf, size_t n);

// After tp_import_peer_descs: the exchanges run inside the GEMV kernels (push in the epilogue of the producer, pull
// in the prologue of the consumer; xchg_protocol.h). tp_hooks gives the view, epoch word and wait budget.
bool tp_push_ready(const TpComm* tp);
XchgHooks tp_hooks(TpComm* tp);
// Local word for the "last CTA reduces" ticket of the vocabulary-sharded LM head.
uint32_t* tp_ticket_ptr(TpComm* tp);
void tp_set_wait_ns(TpComm* tp, unsigned long long ns);

// Peer-memory exchange buffers. Every rank exports a 128-byte descriptor of its buffer (process id, device
// pointer, CUDA IPC handle); the host gathers the descriptors of all ranks and hands them to every rank. After the
// import the all-reduce runs as this library's own kernel over NVLink stores instead of an NCCL call.
constexpr size_t kTpPeerDescBytes = 128;
int tp_export_peer_desc(TpComm* tp, void* out, size_t out_bytes, std::string& err);
int tp_import_peer_descs(TpComm* tp, const void* descs, int n, std::string& err);

// part_val/part_idx hold nparts per-CTA arg-max partials with rank-local row indices; afterwards entries
// [0, world) hold one (max, global lowest index) pair per rank, on every rank.
cudaError_t tp_gather_argmax(TpComm* tp, cudaStream_t s, float* part_val, uint32_t* part_idx, uint32_t nparts,
                             uint32_t v_lo, int* launches);

// All ranks' logits shards, in rank order, into pinned host memory (V = world * Vl floats).
int tp_allgather_logits(TpComm* tp, cudaStream_t s, const float* logits_local, uint32_t Vl, float* host_out,
                        std::string& err);

}  // namespace nfai
