// Descriptor of the fused decode step (internal).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"

namespace nfai {

struct LayerDesc {
  const void* qkv;
  const void* o;
  const void* gateup;
  const void* down;
  const float* attn_norm;
  const float* ffn_norm;
};

struct StepDesc {
  uint32_t H, L, qH, kvH, d, ropeDim, F, V, ctx;  // local (per-rank) head counts and widths
  float eps;
  const void* embd;       // [V_total][H], replicated
  uint32_t embd_rows;     // V_total (token ids are checked against it)
  const void* head;       // [V][H] rows of this rank
  const float* out_norm;
  const float2* rope_cs;
  StepState* state;
  const uint32_t* prompt;  // non-null: head-less prompt step, token = prompt[state->prompt_idx]
  float* xbuf;             // [(2L+1)][H]
  float* q;
  float* attn_out;
  float* hbuf;
  float* logits;
  float* part_val;
  uint32_t* part_idx;
  float* attn_part;
  uint32_t* tickets;
  uint32_t S_max;
  uint32_t attn_heads;      // query heads per attention CTA (ring variant: 1 or 4)
  uint32_t attn_min_chunk;  // fewest positions per attention CTA before the range is split
  void* kc;
  void* vc;
  unsigned long long kv_layer_bytes;
  uint32_t* sync_counter;  // zeroed before every launch
  uint32_t* abort_flag;
  uint32_t* history;
  uint32_t history_cap;
  int with_head;
  const LayerDesc* layers;
  unsigned long long* trace;  // optional: CTA 0 stamps %globaltimer after every barrier and at every phase end
};
constexpr int kTraceSlots = 2048;

constexpr uint32_t kMegaMinChunk = 256;  // fewest positions one attention CTA takes inside the fused step
constexpr uint32_t kMegaHeadsPerCta = 2;

// Shared memory the kernel needs, the largest grid that is co-resident, and the launch itself.
size_t megastep_smem(uint32_t H, uint32_t F, uint32_t qDim);
cudaError_t megastep_max_grid(int wdtype, int kvdtype, uint32_t d, size_t smem, int* grid_out);
cudaError_t launch_megastep(cudaStream_t s, int wdtype, int kvdtype, uint32_t d, const StepDesc* desc_dev, int grid,
                            size_t smem);

// Ring variant (fused_ring.cu): weights stream through per-warp shared-memory rings across the grid barriers.
cudaError_t fused_ring_prepare(int wdtype, int kvdtype, uint32_t d, uint32_t H, uint32_t F, uint32_t qDim, int* grid_out,
                               int* stages_out, size_t* smem_out);
cudaError_t launch_fused_ring(cudaStream_t s, int wdtype, int kvdtype, uint32_t d, const StepDesc* desc_dev, int grid,
                              size_t smem, int stages);

}  // namespace nfai
