// The tensor-parallel exchange protocol, written once for the device kernels and for the host model of it.
//
// Every rank owns an exchange area in its own memory that all ranks can write:
//   slots[parity][src][kMaxH]   float32 partial vectors, one per source rank, two parities
//   flags[src]                  the epoch of the last exchange whose vector `src` has delivered here
//   pair_slots[parity][src]     (value bits, index) of `src`'s best logit, for the arg-max exchange
//   pair_flags[src]             the same kind of epoch word for the pair exchange
// One exchange = every rank stores its partial vector into ITS slot in EVERY rank's area, then publishes the
// exchange's epoch into its flag word in every area with release semantics. A consumer waits (bounded) until all
// flags in its OWN area have reached the epoch, and sums the slots of its own area in rank order: the same order
// on every rank, so all ranks compute bit-identical results. Nothing ever reads another rank's memory.
//
// Epochs count exchanges since the context was created (mod 2^32, compared with wrap-around). Two parities are
// enough: a rank can run at most one exchange ahead of the slowest one, because publishing exchange e+1 comes after
// consuming exchange e, which needs every rank's flag for e.
//
// The memory operations are a policy (`Mem`): on the device they are system-scope PTX loads and stores over
// NVLink, in the host model they are C++ atomics shared by CPU threads. The reference has no counterpart (one
// device); the sums this protocol produces stand where the host residual adds of
// NFAI.Vulkan.Shaders/TransformerBlock.cs:151-161,174-181 stand.
#pragma once
#include <stddef.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define NFAI_XHD __host__ __device__ __forceinline__
#else
#define NFAI_XHD inline
#endif

namespace nfai {
namespace xchg {

constexpr uint32_t kMaxH = 16384;  // longest vector one exchange carries
constexpr int kMaxWorld = 8;

// Byte layout of one rank's exchange area.
constexpr size_t kSlotFloats = (size_t)2 * kMaxWorld * kMaxH;
constexpr size_t kFlagsOffset = kSlotFloats * 4;                    // kMaxWorld words, padded to 256 bytes
constexpr size_t kPairSlotsOffset = kFlagsOffset + 256;             // [2][kMaxWorld] x 8 bytes
constexpr size_t kPairFlagsOffset = kPairSlotsOffset + 256;         // kMaxWorld words
constexpr size_t kLocalOffset = kPairFlagsOffset + 256;             // words only this rank touches (epoch, tickets)
constexpr size_t kAreaBytes = kLocalOffset + 256;

NFAI_XHD uint32_t parity_of(uint32_t epoch) { return epoch & 1u; }

// Offset (in floats) of `src`'s vector for the exchange `epoch` inside one area's slots.
NFAI_XHD size_t slot_offset(uint32_t epoch, int src) { return ((size_t)parity_of(epoch) * kMaxWorld + (size_t)src) * kMaxH; }

// Index of `src`'s pair for the exchange `epoch` inside one area's pair slots.
NFAI_XHD size_t pair_index(uint32_t epoch, int src) { return (size_t)parity_of(epoch) * kMaxWorld + (size_t)src; }

// Has a flag word reached `epoch`? Wrap-around safe as long as ranks stay within 2^31 exchanges of each other.
NFAI_XHD bool reached(uint32_t seen, uint32_t epoch) { return (int32_t)(seen - epoch) >= 0; }

// The view one rank has of all areas.
struct View {
  float* slots[kMaxWorld];
  uint32_t* flags[kMaxWorld];
  unsigned long long* pair_slots[kMaxWorld];
  uint32_t* pair_flags[kMaxWorld];
  int rank, world;
};

NFAI_XHD View make_view(char* const* area_base, int rank, int world) {
  View v{};
  v.rank = rank;
  v.world = world;
  for (int r = 0; r < world && r < kMaxWorld; ++r) {
    v.slots[r] = reinterpret_cast<float*>(area_base[r]);
    v.flags[r] = reinterpret_cast<uint32_t*>(area_base[r] + kFlagsOffset);
    v.pair_slots[r] = reinterpret_cast<unsigned long long*>(area_base[r] + kPairSlotsOffset);
    v.pair_flags[r] = reinterpret_cast<uint32_t*>(area_base[r] + kPairFlagsOffset);
  }
  return v;
}

// ---- producer side ---------------------------------------------------------------------------------------------
// Store element i of this rank's partial vector into its slot on every rank.
template <class Mem>
NFAI_XHD void push_value(Mem& mem, const View& v, uint32_t epoch, uint32_t i, float value) {
  const size_t off = slot_offset(epoch, v.rank) + i;
  for (int dst = 0; dst < v.world; ++dst) mem.store_f32(v.slots[dst] + off, value);
}

// After ALL of this rank's values of the exchange are stored (and ordered before this call): tell every rank.
template <class Mem>
NFAI_XHD void publish(Mem& mem, const View& v, uint32_t epoch) {
  for (int dst = 0; dst < v.world; ++dst) mem.store_release_u32(v.flags[dst] + v.rank, epoch);
}

template <class Mem>
NFAI_XHD void push_pair(Mem& mem, const View& v, uint32_t epoch, float best, uint32_t index) {
  unsigned long long bits;
  {
    union { float f; uint32_t u; } cv;
    cv.f = best;
    bits = ((unsigned long long)index << 32) | cv.u;
  }
  for (int dst = 0; dst < v.world; ++dst) mem.store_u64(v.pair_slots[dst] + pair_index(epoch, v.rank), bits);
  mem.fence_system();
  for (int dst = 0; dst < v.world; ++dst) mem.store_release_u32(v.pair_flags[dst] + v.rank, epoch);
}

// ---- consumer side ---------------------------------------------------------------------------------------------
// Wait until rank `src`'s flag in this rank's own area has reached `epoch`; false when `budget_ns` ran out.
template <class Mem>
NFAI_XHD bool wait_flag(Mem& mem, const uint32_t* flag, uint32_t epoch, unsigned long long budget_ns) {
  if (reached(mem.load_acquire_u32(flag), epoch)) return true;
  const unsigned long long t0 = mem.now_ns();
  uint32_t polls = 0;
  while (true) {
    if (reached(mem.load_acquire_u32(flag), epoch)) return true;
    if ((++polls & 31u) == 0 && mem.now_ns() - t0 > budget_ns) return false;
  }
}

// Sum of element i over the ranks' slots of this rank's own area, in rank order, plus the residual.
template <class Mem>
NFAI_XHD float sum_slots(Mem& mem, const View& v, uint32_t epoch, uint32_t i, float resid) {
  const float* mine = v.slots[v.rank];
  float sum = 0.f;
  for (int src = 0; src < v.world; ++src) sum += mem.load_f32(mine + slot_offset(epoch, src) + i);
  return resid + sum;
}

// Best (value, lowest index) over the ranks' pairs of this rank's own area (index 0xffffffff = no candidate).
template <class Mem>
NFAI_XHD void best_pair(Mem& mem, const View& v, uint32_t epoch, float* best, uint32_t* index) {
  float bv = 0.f;
  uint32_t bi = 0xffffffffu;
  for (int src = 0; src < v.world; ++src) {
    const unsigned long long bits = mem.load_u64(v.pair_slots[v.rank] + pair_index(epoch, src));
    union { float f; uint32_t u; } cv;
    cv.u = (uint32_t)bits;
    const uint32_t ix = (uint32_t)(bits >> 32);
    if (ix != 0xffffffffu && (bi == 0xffffffffu || cv.f > bv || (cv.f == bv && ix < bi))) {
      bv = cv.f;
      bi = ix;
    }
  }
  *best = bv;
  *index = bi;
}

}  // namespace xchg
}  // namespace nfai
