// The tensor-parallel exchange protocol, written once for the device kernels and for the host model of it.
//
// Every rank owns an exchange area in its own memory that all ranks can write:
//   slots[parity][src][kMaxH]   one 8-byte word per element: (float32 bits, epoch) of `src`'s partial vector
//   pair_slots[parity][src][2]  two 8-byte words: (best logit bits, epoch) and (its global index, epoch)
// One exchange = every rank stores its partial vector, element by element, into ITS slot in EVERY rank's area. Each
// word carries the value together with the epoch of the exchange and is written with one 8-byte store, which the
// memory system delivers whole: a reader that sees the epoch it waits for also sees the value. There are no flags,
// fences or tickets, so an element can be consumed one NVLink latency after it was produced. A consumer polls
// (bounded) the words of its OWN area until each shows the epoch, and adds the values in rank order: the same order
// on every rank, so all ranks compute bit-identical results. Nothing ever reads another rank's memory.
//
// Epochs count exchanges since the context was created (mod 2^32; never 0, the value of fresh memory). Two parities
// are enough: a rank can run at most one exchange ahead of the slowest one, because producing exchange e+1 comes
// after consuming exchange e, which needs every rank's words of e; so a slot of parity e&1 is overwritten (by e+2)
// only after every rank has consumed e.
//
// The memory operations are a policy (`Mem`): on the device they are 8-byte stores into peer memory over NVLink and
// volatile loads of local memory, in the host model they are C++ atomics shared by CPU threads. The reference has no
// counterpart (one device); the sums this protocol produces stand where the host residual adds of
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
constexpr size_t kSlotWords = (size_t)2 * kMaxWorld * kMaxH;        // 8-byte words
constexpr size_t kPairSlotsOffset = kSlotWords * 8;                 // [2][kMaxWorld][2] words
constexpr size_t kLocalOffset = kPairSlotsOffset + 256;             // words only this rank touches (epoch counter)
constexpr size_t kAreaBytes = kLocalOffset + 256;

NFAI_XHD uint32_t parity_of(uint32_t epoch) { return epoch & 1u; }

// Index of the word of element 0 of `src`'s vector for the exchange `epoch` inside one area's slots.
NFAI_XHD size_t slot_offset(uint32_t epoch, int src) { return ((size_t)parity_of(epoch) * kMaxWorld + (size_t)src) * kMaxH; }

// Index of `src`'s first pair word for the exchange `epoch` inside one area's pair slots.
NFAI_XHD size_t pair_index(uint32_t epoch, int src) { return ((size_t)parity_of(epoch) * kMaxWorld + (size_t)src) * 2; }

NFAI_XHD unsigned long long pack(uint32_t bits, uint32_t epoch) { return ((unsigned long long)epoch << 32) | bits; }
NFAI_XHD uint32_t epoch_of(unsigned long long word) { return (uint32_t)(word >> 32); }
NFAI_XHD uint32_t bits_of(unsigned long long word) { return (uint32_t)word; }
NFAI_XHD uint32_t float_bits(float f) {
  union { float f; uint32_t u; } cv;
  cv.f = f;
  return cv.u;
}
NFAI_XHD float bits_float(uint32_t u) {
  union { float f; uint32_t u; } cv;
  cv.u = u;
  return cv.f;
}

// The view one rank has of all areas.
struct View {
  unsigned long long* slots[kMaxWorld];
  unsigned long long* pair_slots[kMaxWorld];
  int rank, world;
};

NFAI_XHD View make_view(char* const* area_base, int rank, int world) {
  View v{};
  v.rank = rank;
  v.world = world;
  for (int r = 0; r < world && r < kMaxWorld; ++r) {
    v.slots[r] = reinterpret_cast<unsigned long long*>(area_base[r]);
    v.pair_slots[r] = reinterpret_cast<unsigned long long*>(area_base[r] + kPairSlotsOffset);
  }
  return v;
}

// ---- producer side ---------------------------------------------------------------------------------------------
// Element i of this rank's partial vector goes into its slot on every rank.
template <class Mem>
NFAI_XHD void push_value(Mem& mem, const View& v, uint32_t epoch, uint32_t i, float value) {
  const size_t off = slot_offset(epoch, v.rank) + i;
  const unsigned long long word = pack(float_bits(value), epoch);
  for (int dst = 0; dst < v.world; ++dst) mem.store_u64(v.slots[dst] + off, word);
}

template <class Mem>
NFAI_XHD void push_pair(Mem& mem, const View& v, uint32_t epoch, float best, uint32_t index) {
  const size_t off = pair_index(epoch, v.rank);
  for (int dst = 0; dst < v.world; ++dst) {
    mem.store_u64(v.pair_slots[dst] + off, pack(float_bits(best), epoch));
    mem.store_u64(v.pair_slots[dst] + off + 1, pack(index, epoch));
  }
}

// ---- consumer side ---------------------------------------------------------------------------------------------
// Poll one word of this rank's own area until it carries `epoch`; false when `budget_ns` ran out.
template <class Mem>
NFAI_XHD bool wait_word(Mem& mem, const unsigned long long* word, uint32_t epoch, unsigned long long budget_ns,
                        uint32_t* bits) {
  unsigned long long w = mem.load_u64(word);
  if (epoch_of(w) != epoch) {
    const unsigned long long t0 = mem.now_ns();
    uint32_t polls = 0;
    while (true) {
      w = mem.load_u64(word);
      if (epoch_of(w) == epoch) break;
      if ((++polls & 31u) == 0 && mem.now_ns() - t0 > budget_ns) return false;
    }
  }
  *bits = bits_of(w);
  return true;
}

// Element i: residual + (sum over the ranks' slots of this rank's own area, from zero, in rank order).
// false when a word did not arrive in time (*out is then not written).
template <class Mem>
NFAI_XHD bool sum_slots(Mem& mem, const View& v, uint32_t epoch, uint32_t i, float resid, unsigned long long budget_ns,
                        float* out) {
  const unsigned long long* mine = v.slots[v.rank];
  float sum = 0.f;
  for (int src = 0; src < v.world; ++src) {
    uint32_t bits;
    if (!wait_word(mem, mine + slot_offset(epoch, src) + i, epoch, budget_ns, &bits)) return false;
    sum += bits_float(bits);
  }
  *out = resid + sum;
  return true;
}

// Best (value, lowest index) over the ranks' pairs of this rank's own area (index 0xffffffff = no candidate).
template <class Mem>
NFAI_XHD bool best_pair(Mem& mem, const View& v, uint32_t epoch, unsigned long long budget_ns, float* best, uint32_t* index) {
  float bv = 0.f;
  uint32_t bi = 0xffffffffu;
  for (int src = 0; src < v.world; ++src) {
    uint32_t vb, ix;
    const unsigned long long* p = v.pair_slots[v.rank] + pair_index(epoch, src);
    if (!wait_word(mem, p, epoch, budget_ns, &vb) || !wait_word(mem, p + 1, epoch, budget_ns, &ix)) return false;
    const float val = bits_float(vb);
    if (ix != 0xffffffffu && (bi == 0xffffffffu || val > bv || (val == bv && ix < bi))) {
      bv = val;
      bi = ix;
    }
  }
  *best = bv;
  *index = bi;
  return true;
}

}  // namespace xchg
}  // namespace nfai
