// Host model of the tensor-parallel exchange: the ranks are CPU threads, the exchange areas are host memory, and
// the protocol code is the very header the device kernels compile (nfai_b200/csrc/xchg_protocol.h) with a memory
// policy made of C++ atomics instead of system-scope PTX.
//
//   xchg_model <world> <exchanges> <H> [stall_rank stall_at]
//
// Every rank runs `exchanges` rounds shaped like a one-layer decode step: two vector exchanges back to back (push a
// partial vector as (value, epoch) words, poll the own area until every word carries the epoch (bounded), sum in rank
// order with a residual), then the arg-max pair exchange. The only synchronisation is the 8-byte word itself
// (relaxed atomics here, single 8-byte stores on the device). Ranks are delayed at random so that they drift as far apart
// as the protocol allows. Checked: every rank computes bit-identical sums, equal to the sum taken in rank order on
// one thread; the pair exchange picks the lowest index among equal maxima; epochs survive the 2^32 wrap.
// With stall_rank/stall_at, that rank stops before publishing exchange stall_at: the others must give up after
// their wait budget with a time-out status -- no thread may hang -- and their earlier results must still be right.
// Exit code 0 = all checks passed.
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <thread>
#include <vector>

#include "xchg_protocol.h"

using namespace nfai::xchg;

struct HostMem {
  void store_u64(unsigned long long* p, unsigned long long v) { __atomic_store_n(p, v, __ATOMIC_RELAXED); }
  unsigned long long load_u64(const unsigned long long* p) { return __atomic_load_n(p, __ATOMIC_RELAXED); }
  unsigned long long now_ns() {
    return (unsigned long long)std::chrono::duration_cast<std::chrono::nanoseconds>(
               std::chrono::steady_clock::now().time_since_epoch())
        .count();
  }
};

static float partial_of(int rank, uint32_t e, uint32_t i) {
  // values whose float32 sum depends on the order of the additions
  uint32_t h = (uint32_t)rank * 2654435761u ^ e * 40503u ^ i * 2246822519u;
  h ^= h >> 15;
  return ((int)(h % 20001) - 10000) * (1.0f / 3.0f) * (rank % 2 ? 1e-3f : 1.0f);
}

int main(int argc, char** argv) {
  const int world = argc > 1 ? atoi(argv[1]) : 4;
  const uint32_t rounds = argc > 2 ? (uint32_t)atoi(argv[2]) : 200;
  const uint32_t H = argc > 3 ? (uint32_t)atoi(argv[3]) : 64;
  const int stall_rank = argc > 5 ? atoi(argv[4]) : -1;
  const uint32_t stall_at = argc > 5 ? (uint32_t)atoi(argv[5]) : 0;
  if (world < 1 || world > kMaxWorld || H == 0 || H > kMaxH) return 2;
  const unsigned long long budget_ns = stall_rank >= 0 ? 20ull * 1000 * 1000 : 5ull * 1000 * 1000 * 1000;
  // epochs start just below the 32-bit wrap so that the comparison is exercised across it
  // three epochs per round: the count passes the 32-bit wrap a third of the way in (epoch 0 then names an exchange
  // whose slots have long been written, so it cannot be mistaken for fresh memory)
  const uint32_t epoch0 = 0xffffffffu - rounds;

  std::vector<std::vector<char>> areas(world, std::vector<char>(kAreaBytes));
  std::vector<char*> base(world);
  for (int r = 0; r < world; ++r) {
    base[r] = areas[r].data();
  }
  std::vector<std::vector<float>> results(world, std::vector<float>((size_t)2 * rounds * H, 0.f));
  std::vector<std::vector<uint32_t>> winners(world, std::vector<uint32_t>(rounds, 0));
  std::vector<uint32_t> completed(world, 0);
  std::vector<int> timed_out(world, 0);

  auto rank_main = [&](int rank) {
    HostMem mem;
    View v = make_view(base.data(), rank, world);
    std::mt19937 rng(1234 + rank);
    for (uint32_t e = 0; e < rounds; ++e) {
      if (rank == stall_rank && e == stall_at) return;  // this rank is gone: it never publishes again
      for (uint32_t half = 0; half < 2; ++half) {
        const uint32_t epoch = epoch0 + 3 * e + 1 + half;  // consecutive epochs: the two parities alternate
        if (rng() % 4 == 0) std::this_thread::sleep_for(std::chrono::microseconds(rng() % 200));
        for (uint32_t i = 0; i < H; ++i) push_value(mem, v, epoch, i, partial_of(rank, 2 * e + half, i));
        for (uint32_t i = 0; i < H; ++i) {
          float x;
          if (!sum_slots(mem, v, epoch, i, 0.25f * i, budget_ns, &x)) {
            timed_out[rank] = 1;
            return;
          }
          results[rank][((size_t)2 * e + half) * H + i] = x;
        }
      }
      // pair exchange: ranks r and r^1 tie on the value, the lower global index must win
      const uint32_t pe = epoch0 + 3 * e + 3;
      push_pair(mem, v, pe, (float)((e + rank / 2) % 7), 1000u * (uint32_t)rank + e % 5);
      float bv;
      uint32_t bi;
      if (!best_pair(mem, v, pe, budget_ns, &bv, &bi)) {
        timed_out[rank] = 1;
        return;
      }
      winners[rank][e] = bi;
      completed[rank] = e + 1;
    }
  };
  std::vector<std::thread> th;
  for (int r = 0; r < world; ++r) th.emplace_back(rank_main, r);
  for (auto& t : th) t.join();  // returns only if nothing hangs

  int bad = 0;
  for (int r = 0; r < world; ++r) {
    const uint32_t want_done = stall_rank < 0 ? rounds : (r == stall_rank ? stall_at : stall_at);
    if (stall_rank < 0 && (completed[r] != rounds || timed_out[r])) { printf("rank %d completed %u of %u\n", r, completed[r], rounds); ++bad; }
    if (stall_rank >= 0 && r != stall_rank && !timed_out[r]) { printf("rank %d did not time out\n", r); ++bad; }
    if (stall_rank >= 0 && completed[r] != want_done) { printf("rank %d completed %u, expected %u\n", r, completed[r], want_done); ++bad; }
    for (uint32_t e = 0; e < completed[r]; ++e) {
      for (uint32_t x = 2 * e; x < 2 * e + 2; ++x)
        for (uint32_t i = 0; i < H; ++i) {
          float sum = 0.f;
          for (int src = 0; src < world; ++src) sum += partial_of(src, x, i);
          const float want = 0.25f * i + sum;
          const float got = results[r][(size_t)x * H + i];
          if (memcmp(&want, &got, 4) != 0) {
            if (bad < 5) printf("rank %d exchange %u element %u: %.9g != %.9g\n", r, x, i, got, want);
            ++bad;
          }
        }
      float bv = 0.f;
      uint32_t bi = 0xffffffffu;
      for (int src = 0; src < world; ++src) {
        const float val = (float)((e + src / 2) % 7);
        const uint32_t ix = 1000u * (uint32_t)src + e % 5;
        if (bi == 0xffffffffu || val > bv || (val == bv && ix < bi)) { bv = val; bi = ix; }
      }
      if (winners[r][e] != bi) { if (bad < 5) printf("rank %d exchange %u winner %u != %u\n", r, e, winners[r][e], bi); ++bad; }
    }
  }
  printf("%s world=%d rounds=%u H=%u stall=%d\n", bad ? "FAILED" : "ok", world, rounds, H, stall_rank);
  return bad ? 1 : 0;
}
