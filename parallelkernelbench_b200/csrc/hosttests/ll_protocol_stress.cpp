// Host stress of the no-barrier exchange protocol (data word + epoch word in one 8-byte store, two slot sets alternating by
// the parity of a per-rank epoch) with real threads as ranks. The device kernels use 8-byte volatile stores and loads of
// {data, epoch}; here they are relaxed 64-bit atomics, which is the same guarantee (single-copy atomicity of the pair, no
// ordering between different words). The reduction must be exact for every call although ranks drift apart by up to one
// call. Build with -fsanitize=thread to let ThreadSanitizer watch the non-atomic bookkeeping as well.
//   usage: ll_protocol_stress <ranks> <calls> <max_units> [single]     ("single" aliases the two slot sets: must FAIL)
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <thread>
#include <vector>

struct Rank {
  uint32_t epoch = 0;                                   // header word: read and written by its own rank only
  std::vector<std::atomic<uint64_t>> slots;             // [2 parities][world][cap]
};

static inline uint64_t pack(uint32_t data, uint32_t epoch) { return (uint64_t)epoch << 32 | data; }

int main(int argc, char** argv) {
  const int world = argc > 1 ? atoi(argv[1]) : 4, calls = argc > 2 ? atoi(argv[2]) : 2000, cap = argc > 3 ? atoi(argv[3]) : 64;
  const bool single = argc > 4 && strcmp(argv[4], "single") == 0;
  std::vector<Rank> ranks(world);
  for (auto& r : ranks) {
    r.slots = std::vector<std::atomic<uint64_t>>((size_t)2 * world * cap);
    for (auto& s : r.slots) s.store(0, std::memory_order_relaxed);
  }
  auto slot = [&](int rank, uint32_t parity, int src, int i) -> std::atomic<uint64_t>& {
    return ranks[rank].slots[((size_t)(single ? 0 : parity) * world + src) * cap + i];
  };
  // inputs are a pure function of (rank, call, unit) so that every thread can compute the expected sums itself
  auto input = [](int r, int c, int i) { return (uint32_t)((r + 1) * 2654435761u + c * 40503u + i * 9176u) & 0xffffu; };
  std::mt19937 seed_rng(7);
  std::vector<int> units(calls);
  for (auto& u : units) u = 1 + seed_rng() % cap;
  std::atomic<int> failures{0}, future{0}, timeouts{0};
  auto body = [&](int me) {
    std::mt19937 rng(100 + me);
    for (int c = 0; c < calls && !failures.load(std::memory_order_relaxed); ++c) {
      if (rng() % 16 == 0) std::this_thread::sleep_for(std::chrono::microseconds(rng() % 200));   // fall behind for a while
      const uint32_t epoch = ranks[me].epoch + 1, parity = epoch & 1u;
      for (int i = 0; i < units[c]; ++i)
        for (int g = 0; g < world; ++g) slot(g, parity, me, i).store(pack(input(me, c, i), epoch), std::memory_order_relaxed);
      const auto t0 = std::chrono::steady_clock::now();
      for (int i = 0; i < units[c]; ++i) {
        uint32_t acc = 0, want = 0;
        for (int g = 0; g < world; ++g) {
          uint64_t v;
          while ((uint32_t)((v = slot(me, parity, g, i).load(std::memory_order_relaxed)) >> 32) != epoch) {
            if ((uint32_t)(v >> 32) > epoch) { future.fetch_add(1); failures.fetch_add(1); return; }   // a word of a later call
            if (failures.load(std::memory_order_relaxed)) return;                        // another rank already failed
            if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(20)) { timeouts.fetch_add(1); failures.fetch_add(1); return; }
            std::this_thread::yield();
          }
          acc += (uint32_t)v;
          want += input(g, c, i);
        }
        if (acc != want) { failures.fetch_add(1); return; }
      }
      ranks[me].epoch = epoch;                             // "the last block advances the epoch"
    }
  };
  std::vector<std::thread> th;
  for (int r = 0; r < world; ++r) th.emplace_back(body, r);
  for (auto& t : th) t.join();
  printf("ranks=%d calls=%d failures=%d future_epoch=%d timeouts=%d %s\n", world, calls, failures.load(), future.load(), timeouts.load(),
         failures.load() ? "FAIL" : "OK");
  return failures.load() ? 1 : 0;
}
