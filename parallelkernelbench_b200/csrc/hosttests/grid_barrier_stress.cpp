// Host model of the grid-wide cross-rank barrier (`symm_grid_barrier`): every "block" is a thread, R ranks x B blocks.
// Memory orders mirror the device code: arrive = __threadfence + atomicAdd (release RMW), block 0 waits with acquire loads,
// exchanges release-stored / acquire-polled epoch flags with block 0 of every peer, resets the arrive counter and
// release-stores the rank's release word, which the other blocks poll with acquire loads.
// The payload is written with PLAIN stores before the barrier and read with plain loads after it, by a different block index
// of a different rank - exactly the access pattern the barrier exists for - so under -fsanitize=thread any missing
// happens-before edge is reported as a data race, and without the sanitizer a stale value fails the check.
//   usage: grid_barrier_stress <ranks> <blocks> <iterations> [blockonly]
// "blockonly" replaces the barrier by the per-block-index form (same-index blocks of all ranks only), which does NOT order a
// block against other block indices: the cross-index read must then be caught (it is the defect the grid-wide form fixed).
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <thread>
#include <vector>

struct RankState {
  std::atomic<uint32_t> arrive{0}, release{0};
  std::vector<std::atomic<uint32_t>> flags;   // flags[p]: epoch published by rank p's block 0
  uint32_t epoch0 = 0;                        // block 0 only
  std::vector<uint32_t> payload;              // payload[b]: plain data written by block b
  std::vector<std::atomic<uint32_t>> bflags;  // block-only form: bflags[b * R + p]
  std::vector<uint32_t> bepoch;               // block-only form: epoch of block b
};

int main(int argc, char** argv) {
  const int R = argc > 1 ? atoi(argv[1]) : 4, B = argc > 2 ? atoi(argv[2]) : 6, iters = argc > 3 ? atoi(argv[3]) : 2000;
  const bool block_only = argc > 4 && strcmp(argv[4], "blockonly") == 0;
  std::vector<RankState> rk(R);
  for (auto& r : rk) {
    r.flags = std::vector<std::atomic<uint32_t>>(R);
    for (auto& f : r.flags) f.store(0);
    r.payload.assign(B, 0);
    r.bflags = std::vector<std::atomic<uint32_t>>((size_t)B * R);
    for (auto& f : r.bflags) f.store(0);
    r.bepoch.assign(B, 0);
  }
  std::atomic<int> failures{0};
  auto wait_ge = [&](std::atomic<uint32_t>& w, uint32_t target) {
    const auto t0 = std::chrono::steady_clock::now();
    while ((int32_t)(w.load(std::memory_order_acquire) - target) < 0) {
      if (failures.load(std::memory_order_relaxed)) return false;      // another block already failed: do not wait for it
      if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(30)) return false;
      std::this_thread::yield();
    }
    return true;
  };
  auto barrier = [&](int r, int b) -> bool {
    RankState& me = rk[r];
    if (block_only) {
      const uint32_t e = ++me.bepoch[b];
      for (int p = 0; p < R; ++p) rk[p].bflags[(size_t)b * R + r].store(e, std::memory_order_release);
      for (int p = 0; p < R; ++p)
        if (!wait_ge(me.bflags[(size_t)b * R + p], e)) return false;
      return true;
    }
    const uint32_t target = me.release.load(std::memory_order_acquire) + 1u;   // cannot advance before this block has arrived
    me.arrive.fetch_add(1u, std::memory_order_release);
    if (b == 0) {
      if (!wait_ge(me.arrive, (uint32_t)B)) return false;
      me.arrive.store(0u, std::memory_order_relaxed);
      const uint32_t e = ++me.epoch0;
      for (int p = 0; p < R; ++p) rk[p].flags[r].store(e, std::memory_order_release);
      for (int p = 0; p < R; ++p)
        if (!wait_ge(me.flags[p], e)) return false;
      me.release.store(target, std::memory_order_release);
      return true;
    }
    return wait_ge(me.release, target);
  };
  auto body = [&](int r, int b) {
    std::mt19937 rng(r * 100 + b);
    for (int k = 1; k <= iters && !failures.load(std::memory_order_relaxed); ++k) {
      if (rng() % 32 == 0) std::this_thread::sleep_for(std::chrono::microseconds(rng() % 100));
      rk[r].payload[b] = (uint32_t)k;                      // stage (plain store)
      if (!barrier(r, b)) { failures.fetch_add(1); return; }
      // read what ANOTHER block index of ANOTHER rank staged (plain load): must be this iteration's value
      const int pr = (r + 1 + (int)(rng() % R)) % R, pb = (b + 1 + (int)(rng() % B)) % B;
      if (rk[pr].payload[pb] != (uint32_t)k) { failures.fetch_add(1); return; }
      if (!barrier(r, b)) { failures.fetch_add(1); return; }   // nobody restages before everyone has read
    }
  };
  std::vector<std::thread> th;
  for (int r = 0; r < R; ++r)
    for (int b = 0; b < B; ++b) th.emplace_back(body, r, b);
  for (auto& t : th) t.join();
  printf("ranks=%d blocks=%d iterations=%d failures=%d %s\n", R, B, iters, failures.load(), failures.load() ? "FAIL" : "OK");
  return failures.load() ? 1 : 0;
}
