// Host emulation of the synchronisation protocols of the peer-memory kernels: one std::thread per rank, the symmetric
// buffers as arrays of std::atomic words, the same state machines as the device code.  Runs under any thread
// interleaving the host scheduler produces (plus random yields), so protocol errors (a slot refilled too early, a
// staging buffer reused while a peer still reads it) show up as wrong sums without a GPU, and the file can be built
// with -fsanitize=thread.
//
//   sim_lamport_allreduce   csrc/collective/ar_residual_norm.cu: self-validating pushes into `slots` receive buffers
//                           per rank (3 in the kernel), sentinel 0x8000 per 16-bit lane, sender rewrites -0 to +0,
//                           call k re-arms slot (k + 2) mod slots.
//   sim_epoch_counters      csrc/collective/tp_gemm.cu (GEMM -> reduce-scatter): sources write tiles into the owner's
//                           staging (double-buffered by call parity) and release-add a per-(block, source) counter;
//                           the owner acquires counter >= epoch * tiles and reads.
//
// The reference has no such protocols: its collectives are host loops under a mutex (src/gpu/multi_gpu.rs:583-700).
#include "protocol_sim.h"

#include <atomic>
#include <chrono>
#include <memory>
#include <random>
#include <thread>
#include <vector>

namespace rt_host {

namespace {

constexpr uint32_t kSentinel = 0x80008000u;

inline uint32_t mix(uint64_t x) {  // splitmix64 -> 32 bits
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return static_cast<uint32_t>((x ^ (x >> 31)) >> 16);
}

// The word rank `r` contributes at position i of call k; every 7th word carries a -0 lane on purpose.
inline uint32_t payload(int r, long long k, int i) {
  uint32_t w = mix((static_cast<uint64_t>(r) << 48) ^ (static_cast<uint64_t>(k) << 20) ^ static_cast<uint64_t>(i));
  if (i % 7 == 3) w = (w & 0xffff0000u) | 0x8000u;
  return w;
}
inline uint32_t fix_word(uint32_t w) {  // -0 -> +0 in both 16-bit lanes, as the sender does
  if ((w & 0xffffu) == 0x8000u) w &= 0xffff0000u;
  if ((w >> 16) == 0x8000u) w &= 0x0000ffffu;
  return w;
}
inline bool pending(uint32_t w) { return (w & 0xffffu) == 0x8000u || (w >> 16) == 0x8000u; }

inline void jitter(std::mt19937& g, int slow_us) {
  const unsigned v = g() & 63u;
  if (v == 0) std::this_thread::yield();
  if (slow_us > 0 && v < 8) std::this_thread::sleep_for(std::chrono::microseconds(slow_us));
}

}  // namespace

SimResult sim_lamport_allreduce(int world, long long calls, int words, int slots, int slow_rank, int slow_us, unsigned seed) {
  SimResult res{};
  if (world < 1 || words < 1 || slots < 1 || calls < 0) return res;
  // recv[rank][slot][src][word]
  const size_t per_rank = static_cast<size_t>(slots) * world * words;
  std::unique_ptr<std::atomic<uint32_t>[]> recv(new std::atomic<uint32_t>[per_rank * world]);
  for (size_t i = 0; i < per_rank * world; ++i) recv[i].store(kSentinel, std::memory_order_relaxed);
  std::atomic<long long> mismatches{0}, timeouts{0};
  auto at = [&](int rank, int slot, int src, int i) -> std::atomic<uint32_t>& {
    return recv[static_cast<size_t>(rank) * per_rank + (static_cast<size_t>(slot) * world + src) * words + i];
  };
  auto body = [&](int r) {
    std::mt19937 g(seed * 977u + r);
    for (long long k = 0; k < calls; ++k) {
      const int slot = static_cast<int>(k % slots);
      for (int pi = 0; pi < world; ++pi) {  // push to every peer, own copy included, starting with the next rank
        const int p = (r + 1 + pi) % world;
        for (int i = 0; i < words; ++i) at(p, slot, r, i).store(fix_word(payload(r, k, i)), std::memory_order_relaxed);
        jitter(g, r == slow_rank ? slow_us : 0);
      }
      bool gave_up = false;
      for (int i = 0; i < words && !gave_up; ++i) {
        uint64_t sum = 0, want = 0;
        for (int src = 0; src < world; ++src) {
          uint32_t w;
          long long spins = 0;
          while (pending(w = at(r, slot, src, i).load(std::memory_order_relaxed))) {
            if (++spins > 200000000LL) {  // bounded like the device poll
              gave_up = true;
              break;
            }
            if ((spins & 1023) == 0) std::this_thread::yield();
          }
          if (gave_up) break;
          sum += w;
          want += fix_word(payload(src, k, i));
        }
        if (!gave_up && sum != want) mismatches.fetch_add(1, std::memory_order_relaxed);
      }
      if (gave_up) {
        timeouts.fetch_add(1, std::memory_order_relaxed);
        return;
      }
      // re-arm the slot furthest from use: call k + 2 with three slots (no peer can be writing it yet); with two slots
      // it is the slot of call k + 1, which a faster peer may already be filling - the race this emulation exposes
      const int rearm = static_cast<int>((k + slots - 1) % slots);
      if (rearm != slot || slots == 1)
        for (int src = 0; src < world; ++src)
          for (int i = 0; i < words; ++i) at(r, rearm, src, i).store(kSentinel, std::memory_order_relaxed);
      jitter(g, r == slow_rank ? slow_us : 0);
    }
  };
  std::vector<std::thread> th;
  for (int r = 0; r < world; ++r) th.emplace_back(body, r);
  for (auto& t : th) t.join();
  res.mismatches = mismatches.load();
  res.timeouts = timeouts.load();
  res.checked = calls * world * static_cast<long long>(words);
  return res;
}

SimResult sim_epoch_counters(int world, long long calls, int blocks, int tiles, int parities, int slow_rank, int slow_us,
                             unsigned seed) {
  SimResult res{};
  if (world < 1 || blocks < 1 || tiles < 1 || parities < 1 || calls < 0) return res;
  // stage[owner][parity][src][block][tile], count[owner][block][src]
  const size_t per_owner = static_cast<size_t>(parities) * world * blocks * tiles;
  std::unique_ptr<std::atomic<uint32_t>[]> stage(new std::atomic<uint32_t>[per_owner * world]);
  std::unique_ptr<std::atomic<long long>[]> count(new std::atomic<long long>[static_cast<size_t>(world) * blocks * world]);
  for (size_t i = 0; i < per_owner * world; ++i) stage[i].store(0, std::memory_order_relaxed);
  for (size_t i = 0; i < static_cast<size_t>(world) * blocks * world; ++i) count[i].store(0, std::memory_order_relaxed);
  std::atomic<long long> mismatches{0}, timeouts{0};
  auto st = [&](int owner, int par, int src, int b, int t) -> std::atomic<uint32_t>& {
    return stage[static_cast<size_t>(owner) * per_owner + ((static_cast<size_t>(par) * world + src) * blocks + b) * tiles + t];
  };
  auto cnt = [&](int owner, int b, int src) -> std::atomic<long long>& {
    return count[(static_cast<size_t>(owner) * blocks + b) * world + src];
  };
  auto body = [&](int r) {
    std::mt19937 g(seed * 131u + r);
    for (long long e = 1; e <= calls; ++e) {
      const int par = static_cast<int>(e % parities);
      // tiles for remote owners first, in ring order; then the own rows
      for (int s = 1; s < world; ++s) {
        const int owner = (r + s) % world;
        for (int b = 0; b < blocks; ++b) {
          for (int t = 0; t < tiles; ++t) {
            st(owner, par, r, b, t).store(payload(r, e, b * tiles + t) ^ static_cast<uint32_t>(owner), std::memory_order_relaxed);
            cnt(owner, b, r).fetch_add(1, std::memory_order_release);
          }
          jitter(g, r == slow_rank ? slow_us : 0);
        }
      }
      for (int b = 0; b < blocks; ++b) {
        for (int src = 0; src < world; ++src) {
          if (src == r) continue;
          long long spins = 0;
          while (cnt(r, b, src).load(std::memory_order_acquire) < e * tiles) {
            if (++spins > 200000000LL) {
              timeouts.fetch_add(1, std::memory_order_relaxed);
              return;
            }
            if ((spins & 1023) == 0) std::this_thread::yield();
          }
          for (int t = 0; t < tiles; ++t) {
            const uint32_t got = st(r, par, src, b, t).load(std::memory_order_relaxed);
            if (got != (payload(src, e, b * tiles + t) ^ static_cast<uint32_t>(r))) mismatches.fetch_add(1, std::memory_order_relaxed);
          }
        }
        jitter(g, r == slow_rank ? slow_us : 0);
      }
    }
  };
  std::vector<std::thread> th;
  for (int r = 0; r < world; ++r) th.emplace_back(body, r);
  for (auto& t : th) t.join();
  res.mismatches = mismatches.load();
  res.timeouts = timeouts.load();
  res.checked = calls * world * static_cast<long long>(world - 1) * blocks * tiles;
  return res;
}

}  // namespace rt_host
