// Host emulation of the peer-memory kernels' synchronisation protocols (see protocol_sim.cpp).
#pragma once

#include <cstdint>

namespace rt_host {

struct SimResult {
  long long mismatches = 0;  // values that differed from the expected ones
  long long timeouts = 0;    // ranks that gave up in a bounded wait
  long long checked = 0;     // values compared
};

// `slots` receive buffers per rank (the kernel uses 3); `slow_rank` >= 0 sleeps `slow_us` at random points.
SimResult sim_lamport_allreduce(int world, long long calls, int words, int slots, int slow_rank, int slow_us, unsigned seed);

// `parities` staging buffers (the kernel uses 2, selected by call parity).
SimResult sim_epoch_counters(int world, long long calls, int blocks, int tiles, int parities, int slow_rank, int slow_us,
                             unsigned seed);

}  // namespace rt_host
