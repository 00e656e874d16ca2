// Offset allocator over one contiguous arena; see arena.cpp.
#pragma once
#include <cstdint>

namespace rt {

struct ArenaStats {
  uint64_t capacity, in_use, peak, n_alloc, n_free, n_fail, live_blocks, free_ranges, largest_free;
  double fragmentation;  // 1 - largest free range / total free bytes
};

class Arena {
 public:
  Arena(uint64_t capacity, uint64_t alignment = 256);
  ~Arena();
  Arena(const Arena&) = delete;
  Arena& operator=(const Arena&) = delete;
  // Returns the offset of a block of at least `size` bytes, or -1 when no free range fits.
  int64_t allocate(uint64_t size);
  void release(uint64_t offset);
  void reset();
  ArenaStats stats() const;
  uint64_t size_of(uint64_t offset) const;  // 0 if not allocated

 private:
  struct Impl;
  Impl* p_;
};

}  // namespace rt
