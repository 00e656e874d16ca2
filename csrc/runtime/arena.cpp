// Offset allocator over one contiguous arena (device memory pool bookkeeping).
//
// The reference's GpuMemoryPool walks a Vec of blocks first-fit and never merges neighbours
// (src/gpu/memory.rs:11-200).  This allocator keeps the free ranges in two ordered maps (by offset for
// coalescing, by size for best-fit lookup), so allocate / free are O(log n), freed neighbours merge at
// once, and fragmentation statistics are exact.  It hands out offsets only: the Python side owns one large
// device buffer and views it, so a training step's temporaries never touch cudaMalloc.
#include <cstdint>
#include <map>
#include <mutex>
#include <set>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <utility>

#include "arena.h"

namespace rt {

struct Arena::Impl {
  uint64_t capacity, alignment;
  std::map<uint64_t, uint64_t> free_by_off;               // offset -> size
  std::set<std::pair<uint64_t, uint64_t>> free_by_size;   // (size, offset)
  std::unordered_map<uint64_t, uint64_t> live;            // offset -> size
  uint64_t in_use = 0, peak = 0, n_alloc = 0, n_free = 0, n_fail = 0;
  std::mutex mu;

  void add_free(uint64_t off, uint64_t size) {
    free_by_off[off] = size;
    free_by_size.insert({size, off});
  }
  void del_free(uint64_t off, uint64_t size) {
    free_by_off.erase(off);
    free_by_size.erase({size, off});
  }
};

Arena::Arena(uint64_t capacity, uint64_t alignment) : p_(new Impl) {
  if (alignment == 0 || (alignment & (alignment - 1))) throw std::invalid_argument("arena: alignment must be a power of two");
  p_->capacity = capacity / alignment * alignment;
  p_->alignment = alignment;
  if (p_->capacity) p_->add_free(0, p_->capacity);
}

Arena::~Arena() { delete p_; }

int64_t Arena::allocate(uint64_t size) {
  std::lock_guard<std::mutex> lk(p_->mu);
  const uint64_t a = p_->alignment;
  const uint64_t need = size == 0 ? a : (size + a - 1) / a * a;
  auto it = p_->free_by_size.lower_bound({need, 0});  // best fit: smallest range that is large enough
  if (it == p_->free_by_size.end()) {
    ++p_->n_fail;
    return -1;
  }
  const uint64_t fsize = it->first, off = it->second;
  p_->del_free(off, fsize);
  if (fsize > need) p_->add_free(off + need, fsize - need);
  p_->live[off] = need;
  p_->in_use += need;
  if (p_->in_use > p_->peak) p_->peak = p_->in_use;
  ++p_->n_alloc;
  return (int64_t)off;
}

void Arena::release(uint64_t off) {
  std::lock_guard<std::mutex> lk(p_->mu);
  auto it = p_->live.find(off);
  if (it == p_->live.end()) throw std::invalid_argument("arena: release of an offset that is not allocated: " + std::to_string(off));
  uint64_t size = it->second;
  p_->live.erase(it);
  p_->in_use -= size;
  ++p_->n_free;
  // merge with the following and the preceding free range
  auto next = p_->free_by_off.find(off + size);
  if (next != p_->free_by_off.end()) {
    const uint64_t nsize = next->second;
    p_->del_free(off + size, nsize);
    size += nsize;
  }
  auto after = p_->free_by_off.lower_bound(off);
  if (after != p_->free_by_off.begin()) {
    auto prev = std::prev(after);
    if (prev->first + prev->second == off) {
      const uint64_t poff = prev->first, psize = prev->second;
      p_->del_free(poff, psize);
      off = poff;
      size += psize;
    }
  }
  p_->add_free(off, size);
}

void Arena::reset() {
  std::lock_guard<std::mutex> lk(p_->mu);
  p_->free_by_off.clear();
  p_->free_by_size.clear();
  p_->live.clear();
  p_->in_use = 0;
  if (p_->capacity) p_->add_free(0, p_->capacity);
}

ArenaStats Arena::stats() const {
  std::lock_guard<std::mutex> lk(p_->mu);
  ArenaStats s{};
  s.capacity = p_->capacity;
  s.in_use = p_->in_use;
  s.peak = p_->peak;
  s.n_alloc = p_->n_alloc;
  s.n_free = p_->n_free;
  s.n_fail = p_->n_fail;
  s.live_blocks = p_->live.size();
  s.free_ranges = p_->free_by_off.size();
  s.largest_free = p_->free_by_size.empty() ? 0 : p_->free_by_size.rbegin()->first;
  const uint64_t total_free = p_->capacity - p_->in_use;
  s.fragmentation = total_free ? 1.0 - (double)s.largest_free / (double)total_free : 0.0;
  return s;
}

uint64_t Arena::size_of(uint64_t off) const {
  std::lock_guard<std::mutex> lk(p_->mu);
  auto it = p_->live.find(off);
  return it == p_->live.end() ? 0 : it->second;
}

}  // namespace rt
