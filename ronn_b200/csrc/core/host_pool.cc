// Host memory allocators.
//
// One implementation backs three reference components:
//   * the size-class byte-buffer pool (crates/ronn-core/src/memory_pool.rs:74-239:
//     power-of-two classes, per-class and total buffer caps, hit/miss counters),
//   * the aligned allocator (crates/ronn-providers/src/allocator.rs:158-255, 64-byte),
//   * the bucketed pooled allocator (crates/ronn-providers/src/allocator.rs:259-505:
//     granularity buckets, max buffers per bucket, max pooled bytes, hit rate).
// Thread-safe; all entry points extern "C".
#include <atomic>
#include <cstdint>
#include <cstdlib>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace {

struct Pool {
  std::mutex mu;
  uint64_t granularity;       // bucket rounding; 0 = power-of-two classes
  uint64_t alignment;
  uint64_t max_per_bucket;
  uint64_t max_pool_bytes;    // cap on bytes parked in the pool
  uint64_t max_total_buffers; // cap on buffers parked in the pool (0 = unlimited)
  std::unordered_map<uint64_t, std::vector<void*>> buckets;
  std::unordered_map<void*, uint64_t> live;   // ptr -> bucket size
  uint64_t pooled_bytes = 0, pooled_buffers = 0;
  uint64_t hits = 0, misses = 0, allocated_bytes = 0, peak_bytes = 0, alloc_count = 0, free_count = 0;

  uint64_t bucket_of(uint64_t n) const {
    if (granularity) return (n + granularity - 1) / granularity * granularity;
    uint64_t c = 64;
    while (c < n) c <<= 1;
    return c;
  }
};

}  // namespace

extern "C" {

void* ronn_pool_new(uint64_t granularity, uint64_t alignment, uint64_t max_per_bucket, uint64_t max_pool_bytes,
                    uint64_t max_total_buffers) {
  if (alignment == 0 || (alignment & (alignment - 1))) return nullptr;
  Pool* p = new Pool();
  p->granularity = granularity;
  p->alignment = alignment < sizeof(void*) ? sizeof(void*) : alignment;
  p->max_per_bucket = max_per_bucket;
  p->max_pool_bytes = max_pool_bytes;
  p->max_total_buffers = max_total_buffers;
  return p;
}

void ronn_pool_clear(void* h) {
  Pool* p = static_cast<Pool*>(h);
  std::lock_guard<std::mutex> g(p->mu);
  for (auto& kv : p->buckets)
    for (void* b : kv.second) free(b);
  p->buckets.clear();
  p->pooled_bytes = 0;
  p->pooled_buffers = 0;
}

void ronn_pool_free(void* h) {
  Pool* p = static_cast<Pool*>(h);
  ronn_pool_clear(h);
  for (auto& kv : p->live) free(kv.first);
  delete p;
}

// Returns nullptr for zero-size requests or when the system allocator fails.
void* ronn_pool_alloc(void* h, uint64_t nbytes) {
  Pool* p = static_cast<Pool*>(h);
  if (nbytes == 0 || nbytes > (uint64_t(1) << 46)) return nullptr;
  uint64_t b = p->bucket_of(nbytes);
  std::lock_guard<std::mutex> g(p->mu);
  void* ptr = nullptr;
  auto it = p->buckets.find(b);
  if (it != p->buckets.end() && !it->second.empty()) {
    ptr = it->second.back();
    it->second.pop_back();
    p->pooled_bytes -= b;
    p->pooled_buffers -= 1;
    p->hits += 1;
  } else {
    uint64_t sz = (b + p->alignment - 1) / p->alignment * p->alignment;
    if (posix_memalign(&ptr, size_t(p->alignment), size_t(sz)) != 0) return nullptr;
    p->misses += 1;
  }
  p->live[ptr] = b;
  p->allocated_bytes += b;
  if (p->allocated_bytes > p->peak_bytes) p->peak_bytes = p->allocated_bytes;
  p->alloc_count += 1;
  return ptr;
}

// Returns 0 ok, -1 when the pointer is unknown (double free or foreign pointer).
int32_t ronn_pool_release(void* h, void* ptr) {
  Pool* p = static_cast<Pool*>(h);
  std::lock_guard<std::mutex> g(p->mu);
  auto it = p->live.find(ptr);
  if (it == p->live.end()) return -1;
  uint64_t b = it->second;
  p->live.erase(it);
  p->allocated_bytes -= b;
  p->free_count += 1;
  auto& bucket = p->buckets[b];
  bool room = bucket.size() < p->max_per_bucket && p->pooled_bytes + b <= p->max_pool_bytes &&
              (p->max_total_buffers == 0 || p->pooled_buffers < p->max_total_buffers);
  if (room) {
    bucket.push_back(ptr);
    p->pooled_bytes += b;
    p->pooled_buffers += 1;
  } else {
    free(ptr);
  }
  return 0;
}

// out[0..8] = hits, misses, allocated_bytes, peak_bytes, pooled_bytes, pooled_buffers, alloc_count, free_count, live
void ronn_pool_stats(void* h, uint64_t* out) {
  Pool* p = static_cast<Pool*>(h);
  std::lock_guard<std::mutex> g(p->mu);
  out[0] = p->hits; out[1] = p->misses; out[2] = p->allocated_bytes; out[3] = p->peak_bytes;
  out[4] = p->pooled_bytes; out[5] = p->pooled_buffers; out[6] = p->alloc_count; out[7] = p->free_count;
  out[8] = p->live.size();
}

uint64_t ronn_pool_bucket_size(void* h, uint64_t nbytes) { return static_cast<Pool*>(h)->bucket_of(nbytes); }

}  // extern "C"
