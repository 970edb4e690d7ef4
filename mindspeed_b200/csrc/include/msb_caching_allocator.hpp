// Block-splitting caching allocator with memory-pressure hooks and lifetime tracing.
//
// Backend-agnostic core: the owner supplies raw segment malloc/free functions (cudaMalloc/cudaFree in the device
// build, malloc/free in the host build that the CPU tests drive).  Design, sized for a 180 GB HBM3e device:
//
//   * requests are rounded to 512 B; requests < 1 MiB are served from 2 MiB "small" segments, larger ones from
//     segments of max(20 MiB, request rounded to 2 MiB) - large segments are what fragment, so they are split
//     only when the remainder is >= 1 MiB;
//   * free blocks live in one ordered set per (pool, stream) keyed by (size, address): best-fit in O(log n);
//     neighbouring free blocks of a segment are merged on free;
//   * a soft limit (set_limit) and the backend's own failure both trigger the pressure path: first cached
//     segments that are entirely free are returned to the backend, then the registered pressure callback is
//     invoked (it may swap tensors out or drop recomputable activations and reports how many bytes it released),
//     then the request is retried once;
//   * every malloc/free can be appended to a trace ring (sequence number, address, size, stream, user "step" and
//     "phase" tags) - the raw material of the swap policy search.
//
// Not thread-hot: one mutex around everything; the torch caching layer above calls in rarely compared to
// kernel launches.  No counterpart of this file exists in the reference as portable source: its allocator is a
// fork of the Ascend caching allocator (mindspeed/ops/csrc/pluggable_allocator/smart_swap/DeviceCachingAllocator.cpp,
// adaptive_recomputing/NpuCachingCustomAllocator.cpp); this one is written from the behaviour described there.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <map>
#include <mutex>
#include <set>
#include <unordered_map>
#include <vector>

namespace msb { namespace alloc {

struct Stats {
  uint64_t allocated_bytes, reserved_bytes, peak_allocated_bytes, peak_reserved_bytes;
  uint64_t num_mallocs, num_frees, num_segments, num_segment_allocs, num_pressure_events, num_cache_flushes;
  uint64_t largest_free_block, free_bytes_in_cache;
};

struct TraceEvent {
  uint64_t seq;
  uint64_t addr;
  uint64_t size;
  uint64_t stream;
  int32_t step;
  int32_t phase;     // user tag, e.g. 0 = forward, 1 = backward, 2 = optimizer
  int32_t is_free;   // 0 = malloc, 1 = free
  int32_t pad;
};

typedef void* (*RawMalloc)(size_t bytes, int device);
typedef int (*RawFree)(void* p, int device);
// returns the number of bytes the callee released back to this allocator (by freeing tensors)
typedef uint64_t (*PressureCallback)(uint64_t bytes_needed, int device, void* user);

class CachingAllocator {
 public:
  static constexpr size_t kRound = 512;
  static constexpr size_t kSmallLimit = 1u << 20;
  static constexpr size_t kSmallSegment = 2u << 20;
  static constexpr size_t kLargeSegmentMin = 20u << 20;
  static constexpr size_t kLargeRound = 2u << 20;

  CachingAllocator(RawMalloc m, RawFree f, int device) : raw_malloc_(m), raw_free_(f), device_(device) {}
  ~CachingAllocator() { release_all(); }

  void* malloc(size_t bytes, uint64_t stream) {
    std::lock_guard<std::mutex> g(mu_);
    if (bytes == 0) return nullptr;
    const size_t size = round_size(bytes);
    const bool small = size < kSmallLimit;
    Block* b = find_free(size, small, stream);
    if (!b) b = grow(size, small, stream);
    if (!b) {
      // pressure path: drop cached segments, ask the owner to release memory, retry once
      ++stats_.num_pressure_events;
      flush_free_segments();
      b = grow(size, small, stream);
      if (!b && pressure_cb_) {
        in_callback_ = true;
        mu_.unlock();
        const uint64_t released = pressure_cb_(size, device_, pressure_user_);
        mu_.lock();
        in_callback_ = false;
        (void)released;
        b = find_free(size, small, stream);
        if (!b) { flush_free_segments(); b = grow(size, small, stream); }
      }
      if (!b) return nullptr;
    }
    b = maybe_split(b, size, small);
    b->allocated = true;
    b->requested = bytes;
    live_[b->ptr] = b;
    stats_.allocated_bytes += b->size;
    if (stats_.allocated_bytes > stats_.peak_allocated_bytes) stats_.peak_allocated_bytes = stats_.allocated_bytes;
    ++stats_.num_mallocs;
    trace(b, 0);
    return b->ptr;
  }

  // returns 0 on success, 1 when the pointer is unknown
  int free(void* p) {
    std::lock_guard<std::mutex> g(mu_);
    if (!p) return 0;
    auto it = live_.find(p);
    if (it == live_.end()) return 1;
    Block* b = it->second;
    live_.erase(it);
    b->allocated = false;
    stats_.allocated_bytes -= b->size;
    ++stats_.num_frees;
    trace(b, 1);
    // merge with free neighbours of the same segment
    if (b->prev && !b->prev->allocated) b = merge(b->prev, b);
    if (b->next && !b->next->allocated) b = merge(b, b->next);
    pool(b->small, b->stream).insert(b);
    return 0;
  }

  // Return every completely free segment to the backend; returns bytes released.
  uint64_t empty_cache() {
    std::lock_guard<std::mutex> g(mu_);
    return flush_free_segments();
  }

  void set_limit(uint64_t bytes) { std::lock_guard<std::mutex> g(mu_); limit_ = bytes; }
  void set_pressure_callback(PressureCallback cb, void* user) { std::lock_guard<std::mutex> g(mu_); pressure_cb_ = cb; pressure_user_ = user; }
  void set_tags(int step, int phase) { std::lock_guard<std::mutex> g(mu_); step_ = step; phase_ = phase; }
  void enable_trace(size_t capacity) {
    std::lock_guard<std::mutex> g(mu_);
    trace_.clear(); trace_.reserve(capacity); trace_cap_ = capacity; trace_dropped_ = 0;
  }
  size_t read_trace(TraceEvent* out, size_t max_events, bool clear) {
    std::lock_guard<std::mutex> g(mu_);
    const size_t n = trace_.size() < max_events ? trace_.size() : max_events;
    for (size_t i = 0; i < n; ++i) out[i] = trace_[i];
    if (clear) trace_.clear();
    return n;
  }
  uint64_t trace_dropped() { std::lock_guard<std::mutex> g(mu_); return trace_dropped_; }

  Stats stats() {
    std::lock_guard<std::mutex> g(mu_);
    Stats s = stats_;
    s.largest_free_block = 0; s.free_bytes_in_cache = 0;
    for (auto& kv : pools_) for (Block* b : kv.second) { s.free_bytes_in_cache += b->size; if (b->size > s.largest_free_block) s.largest_free_block = b->size; }
    return s;
  }
  uint64_t block_size(void* p) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = live_.find(p);
    return it == live_.end() ? 0 : it->second->size;
  }
  void reset_peaks() { std::lock_guard<std::mutex> g(mu_); stats_.peak_allocated_bytes = stats_.allocated_bytes; stats_.peak_reserved_bytes = stats_.reserved_bytes; }

  static size_t round_size(size_t bytes) { return bytes < kRound ? kRound : ((bytes + kRound - 1) / kRound) * kRound; }

 private:
  struct Block {
    void* ptr; size_t size; size_t requested; uint64_t stream; bool small; bool allocated;
    Block* prev; Block* next; void* segment; size_t segment_size;
  };
  struct Cmp {
    bool operator()(const Block* a, const Block* b) const {
      if (a->size != b->size) return a->size < b->size;
      return reinterpret_cast<uintptr_t>(a->ptr) < reinterpret_cast<uintptr_t>(b->ptr);
    }
  };
  typedef std::set<Block*, Cmp> Pool;

  Pool& pool(bool small, uint64_t stream) { return pools_[(stream << 1) | (small ? 1u : 0u)]; }

  Block* find_free(size_t size, bool small, uint64_t stream) {
    Pool& pl = pool(small, stream);
    Block key{nullptr, size, 0, stream, small, false, nullptr, nullptr, nullptr, 0};
    auto it = pl.lower_bound(&key);
    if (it == pl.end()) return nullptr;
    // do not hand a huge cached block to a much smaller large request: it would pin the segment (fragmentation guard)
    if (!small && (*it)->size > size * 4 && (*it)->size - size >= (200u << 20)) return nullptr;
    Block* b = *it;
    pl.erase(it);
    return b;
  }

  Block* grow(size_t size, bool small, uint64_t stream) {
    size_t seg = small ? kSmallSegment : (size < kLargeSegmentMin ? kLargeSegmentMin : ((size + kLargeRound - 1) / kLargeRound) * kLargeRound);
    if (limit_ && stats_.reserved_bytes + seg > limit_) {
      if (!small && stats_.reserved_bytes + size <= limit_) seg = ((size + kLargeRound - 1) / kLargeRound) * kLargeRound;
      if (stats_.reserved_bytes + seg > limit_) return nullptr;
    }
    void* p = raw_malloc_(seg, device_);
    if (!p) return nullptr;
    ++stats_.num_segments; ++stats_.num_segment_allocs;
    stats_.reserved_bytes += seg;
    if (stats_.reserved_bytes > stats_.peak_reserved_bytes) stats_.peak_reserved_bytes = stats_.reserved_bytes;
    Block* b = new Block{p, seg, 0, stream, small, false, nullptr, nullptr, p, seg};
    return b;
  }

  Block* maybe_split(Block* b, size_t size, bool small) {
    const size_t rest = b->size - size;
    const bool split = small ? rest >= kRound : rest >= kSmallLimit;
    if (!split) return b;
    Block* r = new Block{static_cast<char*>(b->ptr) + size, rest, 0, b->stream, b->small, false, b, b->next, b->segment, b->segment_size};
    if (b->next) b->next->prev = r;
    b->next = r;
    b->size = size;
    pool(r->small, r->stream).insert(r);
    return b;
  }

  Block* merge(Block* a, Block* b) {   // a directly precedes b; at most one of them is in a pool
    pool(a->small, a->stream).erase(a);
    pool(b->small, b->stream).erase(b);
    a->size += b->size;
    a->next = b->next;
    if (b->next) b->next->prev = a;
    delete b;
    return a;
  }

  uint64_t flush_free_segments() {
    uint64_t released = 0;
    for (auto& kv : pools_) {
      Pool& pl = kv.second;
      for (auto it = pl.begin(); it != pl.end();) {
        Block* b = *it;
        if (!b->prev && !b->next && b->ptr == b->segment) {
          raw_free_(b->segment, device_);
          stats_.reserved_bytes -= b->segment_size;
          --stats_.num_segments;
          released += b->segment_size;
          it = pl.erase(it);
          delete b;
        } else {
          ++it;
        }
      }
    }
    if (released) ++stats_.num_cache_flushes;
    return released;
  }

  void release_all() {
    std::lock_guard<std::mutex> g(mu_);
    flush_free_segments();
  }

  void trace(Block* b, int is_free) {
    if (!trace_cap_) return;
    if (trace_.size() >= trace_cap_) { ++trace_dropped_; return; }
    trace_.push_back(TraceEvent{seq_++, (uint64_t)reinterpret_cast<uintptr_t>(b->ptr), (uint64_t)b->size, b->stream, step_, phase_, is_free, 0});
  }

  RawMalloc raw_malloc_;
  RawFree raw_free_;
  int device_;
  std::mutex mu_;
  std::unordered_map<uint64_t, Pool> pools_;
  std::unordered_map<void*, Block*> live_;
  Stats stats_{};
  uint64_t limit_ = 0;
  PressureCallback pressure_cb_ = nullptr;
  void* pressure_user_ = nullptr;
  bool in_callback_ = false;
  std::vector<TraceEvent> trace_;
  size_t trace_cap_ = 0;
  uint64_t trace_dropped_ = 0, seq_ = 0;
  int step_ = 0, phase_ = 0;
};

}}  // namespace msb::alloc
