// Caching device allocator with split / coalesce, stream-aware reuse, statistics, a reservation budget and cache release under pressure.
//
// Two size pools, as in the allocator it replaces: requests below 1 MiB are rounded to 512 B and carved out of 2 MiB segments; larger requests are
// rounded to 512 B, served from 20 MiB segments when below 10 MiB and from their own segment (rounded up to 2 MiB) otherwise. A freed block goes
// back to its pool, merging with free neighbours of the same segment; a block is only re-used on the stream it was freed on, or on any stream
// once every stream recorded for it has been synchronised through an event. Segments come from cudaMalloc, or from the host heap when the
// allocator is created in host mode (which is how the block logic is unit-tested without a GPU).
//
// Capability parity: ferrotorch-gpu/src/allocator.rs:53-69,99,211-253,488-682, pool.rs:33-292 (record_stream, round_len), and the budget /
// pressure half of memory_guard.rs:55-600.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <set>
#include <unordered_map>
#include <vector>

#include "host_common.h"

namespace {

constexpr size_t kMinBlock = 512, kSmallSize = 1 << 20, kSmallBuffer = 2 << 20, kMinLarge = 10 << 20, kLargeBuffer = 20 << 20, kRoundLarge = 2 << 20;

struct Block {
  char* ptr;
  size_t size;
  cudaStream_t stream;          // stream the block was last used on
  bool allocated = false, small = false;
  Block *prev = nullptr, *next = nullptr;   // neighbours inside the segment
  std::vector<cudaEvent_t> pending;         // events of other streams that used the block (record_stream)
  size_t requested = 0;
};

struct Cmp {
  bool operator()(const Block* a, const Block* b) const {
    if (a->stream != b->stream) return (uintptr_t)a->stream < (uintptr_t)b->stream;
    if (a->size != b->size) return a->size < b->size;
    return (uintptr_t)a->ptr < (uintptr_t)b->ptr;
  }
};

struct Allocator {
  bool host_mode;
  std::mutex mu;
  std::set<Block*, Cmp> small_free, large_free;
  std::unordered_map<void*, Block*> live;
  std::vector<Block*> deferred;              // freed blocks still in use on another stream
  int64_t allocated = 0, reserved = 0, peak_allocated = 0, peak_reserved = 0, n_alloc = 0, n_free = 0, n_segment_alloc = 0, n_cache_hit = 0, n_oom = 0;
  int64_t budget = -1;                       // max reserved bytes, -1 = unlimited
  // Debug aid: with canary > 0 every block gets `canary` extra bytes behind the requested size, filled with 0xA5 when the block is handed out
  // and compared when it is freed; a mismatch (a write past the end of the allocation) is counted and reported by the free call.
  size_t canary = 0;
  int64_t n_canary_bad = 0;
  static constexpr unsigned char kCanaryByte = 0xA5;

  static size_t round_size(size_t n) { return n < kMinBlock ? kMinBlock : (n + kMinBlock - 1) / kMinBlock * kMinBlock; }
  static size_t segment_size(size_t n) {
    if (n <= kSmallSize) return kSmallBuffer;
    if (n < kMinLarge) return kLargeBuffer;
    return (n + kRoundLarge - 1) / kRoundLarge * kRoundLarge;
  }

  int raw_alloc(void** p, size_t n) {
    if (budget >= 0 && reserved + (int64_t)n > budget) return FT_ERR_TOO_LARGE;
    if (host_mode) {
      *p = std::malloc(n);
      return *p ? 0 : FT_ERR_TOO_LARGE;
    }
    cudaError_t e = cudaMalloc(p, n);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return FT_ERR_TOO_LARGE;
    }
    return 0;
  }
  void raw_free(void* p) {
    if (host_mode) std::free(p);
    else cudaFree(p);
  }

  void poll_deferred() {
    for (size_t i = 0; i < deferred.size();) {
      Block* b = deferred[i];
      bool done = true;
      for (cudaEvent_t ev : b->pending)
        if (!host_mode && cudaEventQuery(ev) == cudaErrorNotReady) { done = false; break; }
      if (done) {
        for (cudaEvent_t ev : b->pending) if (!host_mode) cudaEventDestroy(ev);
        b->pending.clear();
        deferred[i] = deferred.back();
        deferred.pop_back();
        release(b);
      } else {
        i++;
      }
    }
  }

  void release(Block* b) {
    auto& pool = b->small ? small_free : large_free;
    b->allocated = false;
    for (Block* nb : {b->prev, b->next}) {
      if (!nb || nb->allocated || nb->stream != b->stream || !nb->pending.empty()) continue;
      bool in_deferred = false;
      for (Block* d : deferred) if (d == nb) { in_deferred = true; break; }
      if (in_deferred) continue;
      pool.erase(nb);
      if (nb == b->prev) {
        b->ptr = nb->ptr;
        b->prev = nb->prev;
        if (b->prev) b->prev->next = b;
      } else {
        b->next = nb->next;
        if (b->next) b->next->prev = b;
      }
      b->size += nb->size;
      delete nb;
    }
    pool.insert(b);
  }

  int malloc_(size_t n, cudaStream_t stream, void** out) {
    std::lock_guard<std::mutex> lk(mu);
    if (n == 0) { *out = nullptr; return 0; }
    poll_deferred();
    const size_t size = round_size(n + canary);
    const bool small = size <= kSmallSize;
    auto& pool = small ? small_free : large_free;
    Block key{nullptr, size, stream};
    Block* b = nullptr;
    auto it = pool.lower_bound(&key);
    if (it != pool.end() && (*it)->stream == stream && (small || (*it)->size < kMinLarge || (*it)->size <= size + kLargeBuffer)) {
      b = *it;
      pool.erase(it);
      n_cache_hit++;
    } else {
      const size_t seg = segment_size(size);
      void* p = nullptr;
      int e = raw_alloc(&p, seg);
      if (e) {                                   // release cached segments and retry once
        empty_cache_locked();
        e = raw_alloc(&p, seg);
      }
      if (e) { n_oom++; return e; }
      n_segment_alloc++;
      reserved += seg;
      if (reserved > peak_reserved) peak_reserved = reserved;
      b = new Block{(char*)p, seg, stream};
      b->small = small;
    }
    const size_t rem = b->size - size;
    if (small ? rem >= kMinBlock : rem > kSmallSize) {
      Block* r = new Block{b->ptr + size, rem, stream};
      r->small = small;
      r->prev = b;
      r->next = b->next;
      if (r->next) r->next->prev = r;
      b->next = r;
      b->size = size;
      pool.insert(r);
    }
    b->allocated = true;
    b->requested = n;
    b->stream = stream;
    live[b->ptr] = b;
    allocated += b->size;
    if (allocated > peak_allocated) peak_allocated = allocated;
    n_alloc++;
    *out = b->ptr;
    if (canary) {
      if (host_mode) std::memset(b->ptr + n, kCanaryByte, canary);
      else if (cudaMemsetAsync(b->ptr + n, kCanaryByte, canary, stream) != cudaSuccess) cudaGetLastError();
    }
    return 0;
  }

  // true if the guard bytes behind the block's requested size are intact (device blocks: a synchronous copy back, debug builds only)
  bool canary_intact(const Block* b) {
    if (!canary || b->requested + canary > b->size) return true;
    std::vector<unsigned char> host(canary);
    if (host_mode) std::memcpy(host.data(), b->ptr + b->requested, canary);
    else if (cudaMemcpy(host.data(), b->ptr + b->requested, canary, cudaMemcpyDeviceToHost) != cudaSuccess) { cudaGetLastError(); return true; }
    for (unsigned char c : host) if (c != kCanaryByte) return false;
    return true;
  }

  int free_(void* p) {
    std::lock_guard<std::mutex> lk(mu);
    if (!p) return 0;
    auto it = live.find(p);
    if (it == live.end()) return FT_ERR_ARG;
    Block* b = it->second;
    const bool intact = canary_intact(b);
    if (!intact) n_canary_bad++;
    live.erase(it);
    allocated -= b->size;
    n_free++;
    if (!b->pending.empty()) {
      b->allocated = false;
      deferred.push_back(b);
    } else {
      release(b);
    }
    return intact ? 0 : FT_ERR_CORRUPT;
  }

  int record_stream(void* p, cudaStream_t s) {
    std::lock_guard<std::mutex> lk(mu);
    auto it = live.find(p);
    if (it == live.end()) return FT_ERR_ARG;
    if (s == it->second->stream) return 0;
    cudaEvent_t ev = nullptr;
    if (!host_mode) {
      FT_CUDA_TRY(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
      FT_CUDA_TRY(cudaEventRecord(ev, s));
    }
    it->second->pending.push_back(ev);
    return 0;
  }

  int64_t empty_cache_locked() {
    int64_t freed = 0;
    for (auto* pool : {&small_free, &large_free}) {
      for (auto it = pool->begin(); it != pool->end();) {
        Block* b = *it;
        if (!b->prev && !b->next) {             // a whole, unsplit segment
          raw_free(b->ptr);
          reserved -= (int64_t)b->size;
          freed += (int64_t)b->size;
          it = pool->erase(it);
          delete b;
        } else {
          ++it;
        }
      }
    }
    return freed;
  }
};

std::mutex g_mu;
std::map<int, Allocator*> g_device_alloc;     // per-device instance behind the torch plug-in entry points

Allocator* device_allocator(int dev) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_device_alloc.find(dev);
  if (it != g_device_alloc.end()) return it->second;
  Allocator* a = new Allocator();
  a->host_mode = false;
  g_device_alloc[dev] = a;
  return a;
}

}  // namespace

// host_mode = 1: segments from the host heap (tests); 0: cudaMalloc on the current device.
FT_EXPORT int ft_alloc_create(int host_mode, void** handle) {
  if (!handle) return FT_ERR_ARG;
  Allocator* a = new Allocator();
  a->host_mode = host_mode != 0;
  *handle = a;
  return 0;
}
FT_EXPORT int ft_alloc_destroy(void* h) {
  if (!h) return FT_ERR_ARG;
  Allocator* a = (Allocator*)h;
  {
    std::lock_guard<std::mutex> lk(a->mu);
    a->empty_cache_locked();
  }
  delete a;
  return 0;
}
FT_EXPORT int ft_alloc_malloc(void* h, int64_t bytes, cudaStream_t stream, void** out) {
  if (!h || bytes < 0 || !out) return FT_ERR_ARG;
  return ((Allocator*)h)->malloc_((size_t)bytes, stream, out);
}
FT_EXPORT int ft_alloc_free(void* h, void* p) { return h ? ((Allocator*)h)->free_(p) : FT_ERR_ARG; }
FT_EXPORT int ft_alloc_record_stream(void* h, void* p, cudaStream_t s) { return h ? ((Allocator*)h)->record_stream(p, s) : FT_ERR_ARG; }
FT_EXPORT int ft_alloc_set_budget(void* h, int64_t max_reserved_bytes) {
  if (!h) return FT_ERR_ARG;
  std::lock_guard<std::mutex> lk(((Allocator*)h)->mu);
  ((Allocator*)h)->budget = max_reserved_bytes;
  return 0;
}
// Debug aid: guard bytes behind every later allocation, checked on free (ft_alloc_free then returns FT_ERR_CORRUPT and the block is still
// released). bytes = 0 switches it off. Blocks that are live when the setting changes are not checked.
FT_EXPORT int ft_alloc_set_canary(void* h, int64_t bytes) {
  if (!h || bytes < 0 || bytes > (1 << 20)) return FT_ERR_ARG;
  Allocator* a = (Allocator*)h;
  std::lock_guard<std::mutex> lk(a->mu);
  if (!a->live.empty()) return FT_ERR_ARG;
  a->canary = (size_t)bytes;
  return 0;
}
FT_EXPORT int ft_alloc_canary_violations(void* h, int64_t* out) {
  if (!h || !out) return FT_ERR_ARG;
  std::lock_guard<std::mutex> lk(((Allocator*)h)->mu);
  *out = ((Allocator*)h)->n_canary_bad;
  return 0;
}
FT_EXPORT int ft_alloc_empty_cache(void* h, int64_t* freed) {
  if (!h) return FT_ERR_ARG;
  std::lock_guard<std::mutex> lk(((Allocator*)h)->mu);
  ((Allocator*)h)->poll_deferred();
  const int64_t f = ((Allocator*)h)->empty_cache_locked();
  if (freed) *freed = f;
  return 0;
}
// out[0..9] = allocated, reserved, peak_allocated, peak_reserved, n_alloc, n_free, n_segment_alloc, n_cache_hit, n_oom, live blocks
FT_EXPORT int ft_alloc_stats(void* h, int64_t* out) {
  if (!h || !out) return FT_ERR_ARG;
  Allocator* a = (Allocator*)h;
  std::lock_guard<std::mutex> lk(a->mu);
  const int64_t v[10] = {a->allocated, a->reserved, a->peak_allocated, a->peak_reserved, a->n_alloc, a->n_free, a->n_segment_alloc, a->n_cache_hit, a->n_oom,
                         (int64_t)a->live.size()};
  for (int i = 0; i < 10; i++) out[i] = v[i];
  return 0;
}
FT_EXPORT int ft_alloc_reset_peak(void* h) {
  if (!h) return FT_ERR_ARG;
  Allocator* a = (Allocator*)h;
  std::lock_guard<std::mutex> lk(a->mu);
  a->peak_allocated = a->allocated;
  a->peak_reserved = a->reserved;
  return 0;
}

// Entry points with the signature torch.cuda.memory.CUDAPluggableAllocator expects; a null return makes torch raise its out-of-memory error.
extern "C" __attribute__((visibility("default"))) void* ft_torch_malloc(ssize_t size, int device, cudaStream_t stream) {
  int cur = 0;
  cudaGetDevice(&cur);
  if (cur != device) cudaSetDevice(device);
  void* p = nullptr;
  const int e = device_allocator(device)->malloc_((size_t)size, stream, &p);
  if (cur != device) cudaSetDevice(cur);
  return e ? nullptr : p;
}
extern "C" __attribute__((visibility("default"))) void ft_torch_free(void* ptr, ssize_t, int device, cudaStream_t) { device_allocator(device)->free_(ptr); }
FT_EXPORT int ft_torch_allocator_handle(int device, void** handle) {
  if (!handle) return FT_ERR_ARG;
  *handle = device_allocator(device);
  return 0;
}
