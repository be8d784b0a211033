// Parameter all-gather of the fully sharded (ZeRO-3) engine over NVLink peer memory, in three small kernels that never wait for one another on
// the same GPU:
//
//   ft_fsdp_push_shard   producer: every rank copies ITS shard of a flat unit, piece by piece (512 KiB), into the gather slot of every rank (its own
//                        included) with plain 16-byte loads and posted stores, and after each piece bumps that piece's arrival counter on the
//                        receiving rank (red.release.sys). It runs on a side stream one unit ahead of the compute stream, so the copy overlaps
//                        the previous unit's GEMMs. Before it writes into a rank's slot it waits (bounded) until that rank has released the
//                        slot's previous occupant.
//   ft_fsdp_release      consumer side, on the compute stream after the last kernel that read a slot: tells every rank that this rank's copy of
//                        the slot may be overwritten.
//   ft_fsdp_gate         consumer side: waits (bounded) until a range of pieces has arrived. Used by consumers that are not GEMMs (the norm
//                        weights); the GEMMs wait inside their own TMA producer (gemm_2sm.cu: the consuming GEMM starts on the pieces that are
//                        there and stalls only at tiles whose weights are still in flight).
//
// Counters are monotonic: the n-th gather into a slot sets every piece counter it uses to n (one writer per piece and receiver), and the n-th release raises the releasing
// rank's entry of the slot's free flags to n; nothing is ever reset, so a late or repeated signal cannot be mistaken for a new one.
// Every wait has a deadline; on expiry the kernel records {kernel 9, site, peer / piece} in the status word and returns.
//
// Capability parity: the forward all-gather and restore_shards of ferrotorch-distributed/src/fsdp.rs:389-542,586-609 (host vectors over TCP
// there).
#include <cstdlib>

#include "common.cuh"
#include "host_common.h"

namespace {

constexpr int MAXR = 8;
constexpr uint32_t FT_K_FSDP = 9;
constexpr int PUSH_THREADS = 512;
constexpr int UNROLL = 4;

struct PushArgs {
  const uint4* src;              // this rank's shard (chunk_bytes)
  uint8_t* dst[MAXR];            // every rank's mapping of the slot (the shard of rank r goes to dst[q] + r * chunk_bytes)
  uint32_t* arrive[MAXR];        // every rank's arrival counters of the slot, u32 [world * pieces_per_chunk]
  const uint32_t* free_flags;    // local, u32 [world]: free_flags[q] = number of gathers into this slot that rank q has released
  uint32_t need_free;            // gathers into this slot before this one
  int rank, world;
  unsigned long long chunk_bytes, piece_bytes;
  int pieces_per_chunk;
  int reverse;                   // 1: last piece first (the backward pass consumes a unit from its end)
  unsigned long long timeout_ns;
};

__global__ void __launch_bounds__(PUSH_THREADS) fsdp_push_kernel(const PushArgs a, uint32_t* status) {
  __shared__ int dest_ok[MAXR];                 // 0 unknown, 1 released, -1 timed out
  if (threadIdx.x < MAXR) dest_ok[threadIdx.x] = 0;
  __syncthreads();
  const int items = a.pieces_per_chunk * a.world;
  for (int it = blockIdx.x; it < items; it += gridDim.x) {
    const int j0 = it / a.world, d = it % a.world;
    const int j = a.reverse ? a.pieces_per_chunk - 1 - j0 : j0;
    const int q = (a.rank + 1 + d) % a.world;     // peers first (rotated so that the ranks hit distinct receivers), the local copy last
    if (threadIdx.x == 0 && dest_ok[q] == 0) {
      const bool ok = wait_flag_ge(a.free_flags + q, a.need_free, a.timeout_ns);
      if (!ok) ft_set_status(status, FT_K_FSDP, 1, q);
      dest_ok[q] = ok ? 1 : -1;
    }
    __syncthreads();
    if (dest_ok[q] < 0) continue;                 // uniform for the CTA: the receiver never released the slot
    const unsigned long long off = (unsigned long long)j * a.piece_bytes;
    const unsigned long long n = min(a.piece_bytes, a.chunk_bytes - off);
    const uint4* s = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(a.src) + off);
    uint4* t = reinterpret_cast<uint4*>(a.dst[q] + (unsigned long long)a.rank * a.chunk_bytes + off);
    const unsigned long long nvec = n / 16;
    for (unsigned long long i = threadIdx.x; i < nvec; i += (unsigned long long)blockDim.x * UNROLL) {
      uint4 v[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; u++) {
        const unsigned long long k = i + (unsigned long long)u * blockDim.x;
        if (k < nvec) v[u] = __ldcs(s + k);
      }
#pragma unroll
      for (int u = 0; u < UNROLL; u++) {
        const unsigned long long k = i + (unsigned long long)u * blockDim.x;
        if (k < nvec) t[k] = v[u];
      }
    }
    __threadfence_system();
    __syncthreads();
    // one writer per (piece, receiver) and gather: the counter is SET to the gather number, so units with different piece counts can share a slot
    if (threadIdx.x == 0) st_release_sys(a.arrive[q] + a.rank * a.pieces_per_chunk + j, a.need_free + 1u);
  }
}

struct FreePtrs {
  uint32_t* f[MAXR];
};
__global__ void fsdp_release_kernel(const FreePtrs p, int world, uint32_t value) {
  __threadfence_system();
  if ((int)threadIdx.x < world) st_release_sys(p.f[threadIdx.x], value);
}

__global__ void __launch_bounds__(256) fsdp_gate_kernel(const uint32_t* __restrict__ arrive, int lo, int hi, uint32_t expected, unsigned long long timeout_ns,
                                                        uint32_t* status) {
  for (int p = lo + threadIdx.x; p < hi; p += blockDim.x) {
    if (!wait_flag_ge(arrive + p, expected, timeout_ns)) ft_set_status(status, FT_K_FSDP, 2, (uint32_t)p);
  }
}

// Copy-engine form of the push: the shard travels by cudaMemcpyAsync (no SM is occupied while the GEMMs run); these two small kernels frame it.
__global__ void fsdp_wait_free_kernel(const uint32_t* __restrict__ free_flags, int world, uint32_t need, unsigned long long timeout_ns, uint32_t* status) {
  if ((int)threadIdx.x < world && !wait_flag_ge(free_flags + threadIdx.x, need, timeout_ns)) ft_set_status(status, FT_K_FSDP, 3, threadIdx.x);
}
__global__ void __launch_bounds__(256) fsdp_signal_kernel(uint32_t* __restrict__ arrive, int count, uint32_t value) {
  __threadfence_system();
  for (int i = threadIdx.x; i < count; i += blockDim.x) st_release_sys(arrive + i, value);
}

unsigned long long g_timeout_ns = 0;
unsigned long long gather_timeout_ns() {
  if (g_timeout_ns == 0) {
    const char* e = getenv("FT_COMM_TIMEOUT_MS");
    const long long ms = e ? atoll(e) : 0;
    g_timeout_ns = ms > 0 ? (unsigned long long)ms * 1000000ull : 2000000000ull;
  }
  return g_timeout_ns;
}

}  // namespace

// Deadline (milliseconds) of the waits in the three kernels launched from now on (default 2000, or FT_COMM_TIMEOUT_MS).
FT_EXPORT int ft_fsdp_gather_set_timeout_ms(int ms) {
  if (ms < 1 || ms > 600000) return FT_ERR_ARG;
  g_timeout_ns = (unsigned long long)ms * 1000000ull;
  return FT_OK;
}

// src: this rank's shard, chunk_bytes (multiple of 16, and of piece_bytes unless the chunk is a single piece). slot_ptrs[q] / arrive_ptrs[q]:
// this rank's mappings of rank q's gather slot and of its arrival counters (u32 [world * pieces_per_chunk], zero before the first gather).
// free_flags: local u32 [world]. gather_no: 1 for the first gather into this slot, 2 for the second, ...; the kernel waits for
// free_flags[q] >= gather_no - 1 before it writes into rank q's slot and raises the piece counters to gather_no.
FT_EXPORT int ft_fsdp_push_shard(const void* src, void* const* slot_ptrs, void* const* arrive_ptrs, const void* free_flags, int rank, int world,
                                 int64_t chunk_bytes, int64_t piece_bytes, uint32_t gather_no, int reverse, int max_ctas, cudaStream_t st) {
  if (world < 1 || world > MAXR || rank < 0 || rank >= world || chunk_bytes <= 0 || (chunk_bytes & 15) || piece_bytes <= 0 || (piece_bytes & 15) || gather_no < 1)
    return FT_ERR_ARG;
  if (reinterpret_cast<uintptr_t>(src) & 15) return FT_ERR_ARG;
  PushArgs a = {};
  a.src = (const uint4*)src;
  for (int q = 0; q < world; q++) {
    a.dst[q] = (uint8_t*)slot_ptrs[q];
    a.arrive[q] = (uint32_t*)arrive_ptrs[q];
    if ((reinterpret_cast<uintptr_t>(slot_ptrs[q]) & 15) || arrive_ptrs[q] == nullptr) return FT_ERR_ARG;
  }
  a.free_flags = (const uint32_t*)free_flags;
  a.need_free = gather_no - 1;
  a.rank = rank;
  a.world = world;
  a.chunk_bytes = (unsigned long long)chunk_bytes;
  a.piece_bytes = (unsigned long long)piece_bytes;
  a.pieces_per_chunk = (int)((chunk_bytes + piece_bytes - 1) / piece_bytes);
  a.reverse = reverse ? 1 : 0;
  a.timeout_ns = gather_timeout_ns();
  int grid = a.pieces_per_chunk * world;
  const int cap = max_ctas > 0 ? max_ctas : 24;
  if (grid > cap) grid = cap;
  static int threads = 0;
  if (threads == 0) { const char* e = getenv("FT_FSDP_PUSH_THREADS"); threads = e ? atoi(e) : PUSH_THREADS; if (threads < 32 || threads > PUSH_THREADS) threads = PUSH_THREADS; }
  static bool configured = false;
  if (!configured) { ft_prefer_max_shared(fsdp_push_kernel); ft_prefer_max_shared(fsdp_release_kernel); ft_prefer_max_shared(fsdp_gate_kernel); configured = true; }
  fsdp_push_kernel<<<grid, threads, 0, st>>>(a, ft_status_ptr());
  return (int)cudaGetLastError();
}

// Writes `value` into this rank's entry of the slot's free flags on every rank: free_ptrs[q] is this rank's mapping of the word
// free[slot][rank] in rank q's memory.
FT_EXPORT int ft_fsdp_release(void* const* free_ptrs, int world, uint32_t value, cudaStream_t st) {
  if (world < 1 || world > MAXR) return FT_ERR_ARG;
  FreePtrs p = {};
  for (int q = 0; q < world; q++) p.f[q] = (uint32_t*)free_ptrs[q];
  fsdp_release_kernel<<<1, 32, 0, st>>>(p, world, value);
  return (int)cudaGetLastError();
}

// Waits until the arrival counters [piece_lo, piece_hi) of a slot (local memory) have all reached `expected`.
FT_EXPORT int ft_fsdp_gate(const void* arrive, int piece_lo, int piece_hi, uint32_t expected, cudaStream_t st) {
  if (arrive == nullptr || piece_lo < 0 || piece_hi <= piece_lo) return FT_ERR_ARG;
  fsdp_gate_kernel<<<1, 256, 0, st>>>((const uint32_t*)arrive, piece_lo, piece_hi, expected, gather_timeout_ns(), ft_status_ptr());
  return (int)cudaGetLastError();
}

// Copy-engine push, step 1: wait (bounded) on the gather stream until every rank has released the slot's previous occupant
// (free_flags[q] >= need for q < world; local memory).
FT_EXPORT int ft_fsdp_wait_free(const void* free_flags, int world, uint32_t need, cudaStream_t st) {
  if (world < 1 || world > MAXR || free_flags == nullptr) return FT_ERR_ARG;
  static bool configured = false;
  if (!configured) { ft_prefer_max_shared(fsdp_wait_free_kernel); ft_prefer_max_shared(fsdp_signal_kernel); configured = true; }
  fsdp_wait_free_kernel<<<1, 32, 0, st>>>((const uint32_t*)free_flags, world, need, gather_timeout_ns(), ft_status_ptr());
  return (int)cudaGetLastError();
}

// Step 2: one device-to-device copy per destination (dst may be a peer mapping: the copy engine moves it across NVLink).
FT_EXPORT int ft_memcpy_d2d_async(void* dst, const void* src, int64_t bytes, cudaStream_t st) {
  if (bytes <= 0 || dst == nullptr || src == nullptr) return FT_ERR_ARG;
  return (int)cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToDevice, st);
}

// Step 3, after the copy to a rank in stream order: set `count` arrival counters of that rank (arrive = this rank's mapping of the first one) to
// `value`, the number of this gather.
FT_EXPORT int ft_fsdp_signal(void* arrive, int count, uint32_t value, cudaStream_t st) {
  if (arrive == nullptr || count < 1) return FT_ERR_ARG;
  fsdp_signal_kernel<<<1, 256, 0, st>>>((uint32_t*)arrive, count, value);
  return (int)cudaGetLastError();
}
