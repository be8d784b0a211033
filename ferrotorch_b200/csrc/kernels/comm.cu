// Collectives and fused compute+collective kernels over NVLink peer memory (sm_100a).
//
// Every rank runs one process on its own GPU and maps every peer's symmetric buffers into its address space
// (torch.distributed._symmetric_memory provides the mapping). The kernels below address peers with plain
// ld/st (or multimem.* through the NVSwitch multicast address when one is bound) - no TMA multicast is used anywhere.
//
// Synchronisation: a per-rank flag block in symmetric memory, flags[phase][src_rank] (u32). A rank announces phase
// completion by storing the launch's sequence number into its slot on every peer (st.release.sys) and waits until all
// of its own slots reach that number (ld.acquire.sys). Every wait has a deadline (default 2 s): when it expires the
// kernel records {kernel, site, peer} in the status word and returns without touching peer data, so a missing peer
// turns into an error the host can read instead of a hung GPU.
//
//   ft_comm_allreduce      in-place two-shot all-reduce (each rank reduces its 1/N slice from all peers in fixed rank
//                          order, scales, and pushes the result to every peer), bf16 or f32, optional NVLS path
//   ft_comm_allreduce_1shot small messages: every rank reduces the whole buffer locally from all peers
//   ft_comm_reduce_scatter / ft_comm_allgather
//   ft_fsdp_rs_adamw_ag    reduce-scatter of a flat bf16 gradient unit fused with the sharded AdamW update of the f32
//                          master/moments and the all-gather (push) of the updated bf16 slice to every peer
//
// Capability parity: star all-reduce / all-gather / reduce-scatter on host vectors (ferrotorch-distributed/src/
// collective.rs:64-410), NCCL wrappers (nccl_collective.rs:75-260), FSDP sync_gradients + broadcast_updated_params
// (fsdp.rs:627-845).
#include <cstdlib>

#include "common.cuh"
#include "host_common.h"

namespace {

constexpr int MAX_RANKS = 8;
constexpr uint64_t COMM_TIMEOUT_NS = 2000000000ull;

struct PeerPtrs {
  void* p[MAX_RANKS];
};

// flags block per rank: u32 [4 phases][MAX_RANKS] followed by a u32 grid counter per phase pair
struct CommSync {
  uint32_t* flags[MAX_RANKS];   // flags[r] = base of rank r's flag block (peer mapped)
  uint32_t* counter;            // local device memory, u32[2], zero between launches
  int rank, world;
  uint32_t seq;                 // sequence number of this launch (same on every rank)
  uint32_t* seq_dev;            // optional: the sequence lives in device memory (seq = *seq_dev + 1, written back by the last CTA), so a
                                // launch captured in a CUDA graph advances it on every replay
  // optional per-launch phase stamps (globaltimer ns): record (seq % trace_cap) = {seq | kind << 32, entered, peers ready, body done, retired}
  unsigned long long* trace;
  uint32_t trace_cap, trace_kind;
  uint64_t timeout_ns;          // deadline of every wait on a peer in this launch
};
constexpr int TRACE_WORDS = 5;
FT_DEVICE void trace_stamp(const CommSync& s, int word) {
  if (s.trace == nullptr) return;
  unsigned long long* rec = s.trace + (size_t)(s.seq % s.trace_cap) * TRACE_WORDS;
  if (word == 1) rec[0] = (unsigned long long)s.seq | ((unsigned long long)s.trace_kind << 32);
  rec[word] = globaltimer_ns();
}

// One thread per peer: tell every peer that this rank reached `phase` of launch `seq`.
FT_DEVICE void signal_peers(const CommSync& s, int phase) {
  if (threadIdx.x < s.world) st_release_sys(s.flags[threadIdx.x] + phase * MAX_RANKS + s.rank, s.seq);
}
// Every thread < world polls one local slot. Returns false on timeout (warp-uniform result for warp 0).
FT_DEVICE bool wait_peers(const CommSync& s, int phase, uint32_t* status, int site) {
  bool ok = true;
  if (threadIdx.x < s.world) {
    ok = wait_flag_ge(s.flags[s.rank] + phase * MAX_RANKS + threadIdx.x, s.seq, s.timeout_ns);
    if (!ok) ft_set_status(status, FT_K_COMM, site, threadIdx.x);
  }
  return ok;
}

// Start-of-kernel rendezvous: CTA 0 signals; every CTA waits on the local flags. Returns false if any peer is missing.
FT_DEVICE bool comm_begin(CommSync& s, uint32_t* status) {
  if (s.seq_dev) s.seq = *reinterpret_cast<volatile uint32_t*>(s.seq_dev) + 1;   // read before any CTA can reach comm_end's write-back
  __shared__ int ok_sh;
  if (threadIdx.x == 0) ok_sh = 1;
  if (blockIdx.x == 0 && threadIdx.x == 0) trace_stamp(s, 1);
  __syncthreads();
  if (blockIdx.x == 0) signal_peers(s, 0);
  if (!wait_peers(s, 0, status, 1)) ok_sh = 0;
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x == 0) trace_stamp(s, 2);
  return ok_sh != 0;
}

// End-of-kernel rendezvous: the last CTA to finish announces completion to the peers and waits for theirs, so that when
// the kernel retires (a) every peer has finished reading this rank's buffers and (b) every peer's pushes into this
// rank's buffers have landed.
FT_DEVICE void comm_end(const CommSync& s, uint32_t* status) {
  __threadfence_system();
  __syncthreads();
  __shared__ int last;
  if (threadIdx.x == 0) {
    uint32_t prev = atomicAdd(s.counter, 1u);
    last = (prev == gridDim.x - 1);
  }
  __syncthreads();
  if (!last) return;
  if (threadIdx.x == 0) { *s.counter = 0; trace_stamp(s, 3); }    // counter: ready for the next launch on this stream
  __threadfence_system();
  signal_peers(s, 1);
  wait_peers(s, 1, status, 2);
  if (threadIdx.x == 0) trace_stamp(s, 4);
  if (s.seq_dev && threadIdx.x == 0) *s.seq_dev = s.seq;
}

// A CTA whose opening rendezvous timed out still takes part in the grid's bookkeeping: it is counted, and if it is the last one it zeroes the
// counter and advances the device-side sequence number. Without this a launch in which only some CTAs time out (or a peer's flag arrives just
// after the deadline) would leave the counter non-zero and every later collective on the communicator would fail to elect a last CTA.
// The data phase and the closing handshake are skipped: nothing of a peer is touched after a timeout.
FT_DEVICE void comm_abort(const CommSync& s) {
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(s.counter, 1u);
    if (prev == gridDim.x - 1) {
      *s.counter = 0;
      if (s.seq_dev) *s.seq_dev = s.seq;
    }
  }
}

template <typename T> struct Vec16;
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static FT_DEVICE void load(const __nv_bfloat16* p, float* f) { bf16x8 v = *reinterpret_cast<const bf16x8*>(p); bf16x8_to_float(v, f); }
  static FT_DEVICE void store(__nv_bfloat16* p, const float* f) { *reinterpret_cast<bf16x8*>(p) = float_to_bf16x8(f); }
};
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static FT_DEVICE void load(const float* p, float* f) { float4 v = *reinterpret_cast<const float4*>(p); f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w; }
  static FT_DEVICE void store(float* p, const float* f) { *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]); }
};

// ---------------------------------------------------------------------------------------------------------
// two-shot all-reduce, in place: buf_p[i] <- scale * sum_q buf_q[i]
// ---------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(512) allreduce_2shot_kernel(PeerPtrs bufs, CommSync s, size_t n, float scale, uint32_t* status) {
  if (!comm_begin(s, status)) { comm_abort(s); return; }
  constexpr int V = Vec16<T>::N;
  const size_t nvec = n / V;
  const size_t per = (nvec + s.world - 1) / s.world;
  const size_t lo = per * s.rank, hi = min(nvec, lo + per);
  for (size_t i = lo + blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < hi; i += (size_t)gridDim.x * blockDim.x) {
    float acc[V];
#pragma unroll
    for (int e = 0; e < V; e++) acc[e] = 0.f;
    float f[MAX_RANKS][V];
#pragma unroll
    for (int q = 0; q < MAX_RANKS; q++)
      if (q < s.world) Vec16<T>::load(reinterpret_cast<const T*>(bufs.p[q]) + i * V, f[q]);
#pragma unroll
    for (int q = 0; q < MAX_RANKS; q++)
      if (q < s.world)
#pragma unroll
        for (int e = 0; e < V; e++) acc[e] += f[q][e];
#pragma unroll
    for (int e = 0; e < V; e++) acc[e] *= scale;
#pragma unroll
    for (int q = 0; q < MAX_RANKS; q++)
      if (q < s.world) Vec16<T>::store(reinterpret_cast<T*>(bufs.p[q]) + i * V, acc);
  }
  // scalar tail (n % V) handled by rank 0
  if (s.rank == 0 && blockIdx.x == 0) {
    for (size_t i = nvec * V + threadIdx.x; i < n; i += blockDim.x) {
      float a = 0.f;
      for (int q = 0; q < s.world; q++) a += (float)reinterpret_cast<const T*>(bufs.p[q])[i];
      a *= scale;
      for (int q = 0; q < s.world; q++) reinterpret_cast<T*>(bufs.p[q])[i] = (T)a;
    }
  }
  comm_end(s, status);
}

// NVLS (NVSwitch multicast) helpers: one multimem.ld_reduce returns the sum over every rank's copy of 16 bytes (reduced inside the switch, f32
// accumulation), one multimem.st writes 16 bytes into every rank's copy. `mc` is this rank's mapping of the multicast address of the buffer.
template <typename T> struct Nvls;
template <> struct Nvls<__nv_bfloat16> {
  static FT_DEVICE uint4 ld_reduce(const void* p) {
    uint4 r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
    return r;
  }
  static FT_DEVICE uint4 scale(uint4 v, float s) {
    uint32_t r[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&r[e]));
      const __nv_bfloat162 h = __floats2bfloat162_rn(f.x * s, f.y * s);
      r[e] = *reinterpret_cast<const uint32_t*>(&h);
    }
    return make_uint4(r[0], r[1], r[2], r[3]);
  }
};
template <> struct Nvls<float> {
  static FT_DEVICE uint4 ld_reduce(const void* p) {
    uint4 r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
    return r;
  }
  static FT_DEVICE uint4 scale(uint4 v, float s) {
    return make_uint4(__float_as_uint(__uint_as_float(v.x) * s), __float_as_uint(__uint_as_float(v.y) * s), __float_as_uint(__uint_as_float(v.z) * s),
                      __float_as_uint(__uint_as_float(v.w) * s));
  }
};
FT_DEVICE void multimem_st_v4(void* p, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// NVLS all-reduce, in place: every rank reduces its 1/N slice inside the switch and broadcasts the result through the switch.
template <typename T>
__global__ void __launch_bounds__(512) allreduce_nvls_kernel(T* mc, CommSync s, size_t n, float scale, uint32_t* status) {
  if (!comm_begin(s, status)) { comm_abort(s); return; }
  constexpr int V = Vec16<T>::N;
  const size_t nvec = n / V;
  const size_t per = (nvec + s.world - 1) / s.world;
  const size_t lo = per * s.rank, hi = min(nvec, lo + per);
  for (size_t i = lo + blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < hi; i += (size_t)gridDim.x * blockDim.x) {
    uint4 r = Nvls<T>::ld_reduce(mc + i * V);
    if (scale != 1.f) r = Nvls<T>::scale(r, scale);
    multimem_st_v4(mc + i * V, r);
  }
  comm_end(s, status);
}

// NVLS reduce-scatter: out_local = scale * (sum over ranks of buf_q[rank * chunk ...]), one in-switch reduction per 16 bytes. The slice is read as
// `rows` rows of `cols` elements (contiguous in the buffer) and written with a row pitch of out_ld elements, so a column block of a wider output
// can be the destination. 256 threads per CTA: the kernel may run beside a GEMM (see host_common.h).
template <typename T>
__global__ void __launch_bounds__(256) reduce_scatter_nvls_kernel(const T* mc, T* __restrict__ out, CommSync s, size_t rows, size_t cols, size_t out_ld,
                                                                  float scale, uint32_t* status) {
  if (!comm_begin(s, status)) { comm_abort(s); return; }
  constexpr int V = Vec16<T>::N;
  constexpr int U = 4;                                       // in-switch reductions in flight per thread: the round trip through the switch is long
  const size_t vpr = cols / V, nvec = rows * vpr, base = rows * cols * s.rank;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i0 = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i0 < nvec; i0 += stride * U) {
    uint4 r[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const size_t i = i0 + u * stride;
      if (i < nvec) r[u] = Nvls<T>::ld_reduce(mc + base + i * V);
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      const size_t i = i0 + u * stride;
      if (i < nvec) *reinterpret_cast<uint4*>(out + (i / vpr) * out_ld + (i % vpr) * V) = scale != 1.f ? Nvls<T>::scale(r[u], scale) : r[u];
    }
  }
  comm_end(s, status);
}

// one-shot: out_local[i] = scale * sum_q buf_q[i]; for messages small enough that latency dominates
template <typename T>
__global__ void __launch_bounds__(512) allreduce_1shot_kernel(PeerPtrs bufs, T* __restrict__ out, CommSync s, size_t n, float scale,
                                                              uint32_t* status) {
  if (!comm_begin(s, status)) { comm_abort(s); return; }
  constexpr int V = Vec16<T>::N;
  const size_t nvec = n / V;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
    float acc[V];
#pragma unroll
    for (int e = 0; e < V; e++) acc[e] = 0.f;
    for (int q = 0; q < s.world; q++) {
      float f[V];
      Vec16<T>::load(reinterpret_cast<const T*>(bufs.p[q]) + i * V, f);
#pragma unroll
      for (int e = 0; e < V; e++) acc[e] += f[e];
    }
#pragma unroll
    for (int e = 0; e < V; e++) acc[e] *= scale;
    Vec16<T>::store(out + i * V, acc);
  }
  if (blockIdx.x == 0)
    for (size_t i = nvec * V + threadIdx.x; i < n; i += blockDim.x) {
      float a = 0.f;
      for (int q = 0; q < s.world; q++) a += (float)reinterpret_cast<const T*>(bufs.p[q])[i];
      out[i] = (T)(a * scale);
    }
  comm_end(s, status);
}

// reduce-scatter: out_local[i] = scale * sum_q buf_q[rank*chunk + i], i < chunk
template <typename T>
__global__ void __launch_bounds__(512) reduce_scatter_kernel(PeerPtrs bufs, T* __restrict__ out, CommSync s, size_t chunk, float scale,
                                                             uint32_t* status) {
  if (!comm_begin(s, status)) { comm_abort(s); return; }
  constexpr int V = Vec16<T>::N;
  const size_t nvec = chunk / V, base = chunk * s.rank;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
    uint4 raw[MAX_RANKS];                                  // every peer's 16 bytes are requested before any is used: the NVLink loads overlap
#pragma unroll
    for (int q = 0; q < MAX_RANKS; q++)
      if (q < s.world) raw[q] = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(bufs.p[q]) + base + i * V);
    float acc[V];
#pragma unroll
    for (int e = 0; e < V; e++) acc[e] = 0.f;
#pragma unroll
    for (int q = 0; q < MAX_RANKS; q++)
      if (q < s.world) {
        float f[V];
        Vec16<T>::load(reinterpret_cast<const T*>(&raw[q]), f);
#pragma unroll
        for (int e = 0; e < V; e++) acc[e] += f[e];          // fixed rank order
      }
#pragma unroll
    for (int e = 0; e < V; e++) acc[e] *= scale;
    Vec16<T>::store(out + i * V, acc);
  }
  comm_end(s, status);
}

// all-gather (push): buf_q[rank*chunk + i] = src_local[i] for every q
template <typename T>
__global__ void __launch_bounds__(512) allgather_kernel(PeerPtrs bufs, const T* __restrict__ src, CommSync s, size_t chunk, uint32_t* status) {
  if (!comm_begin(s, status)) { comm_abort(s); return; }
  constexpr int V = Vec16<T>::N;
  const size_t nvec = chunk / V, base = chunk * s.rank;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
    const uint4 v = *reinterpret_cast<const uint4*>(src + i * V);
    for (int q = 0; q < s.world; q++) *reinterpret_cast<uint4*>(reinterpret_cast<T*>(bufs.p[q]) + base + i * V) = v;
  }
  comm_end(s, status);
}

// all-to-all (pull): out[q*chunk + i] = buf_q[rank*chunk + i]: every rank exposes W chunks (chunk q is addressed to rank q) and pulls the chunks
// addressed to itself from every peer. The building block of Ulysses sequence parallelism and of expert dispatch / combine.
template <typename T>
__global__ void __launch_bounds__(512) alltoall_kernel(PeerPtrs bufs, T* __restrict__ out, CommSync s, size_t chunk, uint32_t* status) {
  if (!comm_begin(s, status)) { comm_abort(s); return; }
  constexpr int V = Vec16<T>::N;
  const size_t nvec = chunk / V, total = nvec * s.world;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int q = (int)(i / nvec);
    const size_t k = i % nvec;
    const int src = (s.rank + q) % s.world;                 // start at the own chunk so the ranks do not all read the same peer first
    const uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(bufs.p[src]) + chunk * s.rank + k * V);
    *reinterpret_cast<uint4*>(out + chunk * src + k * V) = v;
  }
  comm_end(s, status);
}

// broadcast (pull): out[i] = buf_root[i] on every rank
template <typename T>
__global__ void __launch_bounds__(512) broadcast_kernel(PeerPtrs bufs, T* __restrict__ out, CommSync s, int root, size_t n, uint32_t* status) {
  if (!comm_begin(s, status)) { comm_abort(s); return; }
  constexpr int V = Vec16<T>::N;
  const size_t nvec = n / V;
  if (s.rank != root || out != bufs.p[root]) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x)
      *reinterpret_cast<uint4*>(out + i * V) = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(bufs.p[root]) + i * V);
  }
  comm_end(s, status);
}

// ---------------------------------------------------------------------------------------------------------
// FSDP: reduce-scatter(mean) of the bf16 gradient unit + AdamW on the owned f32 slice + push all-gather
// ---------------------------------------------------------------------------------------------------------
struct AdamWArgsC { float lr, beta1, beta2, eps, weight_decay, bias_c1, bias_c2; };

// local_out != null: the fully sharded form. The refreshed bf16 slice is written to this rank's own shard only (local_out[i]); nothing is pushed,
// the parameters are gathered again when the next forward pass needs them (fsdp_gather.cu).
// 256 threads and raw 16-byte gradient loads keep the kernel light (registers, warps per SM sub-partition): it runs on a side stream BESIDE the
// backward GEMMs, and a CTA that does not fit next to a GEMM CTA would make the GEMM wait for it instead.
__global__ void __maxnreg__(80) fsdp_rs_adamw_ag_kernel(PeerPtrs grads, PeerPtrs params, CommSync s, float* __restrict__ master,
                                                               float* __restrict__ m, float* __restrict__ v, size_t chunk, AdamWArgsC a,
                                                               const float* __restrict__ grad_scale_ptr, __nv_bfloat16* __restrict__ local_out,
                                                               uint32_t* status) {
  if (!comm_begin(s, status)) { comm_abort(s); return; }
  const float inv_world = (grad_scale_ptr ? *grad_scale_ptr : 1.f) / (float)s.world;
  const float decay = 1.f - a.lr * a.weight_decay, step = a.lr / a.bias_c1, inv_c2 = rsqrtf(a.bias_c2);
  const size_t nvec = chunk / 8, base = chunk * s.rank;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
    uint4 raw[MAX_RANKS];                                     // every peer's slice is requested before any is used: the loads overlap
#pragma unroll
    for (int q = 0; q < MAX_RANKS; q++)
      if (q < s.world) raw[q] = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(grads.p[q]) + base + i * 8);
    float g[8];
#pragma unroll
    for (int e = 0; e < 8; e++) g[e] = 0.f;
#pragma unroll
    for (int q = 0; q < MAX_RANKS; q++)
      if (q < s.world) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[q]);
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const float2 f2 = __bfloat1622float2(h[e]);
          g[2 * e] += f2.x;                                   // fixed rank order: identical bits on every rank
          g[2 * e + 1] += f2.y;
        }
      }
    float4* pm = reinterpret_cast<float4*>(master + i * 8);
    float4* mm = reinterpret_cast<float4*>(m + i * 8);
    float4* vv = reinterpret_cast<float4*>(v + i * 8);
    float p[8], m1[8], v1[8];
    { float4 t0 = pm[0], t1 = pm[1]; p[0] = t0.x; p[1] = t0.y; p[2] = t0.z; p[3] = t0.w; p[4] = t1.x; p[5] = t1.y; p[6] = t1.z; p[7] = t1.w; }
    { float4 t0 = mm[0], t1 = mm[1]; m1[0] = t0.x; m1[1] = t0.y; m1[2] = t0.z; m1[3] = t0.w; m1[4] = t1.x; m1[5] = t1.y; m1[6] = t1.z; m1[7] = t1.w; }
    { float4 t0 = vv[0], t1 = vv[1]; v1[0] = t0.x; v1[1] = t0.y; v1[2] = t0.z; v1[3] = t0.w; v1[4] = t1.x; v1[5] = t1.y; v1[6] = t1.z; v1[7] = t1.w; }
#pragma unroll
    for (int e = 0; e < 8; e++) {
      const float gg = g[e] * inv_world;
      p[e] *= decay;
      m1[e] = a.beta1 * m1[e] + (1.f - a.beta1) * gg;
      v1[e] = a.beta2 * v1[e] + (1.f - a.beta2) * gg * gg;
      p[e] -= step * m1[e] / (sqrtf(v1[e]) * inv_c2 + a.eps);
    }
    pm[0] = make_float4(p[0], p[1], p[2], p[3]); pm[1] = make_float4(p[4], p[5], p[6], p[7]);
    mm[0] = make_float4(m1[0], m1[1], m1[2], m1[3]); mm[1] = make_float4(m1[4], m1[5], m1[6], m1[7]);
    vv[0] = make_float4(v1[0], v1[1], v1[2], v1[3]); vv[1] = make_float4(v1[4], v1[5], v1[6], v1[7]);
    const bf16x8 out = float_to_bf16x8(p);
    if (local_out != nullptr) {
      *reinterpret_cast<bf16x8*>(local_out + i * 8) = out;
    } else {
#pragma unroll
      for (int q = 0; q < MAX_RANKS; q++)
        if (q < s.world) *reinterpret_cast<bf16x8*>(reinterpret_cast<__nv_bfloat16*>(params.p[q]) + base + i * 8) = out;
    }
  }
  comm_end(s, status);
}

// stand-alone device barrier (phase 0 + phase 1 rendezvous, no data)
__global__ void comm_barrier_kernel(CommSync s, uint32_t* status) {
  if (!comm_begin(s, status)) { comm_abort(s); return; }
  comm_end(s, status);
}

inline int comm_grid(size_t work, int max_ctas) {
  size_t g = (work + 511) / 512;
  if (g < 1) g = 1;
  return (int)(g < (size_t)max_ctas ? g : (size_t)max_ctas);
}

// Phase-stamp ring of the current device (null = off), set by ft_comm_set_trace.
unsigned long long* g_trace[64] = {nullptr};
uint32_t g_trace_cap[64] = {0};
// Deadline of the waits on peers inside the collective kernels: 2 s unless FT_COMM_TIMEOUT_MS or ft_comm_set_timeout_ms says otherwise.
uint64_t g_timeout_ns = 0;
uint64_t comm_timeout_ns() {
  if (g_timeout_ns == 0) {
    const char* e = getenv("FT_COMM_TIMEOUT_MS");
    const long long ms = e ? atoll(e) : 0;
    g_timeout_ns = ms > 0 ? (uint64_t)ms * 1000000ull : COMM_TIMEOUT_NS;
  }
  return g_timeout_ns;
}

int fill_sync(CommSync& s, void* const* flag_ptrs, uint32_t* counter, int rank, int world, uint32_t seq, uint32_t kind = 0) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return FT_ERR_ARG;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  s.trace = g_trace[dev];
  s.trace_cap = g_trace_cap[dev];
  s.trace_kind = kind;
  s.timeout_ns = comm_timeout_ns();
  for (int i = 0; i < MAX_RANKS; i++) s.flags[i] = i < world ? reinterpret_cast<uint32_t*>(flag_ptrs[i]) : nullptr;
  s.counter = counter;
  s.rank = rank;
  s.world = world;
  s.seq = seq;
  s.seq_dev = nullptr;
  return FT_OK;
}

// ---------------------------------------------------------------------------------------------------------
// point-to-point: put into a slot of the receiver's ring + flag; the receiver waits for the flag and copies out
// ---------------------------------------------------------------------------------------------------------
// ring slot layout on the receiver: [payload bytes ...]; flags: u32 per slot holding the message number that filled it (1, 2, ...),
// ack: u32 per slot on the SENDER holding the number of the last message the receiver consumed from that slot.
// Both point-to-point kernels count their CTAs in one u32: the low half counts CTAs that are through, the high half those whose wait ran
// out. The last CTA always resets the word (so a partial timeout leaves the channel usable) and raises the flag / acknowledgement only when
// no CTA failed.
FT_DEVICE void p2p_finish(unsigned int* counter, bool ok, uint32_t* signal, uint32_t msg, bool fence) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(counter, ok ? 1u : 0x10001u);
    if ((prev & 0xffffu) == gridDim.x - 1) {
      const unsigned int fails = (prev >> 16) + (ok ? 0u : 1u);
      *counter = 0;
      if (fence) __threadfence_system();
      if (fails == 0) st_release_sys(signal, msg);
    }
  }
}

__global__ void __launch_bounds__(512) p2p_put_kernel(const uint4* __restrict__ src, uint4* __restrict__ peer_slot, size_t nvec, uint32_t* __restrict__ peer_flag,
                                                      const uint32_t* __restrict__ my_ack, uint32_t msg, uint32_t prev_msg_in_slot, unsigned int* __restrict__ counter,
                                                      uint64_t timeout_ns, uint32_t* status) {
  // the slot must have been drained by the receiver (its ack names the previous message that used this slot)
  __shared__ int ok_sh;
  if (threadIdx.x == 0) {
    ok_sh = 1;
    if (prev_msg_in_slot != 0 && !wait_flag_ge(my_ack, prev_msg_in_slot, timeout_ns)) {
      ft_set_status(status, FT_K_COMM, 21, msg);
      ok_sh = 0;
    }
  }
  __syncthreads();
  const bool ok = ok_sh != 0;
  if (ok)
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) peer_slot[i] = src[i];
  p2p_finish(counter, ok, peer_flag, msg, true);
}

__global__ void __launch_bounds__(512) p2p_get_kernel(uint4* __restrict__ dst, const uint4* __restrict__ my_slot, size_t nvec, const uint32_t* __restrict__ my_flag,
                                                      uint32_t* __restrict__ peer_ack, uint32_t msg, unsigned int* __restrict__ counter, uint64_t timeout_ns,
                                                      uint32_t* status) {
  __shared__ int ok_sh;
  if (threadIdx.x == 0) {
    ok_sh = wait_flag_ge(my_flag, msg, timeout_ns) ? 1 : 0;
    if (!ok_sh) ft_set_status(status, FT_K_COMM, 22, msg);
  }
  __syncthreads();
  const bool ok = ok_sh != 0;
  if (ok)
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) dst[i] = __ldcg(my_slot + i);
  p2p_finish(counter, ok, peer_ack, msg, false);                // the sender may overwrite the slot
}

}  // namespace

// Phase stamps of the collective kernels launched on the current device from now on: `ring` is device memory for `capacity` records of five
// u64 words {launch number | kind << 32, entered, peers ready, body done, retired} in globaltimer nanoseconds; record index = launch number
// modulo capacity. kind: 1 all-reduce, 2 one-shot all-reduce, 3 reduce-scatter, 4 all-gather, 5 all-to-all, 6 broadcast, 7 barrier,
// 8 fused reduce-scatter + AdamW + all-gather. ring = null switches the stamps off (the default).
FT_EXPORT int ft_comm_set_trace(void* ring, int capacity) {
  int dev = 0;
  FT_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || (ring != nullptr && capacity < 1)) return FT_ERR_ARG;
  g_trace[dev] = (unsigned long long*)ring;
  g_trace_cap[dev] = ring ? (uint32_t)capacity : 0u;
  return FT_OK;
}

// Deadline (milliseconds, 1 .. 600 000) of the waits on peers in the collective kernels launched from now on; every rank of a group should
// use the same value. The environment variable FT_COMM_TIMEOUT_MS sets the initial value (default 2000).
FT_EXPORT int ft_comm_set_timeout_ms(int ms) {
  if (ms < 1 || ms > 600000) return FT_ERR_ARG;
  g_timeout_ns = (uint64_t)ms * 1000000ull;
  return FT_OK;
}

// Size in bytes of the per-rank flag block the kernels expect (zero-initialised symmetric memory).
FT_EXPORT int ft_comm_flag_bytes() { return 4 * MAX_RANKS * 4; }

// buf_ptrs / flag_ptrs: host arrays of `world` device pointers (this rank's mappings of every rank's buffer / flag block).
// counter: local device u32[2], zeroed once. seq: launch sequence number, identical on all ranks, increasing by one per launch.
// dtype: 0 bf16, 1 f32. mc_ptr: multicast mapping of the same buffer or null (NVLS used only when non-null, bf16, n % (8*world) == 0).
FT_EXPORT int ft_comm_allreduce(void* const* buf_ptrs, void* const* flag_ptrs, uint32_t* counter, int rank, int world, uint32_t seq,
                                int64_t n, int dtype, float scale, void* mc_ptr, int max_ctas, cudaStream_t st) {
  CommSync s;
  int r = fill_sync(s, flag_ptrs, counter, rank, world, seq, 1);
  if (r) return r;
  if (n <= 0) return FT_ERR_ARG;
  PeerPtrs b;
  for (int i = 0; i < MAX_RANKS; i++) b.p[i] = i < world ? buf_ptrs[i] : nullptr;
  uint32_t* status = ft_status_ptr();
  const int V = dtype == 0 ? 8 : 4;
  const int grid = comm_grid((size_t)n / V / world + 1, max_ctas > 0 ? max_ctas : 64);
  if (mc_ptr && dtype == 0 && (n % (8 * (int64_t)world)) == 0)
    allreduce_nvls_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>((__nv_bfloat16*)mc_ptr, s, (size_t)n, scale, status);
  else if (mc_ptr && dtype == 1 && (n % (4 * (int64_t)world)) == 0)
    allreduce_nvls_kernel<float><<<grid, 512, 0, st>>>((float*)mc_ptr, s, (size_t)n, scale, status);
  else if (dtype == 0)
    allreduce_2shot_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>(b, s, (size_t)n, scale, status);
  else
    allreduce_2shot_kernel<float><<<grid, 512, 0, st>>>(b, s, (size_t)n, scale, status);
  return (int)cudaGetLastError();
}

// seq_dev (optional, device u32): when non-null the launch takes its sequence number from device memory and advances it, which makes
// the launch replayable from a CUDA graph; `seq` is then ignored. All ranks must use the same mode for a given flag block.
FT_EXPORT int ft_comm_allreduce_1shot(void* const* buf_ptrs, void* out, void* const* flag_ptrs, uint32_t* counter, int rank, int world,
                                      uint32_t seq, int64_t n, int dtype, float scale, int max_ctas, uint32_t* seq_dev, cudaStream_t st) {
  CommSync s;
  int r = fill_sync(s, flag_ptrs, counter, rank, world, seq, 2);
  if (r) return r;
  s.seq_dev = seq_dev;
  if (n <= 0) return FT_ERR_ARG;
  PeerPtrs b;
  for (int i = 0; i < MAX_RANKS; i++) b.p[i] = i < world ? buf_ptrs[i] : nullptr;
  const int V = dtype == 0 ? 8 : 4;
  const int grid = comm_grid((size_t)n / V + 1, max_ctas > 0 ? max_ctas : 32);
  if (dtype == 0) allreduce_1shot_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>(b, (__nv_bfloat16*)out, s, (size_t)n, scale, ft_status_ptr());
  else allreduce_1shot_kernel<float><<<grid, 512, 0, st>>>(b, (float*)out, s, (size_t)n, scale, ft_status_ptr());
  return (int)cudaGetLastError();
}

// out[chunk] = scale * sum over ranks of buf_q[rank*chunk : (rank+1)*chunk]; chunk % (16/elem) == 0
FT_EXPORT int ft_comm_reduce_scatter(void* const* buf_ptrs, void* out, void* const* flag_ptrs, uint32_t* counter, int rank, int world,
                                     uint32_t seq, int64_t chunk, int dtype, float scale, int max_ctas, cudaStream_t st) {
  CommSync s;
  int r = fill_sync(s, flag_ptrs, counter, rank, world, seq, 3);
  if (r) return r;
  const int V = dtype == 0 ? 8 : 4;
  if (chunk <= 0 || chunk % V) return FT_ERR_ARG;
  PeerPtrs b;
  for (int i = 0; i < MAX_RANKS; i++) b.p[i] = i < world ? buf_ptrs[i] : nullptr;
  const int grid = comm_grid((size_t)chunk / V, max_ctas > 0 ? max_ctas : 64);
  if (dtype == 0) reduce_scatter_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>(b, (__nv_bfloat16*)out, s, (size_t)chunk, scale, ft_status_ptr());
  else reduce_scatter_kernel<float><<<grid, 512, 0, st>>>(b, (float*)out, s, (size_t)chunk, scale, ft_status_ptr());
  return (int)cudaGetLastError();
}

// Two-dimensional form of the in-switch reduce-scatter: this rank's slice is `rows` x `cols` elements, contiguous in the exposed buffer at
// element offset rank * rows * cols; it is written to `out` with a row pitch of out_ld elements (cols and out_ld multiples of 16 bytes).
FT_EXPORT int ft_comm_reduce_scatter_nvls_2d(void* mc_ptr, void* out, void* const* flag_ptrs, uint32_t* counter, int rank, int world, uint32_t seq,
                                             int64_t rows, int64_t cols, int64_t out_ld, int dtype, float scale, int max_ctas, cudaStream_t st) {
  CommSync s;
  int r = fill_sync(s, flag_ptrs, counter, rank, world, seq, 3);
  if (r) return r;
  const int V = dtype == 0 ? 8 : 4;
  if (mc_ptr == nullptr || rows <= 0 || cols <= 0 || cols % V || out_ld % V || out_ld < cols) return FT_ERR_ARG;
  size_t g = ((size_t)rows * cols / V / 4 + 255) / 256;
  const size_t cap = max_ctas > 0 ? max_ctas : 148;
  const int grid = (int)(g < 1 ? 1 : (g < cap ? g : cap));
  static bool configured = false;
  if (!configured) { ft_prefer_max_shared(reduce_scatter_nvls_kernel<__nv_bfloat16>); ft_prefer_max_shared(reduce_scatter_nvls_kernel<float>); configured = true; }
  if (dtype == 0) reduce_scatter_nvls_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)mc_ptr, (__nv_bfloat16*)out, s, (size_t)rows, (size_t)cols, (size_t)out_ld, scale, ft_status_ptr());
  else reduce_scatter_nvls_kernel<float><<<grid, 256, 0, st>>>((const float*)mc_ptr, (float*)out, s, (size_t)rows, (size_t)cols, (size_t)out_ld, scale, ft_status_ptr());
  return (int)cudaGetLastError();
}

// The same through the switch: mc_ptr is the multicast mapping of the buffer the ranks exposed (NVLS). One multimem.ld_reduce per 16 bytes replaces
// `world` peer loads, so the ingress of a rank is one slice instead of `world - 1`.
FT_EXPORT int ft_comm_reduce_scatter_nvls(void* mc_ptr, void* out, void* const* flag_ptrs, uint32_t* counter, int rank, int world, uint32_t seq,
                                          int64_t chunk, int dtype, float scale, int max_ctas, cudaStream_t st) {
  return ft_comm_reduce_scatter_nvls_2d(mc_ptr, out, flag_ptrs, counter, rank, world, seq, 1, chunk, chunk, dtype, scale, max_ctas, st);
}

// every rank's buf[rank*chunk : (rank+1)*chunk] on every peer = src[chunk]
FT_EXPORT int ft_comm_allgather(void* const* buf_ptrs, const void* src, void* const* flag_ptrs, uint32_t* counter, int rank, int world,
                                uint32_t seq, int64_t chunk, int dtype, int max_ctas, cudaStream_t st) {
  CommSync s;
  int r = fill_sync(s, flag_ptrs, counter, rank, world, seq, 4);
  if (r) return r;
  const int V = dtype == 0 ? 8 : 4;
  if (chunk <= 0 || chunk % V) return FT_ERR_ARG;
  PeerPtrs b;
  for (int i = 0; i < MAX_RANKS; i++) b.p[i] = i < world ? buf_ptrs[i] : nullptr;
  const int grid = comm_grid((size_t)chunk / V, max_ctas > 0 ? max_ctas : 64);
  if (dtype == 0) allgather_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>(b, (const __nv_bfloat16*)src, s, (size_t)chunk, ft_status_ptr());
  else allgather_kernel<float><<<grid, 512, 0, st>>>(b, (const float*)src, s, (size_t)chunk, ft_status_ptr());
  return (int)cudaGetLastError();
}

// out[q*chunk : (q+1)*chunk] = rank q's buf[rank*chunk : (rank+1)*chunk]; buf holds world*chunk elements on every rank.
FT_EXPORT int ft_comm_alltoall(void* const* buf_ptrs, void* out, void* const* flag_ptrs, uint32_t* counter, int rank, int world, uint32_t seq,
                               int64_t chunk, int dtype, int max_ctas, cudaStream_t st) {
  CommSync s;
  int r = fill_sync(s, flag_ptrs, counter, rank, world, seq, 5);
  if (r) return r;
  const int V = dtype == 0 ? 8 : 4;
  if (chunk <= 0 || chunk % V) return FT_ERR_ARG;
  PeerPtrs b;
  for (int i = 0; i < MAX_RANKS; i++) b.p[i] = i < world ? buf_ptrs[i] : nullptr;
  const int grid = comm_grid((size_t)chunk * world / V, max_ctas > 0 ? max_ctas : 64);
  if (dtype == 0) alltoall_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>(b, (__nv_bfloat16*)out, s, (size_t)chunk, ft_status_ptr());
  else alltoall_kernel<float><<<grid, 512, 0, st>>>(b, (float*)out, s, (size_t)chunk, ft_status_ptr());
  return (int)cudaGetLastError();
}

// out[0:n] on every rank = root's buf[0:n].
FT_EXPORT int ft_comm_broadcast(void* const* buf_ptrs, void* out, void* const* flag_ptrs, uint32_t* counter, int rank, int world, uint32_t seq,
                                int root, int64_t n, int dtype, int max_ctas, cudaStream_t st) {
  CommSync s;
  int r = fill_sync(s, flag_ptrs, counter, rank, world, seq, 6);
  if (r) return r;
  const int V = dtype == 0 ? 8 : 4;
  if (n <= 0 || n % V || root < 0 || root >= world) return FT_ERR_ARG;
  PeerPtrs b;
  for (int i = 0; i < MAX_RANKS; i++) b.p[i] = i < world ? buf_ptrs[i] : nullptr;
  const int grid = comm_grid((size_t)n / V, max_ctas > 0 ? max_ctas : 64);
  if (dtype == 0) broadcast_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>(b, (__nv_bfloat16*)out, s, root, (size_t)n, ft_status_ptr());
  else broadcast_kernel<float><<<grid, 512, 0, st>>>(b, (float*)out, s, root, (size_t)n, ft_status_ptr());
  return (int)cudaGetLastError();
}

// Sender side of a point-to-point message: copies `bytes` (multiple of 16) from src into the receiver's ring slot (peer mapping) and then sets the
// receiver's flag to `msg` (1, 2, ... per channel). If the slot was used before (prev_msg_in_slot != 0) the kernel first waits, bounded, until the
// receiver acknowledged that message in `my_ack` (local memory the receiver writes through its mapping). counter: local u32, zero between launches.
FT_EXPORT int ft_comm_p2p_put(const void* src, void* peer_slot, int64_t bytes, void* peer_flag, const void* my_ack, uint32_t msg, uint32_t prev_msg_in_slot,
                              uint32_t* counter, cudaStream_t st) {
  if (bytes <= 0 || bytes % 16 || msg == 0) return FT_ERR_ARG;
  const int grid = comm_grid((size_t)bytes / 16, 32);
  p2p_put_kernel<<<grid, 512, 0, st>>>((const uint4*)src, (uint4*)peer_slot, (size_t)bytes / 16, (uint32_t*)peer_flag, (const uint32_t*)my_ack, msg, prev_msg_in_slot,
                                       counter, comm_timeout_ns(), ft_status_ptr());
  return (int)cudaGetLastError();
}

// Receiver side: waits (bounded) until the local flag reaches `msg`, copies the slot into dst and acknowledges on the sender.
FT_EXPORT int ft_comm_p2p_get(void* dst, const void* my_slot, int64_t bytes, const void* my_flag, void* peer_ack, uint32_t msg, uint32_t* counter, cudaStream_t st) {
  if (bytes <= 0 || bytes % 16 || msg == 0) return FT_ERR_ARG;
  const int grid = comm_grid((size_t)bytes / 16, 32);
  p2p_get_kernel<<<grid, 512, 0, st>>>((uint4*)dst, (const uint4*)my_slot, (size_t)bytes / 16, (const uint32_t*)my_flag, (uint32_t*)peer_ack, msg, counter,
                                       comm_timeout_ns(), ft_status_ptr());
  return (int)cudaGetLastError();
}

FT_EXPORT int ft_comm_barrier(void* const* flag_ptrs, uint32_t* counter, int rank, int world, uint32_t seq, cudaStream_t st) {
  CommSync s;
  int r = fill_sync(s, flag_ptrs, counter, rank, world, seq, 7);
  if (r) return r;
  comm_barrier_kernel<<<1, 32, 0, st>>>(s, ft_status_ptr());
  return (int)cudaGetLastError();
}

// grad_ptrs / param_ptrs: `world` mappings of every rank's full bf16 gradient / parameter unit (padded = world*chunk elements).
// master, m, v: this rank's f32 slices [chunk]. chunk % 8 == 0. step >= 1 (bias correction).
FT_EXPORT int ft_fsdp_rs_adamw_ag(void* const* grad_ptrs, void* const* param_ptrs, void* const* flag_ptrs, uint32_t* counter, int rank,
                                  int world, uint32_t seq, float* master, float* m, float* v, int64_t chunk, float lr, float beta1,
                                  float beta2, float eps, float weight_decay, int step, const float* grad_scale_ptr, int max_ctas,
                                  cudaStream_t st) {
  CommSync s;
  int r = fill_sync(s, flag_ptrs, counter, rank, world, seq, 8);
  if (r) return r;
  if (chunk <= 0 || chunk % 8 || step < 1) return FT_ERR_ARG;
  PeerPtrs g, p;
  for (int i = 0; i < MAX_RANKS; i++) { g.p[i] = i < world ? grad_ptrs[i] : nullptr; p.p[i] = i < world ? param_ptrs[i] : nullptr; }
  AdamWArgsC a{lr, beta1, beta2, eps, weight_decay, 1.f - powf(beta1, (float)step), 1.f - powf(beta2, (float)step)};
  const int grid = comm_grid((size_t)chunk / 8, max_ctas > 0 ? max_ctas : 148);     // one CTA per SM beside the GEMM
  static bool configured = false;
  if (!configured) { ft_prefer_max_shared(fsdp_rs_adamw_ag_kernel); configured = true; }
  fsdp_rs_adamw_ag_kernel<<<grid, 256, 0, st>>>(g, p, s, master, m, v, (size_t)chunk, a, grad_scale_ptr, nullptr, ft_status_ptr());
  return (int)cudaGetLastError();
}

// The same without the all-gather (fully sharded parameters): the reduced gradient slice updates master / m / v and the bf16 result goes to
// `shard_out` [chunk], this rank's own shard of the unit. grad_ptrs as above.
FT_EXPORT int ft_fsdp_rs_adamw(void* const* grad_ptrs, void* shard_out, void* const* flag_ptrs, uint32_t* counter, int rank, int world, uint32_t seq,
                               float* master, float* m, float* v, int64_t chunk, float lr, float beta1, float beta2, float eps, float weight_decay,
                               int step, const float* grad_scale_ptr, int max_ctas, cudaStream_t st) {
  CommSync s;
  int r = fill_sync(s, flag_ptrs, counter, rank, world, seq, 8);
  if (r) return r;
  if (chunk <= 0 || chunk % 8 || step < 1 || shard_out == nullptr) return FT_ERR_ARG;
  PeerPtrs g, p;
  for (int i = 0; i < MAX_RANKS; i++) { g.p[i] = i < world ? grad_ptrs[i] : nullptr; p.p[i] = nullptr; }
  AdamWArgsC a{lr, beta1, beta2, eps, weight_decay, 1.f - powf(beta1, (float)step), 1.f - powf(beta2, (float)step)};
  const int grid = comm_grid((size_t)chunk / 8, max_ctas > 0 ? max_ctas : 148);
  static bool configured = false;
  if (!configured) { ft_prefer_max_shared(fsdp_rs_adamw_ag_kernel); configured = true; }
  fsdp_rs_adamw_ag_kernel<<<grid, 256, 0, st>>>(g, p, s, master, m, v, (size_t)chunk, a, grad_scale_ptr, (__nv_bfloat16*)shard_out, ft_status_ptr());
  return (int)cudaGetLastError();
}
