// Tensor-parallel GEMMs fused with their collective over peer-mapped (symmetric) memory, bf16, NT layout (x [rows, K] . w[N, K]^T).
//
//  MODE 1  all-gather -> GEMM (column-parallel Linear): every rank holds a row shard X_r [M/W, K] and a weight shard W_r [N/W, K] and wants
//          Y_r = [X_0; ..; X_{W-1}] W_r^T. A few CTAs of the kernel are copiers: they PUSH this rank's shard, 32 KiB at a time, through a
//          shared-memory ring with bulk async copies (local global -> smem -> every peer's gathered buffer; posted writes, no multicast)
//          and bump a per-row-tile counter on each peer. The other CTAs run the tcgen05 GEMM: tiles over the local shard first (no
//          waiting), then over the peers' rows in ring order, each tile's TMA producer waiting (bounded) for the row tile's counter. The
//          gathered buffer is double-buffered by launch parity; a pusher checks the peer's `done` flag of two launches before.
//
//  MODE 2  GEMM -> reduce-scatter (row-parallel Linear): every rank holds X[:, K/W slice] and W[:, K/W slice]; the partial product of each
//          128 x 256 tile goes from TMEM through swizzled shared memory straight into the OWNER rank's staging buffer with TMA stores
//          (bf16, peer-mapped destination), followed -- once the stores have completed -- by a release-add on the owner's tile counter. Tiles are visited owner (rank+1), (rank+2), ... with the
//          rank's own rows last. When a CTA runs out of GEMM tiles its epilogue warps reduce the tiles this rank owns: wait (bounded) for the
//          counter to reach 4 W, sum the W partials in fixed rank order in f32, write bf16. The staging buffer is double-buffered by the parity
//          of the launch number; a writer checks that the owner finished the launch two before (the `done` flag) before touching a slot.
//
// All cross-rank waits poll flags with a 2 s deadline; on expiry the kernel records the site in the status word, tears down (TMEM freed, copies
// drained) and returns. Launch numbers (`seq`) start at 1 and must be the same on every rank.
//
// The reference has no tensor parallelism (ferrotorch-distributed has DDP / FSDP / pipeline only); these kernels are the tile-level form of the
// Column/RowParallelLinear layers this framework adds for the 70B inference path.
#include "common.cuh"
#include "host_common.h"

namespace {

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int B_STAGE_BYTES = BN * BK * 2;
constexpr int EPI_WARPS = 4;
constexpr int EPI_BUF_BYTES = 32 * 128;
constexpr int NUM_THREADS = 32 * (2 + EPI_WARPS);
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + EPI_WARPS * EPI_BUF_BYTES + 256 + 1024;
constexpr int MAXR = 8;
constexpr uint64_t WAIT_NS = 2000000000ull;
constexpr int COPY_CHUNK = 32768, COPY_STAGES = 6, COPY_AHEAD = 4;      // COPY_STAGES >= COPY_AHEAD + 2
constexpr uint32_t FT_K_TP = 7;

struct StageMaps {
  CUtensorMap m[MAXR];                    // MODE 2: tensor map of this rank's slot in every owner's staging buffer (current parity)
};

struct TpArgs {
  int rank, world;
  uint32_t seq;
  int ncopy;                              // MODE 1: number of copier CTAs (blockIdx.x < ncopy)
  int split;                              // MODE 1: copier work items per local row tile (each pushes a contiguous range of chunks)
  const __nv_bfloat16* x_local;           // MODE 1: this rank's shard [M/W, K]
  __nv_bfloat16* xg[MAXR];                // MODE 1: every rank's gathered buffer [2][M][K] (symmetric)
  uint32_t* tile_cnt[MAXR];               // MODE 1: every rank's counters u32[2][M / 128] (symmetric): pushes received per row tile and parity
  __nv_bfloat16* stage[MAXR];             // MODE 2: every rank's staging buffer [2][W][M/W][N]
  uint32_t* cnt[MAXR];                    // MODE 2: every rank's counters u32[2][tiles_m_local * tiles_n]
  __nv_bfloat16* out;                     // MODE 2: local result [M/W, N]
  uint32_t* flags[MAXR];                  // every rank's flag block u32[2][MAXR]: [0][q] = rank q's shard is ready (seq), [1][q] = rank q finished (seq)
  unsigned long long* cta_done;           // local counter of CTAs that finished (monotonic over launches)
};

FT_DEVICE bool mbar_wait_deadline(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = globaltimer_ns();
  for (uint32_t i = 1;; i++) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 0xff) == 0 && globaltimer_ns() - t0 > WAIT_NS) return false;
  }
}
FT_DEVICE void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes),
               "r"(smem_u32(bar))
               : "memory");
}
FT_DEVICE void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
FT_DEVICE void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }
FT_DEVICE void red_release_sys_add(uint32_t* p, uint32_t v) { asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
FT_DEVICE void st_peer_v4(void* p, uint4 v) { asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory"); }

// After the CTA is finished: count it; the last CTA of the launch tells every peer that this rank is done with launch `seq`.
FT_DEVICE void publish_done(const TpArgs& a) {
  __threadfence_system();
  const unsigned long long prev = atomicAdd(a.cta_done, 1ull);
  if (prev + 1 == (unsigned long long)gridDim.x * a.seq) {
    for (int q = 0; q < a.world; q++) st_release_sys(a.flags[q] + MAXR + a.rank, a.seq);
  }
}

template <int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
ft_tp_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmAg, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmD, const __grid_constant__ StageMaps stage_maps, const TpArgs a, int M, int N, int K,
                  uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int W = a.world;
  const int tiles_m = M / BM, tiles_n = (N + BN - 1) / BN, tpr = tiles_m / W;     // tpr: row tiles per rank
  const int m_loc = M / W;

  const uint32_t par = a.seq & 1u;
  const uint32_t launches_this_parity = (a.seq + 1u) >> 1;

  // ------------------------------------------------------------------ copier CTAs (MODE 1) ---------------------------------------------
  if (MODE == 1 && (int)blockIdx.x < a.ncopy) {
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + COPY_STAGES * COPY_CHUNK);
    if (threadIdx.x == 0) {
      for (int s = 0; s < COPY_STAGES; s++) mbar_init(&full[s], 1);
      mbar_fence_init();
      const size_t tile_bytes = (size_t)BM * K * 2;
      const int nchunks = (int)((tile_bytes + COPY_CHUNK - 1) / COPY_CHUNK);
      uint32_t issued = 0;                                                         // chunks loaded so far by this CTA (ring position / parity)
      bool ok = true;
      // nobody may still be reading the parity slot this launch overwrites: every peer finished launch seq - 2
      if (a.seq > 2) {
        for (int q = 0; q < W && ok; q++) {
          if (q == a.rank) continue;
          if (!wait_flag_ge(a.flags[a.rank] + MAXR + q, a.seq - 2, WAIT_NS)) { ft_set_status(status, FT_K_TP, 1, q); ok = false; }
        }
      }
      // destination-major order: everything for the peer that consumes this rank's rows first (rank - 1), then rank - 2, ... At any moment the
      // ranks send to distinct destinations, and a consumer receives the shards in the order its tile loop visits them.
      const int per_dst = tpr * a.split;
      for (int item = blockIdx.x; item < (W - 1) * per_dst && ok; item += a.ncopy) {
        const int q = (a.rank - 1 - item / per_dst + 2 * W) % W;
        const int t = (item % per_dst) / a.split, part = item % a.split;
        const int c_begin = (int)((long long)nchunks * part / a.split), c_end = (int)((long long)nchunks * (part + 1) / a.split);
        const int n_it = c_end - c_begin;
        const uint8_t* src = reinterpret_cast<const uint8_t*>(a.x_local) + (size_t)t * tile_bytes;
        uint8_t* dst = reinterpret_cast<uint8_t*>(a.xg[q]) + ((size_t)par * tiles_m + (size_t)(a.rank * tpr + t)) * tile_bytes;
        const uint32_t base = issued;
        for (int c = 0; c < n_it + COPY_AHEAD && ok; c++) {
          if (c < n_it) {
            const uint32_t g = base + c, s = g % COPY_STAGES;
            if (g >= (uint32_t)COPY_STAGES) tma_store_wait_read<COPY_STAGES - COPY_AHEAD - 1>();   // the store that last read this stage is done with it
            const size_t off = (size_t)(c_begin + c) * COPY_CHUNK;
            const uint32_t bytes = (uint32_t)min((size_t)COPY_CHUNK, tile_bytes - off);
            mbar_expect_tx(&full[s], bytes);
            bulk_load(smem + s * COPY_CHUNK, src + off, bytes, &full[s]);
            issued++;
          }
          if (c >= COPY_AHEAD) {
            const int cc = c - COPY_AHEAD;
            const uint32_t g = base + cc, s = g % COPY_STAGES;
            if (!mbar_wait_deadline(&full[s], (g / COPY_STAGES) & 1)) { ft_set_status(status, FT_K_TP, 2, s); ok = false; break; }
            const size_t off = (size_t)(c_begin + cc) * COPY_CHUNK;
            const uint32_t bytes = (uint32_t)min((size_t)COPY_CHUNK, tile_bytes - off);
            bulk_store(dst + off, smem + s * COPY_CHUNK, bytes);
            tma_store_commit();
          }
        }
        if (!ok) break;
        tma_store_wait<0>();                                                       // the peer has this item's bytes
        __threadfence_system();
        red_release_sys_add(a.tile_cnt[q] + (size_t)par * tiles_m + (a.rank * tpr + t), 1u);
      }
      if (!ok) {
        tma_store_wait<0>();
        for (int k = 0; k < 64; k++) __nanosleep(1000);                            // loads already in flight land before smem goes away
      }
      publish_done(a);
    }
    return;
  }

  // ------------------------------------------------------------------ GEMM CTAs -----------------------------------------------------------
  uint8_t* sA = smem;
  uint8_t* sB = sA + STAGES * A_STAGE_BYTES;
  uint8_t* sEpi = sB + STAGES * B_STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sEpi + EPI_WARPS * EPI_BUF_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);

  const int first = MODE == 1 ? a.ncopy : 0;
  const int g_id = blockIdx.x - first, g_n = gridDim.x - first;
  const int num_kb = (K + BK - 1) / BK;
  const int num_tiles = tiles_m * tiles_n;

  // tile -> (owner rank of the rows, row tile inside the owner, column tile). MODE 1 starts at the local shard, MODE 2 ends with it.
  auto tile_map = [&](int tile, int& p, int& tin, int& ni) {
    const int mi = tile / tiles_n;
    ni = tile % tiles_n;
    p = (a.rank + (MODE == 2 ? 1 : 0) + mi / tpr) % W;
    tin = mi % tpr;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int k = 0; k < 2; k++) { mbar_init(&tfull_bar[k], 1); mbar_init(&tempty_bar[k], EPI_WARPS); }
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB); if (MODE == 1) { tma_prefetch_desc(&tmAg); tma_prefetch_desc(&tmD); } }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t s = 0, phase = 0;
      bool ok = true;
      for (int tile = g_id; tile < num_tiles && ok; tile += g_n) {
        int p, tin, ni;
        tile_map(tile, p, tin, ni);
        const int n0 = ni * BN;
        const bool remote = MODE == 1 && p != a.rank;
        if (remote) {
          if (!wait_flag_ge(a.tile_cnt[a.rank] + (size_t)par * tiles_m + (p * tpr + tin), launches_this_parity * (uint32_t)a.split, WAIT_NS)) {
            ft_set_status(status, FT_K_TP, 3, p);
            ok = false;
            break;
          }
          fence_proxy_async_global();
        }
        const int a_row = (MODE == 1 && !remote) ? tin * BM : (p * tpr + tin) * BM;
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait_deadline(&empty_bar[s], phase ^ 1)) { ft_set_status(status, FT_K_TP, 4, s); ok = false; break; }
          mbar_expect_tx(&full_bar[s], A_STAGE_BYTES + B_STAGE_BYTES);
          tma_load_2d(sA + s * A_STAGE_BYTES, remote ? &tmAg : &tmA, &full_bar[s], kb * BK, a_row);
          tma_load_2d(sB + s * B_STAGE_BYTES, &tmB, &full_bar[s], kb * BK, n0);
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
      }
      if (!ok) for (int k = 0; k < 64; k++) __nanosleep(1000);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(BM, BN, 1, 0, 0);
      uint32_t s = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = g_id; tile < num_tiles && ok; tile += g_n) {
        if (!mbar_wait_deadline(&tempty_bar[acc], acc_phase ^ 1)) { ft_set_status(status, FT_K_TP, 5, acc); ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait_deadline(&full_bar[s], phase)) { ft_set_status(status, FT_K_TP, 6, s); ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = smem_u32(sA + s * A_STAGE_BYTES), b_base = smem_u32(sB + s * B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; k++) {
            const uint64_t adesc = make_smem_desc(a_base + k * (UMMA_K * 2), 16, 1024, FT_SWZ_128B);
            const uint64_t bdesc = make_smem_desc(b_base + k * (UMMA_K * 2), 16, 1024, FT_SWZ_128B);
            umma_f16_ss(d_tmem, adesc, bdesc, idesc, (kb != 0 || k != 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    const int q = warp & 3, ew = warp - 2;
    uint8_t* buf = sEpi + ew * EPI_BUF_BYTES;
    constexpr int CHUNKS = BN / 64;
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    for (int tile = g_id; tile < num_tiles && ok; tile += g_n) {
      int p, tin, ni;
      tile_map(tile, p, tin, ni);
      const int n0 = ni * BN;
      if (!mbar_wait_deadline(&tfull_bar[acc], acc_phase)) { if (lane == 0) ft_set_status(status, FT_K_TP, 7, acc); ok = false; break; }
      tc_fence_after();
      if (MODE == 2 && a.seq > 2) {
        // the owner must have finished reducing the launch that last used this staging parity
        bool fine = true;
        if (lane == 0) fine = wait_flag_ge(a.flags[a.rank] + MAXR + p, a.seq - 2, WAIT_NS);
        fine = __shfl_sync(0xffffffffu, fine, 0);
        if (!fine) { if (lane == 0) ft_set_status(status, FT_K_TP, 8, p); ok = false; break; }
      }
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < CHUNKS; c++) {
        uint32_t v[64];
        tmem_ld_32x32b_x32(t_row + c * 64, v);
        tmem_ld_32x32b_x32(t_row + c * 64 + 32, v + 32);
        if (lane == 0) tma_store_wait_read<0>();                   // the previous store from this buffer has been read out
        __syncwarp();
        tmem_ld_wait();
        uint8_t* row = buf + lane * 128;
#pragma unroll
        for (int j = 0; j < 8; j++) {
          uint32_t pk[4];
#pragma unroll
          for (int e = 0; e < 4; e++) {
            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[8 * j + 2 * e]), __uint_as_float(v[8 * j + 2 * e + 1]));
            pk[e] = *reinterpret_cast<uint32_t*>(&h);
          }
          *reinterpret_cast<uint4*>(row + ((j ^ (lane & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
        const int col0 = n0 + c * 64;
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && col0 < N) {
          if (MODE == 1) tma_store_2d(&tmD, buf, col0, (p * tpr + tin) * BM + q * 32);
          else tma_store_2d(&stage_maps.m[p], buf, col0, tin * BM + q * 32);      // this rank's slot in owner p's staging buffer
        }
        if (lane == 0) tma_store_commit();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if (lane == 0) {
      // the partial tiles are only needed once every rank is through its GEMM phase, so nothing is gained by announcing them one by one (and
      // waiting for a store to complete across NVLink in the middle of the epilogue costs a round trip per tile): wait once, then bump every
      // counter this warp owes
      tma_store_wait<0>();
      if (MODE == 2 && ok) {
        __threadfence_system();
        for (int tile = g_id; tile < num_tiles; tile += g_n) {
          int p, tin, ni;
          tile_map(tile, p, tin, ni);
          red_release_sys_add(a.cnt[p] + (size_t)par * tpr * tiles_n + tin * tiles_n + ni, 1u);
        }
      }
    }
    __syncwarp();

    if (MODE == 2 && ok) {
      // ---- reduce the tiles this rank owns: partial from rank s is at stage[rank][par][s][rows][N] ----
      const uint32_t want = launches_this_parity * 4u * (uint32_t)W;
      const __nv_bfloat16* mine = a.stage[a.rank] + (size_t)par * W * m_loc * N;
      const int et = threadIdx.x - 64;                              // 0..127 over the four epilogue warps
      for (int ut = g_id; ut < tpr * tiles_n; ut += g_n) {
        bool fine = true;
        if (lane == 0) fine = wait_flag_ge(a.cnt[a.rank] + (size_t)par * tpr * tiles_n + ut, want, WAIT_NS);
        fine = __shfl_sync(0xffffffffu, fine, 0);
        __syncwarp();                                               // lane 0's acquire orders the whole warp's reads of the partials
        if (!fine) { if (lane == 0) ft_set_status(status, FT_K_TP, 9, ut); break; }
        const int tin = ut / tiles_n, n0 = (ut % tiles_n) * BN;
        // four 16-byte vectors per thread per pass and all W partials of each issued before use: the reduce is a pure stream of local
        // memory and needs many loads in flight per thread to run at bandwidth
        constexpr int UNR = 4;
        for (int vb = et; vb < BM * (BN / 8); vb += 128 * UNR) {
          float accv[UNR][8];
          size_t off[UNR];
          bool live[UNR];
#pragma unroll
          for (int u = 0; u < UNR; u++) {
            const int vix = vb + u * 128;
            const int r = vix / (BN / 8), cv = vix % (BN / 8);
            live[u] = vix < BM * (BN / 8) && n0 + cv * 8 < N;
            off[u] = ((size_t)tin * BM + r) * N + n0 + cv * 8;
#pragma unroll
            for (int e = 0; e < 8; e++) accv[u][e] = 0.f;
          }
#pragma unroll
          for (int s = 0; s < MAXR; s++) {
            if (s < W) {
              uint4 raw[UNR];
#pragma unroll
              for (int u = 0; u < UNR; u++) raw[u] = live[u] ? __ldcg(reinterpret_cast<const uint4*>(mine + (size_t)s * m_loc * N + off[u])) : make_uint4(0, 0, 0, 0);
#pragma unroll
              for (int u = 0; u < UNR; u++) {
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
#pragma unroll
                for (int e = 0; e < 4; e++) {
                  const float2 f = __bfloat1622float2(h[e]);
                  accv[u][2 * e] += f.x;
                  accv[u][2 * e + 1] += f.y;
                }
              }
            }
          }
#pragma unroll
          for (int u = 0; u < UNR; u++) {
            if (!live[u]) continue;
            uint4 o;
            __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int e = 0; e < 4; e++) oh[e] = __floats2bfloat162_rn(accv[u][2 * e], accv[u][2 * e + 1]);
            *reinterpret_cast<uint4*>(a.out + off[u]) = o;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0) publish_done(a);
}

int g_sms[64] = {0};

int fill_common(TpArgs& a, int rank, int world, int64_t seq, void* const* flag_ptrs, void* cta_done) {
  if (world < 1 || world > MAXR || rank < 0 || rank >= world || seq < 1 || seq > 0xffffffffLL) return FT_ERR_ARG;
  a.rank = rank;
  a.world = world;
  a.seq = (uint32_t)seq;
  for (int r = 0; r < world; r++) a.flags[r] = (uint32_t*)flag_ptrs[r];
  a.cta_done = (unsigned long long*)cta_done;
  return 0;
}

}  // namespace

// Bytes of the per-rank flag block (symmetric, zeroed once before the first launch).
FT_EXPORT int ft_tp_flag_bytes() { return 2 * MAXR * 4; }

// Column-parallel forward: out[M, n_loc] = gather(x shards)[M, K] . w_loc[n_loc, K]^T.
//   x_local: this rank's shard [M/world, K] bf16; xg_ptrs[r]: rank r's gathered buffer [2][M][K] bf16 (symmetric memory);
//   cnt_ptrs[r]: rank r's tile counters u32[2][M/128] (symmetric, zeroed once); flag_ptrs[r]: rank r's flag block; cta_done: local u64 zeroed once.
//   M/world must be a multiple of 128, K and n_loc of 8. ncopy: copier CTAs (0 = default).
FT_EXPORT int ft_tp_ag_gemm(const void* x_local, void* const* xg_ptrs, void* const* cnt_ptrs, const void* w_loc, void* out, int M, int n_loc, int K, int rank,
                            int world, int64_t seq, void* const* flag_ptrs, void* cta_done, int ncopy, cudaStream_t st) {
  TpArgs a = {};
  if (int e = fill_common(a, rank, world, seq, flag_ptrs, cta_done)) return e;
  if (M < 1 || n_loc < 1 || K < 1 || (M % (BM * world)) || (K & 7) || (n_loc & 7)) return FT_ERR_ARG;
  int dev = 0;
  FT_CUDA_TRY(cudaGetDevice(&dev));
  FT_CUDA_TRY(ft_bind_context(dev));
  if (!g_sms[dev]) FT_CUDA_TRY(cudaDeviceGetAttribute(&g_sms[dev], cudaDevAttrMultiProcessorCount, dev));
  const int tpr = M / BM / world;
  for (int r = 0; r < world; r++) {
    a.xg[r] = (__nv_bfloat16*)xg_ptrs[r];
    a.tile_cnt[r] = (uint32_t*)cnt_ptrs[r];
  }
  a.x_local = (const __nv_bfloat16*)x_local;
  a.ncopy = world > 1 ? (ncopy > 0 ? ncopy : 16) : 0;
  a.split = a.ncopy > tpr ? a.ncopy / tpr : 1;
  if (a.ncopy >= g_sms[dev]) return FT_ERR_ARG;
  const size_t par_off = (size_t)((uint32_t)seq & 1u) * (size_t)M * K;
  CUtensorMap tA, tAg, tB, tD;
  StageMaps sm = {};
  int r;
  if ((r = ft_make_tmap_2d(&tA, x_local, 2, true, (uint64_t)K, (uint64_t)(M / world), (uint64_t)K * 2, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B))) return r;
  if ((r = ft_make_tmap_2d(&tAg, (const __nv_bfloat16*)xg_ptrs[rank] + par_off, 2, true, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B))) return r;
  if ((r = ft_make_tmap_2d(&tB, w_loc, 2, true, (uint64_t)K, (uint64_t)n_loc, (uint64_t)K * 2, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B))) return r;
  if ((r = ft_make_tmap_2d(&tD, out, 2, true, (uint64_t)n_loc, (uint64_t)M, (uint64_t)n_loc * 2, 64, 32, CU_TENSOR_MAP_SWIZZLE_128B))) return r;
  static bool configured = false;
  if (!configured) {
    FT_CUDA_TRY(cudaFuncSetAttribute(ft_tp_gemm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    configured = true;
  }
  const int tiles = (M / BM) * ((n_loc + BN - 1) / BN);
  int gemm_ctas = g_sms[dev] - a.ncopy;
  if (tiles < gemm_ctas) gemm_ctas = tiles;
  // the grid size enters the `done` accounting, so it must not change between launches of one context: shapes are fixed per context
  ft_tp_gemm_kernel<1><<<a.ncopy + gemm_ctas, NUM_THREADS, SMEM_BYTES, st>>>(tA, tAg, tB, tD, sm, a, M, n_loc, K, ft_status_ptr());
  return (int)cudaGetLastError();
}

// Row-parallel forward: out[M/world, N] (this rank's rows) = sum over ranks of x[:, k slice] . w[:, k slice]^T.
//   x: local [M, k_loc] bf16; w: local [N, k_loc] bf16; stage_ptrs[r]: rank r's staging [2][world][M/world][N] bf16 (symmetric);
//   cnt_ptrs[r]: rank r's counters u32[2][(M/world/128) * ceil(N/256)] (symmetric, zeroed once); out: local [M/world, N] bf16.
FT_EXPORT int ft_tp_gemm_rs(const void* x, const void* w, void* const* stage_ptrs, void* const* cnt_ptrs, void* out, int M, int N, int k_loc, int rank,
                            int world, int64_t seq, void* const* flag_ptrs, void* cta_done, cudaStream_t st) {
  TpArgs a = {};
  if (int e = fill_common(a, rank, world, seq, flag_ptrs, cta_done)) return e;
  if (M < 1 || N < 1 || k_loc < 1 || (M % (BM * world)) || (k_loc & 7) || (N & 7)) return FT_ERR_ARG;
  int dev = 0;
  FT_CUDA_TRY(cudaGetDevice(&dev));
  FT_CUDA_TRY(ft_bind_context(dev));
  if (!g_sms[dev]) FT_CUDA_TRY(cudaDeviceGetAttribute(&g_sms[dev], cudaDevAttrMultiProcessorCount, dev));
  const size_t m_loc = (size_t)M / world;
  const uint32_t par = (uint32_t)seq & 1u;
  StageMaps sm = {};
  int r;
  for (int q = 0; q < world; q++) {
    a.stage[q] = (__nv_bfloat16*)stage_ptrs[q];
    a.cnt[q] = (uint32_t*)cnt_ptrs[q];
    const __nv_bfloat16* slot = (const __nv_bfloat16*)stage_ptrs[q] + ((size_t)par * world + rank) * m_loc * N;
    if ((r = ft_make_tmap_2d(&sm.m[q], slot, 2, true, (uint64_t)N, (uint64_t)m_loc, (uint64_t)N * 2, 64, 32, CU_TENSOR_MAP_SWIZZLE_128B))) return r;
  }
  a.out = (__nv_bfloat16*)out;
  CUtensorMap tA, tB;
  if ((r = ft_make_tmap_2d(&tA, x, 2, true, (uint64_t)k_loc, (uint64_t)M, (uint64_t)k_loc * 2, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B))) return r;
  if ((r = ft_make_tmap_2d(&tB, w, 2, true, (uint64_t)k_loc, (uint64_t)N, (uint64_t)k_loc * 2, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B))) return r;
  static bool configured = false;
  if (!configured) {
    FT_CUDA_TRY(cudaFuncSetAttribute(ft_tp_gemm_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    configured = true;
  }
  const int tiles = (M / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < g_sms[dev] ? tiles : g_sms[dev];
  ft_tp_gemm_kernel<2><<<grid, NUM_THREADS, SMEM_BYTES, st>>>(tA, tA, tB, tA, sm, a, M, N, k_loc, ft_status_ptr());
  return (int)cudaGetLastError();
}
