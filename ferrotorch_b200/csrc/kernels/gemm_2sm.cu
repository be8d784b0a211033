// Two-SM persistent bf16/fp16 GEMM for sm_100a: one 256 x 256 output tile per CTA PAIR (thread-block cluster of two, tcgen05 cta_group::2).
//
//   D[M,N] = A (x) B (+ bias[N]) (activation) (+ residual), f32 accumulation in TMEM, bf16/fp16 or f32 output; layouts as in gemm_tcgen05.cu
//   (a_mn / b_mn select K-major or MN-major operands, so forward, dgrad and wgrad need no transposes).
//
// Why pairs: with cta_group::2 the two SMs of a pair execute ONE 256 x 256 x 16 MMA per instruction. Each CTA stages only its own 128 rows of A and
// its own HALF (128 columns) of B; the tensor cores of both SMs read both B halves. Per SM and k-block that is 16 KiB + 16 KiB of shared memory
// written by TMA and read by the MMA instead of 16 + 32 KiB in the one-SM kernel, which takes the kernel off the shared-memory bandwidth limit and
// leaves room for a six-stage operand ring.
//
// Roles per CTA (192 threads):
//   warp 0      TMA producer. Both CTAs load their own A rows and B half (cp.async.bulk.tensor ... cta_group::2, no multicast) and complete the
//               transaction on the LEADER CTA's full barrier (the leader posted the expected bytes of both CTAs).
//   warp 1      allocates TMEM (cta_group::2, 512 columns = two accumulators); in the leader CTA one lane issues tcgen05.mma.cta_group::2 and
//               commits to the stage-empty / accumulator-full barriers of BOTH CTAs (tcgen05.commit with a CTA mask).
//   warps 2..5  epilogue of the CTA's own 128 accumulator rows: tcgen05.ld -> (+bias, act, +residual) -> swizzled smem -> TMA store; they release
//               the accumulator on the leader's barrier (remote mbarrier arrive for the peer CTA).
// Every wait is bounded (2 s): on expiry the role records its site in the status word and falls through to the teardown (cluster barrier,
// TMEM freed by both CTAs).
//
// Capability parity: the cuBLAS GemmEx wrappers of ferrotorch-gpu/src/blas.rs:1964-2922.
#include <cstdlib>

#include "common.cuh"
#include "host_common.h"
#include "gemm_2sm.h"

namespace {

constexpr int BM = 128;              // accumulator rows per CTA (256 per pair)
constexpr int BN = 256;              // tile columns per pair
constexpr int BNH = BN / 2;          // B rows staged by each CTA
constexpr int BK = 64, UMMA_K = 16;
constexpr int STAGES = 6;
constexpr int A_STAGE_BYTES = BM * BK * 2;    // 16 KiB
constexpr int B_STAGE_BYTES = BNH * BK * 2;   // 16 KiB
constexpr int EPI_WARPS = 4;
constexpr int EPI_BUF_BYTES = 32 * 128;
constexpr int NUM_THREADS = 32 * (2 + EPI_WARPS);
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + EPI_WARPS * EPI_BUF_BYTES + 256 + 1024;
constexpr int RASTER_GM = 8;         // tile rows per raster group: ~74 pairs in flight cover an 8 x ~9 patch of 256 x 256 tiles
constexpr uint32_t FT_K_GEMM2 = 8;

FT_DEVICE uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
FT_DEVICE void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in the CTA of rank `rank`
FT_DEVICE uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
FT_DEVICE void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// tile load whose completion is signalled on a barrier that may live in the peer CTA of the pair (no multicast: the data lands in this CTA only)
FT_DEVICE void tma_load_2d_pair(void* smem_dst, const void* tmap, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
FT_DEVICE void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
}
FT_DEVICE void tmem_relinquish_pair() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
FT_DEVICE void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
FT_DEVICE void umma_pair_f16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on the barrier at this shared-memory offset in every CTA of `cta_mask` once the MMAs issued so far have retired
FT_DEVICE void umma_pair_commit(uint64_t* bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)), "h"(cta_mask)
               : "memory");
}

FT_DEVICE bool mbar_wait_deadline(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t i = 1;; i++) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 0xff) == 0 && globaltimer_ns() - t0 > 2000000000ull) return false;
  }
}

FT_DEVICE float epi_act(int act, float x) {
  switch (act) {
    case 1: return fmaxf(x, 0.f);
    case 2: return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
    case 3: return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
    case 4: return x / (1.f + __expf(-x));
    default: return x;
  }
}

FT_DEVICE void tile_coords(int tile, int tiles_m, int tiles_n, int m_rot, int& m0, int& n0) {
  const int group_size = RASTER_GM * tiles_n;
  const int first_m = (tile / group_size) * RASTER_GM;
  const int gm = min(RASTER_GM, tiles_m - first_m);
  const int local = tile % group_size;
  m0 = ((first_m + local % gm + m_rot) % tiles_m) * (2 * BM);
  n0 = (local / gm) * BN;
}

// At most 128 registers per thread: two warps of the CTA share an SM sub-partition (6 warps on 4 sub-partitions), so the CTA claims at most half
// of each 16K-register sub-partition file and the other half stays available to co-resident kernels of other streams.
template <bool A_MN, bool B_MN, bool OUT_F32>
__global__ void __maxnreg__(128)
ft_gemm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmD,
                const __nv_bfloat16* __restrict__ bias, int M, int N, int K, int k_splits, uint32_t* status, const Gemm2Epi epi, const Gemm2Gate gate,
                long long ldb_bytes) {
  extern __shared__ uint8_t smem_raw[];
  // the dynamic shared window starts at the same offset in both CTAs of the pair, so the rounded pointers (and with them every barrier and
  // operand offset) are the same in both: the MMA descriptors built by the leader address the peer's tiles at the same offsets
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + STAGES * A_STAGE_BYTES;
  uint8_t* sEpi = sB + STAGES * B_STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sEpi + EPI_WARPS * EPI_BUF_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int tiles_m = (M + 2 * BM - 1) / (2 * BM);
  const int tiles_n = (N + BN - 1) / BN;
  const int num_kb_total = (K + BK - 1) / BK;
  const int kb_per = (num_kb_total + k_splits - 1) / k_splits;
  const int num_items = tiles_m * tiles_n * k_splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    // the accumulator-empty barrier of the leader collects the epilogue warps of both CTAs
    for (int a = 0; a < 2; a++) { mbar_init(&tfull_bar[a], 1); mbar_init(&tempty_bar[a], 2 * EPI_WARPS); }
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB); tma_prefetch_desc(&tmD); }
  if (warp == 1) { tmem_alloc_pair(tmem_slot, TMEM_COLS); tmem_relinquish_pair(); }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();              // the peer's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    // Gated operand: one look at all of its pieces by the whole warp. With the gather running a unit ahead they have normally all arrived, and
    // the per-tile waits below then cost nothing; if some are still in flight the tiles wait for exactly the pieces they read.
    long long ready_lo = 0, ready_hi = 0;                 // pieces [ready_lo, ready_hi) of the gated operand are known to have arrived
    if (gate.counters != nullptr) {
      const long long op_lo = gate.b_byte_off / gate.piece_bytes, op_hi = (gate.b_byte_off + gate.b_bytes - 1) / gate.piece_bytes + 1;
      bool mine = true;
      for (long long p = op_lo + lane; p < op_hi; p += 32) mine = mine && (int32_t)(ld_acquire_sys(gate.counters + p) - gate.expected) >= 0;
      if (__all_sync(0xffffffffu, mine)) {
        asm volatile("fence.proxy.async.global;" ::: "memory");
        ready_lo = op_lo;
        ready_hi = op_hi;
      }
    }
    if (lane == 0) {
      uint32_t s = 0, phase = 0;
      bool ok = true;
      for (int item = pair; item < num_items && ok; item += num_pairs) {
        int m0, n0;
        tile_coords(item / k_splits, tiles_m, tiles_n, gate.m_rot, m0, n0);
        const int split = item % k_splits;
        const int kb0 = split * kb_per, kb1 = min(num_kb_total, kb0 + kb_per);
        const int am0 = m0 + (int)cta_rank * BM;          // this CTA's rows of A (and of D)
        const int bn0 = n0 + (int)cta_rank * BNH;         // this CTA's half of the B tile
        if (gate.counters != nullptr && (gate.mode == 2 || (gate.operand == 0 ? bn0 < N : am0 < M))) {
          // the operand rows of this tile may still be on their way from the peers: wait for the pieces that hold them
          long long b0, b1;
          if (gate.mode == 2) { b0 = gate.b_byte_off; b1 = gate.b_byte_off + gate.b_bytes; }
          else if (gate.operand == 0) { b0 = gate.b_byte_off + (long long)bn0 * ldb_bytes; b1 = gate.b_byte_off + (long long)min(bn0 + BNH, N) * ldb_bytes; }
          else { b0 = gate.b_byte_off + am0; b1 = gate.b_byte_off + min(am0 + BM, M); }
          const long long lo = b0 / gate.piece_bytes, hi = (b1 - 1) / gate.piece_bytes + 1;
          if (lo < ready_lo || hi > ready_hi) {
            for (long long p = lo; p < hi && ok; p++) {
              if (p >= ready_lo && p < ready_hi) continue;
              if (!wait_flag_ge(gate.counters + p, gate.expected, 2000000000ull)) { ft_set_status(status, FT_K_GEMM2, 5, (uint32_t)p); ok = false; }
            }
            if (!ok) break;
            // the pieces were written by peers with ordinary stores; the loads below go through the async proxy
            asm volatile("fence.proxy.async.global;" ::: "memory");
            if (lo <= ready_hi && hi >= ready_lo && ready_hi > ready_lo) { ready_lo = min(ready_lo, lo); ready_hi = max(ready_hi, hi); }
            else { ready_lo = lo; ready_hi = hi; }
          }
        }
        for (int kb = kb0; kb < kb1; kb++) {
          if (!mbar_wait_deadline(&empty_bar[s], phase ^ 1)) { ft_set_status(status, FT_K_GEMM2, 1, s); ok = false; break; }
          if (leader) mbar_expect_tx(&full_bar[s], 2 * (A_STAGE_BYTES + B_STAGE_BYTES));
          const uint32_t bar = mapa_u32(smem_u32(&full_bar[s]), 0);
          uint8_t* a_dst = sA + s * A_STAGE_BYTES;
          uint8_t* b_dst = sB + s * B_STAGE_BYTES;
          if constexpr (!A_MN) {
            tma_load_2d_pair(a_dst, &tmA, bar, kb * BK, am0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; j++) tma_load_2d_pair(a_dst + j * (BK * 128), &tmA, bar, am0 + j * 64, kb * BK);
          }
          if constexpr (!B_MN) {
            tma_load_2d_pair(b_dst, &tmB, bar, kb * BK, bn0);
          } else {
#pragma unroll
            for (int j = 0; j < BNH / 64; j++) tma_load_2d_pair(b_dst + j * (BK * 128), &tmB, bar, bn0 + j * 64, kb * BK);
          }
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        for (int i = 0; i < 64; i++) __nanosleep(1000);   // copies already in flight land before the shared memory goes away
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) --------------------------
    if (lane == 0 && leader) {
      const uint32_t idesc = make_idesc_f16(2 * BM, BN, epi.in_f16 ? 0 : 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      uint32_t s = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int item = pair; item < num_items && ok; item += num_pairs) {
        if (!mbar_wait_deadline(&tempty_bar[acc], acc_phase ^ 1)) { ft_set_status(status, FT_K_GEMM2, 2, acc); ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const int split = item % k_splits;
        const int kb0 = split * kb_per, kb1 = min(num_kb_total, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; kb++) {
          if (!mbar_wait_deadline(&full_bar[s], phase)) { ft_set_status(status, FT_K_GEMM2, 3, s); ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = smem_u32(sA + s * A_STAGE_BYTES);
          const uint32_t b_base = smem_u32(sB + s * B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; k++) {
            const uint64_t adesc = A_MN ? make_smem_desc(a_base + k * (UMMA_K * 128), BK * 128, 1024, FT_SWZ_128B)
                                        : make_smem_desc(a_base + k * (UMMA_K * 2), 16, 1024, FT_SWZ_128B);
            const uint64_t bdesc = B_MN ? make_smem_desc(b_base + k * (UMMA_K * 128), BK * 128, 1024, FT_SWZ_128B)
                                        : make_smem_desc(b_base + k * (UMMA_K * 2), 16, 1024, FT_SWZ_128B);
            umma_pair_f16_ss(d_tmem, adesc, bdesc, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
          }
          umma_pair_commit(&empty_bar[s], 3);             // the stage is free in both CTAs
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_pair_commit(&tfull_bar[acc], 3);             // an empty split commits at once: the epilogue stores zeros for it
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) ----------------------------------
    const int q = warp & 3;                      // TMEM lane quarter this warp may access
    const int ew = warp - 2;
    uint8_t* buf = sEpi + ew * EPI_BUF_BYTES;
    constexpr int EPI_COLS = OUT_F32 ? 32 : 64;
    constexpr int CHUNKS = BN / EPI_COLS;
    const uint32_t tempty_leader0 = mapa_u32(smem_u32(&tempty_bar[0]), 0);
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    for (int item = pair; item < num_items && ok; item += num_pairs) {
      int m0, n0;
      tile_coords(item / k_splits, tiles_m, tiles_n, gate.m_rot, m0, n0);
      const int split = item % k_splits;
      const bool empty_split = split * kb_per >= min(num_kb_total, split * kb_per + kb_per);
      const int row0 = m0 + (int)cta_rank * BM + q * 32;
      if (!mbar_wait_deadline(&tfull_bar[acc], acc_phase)) { if (lane == 0) ft_set_status(status, FT_K_GEMM2, 4, acc); ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < CHUNKS; c++) {
        const int col0 = n0 + c * EPI_COLS;
        if (lane == 0) tma_store_wait_read<0>();          // the previous store from this buffer has been read out
        __syncwarp();
        uint8_t* row = buf + lane * 128;
        // 32 accumulator columns at a time: the epilogue warps then need ~100 registers, which keeps the CTA's share of each SM sub-partition's
        // register file small enough for bandwidth-bound kernels of other streams (optimizer, collectives) to be resident beside the GEMM
#pragma unroll 1
        for (int h = 0; h < EPI_COLS / 32; h++) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(t_row + c * EPI_COLS + h * 32, v);
          tmem_ld_wait();
          if (empty_split) {
#pragma unroll
            for (int i = 0; i < 32; i++) v[i] = 0u;
          }
          const int colh = col0 + h * 32;
          if (bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 32; i++) {
              float b = 0.f;
              if (colh + i < N) b = epi.in_f16 ? __half2float(__ldg(reinterpret_cast<const __half*>(bias) + colh + i)) : __bfloat162float(__ldg(bias + colh + i));
              v[i] = __float_as_uint(__uint_as_float(v[i]) + b);
            }
          }
          if (epi.act != 0) {
#pragma unroll
            for (int i = 0; i < 32; i++) v[i] = __float_as_uint(epi_act(epi.act, __uint_as_float(v[i])));
          }
          if (epi.residual != nullptr && row0 + lane < M) {
            const size_t roff = (size_t)(row0 + lane) * (size_t)epi.ldr + colh;
            if constexpr (OUT_F32) {
              const float* rp = reinterpret_cast<const float*>(epi.residual) + roff;
#pragma unroll
              for (int i = 0; i < 32; i++)
                if (colh + i < N) v[i] = __float_as_uint(__uint_as_float(v[i]) + rp[i]);
            } else if (epi.in_f16) {
              const __half* rp = reinterpret_cast<const __half*>(epi.residual) + roff;
#pragma unroll
              for (int i = 0; i < 32; i++)
                if (colh + i < N) v[i] = __float_as_uint(__uint_as_float(v[i]) + __half2float(rp[i]));
            } else {
              const __nv_bfloat16* rp = reinterpret_cast<const __nv_bfloat16*>(epi.residual) + roff;
#pragma unroll
              for (int i = 0; i < 32; i++)
                if (colh + i < N) v[i] = __float_as_uint(__uint_as_float(v[i]) + __bfloat162float(rp[i]));
            }
          }
          if constexpr (OUT_F32) {
#pragma unroll
            for (int j = 0; j < 8; j++) *reinterpret_cast<uint4*>(row + ((j ^ (lane & 7)) << 4)) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 4; j++) {
              uint32_t p[4];
#pragma unroll
              for (int e = 0; e < 4; e++) {
                if (epi.in_f16) {
                  __half2 hh = __floats2half2_rn(__uint_as_float(v[8 * j + 2 * e]), __uint_as_float(v[8 * j + 2 * e + 1]));
                  p[e] = *reinterpret_cast<uint32_t*>(&hh);
                } else {
                  __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(v[8 * j + 2 * e]), __uint_as_float(v[8 * j + 2 * e + 1]));
                  p[e] = *reinterpret_cast<uint32_t*>(&hh);
                }
              }
              *reinterpret_cast<uint4*>(row + (((h * 4 + j) ^ (lane & 7)) << 4)) = make_uint4(p[0], p[1], p[2], p[3]);
            }
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && col0 < N && row0 < M) tma_store_3d(&tmD, buf, col0, row0, split);
        if (lane == 0) tma_store_commit();
      }
      // every TMEM read of this accumulator has completed (tmem_ld_wait above): hand it back to the leader's MMA thread
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(tempty_leader0 + acc * 8);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if (lane == 0) tma_store_wait<0>();
  }

  // Nobody leaves (or frees TMEM) while the other CTA of the pair may still signal its barriers or read the accumulators.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

int g_enabled = -1;
int g_sms[64] = {0};
int g_max_pairs[64] = {0};        // 0 = not queried, -1 = pairs cannot be scheduled

template <bool A_MN, bool B_MN, bool OUT_F32>
int launch(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tD, const void* bias, int M, int N, int K, int k_splits, int dev,
           cudaStream_t stream, const Gemm2Epi& epi, const Gemm2Gate& gate, long long ldb_bytes) {
  auto kern = ft_gemm2_kernel<A_MN, B_MN, OUT_F32>;
  static bool configured = false;
  if (!configured) {
    FT_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  if (g_max_pairs[dev] == 0) {
    cfg.gridDim = dim3(2 * (g_sms[dev] / 2));
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) { cudaGetLastError(); n = -1; }
    g_max_pairs[dev] = n;
  }
  if (g_max_pairs[dev] < 1) return FT_ERR_DRIVER;
  const int items = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN) * k_splits;
  int pairs = g_max_pairs[dev] < g_sms[dev] / 2 ? g_max_pairs[dev] : g_sms[dev] / 2;
  if (items < pairs) pairs = items;
  cfg.gridDim = dim3(2 * pairs);
  cfg.numAttrs = ft_pdl_enabled() ? 2 : 1;
  return (int)cudaLaunchKernelEx(&cfg, kern, tA, tB, tD, reinterpret_cast<const __nv_bfloat16*>(bias), M, N, K, k_splits, ft_status_ptr(), epi, gate, ldb_bytes);
}

}  // namespace

bool ft_gemm2_wanted(int M, int N, int K, int k_splits) {
  if (g_enabled < 0) {
    const char* e = getenv("FT_GEMM_2SM");
    g_enabled = (e && e[0] == '0') ? 0 : 1;
  }
  if (!g_enabled) return false;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || g_max_pairs[dev] < 0) return false;
  // 256-row tiles: take the problem when the padding of the last tile row is small
  if (M < 2 * BM) return false;
  const int padded = (M + 2 * BM - 1) / (2 * BM) * (2 * BM);
  return (padded - M) * 8 <= M && N >= 64 && K >= BK;
}

// Switches the two-SM GEMM on (1) or off (0) for the launches that follow; the environment variable FT_GEMM_2SM=0 switches it off from the start.
FT_EXPORT int ft_gemm_set_2sm(int on) {
  g_enabled = on ? 1 : 0;
  return FT_OK;
}

int ft_gemm2_launch(const void* A, const void* B, void* D, const void* bias, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldd, int a_mn,
                    int b_mn, int out_f32, int k_splits, cudaStream_t stream, const Gemm2Epi& epi, const Gemm2Gate& gate_in) {
  if (epi.act < 0 || epi.act > 4) return FT_ERR_ARG;
  Gemm2Gate gate = gate_in;
  if (gate.counters != nullptr) {
    if (gate.piece_bytes < 1 || gate.b_byte_off < 0 || (gate.mode != 1 && gate.mode != 2) || (gate.operand != 0 && gate.operand != 1)) return FT_ERR_ARG;
    if (gate.mode == 1 && (gate.operand == 0 ? b_mn : a_mn)) gate.mode = 2;      // rows of an MN-major operand are not contiguous per tile
    if (gate.b_bytes <= 0) return FT_ERR_ARG;
  }
  const bool in_bf16 = !epi.in_f16;
  if (M <= 0 || N <= 0 || K <= 0 || k_splits < 1 || k_splits > 256) return FT_ERR_ARG;
  if ((lda & 7) || (ldb & 7) || ((ldd * (out_f32 ? 4 : 2)) & 15)) return FT_ERR_ARG;
  int dev = 0;
  FT_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return FT_ERR_ARG;
  FT_CUDA_TRY(ft_bind_context(dev));
  if (!g_sms[dev]) FT_CUDA_TRY(cudaDeviceGetAttribute(&g_sms[dev], cudaDevAttrMultiProcessorCount, dev));
  CUtensorMap tA, tB, tD;
  int r;
  if (!a_mn) r = ft_make_tmap_2d(&tA, A, 2, in_bf16, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
  else       r = ft_make_tmap_2d(&tA, A, 2, in_bf16, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r;
  if (!b_mn) r = ft_make_tmap_2d(&tB, B, 2, in_bf16, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BK, BNH, CU_TENSOR_MAP_SWIZZLE_128B);
  else       r = ft_make_tmap_2d(&tB, B, 2, in_bf16, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r;
  const uint64_t eb = out_f32 ? 4 : 2;
  r = ft_make_tmap_3d(&tD, D, (int)eb, !out_f32 && in_bf16, (uint64_t)N, (uint64_t)M, (uint64_t)k_splits, (uint64_t)ldd * eb, (uint64_t)M * ldd * eb,
                      out_f32 ? 32 : 64, 32, 1, CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r;
#define FT_GEMM2_CASE(AM, BMN, OF) \
  if (a_mn == AM && b_mn == BMN && out_f32 == OF) return launch<AM, BMN, OF>(tA, tB, tD, bias, M, N, K, k_splits, dev, stream, epi, gate, (long long)ldb * 2);
  FT_GEMM2_CASE(0, 0, 0) FT_GEMM2_CASE(0, 1, 0) FT_GEMM2_CASE(1, 0, 0) FT_GEMM2_CASE(1, 1, 0)
  FT_GEMM2_CASE(0, 0, 1) FT_GEMM2_CASE(0, 1, 1) FT_GEMM2_CASE(1, 0, 1) FT_GEMM2_CASE(1, 1, 1)
#undef FT_GEMM2_CASE
  return FT_ERR_ARG;
}
