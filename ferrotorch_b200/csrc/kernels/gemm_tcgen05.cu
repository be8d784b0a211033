// Persistent warp-specialised bf16 GEMM for sm_100a.
//
//   D[M,N] = A (x) B  (+ bias[N]),  bf16 operands, f32 accumulation in TMEM,
//   bf16 or f32 output.
//
// Operand layouts (row-major memory, leading dimension in elements):
//   a_mn = 0 : A memory is [M,K]  (K contiguous)      a_mn = 1 : A memory is [K,M]  (M contiguous)
//   b_mn = 0 : B memory is [N,K]  (K contiguous)      b_mn = 1 : B memory is [K,N]  (N contiguous)
// so (0,0) is Linear forward x.W^T, (0,1) is dgrad dY.W, (1,1) is wgrad dY^T.X.
//
// Structure per CTA (one CTA per SM, 192 threads):
//   warp 0      TMA producer: cp.async.bulk.tensor tiles into a 4-stage smem ring (128B swizzle)
//   warp 1      allocates TMEM (2 x 256 columns), one lane issues tcgen05.mma (128x256x16)
//   warps 2..5  epilogue: tcgen05.ld -> registers -> (+bias) -> bf16/f32 -> swizzled smem -> TMA store
// The two TMEM accumulators let the epilogue of tile i overlap the main loop of tile i+1.
// Every mbarrier wait is bounded; on expiry the role records its site in the status word and
// the CTA falls through to teardown (TMEM is freed, in-flight stores are drained).
//
// Capability parity: replaces the cuBLAS GemmEx wrappers of ferrotorch-gpu/src/blas.rs:1964-2922
// and the three-launch linear_fused CUDA path of ferrotorch-core/src/grad_fns/linalg.rs:1223-1262.
#include "common.cuh"
#include "host_common.h"
#include "gemm_2sm.h"

namespace {

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;   // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK * 2;   // 32 KiB
constexpr int EPI_WARPS = 4;
constexpr int EPI_BUF_BYTES = 32 * 128;      // 32 rows x 128 B per warp per buffer
constexpr int NUM_THREADS = 32 * (2 + EPI_WARPS);
constexpr int TMEM_COLS = 512;
// One staging buffer per epilogue warp (not two): the CTA then leaves ~18 KiB of the SM's shared memory unclaimed, which is what lets
// CTAs of bandwidth-bound kernels from other streams (the optimizer, the collectives) become resident beside the GEMM instead of
// queueing behind it.
constexpr int EPI_BUFS = 1;
constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + EPI_WARPS * EPI_BUFS * EPI_BUF_BYTES + 256 + 1024;

// Tile order: groups of RASTER_GM tile-rows, walked row-fastest inside a group, so the ~148 tiles in flight
// cover a near-square patch of the output (16 x ~9 tiles) and both operands are re-used out of L2.
constexpr int RASTER_GM = 16;
FT_DEVICE void tile_coords(int tile, int tiles_m, int tiles_n, int& m0, int& n0) {
  const int group_size = RASTER_GM * tiles_n;
  const int first_m = (tile / group_size) * RASTER_GM;
  const int gm = min(RASTER_GM, tiles_m - first_m);
  const int local = tile % group_size;
  m0 = (first_m + local % gm) * BM;
  n0 = (local / gm) * BN;
}

FT_DEVICE bool mbar_wait_deadline(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = globaltimer_ns();
  for (uint32_t i = 1;; i++) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 0xff) == 0 && globaltimer_ns() - t0 > 2000000000ull) return false;
  }
}

// Epilogue extras: activation code applied after the bias, then an optional residual tile added (residual rows are ldr elements apart, same
// dtype as the output); in_f16 selects fp16 operands (bias / residual / bf16-typed output are then fp16 as well).
struct EpiArgs {
  int act;                       // 0 none, 1 relu, 2 gelu (erf), 3 gelu (tanh), 4 silu
  const void* residual;
  int64_t ldr;
  int in_f16;
};

FT_DEVICE float epi_act(int act, float x) {
  switch (act) {
    case 1: return fmaxf(x, 0.f);
    case 2: return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
    case 3: return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
    case 4: return x / (1.f + __expf(-x));
    default: return x;
  }
}

// Tail balancing. With T output tiles on G persistent CTAs the last round holds T % G tiles and the other CTAs idle through it. When that
// remainder is at most G / 2 the launcher cuts each of those tiles into S = G / remainder K slices, one per otherwise idle CTA: slices 1..S-1
// ("helpers") leave their f32 accumulators in a workspace and bump a counter per (tile, TMEM lane quarter); slice 0 (the "owner") adds them to
// its own accumulator and runs the ordinary epilogue. All slices of a tile are the last work item of distinct CTAs of one resident grid and
// helpers never wait, so the owner's (deadline-bounded) wait cannot deadlock. The counters are reset by the owner: the workspace is reusable
// by the next launch on the same stream.
struct TailArgs {
  int tiles;                     // number of output tiles cut into slices (they are the last `tiles` of the tile order); 0 = off
  int slices;                    // S
  float* ws;                     // [tiles][S-1][4 quarters][chunks][EPI_COLS/4][32 lanes] float4
  uint32_t* cnt;                 // [tiles][4], zero between launches
  // Row-shift table of the B operand (MN-major B only; b_atoms_per_tap = 0: off), used by convolution weight gradients: the N axis is
  // [tap][channel] with b_atoms_per_tap 64-channel atoms per filter tap, and the atom of tap t is fetched from B's columns of that channel block
  // at rows k + b_shift[t]. Atoms past the ninth tap and rows outside B read as zeros (TMA fill).
  int b_atoms_per_tap;
  int b_shift[9];
  // The same for a K-major A operand (a_atoms_per_tap = 0: off), used by convolutions evaluated as one GEMM over pixel rows: the K axis is
  // [tap][channel] with a_atoms_per_tap 64-channel k-blocks per filter tap, and k-block kb of tap t = kb / a_atoms_per_tap is fetched from
  // A's columns (kb % a_atoms_per_tap) * 64 at rows m + a_shift[t] (zeros outside A).
  int a_atoms_per_tap;
  int a_shift[9];
};

struct WorkItem {
  int tile, split, kb0, kb1;
  int tail;                      // index of the tail tile or -1
  int slice;                     // K slice of a tail tile (0 = owner)
};

// shift[t] by a chain of selects: the tables are kernel parameters and a run-time index would make the compiler copy them to local memory
FT_DEVICE int pick_shift(const int (&shift)[9], int t) {
  int v = shift[0];
#pragma unroll
  for (int i = 1; i < 9; i++) v = (t == i) ? shift[i] : v;
  return v;
}

FT_DEVICE WorkItem decode_item(int item, int k_splits, int kb_per, int num_kb_total, int full_items, const TailArgs& t) {
  WorkItem w;
  if (item < full_items) {
    w.tile = item / k_splits;
    w.split = item % k_splits;
    w.kb0 = w.split * kb_per;
    w.kb1 = min(num_kb_total, w.kb0 + kb_per);
    w.tail = -1;
    w.slice = 0;
  } else {
    const int j = item - full_items;
    const int per = (num_kb_total + t.slices - 1) / t.slices;
    w.tail = j / t.slices;
    w.slice = j % t.slices;
    w.tile = full_items + w.tail;          // tail balancing runs with k_splits == 1 only
    w.split = 0;
    w.kb0 = w.slice * per;
    w.kb1 = min(num_kb_total, w.kb0 + per);
  }
  return w;
}

template <bool A_MN, bool B_MN, bool OUT_F32>
__global__ void __launch_bounds__(NUM_THREADS, 1)
ft_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmD, const __nv_bfloat16* __restrict__ bias, int M, int N, int K,
               int k_splits, uint32_t* status, const EpiArgs epi, const TailArgs tail) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + STAGES * A_STAGE_BYTES;
  uint8_t* sEpi = sB + STAGES * B_STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sEpi + EPI_WARPS * EPI_BUFS * EPI_BUF_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM;
  const int tiles_n = (N + BN - 1) / BN;
  // A work item is (output tile, K split); split s of a tile accumulates k-blocks [s*kb_per, (s+1)*kb_per) and stores to plane s of D
  // (D's tensor map is 3-D: [splits, M, N]), so short-and-wide problems (decode: a few token rows against a large weight) still
  // spread the weight stream over every SM. k_splits == 1 is the ordinary GEMM.
  const int num_kb_total = (K + BK - 1) / BK;
  const int kb_per = (num_kb_total + k_splits - 1) / k_splits;
  const int full_items = tiles_m * tiles_n * k_splits - tail.tiles;
  const int num_tiles = full_items + tail.tiles * tail.slices;          // work items

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; a++) { mbar_init(&tfull_bar[a], 1); mbar_init(&tempty_bar[a], EPI_WARPS); }
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB); tma_prefetch_desc(&tmD); }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // everything above touched only this CTA's shared memory and TMEM; from here on the kernel reads what its predecessor wrote
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t s = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m0, n0;
        const WorkItem wi = decode_item(tile, k_splits, kb_per, num_kb_total, full_items, tail);
        tile_coords(wi.tile, tiles_m, tiles_n, m0, n0);
        const int kb0 = wi.kb0, kb1 = wi.kb1;
        for (int kb = kb0; kb < kb1; kb++) {
          if (!mbar_wait_deadline(&empty_bar[s], phase ^ 1)) { ft_set_status(status, FT_K_GEMM, 1, s); ok = false; break; }
          mbar_expect_tx(&full_bar[s], A_STAGE_BYTES + B_STAGE_BYTES);
          uint8_t* a_dst = sA + s * A_STAGE_BYTES;
          uint8_t* b_dst = sB + s * B_STAGE_BYTES;
          if constexpr (!A_MN) {
            if (tail.a_atoms_per_tap == 0) tma_load_2d(a_dst, &tmA, &full_bar[s], kb * BK, m0);
            else tma_load_2d(a_dst, &tmA, &full_bar[s], (kb % tail.a_atoms_per_tap) * 64, m0 + pick_shift(tail.a_shift, kb / tail.a_atoms_per_tap));
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; j++) tma_load_2d(a_dst + j * (BK * 128), &tmA, &full_bar[s], m0 + j * 64, kb * BK);
          }
          if constexpr (!B_MN) {
            tma_load_2d(b_dst, &tmB, &full_bar[s], kb * BK, n0);
          } else if (tail.b_atoms_per_tap == 0) {
#pragma unroll
            for (int j = 0; j < BN / 64; j++) tma_load_2d(b_dst + j * (BK * 128), &tmB, &full_bar[s], n0 + j * 64, kb * BK);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; j++) {
              const int g = n0 / 64 + j, tap = g / tail.b_atoms_per_tap;
              // beyond the ninth tap: a column past B's width, so the box is zero filled and the full byte count still arrives
              const int col = tap < 9 ? (g % tail.b_atoms_per_tap) * 64 : tail.b_atoms_per_tap * 64;
              const int row = kb * BK + (tap < 9 ? pick_shift(tail.b_shift, tap) : 0);
              tma_load_2d(b_dst + j * (BK * 128), &tmB, &full_bar[s], col, row);
            }
          }
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // let copies that are already in flight land before the CTA's shared memory goes away
        for (int i = 0; i < 64; i++) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      const uint32_t idesc = epi.in_f16 ? make_idesc_f16(BM, BN, /*f16*/ 0, A_MN ? 1 : 0, B_MN ? 1 : 0)
                                        : make_idesc_f16(BM, BN, /*bf16*/ 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      uint32_t s = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait_deadline(&tempty_bar[acc], acc_phase ^ 1)) { ft_set_status(status, FT_K_GEMM, 2, acc); ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const WorkItem wi = decode_item(tile, k_splits, kb_per, num_kb_total, full_items, tail);
        const int kb0 = wi.kb0, kb1 = wi.kb1;
        if (kb0 >= kb1) {   // an empty split (K not divisible): nothing to accumulate; the epilogue stores zeros for it
          umma_commit(&tfull_bar[acc]);
          acc ^= 1;
          if (acc == 0) acc_phase ^= 1;
          continue;
        }
        for (int kb = kb0; kb < kb1; kb++) {
          if (!mbar_wait_deadline(&full_bar[s], phase)) { ft_set_status(status, FT_K_GEMM, 3, s); ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = smem_u32(sA + s * A_STAGE_BYTES);
          const uint32_t b_base = smem_u32(sB + s * B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; k++) {
            // K-major: 8-row groups 1024 B apart, the K slice moves 32 B inside the 128 B swizzle row.
            // MN-major: 64-element atoms BK*128 B apart (leading offset), 8 k-rows = 1024 B (stride offset),
            //           a K slice of 16 rows moves 2048 B.
            const uint64_t adesc = A_MN ? make_smem_desc(a_base + k * (UMMA_K * 128), BK * 128, 1024, FT_SWZ_128B)
                                        : make_smem_desc(a_base + k * (UMMA_K * 2), 16, 1024, FT_SWZ_128B);
            const uint64_t bdesc = B_MN ? make_smem_desc(b_base + k * (UMMA_K * 128), BK * 128, 1024, FT_SWZ_128B)
                                        : make_smem_desc(b_base + k * (UMMA_K * 2), 16, 1024, FT_SWZ_128B);
            umma_f16_ss(d_tmem, adesc, bdesc, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
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
    // ------------------------------ epilogue ----------------------------------
    const int q = warp & 3;                      // TMEM lane quarter this warp may access
    const int ew = warp - 2;                     // staging slot
    uint8_t* my_buf = sEpi + ew * EPI_BUFS * EPI_BUF_BYTES;
    constexpr int EPI_COLS = OUT_F32 ? 32 : 64;
    constexpr int CHUNKS = BN / EPI_COLS;
    uint32_t acc = 0, acc_phase = 0;
    uint32_t nstore = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int m0, n0;
      const WorkItem wi = decode_item(tile, k_splits, kb_per, num_kb_total, full_items, tail);
      tile_coords(wi.tile, tiles_m, tiles_n, m0, n0);
      const int split = wi.split;
      const bool empty_split = wi.kb0 >= wi.kb1;
      if (!mbar_wait_deadline(&tfull_bar[acc], acc_phase)) { if (lane == 0) ft_set_status(status, FT_K_GEMM, 4, acc); ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
      // tail tile: where this warp's quarter of every helper slice lives, and (owner) the wait for the helpers
      constexpr int WS_CHUNK = (OUT_F32 ? 32 : 64) * 32;          // floats per (quarter, chunk)
      constexpr int WS_SLICE = 4 * (BN / (OUT_F32 ? 32 : 64)) * WS_CHUNK;
      float* ws_q = nullptr;
      if (wi.tail >= 0) {
        ws_q = tail.ws + (size_t)wi.tail * (tail.slices - 1) * WS_SLICE + (size_t)q * (BN / (OUT_F32 ? 32 : 64)) * WS_CHUNK;
        if (wi.slice == 0) {
          uint32_t* c = tail.cnt + wi.tail * 4 + q;
          if (lane == 0) {
            if (!wait_flag_ge_gpu(c, (uint32_t)(tail.slices - 1), 2000000000ull)) ft_set_status(status, FT_K_GEMM, 5, q);
            *c = 0u;
          }
          __syncwarp();
        }
      }
#pragma unroll 1
      for (int c = 0; c < CHUNKS; c++) {
        uint8_t* buf = my_buf + (nstore % EPI_BUFS) * EPI_BUF_BYTES;
        uint32_t v[OUT_F32 ? 32 : 64];
        tmem_ld_32x32b_x32(t_row + c * EPI_COLS, v);
        if constexpr (!OUT_F32) tmem_ld_32x32b_x32(t_row + c * EPI_COLS + 32, v + 32);
        // the previous store from this buffer must have been read out by the TMA engine
        if (lane == 0) tma_store_wait_read<EPI_BUFS - 1>();
        __syncwarp();
        tmem_ld_wait();
        if (empty_split) {
#pragma unroll
          for (int i = 0; i < (OUT_F32 ? 32 : 64); i++) v[i] = 0u;
        }
        if (wi.tail >= 0) {
          if (wi.slice != 0) {                 // helper: park the partial accumulator, nothing else
            uint4* dst = reinterpret_cast<uint4*>(ws_q + (size_t)(wi.slice - 1) * WS_SLICE + (size_t)c * WS_CHUNK);
#pragma unroll
            for (int i = 0; i < EPI_COLS / 4; i++) dst[i * 32 + lane] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            continue;
          }
          for (int hs = 0; hs < tail.slices - 1; hs++) {
            const uint4* src = reinterpret_cast<const uint4*>(ws_q + (size_t)hs * WS_SLICE + (size_t)c * WS_CHUNK);
#pragma unroll
            for (int i = 0; i < EPI_COLS / 4; i++) {
              const uint4 p = __ldcg(src + i * 32 + lane);
              v[4 * i] = __float_as_uint(__uint_as_float(v[4 * i]) + __uint_as_float(p.x));
              v[4 * i + 1] = __float_as_uint(__uint_as_float(v[4 * i + 1]) + __uint_as_float(p.y));
              v[4 * i + 2] = __float_as_uint(__uint_as_float(v[4 * i + 2]) + __uint_as_float(p.z));
              v[4 * i + 3] = __float_as_uint(__uint_as_float(v[4 * i + 3]) + __uint_as_float(p.w));
            }
          }
        }
        const int col0 = n0 + c * EPI_COLS;
        if (bias != nullptr) {
#pragma unroll
          for (int i = 0; i < EPI_COLS; i++) {
            float b = 0.f;
            if (col0 + i < N) b = epi.in_f16 ? __half2float(__ldg(reinterpret_cast<const __half*>(bias) + col0 + i)) : __bfloat162float(__ldg(bias + col0 + i));
            v[i] = __float_as_uint(__uint_as_float(v[i]) + b);
          }
        }
        if (epi.act != 0) {
#pragma unroll
          for (int i = 0; i < EPI_COLS; i++) v[i] = __float_as_uint(epi_act(epi.act, __uint_as_float(v[i])));
        }
        if (epi.residual != nullptr && m0 + q * 32 + lane < M) {
          // the lane owns one output row: its residual segment is EPI_COLS contiguous elements
          const size_t roff = (size_t)(m0 + q * 32 + lane) * (size_t)epi.ldr + col0;
          if constexpr (OUT_F32) {
            const float* rp = reinterpret_cast<const float*>(epi.residual) + roff;
#pragma unroll
            for (int i = 0; i < EPI_COLS; i++)
              if (col0 + i < N) v[i] = __float_as_uint(__uint_as_float(v[i]) + rp[i]);
          } else if (epi.in_f16) {
            const __half* rp = reinterpret_cast<const __half*>(epi.residual) + roff;
#pragma unroll
            for (int i = 0; i < EPI_COLS; i++)
              if (col0 + i < N) v[i] = __float_as_uint(__uint_as_float(v[i]) + __half2float(rp[i]));
          } else {
            const __nv_bfloat16* rp = reinterpret_cast<const __nv_bfloat16*>(epi.residual) + roff;
#pragma unroll
            for (int i = 0; i < EPI_COLS; i++)
              if (col0 + i < N) v[i] = __float_as_uint(__uint_as_float(v[i]) + __bfloat162float(rp[i]));
          }
        }
        uint8_t* row = buf + lane * 128;
        if constexpr (OUT_F32) {
#pragma unroll
          for (int j = 0; j < 8; j++) {
            uint4 pk = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            *reinterpret_cast<uint4*>(row + ((j ^ (lane & 7)) << 4)) = pk;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; j++) {
            uint32_t p[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
              if (epi.in_f16) {
                __half2 h = __floats2half2_rn(__uint_as_float(v[8 * j + 2 * e]), __uint_as_float(v[8 * j + 2 * e + 1]));
                p[e] = *reinterpret_cast<uint32_t*>(&h);
              } else {
                __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[8 * j + 2 * e]), __uint_as_float(v[8 * j + 2 * e + 1]));
                p[e] = *reinterpret_cast<uint32_t*>(&h);
              }
            }
            *reinterpret_cast<uint4*>(row + ((j ^ (lane & 7)) << 4)) = make_uint4(p[0], p[1], p[2], p[3]);
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && col0 < N && (m0 + q * 32) < M) {
          tma_store_3d(&tmD, buf, col0, m0 + q * 32, split);
        }
        if (lane == 0) tma_store_commit();
        nstore++;
      }
      if (wi.tail >= 0 && wi.slice != 0) {   // helper: publish this quarter of the slice to the owner
        __threadfence();
        __syncwarp();
        if (lane == 0) red_release_gpu_add(tail.cnt + wi.tail * 4 + q, 1u);
      }
      // all TMEM reads of this accumulator are complete (tmem_ld_wait above)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if (lane == 0) tma_store_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Workspace of the tail slices: one per (device, stream) that launches GEMMs, so that launches on different streams never share one.
struct TailWs {
  cudaStream_t stream;
  float* ws;
  uint32_t* cnt;
  int sms;
};
constexpr int TAIL_SLOTS = 4, TAIL_MAX_SLICES = 8;
TailWs g_tail_ws[64][TAIL_SLOTS] = {};
int g_tail_enabled = -1;

TailArgs plan_tail(int dev, int tiles, int num_kb, int k_splits, int sms, cudaStream_t stream) {
  TailArgs t{0, 1, nullptr, nullptr, 0, {0, 0, 0, 0, 0, 0, 0, 0, 0}, 0, {0, 0, 0, 0, 0, 0, 0, 0, 0}};
  if (g_tail_enabled < 0) {
    const char* e = getenv("FT_GEMM_TAIL");
    g_tail_enabled = (e && e[0] == '1') ? 1 : 0;
  }
  if (!g_tail_enabled || k_splits != 1 || tiles <= sms) return t;
  const int rem = tiles % sms;
  if (rem == 0) return t;
  int slices = sms / rem;
  if (slices > TAIL_MAX_SLICES) slices = TAIL_MAX_SLICES;
  if (slices > num_kb / 4) slices = num_kb / 4;
  if (slices < 2) return t;
  TailWs* slot = nullptr;
  for (int i = 0; i < TAIL_SLOTS && !slot; i++)
    if (g_tail_ws[dev][i].ws && g_tail_ws[dev][i].stream == stream && g_tail_ws[dev][i].sms == sms) slot = &g_tail_ws[dev][i];
  if (!slot) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) { cudaGetLastError(); return t; }
    for (int i = 0; i < TAIL_SLOTS && !slot; i++)
      if (!g_tail_ws[dev][i].ws) slot = &g_tail_ws[dev][i];
    if (!slot) return t;
    // slices * rem <= sms, so (slices - 1) * rem tile-sized f32 partials fit in sms tiles
    float* ws = nullptr;
    uint32_t* cnt = nullptr;
    if (cudaMalloc(&ws, (size_t)sms * BM * BN * sizeof(float)) != cudaSuccess) { cudaGetLastError(); return t; }
    if (cudaMalloc(&cnt, (size_t)sms * 4 * sizeof(uint32_t)) != cudaSuccess || cudaMemset(cnt, 0, (size_t)sms * 4 * sizeof(uint32_t)) != cudaSuccess) {
      cudaGetLastError();
      cudaFree(ws);
      return t;
    }
    *slot = TailWs{stream, ws, cnt, sms};
  }
  t.tiles = rem;
  t.slices = slices;
  t.ws = slot->ws;
  t.cnt = slot->cnt;
  return t;
}

template <bool A_MN, bool B_MN, bool OUT_F32>
int launch(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tD, const void* bias, int M, int N, int K,
           int k_splits, int num_sms, cudaStream_t stream, const EpiArgs& epi, const TailArgs& tail) {
  auto kern = ft_gemm_kernel<A_MN, B_MN, OUT_F32>;
  static bool configured = false;
  if (!configured) {
    FT_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    configured = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * k_splits;
  const int grid = tiles < num_sms ? tiles : num_sms;
  return (int)ft_launch_pdl(kern, dim3(grid), dim3(NUM_THREADS), (size_t)SMEM_BYTES, stream, tA, tB, tD, reinterpret_cast<const __nv_bfloat16*>(bias), M, N, K,
                            k_splits, ft_status_ptr(), epi, tail);
}

int g_num_sms[64] = {0};

}  // namespace

// b_cols > 0 (with b_atoms_per_tap, b_shift[9]): B is a [K, b_cols] matrix read through the row-shift table of TailArgs while N spans nine taps.
static int gemm_impl(const void* A, const void* B, void* D, const void* bias, int M, int N, int K, int64_t lda, int64_t ldb,
                     int64_t ldd, int a_mn, int b_mn, int out_f32, int k_splits, cudaStream_t stream, EpiArgs epi = EpiArgs{0, nullptr, 0, 0},
                     int b_cols = 0, int b_atoms_per_tap = 0, const int* b_shift = nullptr, int a_cols = 0, int64_t a_rows = 0, int a_taps = 0,
                     const int* a_shift = nullptr, int64_t b_rows = 0) {
  if (epi.act < 0 || epi.act > 4) return FT_ERR_ARG;
  const bool in_bf16 = !epi.in_f16;
  if (M <= 0 || N <= 0 || K <= 0 || k_splits < 1 || k_splits > 256) return FT_ERR_ARG;
  if ((lda & 7) || (ldb & 7) || ((ldd * (out_f32 ? 4 : 2)) & 15)) return FT_ERR_ARG;
  // Large-M problems without a row-shift table go to the CTA-pair kernel (256 x 256 tiles, tcgen05 cta_group::2); FT_ERR_DRIVER from it means
  // that this device cannot co-schedule pairs, and the one-SM kernel below takes over.
  if (a_cols == 0 && b_atoms_per_tap == 0 && ft_gemm2_wanted(M, N, K, k_splits)) {
    const int r2 = ft_gemm2_launch(A, B, D, bias, M, N, K, lda, ldb, ldd, a_mn, b_mn, out_f32, k_splits, stream, Gemm2Epi{epi.act, epi.residual, epi.ldr, epi.in_f16});
    if (r2 != FT_ERR_DRIVER) return r2;
  }
  int dev = 0;
  FT_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return FT_ERR_ARG;
  FT_CUDA_TRY(ft_bind_context(dev));
  if (!g_num_sms[dev]) FT_CUDA_TRY(cudaDeviceGetAttribute(&g_num_sms[dev], cudaDevAttrMultiProcessorCount, dev));

  CUtensorMap tA, tB, tD;
  int r;
  // a_cols > 0: A is an [a_rows, a_cols] matrix read through the A row-shift table (K = a_taps * a_cols)
  if (a_cols > 0 && (a_mn || a_cols % 64 || a_taps < 1 || a_taps > 9 || K != a_taps * a_cols || a_shift == nullptr || a_rows < 1)) return FT_ERR_ARG;
  if (!a_mn) r = ft_make_tmap_2d(&tA, A, 2, in_bf16, (uint64_t)(a_cols > 0 ? a_cols : K), (uint64_t)(a_cols > 0 ? a_rows : M), (uint64_t)lda * 2, BK, BM,
                                 CU_TENSOR_MAP_SWIZZLE_128B);
  else       r = ft_make_tmap_2d(&tA, A, 2, in_bf16, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r;
  if (!b_mn) r = ft_make_tmap_2d(&tB, B, 2, in_bf16, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B);
  else       r = ft_make_tmap_2d(&tB, B, 2, in_bf16, (uint64_t)(b_cols > 0 ? b_cols : N), (uint64_t)(b_rows > 0 ? b_rows : K), (uint64_t)ldb * 2, 64, BK,
                                 CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r;
  const uint64_t eb = out_f32 ? 4 : 2;
  r = ft_make_tmap_3d(&tD, D, (int)eb, !out_f32 && in_bf16, (uint64_t)N, (uint64_t)M, (uint64_t)k_splits, (uint64_t)ldd * eb, (uint64_t)M * ldd * eb,
                      out_f32 ? 32 : 64, 32, 1, CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r;

  const int sms = g_num_sms[dev];
  TailArgs tail = plan_tail(dev, ((M + BM - 1) / BM) * ((N + BN - 1) / BN), (K + BK - 1) / BK, k_splits, sms, stream);
  if (a_cols > 0) {
    tail.a_atoms_per_tap = a_cols / 64;
    for (int t = 0; t < 9; t++) tail.a_shift[t] = t < a_taps ? a_shift[t] : 0;
  }
  if (b_atoms_per_tap > 0) {
    if (!b_mn || b_cols != b_atoms_per_tap * 64 || N != 9 * b_cols || b_shift == nullptr) return FT_ERR_ARG;
    tail.b_atoms_per_tap = b_atoms_per_tap;
    for (int t = 0; t < 9; t++) tail.b_shift[t] = b_shift[t];
  }
#define FT_GEMM_CASE(AM, BMN, OF) \
  if (a_mn == AM && b_mn == BMN && out_f32 == OF) return launch<AM, BMN, OF>(tA, tB, tD, bias, M, N, K, k_splits, sms, stream, epi, tail);
  FT_GEMM_CASE(0, 0, 0) FT_GEMM_CASE(0, 1, 0) FT_GEMM_CASE(1, 0, 0) FT_GEMM_CASE(1, 1, 0)
  FT_GEMM_CASE(0, 0, 1) FT_GEMM_CASE(0, 1, 1) FT_GEMM_CASE(1, 0, 1) FT_GEMM_CASE(1, 1, 1)
#undef FT_GEMM_CASE
  return FT_ERR_ARG;
}

// Switches the tail balancing of ft_gemm_kernel on (1) or off (0). It is off unless the environment variable FT_GEMM_TAIL=1 is set when the
// first GEMM is launched: the sliced schedule has been checked on the host (coverage of every (tile, k-block) exactly once, tail items last
// on distinct CTAs) but not yet timed on hardware.
FT_EXPORT int ft_gemm_set_tail(int on) {
  g_tail_enabled = on ? 1 : 0;
  return FT_OK;
}

// D[M,N] = A (x) B (+bias). All pointers are device pointers; lda/ldb/ldd in elements.
// out_f32 = 0: D is bf16; 1: D is f32. Requirements: base pointers 16-byte aligned,
// lda/ldb multiples of 8, ldd*elem_size a multiple of 16, M,N,K >= 1.
FT_EXPORT int ft_gemm_bf16(const void* A, const void* B, void* D, const void* bias, int M, int N, int K, int64_t lda,
                           int64_t ldb, int64_t ldd, int a_mn, int b_mn, int out_f32, cudaStream_t stream) {
  return gemm_impl(A, B, D, bias, M, N, K, lda, ldb, ldd, a_mn, b_mn, out_f32, 1, stream);
}

// Extended form: fp16 operands (in_f16 = 1; bias, residual and a 16-bit output are fp16 then), an activation after the bias
// (act: 0 none, 1 relu, 2 gelu, 3 gelu-tanh, 4 silu) and a residual matrix [M, N] (rows ldr elements apart, dtype of D) added last.
FT_EXPORT int ft_gemm_ex(const void* A, const void* B, void* D, const void* bias, const void* residual, int M, int N, int K, int64_t lda, int64_t ldb,
                         int64_t ldd, int64_t ldr, int a_mn, int b_mn, int out_f32, int in_f16, int act, cudaStream_t stream) {
  return gemm_impl(A, B, D, bias, M, N, K, lda, ldb, ldd, a_mn, b_mn, out_f32, 1, stream, EpiArgs{act, residual, ldr, in_f16});
}

extern "C" int ft_fsdp_gate(const void* arrive, int piece_lo, int piece_hi, uint32_t expected, cudaStream_t st);

// GEMM whose B operand (a weight) lies in a gather slot that peers are still filling (parallel/fsdp.py, fsdp_gather.cu): `counters` are the
// slot's arrival counters (this GPU's memory), `expected` the number of the current gather, `slot_base` the first byte of the slot and
// `piece_bytes` the arrival granularity. The CTA-pair kernel waits per output-column tile inside its TMA producer, so the product starts on
// the weights that have landed; problems it does not take wait for the whole operand with a gate kernel first. Output bf16 or f32, no epilogue
// extras.
FT_EXPORT int ft_gemm_gated(const void* A, const void* B, void* D, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldd, int a_mn, int b_mn,
                            int out_f32, const void* counters, uint32_t expected, const void* slot_base, int64_t piece_bytes, cudaStream_t stream) {
  if (counters == nullptr || slot_base == nullptr || piece_bytes < 16) return FT_ERR_ARG;
  const long long off = (const char*)B - (const char*)slot_base;
  if (off < 0 || M <= 0 || N <= 0 || K <= 0) return FT_ERR_ARG;
  const long long rows = b_mn ? K : N, row_len = b_mn ? N : K;
  const long long bytes = ((rows - 1) * (long long)ldb + row_len) * 2;
  if ((lda & 7) || (ldb & 7) || ((ldd * (out_f32 ? 4 : 2)) & 15)) return FT_ERR_ARG;
  if (ft_gemm2_wanted(M, N, K, 1)) {
    const Gemm2Gate gate{(const uint32_t*)counters, expected, b_mn ? 2 : 1, off, bytes, (long long)piece_bytes, 0, 0};
    const int r2 = ft_gemm2_launch(A, B, D, nullptr, M, N, K, lda, ldb, ldd, a_mn, b_mn, out_f32, 1, stream, Gemm2Epi{0, nullptr, 0, 0}, gate);
    if (r2 != FT_ERR_DRIVER) return r2;
  }
  const int r = ft_fsdp_gate(counters, (int)(off / piece_bytes), (int)((off + bytes - 1) / piece_bytes) + 1, expected, stream);
  if (r) return r;
  return gemm_impl(A, B, D, nullptr, M, N, K, lda, ldb, ldd, a_mn, b_mn, out_f32, 1, stream);
}

// GEMM whose A operand [M, K] (K contiguous) is being gathered from peers in row pieces (tensor-parallel all-gather -> GEMM): counters[i] reaches
// `expected` when rows [i * rows_per_piece, (i + 1) * rows_per_piece) have arrived. The CTA-pair kernel waits per 128-row tile and walks the
// 256-row tiles starting at tile row m_rot, so a rank starts on its own rows. Refused (FT_ERR_ARG) for problems the pair kernel does not take.
FT_EXPORT int ft_gemm_gated_a(const void* A, const void* B, void* D, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldd, int out_f32,
                              const void* counters, uint32_t expected, int rows_per_piece, int m_rot, cudaStream_t stream) {
  if (counters == nullptr || rows_per_piece < 1 || m_rot < 0 || M <= 0 || N <= 0 || K <= 0) return FT_ERR_ARG;
  if (!ft_gemm2_wanted(M, N, K, 1)) return FT_ERR_ARG;
  const Gemm2Gate gate{(const uint32_t*)counters, expected, 1, 0, (long long)M, (long long)rows_per_piece, 1, m_rot % ((M + 255) / 256)};
  return ft_gemm2_launch(A, B, D, nullptr, M, N, K, lda, ldb, ldd, 0, 0, out_f32, 1, stream, Gemm2Epi{0, nullptr, 0, 0}, gate);
}

// Split-K form: partial[s][M][N] (f32, contiguous planes of M*ldd elements) = A (x) B restricted to the s-th slice of K.
// The caller (or a fused consumer kernel) sums the planes. Used when M*N is small and K large, e.g. decoding, where the
// operand stream has to be spread over all SMs.
FT_EXPORT int ft_gemm_bf16_splitk(const void* A, const void* B, float* partial, int M, int N, int K, int64_t lda, int64_t ldb,
                                  int64_t ldd, int a_mn, int b_mn, int k_splits, cudaStream_t stream) {
  return gemm_impl(A, B, partial, nullptr, M, N, K, lda, ldb, ldd, a_mn, b_mn, 1, k_splits, stream);
}

// Weight gradient of the 3x3 / stride 1 / padding 1 convolution as ONE split-K GEMM: dW[co][tap][ci] = sum_j dYp[j][co] * Xp[j + shift(tap)][ci].
// dyp: bf16 [J, Cout] and xp: bf16 [J, Cin], the output gradient and the input zero-padded by one pixel per side and flattened to rows
// (J = N (H+2) (W+2), row_pitch = W + 2); because dYp is zero on the halo, every tap is the same product with Xp shifted by a constant
// number of rows, which the B loads of the GEMM apply through its row-shift table (rows outside Xp read as zeros).
// planes: f32 [k_splits][Cout][9 * Cin]; the caller sums them (ft_splitk_reduce). Cin must be a multiple of 64, Cout of 8.
FT_EXPORT int ft_conv3x3_wgrad_splitk(const void* dyp, const void* xp, float* planes, int Cout, int Cin, int64_t J, int row_pitch, int k_splits,
                                      cudaStream_t stream) {
  if (Cin <= 0 || Cin % 64 || Cout <= 0 || Cout % 8 || J <= 0 || J > 0x7fffffffll || row_pitch < 3) return FT_ERR_ARG;
  int shift[9];
  for (int t = 0; t < 9; t++) shift[t] = (t / 3 - 1) * row_pitch + (t % 3 - 1);
  return gemm_impl(dyp, xp, planes, nullptr, Cout, 9 * Cin, (int)J, Cout, Cin, 9 * (int64_t)Cin, 1, 1, 1, k_splits, stream, EpiArgs{0, nullptr, 0, 0}, Cin, Cin / 64,
                   shift);
}

// General form: dW[co][t][ci] = sum_{j < J} A[j][co] * B[j + shift[t]][ci] for nine caller-given row shifts (host array of 9 ints); B has b_rows
// rows and reads as zeros outside them. With the input stored as stacked planes (for a stride-2 convolution: the four pixel-parity planes of
// the padded input, one below the other), a tap's plane and its offset inside the plane are both just rows, so the same launch covers strided
// convolutions.
FT_EXPORT int ft_conv_wgrad_shift_splitk(const void* a, const void* b, float* planes, int Cout, int Cin, int64_t J, int64_t b_rows, const int* shift9,
                                         int k_splits, cudaStream_t stream) {
  if (Cin <= 0 || Cin % 64 || Cout <= 0 || Cout % 8 || J <= 0 || J > 0x7fffffffll || b_rows <= 0 || b_rows > 0x7fffffffll || shift9 == nullptr) return FT_ERR_ARG;
  return gemm_impl(a, b, planes, nullptr, Cout, 9 * Cin, (int)J, Cout, Cin, 9 * (int64_t)Cin, 1, 1, 1, k_splits, stream, EpiArgs{0, nullptr, 0, 0}, Cin, Cin / 64,
                   shift9, 0, 0, 0, nullptr, b_rows);
}

// Convolution as one GEMM over pixel rows: Y[j][co] = act(sum_t sum_ci X[j + shift[t]][ci] * W[co][t][ci] + bias[co]) for `taps` <= 9 filter
// taps. x: bf16 [x_rows, Cin] (pixel rows of a zero-padded activation, or stacked parity planes of one for a strided convolution), w: bf16
// [Cout, taps * Cin], y: bf16 [rows, Cout], bias: bf16 [Cout] or null, shift: host array of `taps` row offsets, act as in ft_gemm_ex.
// Rows j + shift[t] outside x read as zeros. Cin must be a multiple of 64, Cout of 8. The caller crops the rows of y that belong to halo
// positions of the padded grid.
FT_EXPORT int ft_conv_rows_gemm(const void* x, const void* w, void* y, const void* bias, int64_t rows, int64_t x_rows, int Cin, int Cout, int taps,
                                const int* shift, int act, cudaStream_t stream) {
  if (Cin <= 0 || Cin % 64 || Cout <= 0 || Cout % 8 || rows <= 0 || rows > 0x7fffffffll || x_rows <= 0 || x_rows > 0x7fffffffll || taps < 1 || taps > 9 ||
      shift == nullptr)
    return FT_ERR_ARG;
  return gemm_impl(x, w, y, bias, (int)rows, Cout, taps * Cin, Cin, (int64_t)taps * Cin, Cout, 0, 0, 0, 1, stream, EpiArgs{act, nullptr, 0, 0}, 0, 0, nullptr, Cin,
                   x_rows, taps, shift);
}
