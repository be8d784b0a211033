// FlashAttention backward for sm_100a (causal / full, GQA, head_dim 128, bf16) on the packed QKV layout.
//
// Three launches, no atomics, results bit-stable run to run:
//   1. delta[b,h,s] = sum_d dO*O                                  (bandwidth kernel)
//   2. dQ:    one CTA per (128-query block, head, batch) walks the key blocks (64 keys):
//             S = Q.K^T, dP = dO.V^T -> dS = P*(dP-delta)*scale -> dQ += dS.K
//   3. dK/dV: one CTA per (128-key block, kv head, batch) walks the query heads of its group and their query
//             blocks (64 queries): S^T = K.Q^T, dP^T = V.dO^T -> P^T, dS^T -> dV += P^T.dO, dK += dS^T.Q
// Every product is a tcgen05.mma with the accumulator in TMEM; the "transposed" operands (K in dS.K, dO in P^T.dO,
// Q in dS^T.Q) are the same shared-memory tiles read through MN-major descriptors, so nothing is transposed or
// loaded twice. Roles per CTA: warp 0 TMA, warp 1 MMA issue, then BWD_PARTS arithmetic warps per TMEM lane quarter, i.e. BWD_PARTS threads per
// accumulator row (64/BWD_PARTS columns each) for the exp2 / dS arithmetic and the final TMEM -> bf16 -> smem -> TMA store.
//
// The reference has no attention backward on the GPU (ferrotorch-gpu/src/flash_attention.rs is forward only;
// ferrotorch-nn/src/flash_attention.rs:373-384 recomputes untiled on the CPU).
#include "common.cuh"
#include "host_common.h"

namespace {

constexpr int BD = 128;                 // head dim
constexpr int BWD_PARTS = 2;                 // arithmetic warps per TMEM lane quarter; each handles 64/BWD_PARTS = 16 score columns
constexpr int BWD_COLS = 64 / BWD_PARTS;
constexpr int BWD_ARITH = 128 * BWD_PARTS;    // arithmetic threads
constexpr int BWD_THREADS = 64 + BWD_ARITH;   // warp 0 TMA, warp 1 MMA, then the arithmetic warps (latency is hidden by warp count: 4 per scheduler)
constexpr float LOG2E = 1.4426950408889634f;

template <int COLS>
FT_DEVICE void tmem_ld_cols(uint32_t taddr, uint32_t* r) {
  if constexpr (COLS == 32) tmem_ld_32x32b_x32(taddr, r);
  else tmem_ld_32x32b_x16(taddr, r);
}

FT_DEVICE bool bw_wait(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = globaltimer_ns();
  for (uint32_t i = 1;; i++) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 0xff) == 0 && globaltimer_ns() - t0 > 2000000000ull) return false;
  }
}

// ------------------------------------------------------------------------------------------------------------
// delta
// ------------------------------------------------------------------------------------------------------------
__global__ void flash_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout, float* __restrict__ delta,
                                   int B, int S, int Hq) {
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int total = B * S * Hq;
  if (warp_global >= total) return;
  const int h = warp_global % Hq;
  const int t = warp_global / Hq;             // token index b*S + s
  const size_t off = ((size_t)t * Hq + h) * BD + lane * 4;
  uint2 a = *reinterpret_cast<const uint2*>(o + off);
  uint2 c = *reinterpret_cast<const uint2*>(dout + off);
  float2 a0 = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&a.x)), a1 = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&a.y));
  float2 c0 = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&c.x)), c1 = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&c.y));
  float s = a0.x * c0.x + a0.y * c0.y + a1.x * c1.x + a1.y * c1.y;
  s = warp_sum(s);
  if (lane == 0) {
    const int b = t / S, sq = t % S;
    delta[((size_t)b * Hq + h) * S + sq] = s;
  }
}

// ------------------------------------------------------------------------------------------------------------
// dQ
// ------------------------------------------------------------------------------------------------------------
constexpr int DQ_BM = 128, DQ_BN = 64;
constexpr int DQ_ST = 3;              // K/V ring depth: a slot is released only after dQ += dS.K of its block, so two blocks must be in flight
constexpr int DQ_SMEM_DATA = 32768 /*Q*/ + 32768 /*dO*/ + DQ_ST * 16384 /*K*/ + DQ_ST * 16384 /*V*/ + 16384 /*dS*/;
constexpr int DQ_SMEM = DQ_SMEM_DATA + 256 + 1024;

__global__ void __launch_bounds__(BWD_THREADS, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ,    // qkv, box {64,128,1}
                    const __grid_constant__ CUtensorMap tmKV,   // qkv, box {64,64,1}
                    const __grid_constant__ CUtensorMap tmdO,   // dout, box {64,128,1}
                    const __grid_constant__ CUtensorMap tmdQ,   // dqkv, box {64,128,1}
                    const float* __restrict__ lse, const float* __restrict__ delta, int S, int Hq, int Hkv, int causal,
                    float scale, uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + 32768;
  uint8_t* sK = sdO + 32768;              // DQ_ST stages x 16 KiB
  uint8_t* sV = sK + DQ_ST * 16384;       // DQ_ST stages x 16 KiB
  uint8_t* sdS = sV + DQ_ST * 16384;      // 16 KiB
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + 16384);
  uint64_t* qdo_full = bars + 0;
  uint64_t* kv_full = bars + 1;   // [DQ_ST]
  uint64_t* kv_empty = bars + 5;  // [DQ_ST]
  uint64_t* sp_full = bars + 9;   // [2]
  uint64_t* ds_ready = bars + 11;
  uint64_t* dq_done = bars + 12;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mblk = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int g = h / (Hq / Hkv);
  const int m0 = mblk * DQ_BM;
  const int kv_end = causal ? min(S, m0 + DQ_BM) : S;
  const int nblk = (kv_end + DQ_BN - 1) / DQ_BN;
  const float scale_log2 = scale * LOG2E;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int i = 0; i < DQ_ST; i++) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    for (int i = 0; i < 2; i++) mbar_init(&sp_full[i], 1);
    mbar_init(ds_ready, BWD_ARITH);
    mbar_init(dq_done, 1);
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmKV); tma_prefetch_desc(&tmdO); tma_prefetch_desc(&tmdQ); }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tdP = tmem_base + 128, tdQ = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(qdo_full, 65536);
      tma_load_3d(sQ, &tmQ, qdo_full, h * BD, m0, b);
      tma_load_3d(sQ + 16384, &tmQ, qdo_full, h * BD + 64, m0, b);
      tma_load_3d(sdO, &tmdO, qdo_full, h * BD, m0, b);
      tma_load_3d(sdO + 16384, &tmdO, qdo_full, h * BD + 64, m0, b);
      const int kcol = (Hq + g) * BD, vcol = (Hq + Hkv + g) * BD;
      for (int j = 0; j < nblk; j++) {
        const int s = j % DQ_ST;
        if (!bw_wait(&kv_empty[s], ((j / DQ_ST) & 1) ^ 1)) { ft_set_status(status, FT_K_FA_BWD, 1, j); break; }
        mbar_expect_tx(&kv_full[s], 32768);
        tma_load_3d(sK + s * 16384, &tmKV, &kv_full[s], kcol, j * DQ_BN, b);
        tma_load_3d(sK + s * 16384 + 8192, &tmKV, &kv_full[s], kcol + 64, j * DQ_BN, b);
        tma_load_3d(sV + s * 16384, &tmKV, &kv_full[s], vcol, j * DQ_BN, b);
        tma_load_3d(sV + s * 16384 + 8192, &tmKV, &kv_full[s], vcol + 64, j * DQ_BN, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_f16(128, 64, 1, 0, 0);
      constexpr uint32_t idesc_dq = make_idesc_f16(128, 128, 1, 0, 1);
      const uint32_t q_base = smem_u32(sQ), do_base = smem_u32(sdO), ds_base = smem_u32(sdS);
      auto issue_s_dp = [&](int j) {
        const uint32_t k_base = smem_u32(sK + (j % DQ_ST) * 16384), v_base = smem_u32(sV + (j % DQ_ST) * 16384);
#pragma unroll
        for (int kk = 0; kk < 8; kk++) {
          const uint32_t ao = (kk >> 2) * 16384 + (kk & 3) * 32, bo = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_f16_ss(tS + (j & 1) * 64, make_smem_desc(q_base + ao, 16, 1024, FT_SWZ_128B),
                      make_smem_desc(k_base + bo, 16, 1024, FT_SWZ_128B), idesc_s, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < 8; kk++) {
          const uint32_t ao = (kk >> 2) * 16384 + (kk & 3) * 32, bo = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_f16_ss(tdP + (j & 1) * 64, make_smem_desc(do_base + ao, 16, 1024, FT_SWZ_128B),
                      make_smem_desc(v_base + bo, 16, 1024, FT_SWZ_128B), idesc_s, kk != 0);
        }
        umma_commit(&sp_full[j & 1]);
      };
      bool ok = bw_wait(qdo_full, 0) && bw_wait(&kv_full[0], 0);
      if (!ok) ft_set_status(status, FT_K_FA_BWD, 2, 0);
      if (ok) {
        tc_fence_after();
        issue_s_dp(0);
        for (int j = 0; j < nblk; j++) {
          if (j + 1 < nblk) {
            if (!bw_wait(&kv_full[(j + 1) % DQ_ST], ((j + 1) / DQ_ST) & 1)) { ft_set_status(status, FT_K_FA_BWD, 3, j); break; }
            tc_fence_after();
            issue_s_dp(j + 1);
          }
          if (!bw_wait(ds_ready, j & 1)) { ft_set_status(status, FT_K_FA_BWD, 4, j); break; }
          tc_fence_after();
          const uint32_t k_base = smem_u32(sK + (j % DQ_ST) * 16384);
#pragma unroll
          for (int kk = 0; kk < 4; kk++)
            umma_f16_ss(tdQ, make_smem_desc(ds_base + kk * 32, 16, 1024, FT_SWZ_128B),
                        make_smem_desc(k_base + kk * 2048, 8192, 1024, FT_SWZ_128B), idesc_dq, (j | kk) != 0);
          umma_commit(dq_done);
          umma_commit(&kv_empty[j % DQ_ST]);
        }
      }
    }
  } else {
    const int q = warp & 3;
    const int part = (warp - 2) >> 2;          // which BWD_COLS of the 64 key columns this warp handles
    const int r = q * 32 + lane;
    const int qidx = m0 + r;
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    const bool qvalid = qidx < S;
    const float lse2 = qvalid ? lse[((size_t)b * Hq + h) * S + qidx] * LOG2E : INFINITY;
    const float dlt = qvalid ? delta[((size_t)b * Hq + h) * S + qidx] : 0.f;
    bool ok = true;
    for (int j = 0; j < nblk && ok; j++) {
      if (!bw_wait(&sp_full[j & 1], (j >> 1) & 1)) { if (lane == 0) ft_set_status(status, FT_K_FA_BWD, 5, j); ok = false; break; }
      tc_fence_after();
      const int kv0 = j * DQ_BN;
      uint32_t pk[BWD_COLS / 2];
      {
        uint32_t sv[BWD_COLS], dv[BWD_COLS];
        tmem_ld_cols<BWD_COLS>(tS + lane_off + (j & 1) * 64 + part * BWD_COLS, sv);
        tmem_ld_cols<BWD_COLS>(tdP + lane_off + (j & 1) * 64 + part * BWD_COLS, dv);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < BWD_COLS / 2; c++) {
          float ds[2];
#pragma unroll
          for (int e = 0; e < 2; e++) {
            const int col = 2 * c + e, kv = kv0 + part * BWD_COLS + col;
            float p = exp2f(__uint_as_float(sv[col]) * scale_log2 - lse2);
            if ((causal && kv > qidx) || kv >= S) p = 0.f;
            ds[e] = p * (__uint_as_float(dv[col]) - dlt) * scale;
          }
          __nv_bfloat162 hh = __floats2bfloat162_rn(ds[0], ds[1]);
          pk[c] = *reinterpret_cast<uint32_t*>(&hh);
        }
      }
      if (j > 0) {
        if (!bw_wait(dq_done, (j - 1) & 1)) { if (lane == 0) ft_set_status(status, FT_K_FA_BWD, 6, j); ok = false; break; }
      }
      uint8_t* row = sdS + r * 128;
#pragma unroll
      for (int c4 = 0; c4 < BWD_COLS / 8; c4++)
        *reinterpret_cast<uint4*>(row + (((part * (BWD_COLS / 8) + c4) ^ (r & 7)) << 4)) = make_uint4(pk[4 * c4], pk[4 * c4 + 1], pk[4 * c4 + 2], pk[4 * c4 + 3]);
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(ds_ready);
    }
    if (ok && !bw_wait(dq_done, (nblk - 1) & 1)) { if (lane == 0) ft_set_status(status, FT_K_FA_BWD, 7, 0); ok = false; }
    if (ok) {
      tc_fence_after();
#pragma unroll 1
      for (int c = part * (4 / BWD_PARTS); c < (part + 1) * (4 / BWD_PARTS); c++) {   // 128 output columns = 4 chunks of 32
        uint32_t ov[32];
        tmem_ld_32x32b_x32(tdQ + lane_off + c * 32, ov);
        tmem_ld_wait();
        uint8_t* orow = sQ + (c >> 1) * 16384 + r * 128;
#pragma unroll
        for (int c8 = 0; c8 < 4; c8++) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; e++) {
            __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(ov[8 * c8 + 2 * e]), __uint_as_float(ov[8 * c8 + 2 * e + 1]));
            w[e] = *reinterpret_cast<uint32_t*>(&hh);
          }
          const int chunk = (c & 1) * 4 + c8;
          *reinterpret_cast<uint4*>(orow + ((chunk ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      fence_proxy_async_smem();
      asm volatile("bar.sync 1, %0;" ::"n"(BWD_ARITH) : "memory");
      if (threadIdx.x == 64) {
        tma_store_3d(&tmdQ, sQ, h * BD, m0, b);
        tma_store_3d(&tmdQ, sQ + 16384, h * BD + 64, m0, b);
        tma_store_commit();
        tma_store_wait<0>();
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// ------------------------------------------------------------------------------------------------------------
// dK / dV
// ------------------------------------------------------------------------------------------------------------
constexpr int DKV_BN = 128 /*keys per CTA*/, DKV_BM = 64 /*queries per step*/;
constexpr int DKV_ST = 3;             // Q/dO ring depth (a slot is released only after dV/dK of its step)
constexpr int DKV_SMEM_DATA = 32768 /*K*/ + 32768 /*V*/ + DKV_ST * 16384 /*Q*/ + DKV_ST * 16384 /*dO*/ + 16384 /*P^T*/ + 16384 /*dS^T*/ + 1024 /*stats*/;
constexpr int DKV_SMEM = DKV_SMEM_DATA + 256 + 1024;

__global__ void __launch_bounds__(BWD_THREADS, 1)
flash_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmKV128,  // qkv, box {64,128,1}  (K, V of this CTA; also the dK/dV store into dqkv)
                     const __grid_constant__ CUtensorMap tmQ64,    // qkv, box {64,64,1}
                     const __grid_constant__ CUtensorMap tmdO64,   // dout, box {64,64,1}
                     const __grid_constant__ CUtensorMap tmdKV,    // dqkv, box {64,128,1}
                     const float* __restrict__ lse, const float* __restrict__ delta, int S, int Hq, int Hkv, int causal,
                     float scale, uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + 32768;
  uint8_t* sQ = sV + 32768;                // DKV_ST stages x 16 KiB
  uint8_t* sdO = sQ + DKV_ST * 16384;      // DKV_ST stages x 16 KiB
  uint8_t* sPt = sdO + DKV_ST * 16384;     // 16 KiB
  uint8_t* sdSt = sPt + 16384;     // 16 KiB
  float* sStat = reinterpret_cast<float*>(sdSt + 16384);   // [2][128]: lse2 (64) | delta (64)
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(sStat) + 1024);
  uint64_t* kv_full = bars + 0;
  uint64_t* qdo_full = bars + 1;   // [DKV_ST]
  uint64_t* qdo_empty = bars + 5;  // [DKV_ST]
  uint64_t* st_full = bars + 9;    // [2]
  uint64_t* pds_ready = bars + 11;
  uint64_t* dkv_done = bars + 12;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = blockIdx.x;                      // key block 0 has the most query blocks and is scheduled first
  const int g = blockIdx.y, b = blockIdx.z;
  const int kv0 = nblk * DKV_BN;
  const int group = Hq / Hkv;
  const int nq = (S + DKV_BM - 1) / DKV_BM;
  const int i_start = causal ? (kv0 / DKV_BM) : 0;
  const int nqi = nq - i_start;                     // query blocks per head
  const int n_it = nqi * group;
  const float scale_log2 = scale * LOG2E;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < DKV_ST; i++) { mbar_init(&qdo_full[i], 1); mbar_init(&qdo_empty[i], 1); }
    for (int i = 0; i < 2; i++) mbar_init(&st_full[i], 1);
    mbar_init(pds_ready, BWD_ARITH);
    mbar_init(dkv_done, 1);
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tmKV128); tma_prefetch_desc(&tmQ64); tma_prefetch_desc(&tmdO64); tma_prefetch_desc(&tmdKV); }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tSt = tmem_base, tdPt = tmem_base + 128, tdV = tmem_base + 256, tdK = tmem_base + 384;
  const int kcol = (Hq + g) * BD, vcol = (Hq + Hkv + g) * BD;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 65536);
      tma_load_3d(sK, &tmKV128, kv_full, kcol, kv0, b);
      tma_load_3d(sK + 16384, &tmKV128, kv_full, kcol + 64, kv0, b);
      tma_load_3d(sV, &tmKV128, kv_full, vcol, kv0, b);
      tma_load_3d(sV + 16384, &tmKV128, kv_full, vcol + 64, kv0, b);
      for (int it = 0; it < n_it; it++) {
        const int s = it % DKV_ST;
        const int hq = g * group + it / nqi, q0 = (i_start + it % nqi) * DKV_BM;
        if (!bw_wait(&qdo_empty[s], ((it / DKV_ST) & 1) ^ 1)) { ft_set_status(status, FT_K_FA_BWD, 11, it); break; }
        mbar_expect_tx(&qdo_full[s], 32768);
        tma_load_3d(sQ + s * 16384, &tmQ64, &qdo_full[s], hq * BD, q0, b);
        tma_load_3d(sQ + s * 16384 + 8192, &tmQ64, &qdo_full[s], hq * BD + 64, q0, b);
        tma_load_3d(sdO + s * 16384, &tmdO64, &qdo_full[s], hq * BD, q0, b);
        tma_load_3d(sdO + s * 16384 + 8192, &tmdO64, &qdo_full[s], hq * BD + 64, q0, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_st = make_idesc_f16(128, 64, 1, 0, 0);
      constexpr uint32_t idesc_acc = make_idesc_f16(128, 128, 1, 0, 1);
      const uint32_t k_base = smem_u32(sK), v_base = smem_u32(sV), pt_base = smem_u32(sPt), dst_base = smem_u32(sdSt);
      auto issue_st = [&](int it) {
        const uint32_t q_base = smem_u32(sQ + (it % DKV_ST) * 16384), do_base = smem_u32(sdO + (it % DKV_ST) * 16384);
#pragma unroll
        for (int kk = 0; kk < 8; kk++) {
          const uint32_t ao = (kk >> 2) * 16384 + (kk & 3) * 32, bo = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_f16_ss(tSt + (it & 1) * 64, make_smem_desc(k_base + ao, 16, 1024, FT_SWZ_128B),
                      make_smem_desc(q_base + bo, 16, 1024, FT_SWZ_128B), idesc_st, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < 8; kk++) {
          const uint32_t ao = (kk >> 2) * 16384 + (kk & 3) * 32, bo = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_f16_ss(tdPt + (it & 1) * 64, make_smem_desc(v_base + ao, 16, 1024, FT_SWZ_128B),
                      make_smem_desc(do_base + bo, 16, 1024, FT_SWZ_128B), idesc_st, kk != 0);
        }
        umma_commit(&st_full[it & 1]);
      };
      bool ok = bw_wait(kv_full, 0) && bw_wait(&qdo_full[0], 0);
      if (!ok) ft_set_status(status, FT_K_FA_BWD, 12, 0);
      if (ok) {
        tc_fence_after();
        issue_st(0);
        for (int it = 0; it < n_it; it++) {
          if (it + 1 < n_it) {
            if (!bw_wait(&qdo_full[(it + 1) % DKV_ST], ((it + 1) / DKV_ST) & 1)) { ft_set_status(status, FT_K_FA_BWD, 13, it); break; }
            tc_fence_after();
            issue_st(it + 1);
          }
          if (!bw_wait(pds_ready, it & 1)) { ft_set_status(status, FT_K_FA_BWD, 14, it); break; }
          tc_fence_after();
          const uint32_t q_base = smem_u32(sQ + (it % DKV_ST) * 16384), do_base = smem_u32(sdO + (it % DKV_ST) * 16384);
#pragma unroll
          for (int kk = 0; kk < 4; kk++)
            umma_f16_ss(tdV, make_smem_desc(pt_base + kk * 32, 16, 1024, FT_SWZ_128B),
                        make_smem_desc(do_base + kk * 2048, 8192, 1024, FT_SWZ_128B), idesc_acc, (it | kk) != 0);
#pragma unroll
          for (int kk = 0; kk < 4; kk++)
            umma_f16_ss(tdK, make_smem_desc(dst_base + kk * 32, 16, 1024, FT_SWZ_128B),
                        make_smem_desc(q_base + kk * 2048, 8192, 1024, FT_SWZ_128B), idesc_acc, (it | kk) != 0);
          umma_commit(dkv_done);
          umma_commit(&qdo_empty[it % DKV_ST]);
        }
      }
    }
  } else {
    const int q = warp & 3;
    const int part = (warp - 2) >> 2;            // which BWD_COLS of the 64 query columns this warp handles
    const int r = q * 32 + lane;                 // key row inside the block
    const int kvidx = kv0 + r;
    const int tid = threadIdx.x - 64;            // index among the arithmetic threads
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    const bool kvalid = kvidx < S;
    bool ok = true;
    // row statistics of a step (threads 0..63 fetch lse in the log2 domain, 64..127 fetch delta) are fetched one step
    // ahead, so the global-memory latency is hidden behind the previous step's arithmetic
    auto fetch_stat = [&](int it2) -> float {
      const int hq2 = g * group + it2 / nqi, qi = (i_start + it2 % nqi) * DKV_BM + (tid & 63);
      if (tid < 64) return (qi < S) ? lse[((size_t)b * Hq + hq2) * S + qi] * LOG2E : INFINITY;
      return (qi < S) ? delta[((size_t)b * Hq + hq2) * S + qi] : 0.f;
    };
    if (tid < 128 && n_it > 0) sStat[tid] = fetch_stat(0);
    for (int it = 0; it < n_it && ok; it++) {
      const int q0 = (i_start + it % nqi) * DKV_BM;
      asm volatile("bar.sync 1, %0;" ::"n"(BWD_ARITH) : "memory");    // publishes sStat[it&1]; everyone has finished reading sStat[(it+1)&1]
      float next_stat = 0.f;
      if (tid < 128 && it + 1 < n_it) next_stat = fetch_stat(it + 1);
      const float* st_lse = sStat + (it & 1) * 128;
      const float* st_dlt = st_lse + 64;
      if (!bw_wait(&st_full[it & 1], (it >> 1) & 1)) { if (lane == 0) ft_set_status(status, FT_K_FA_BWD, 15, it); ok = false; break; }
      tc_fence_after();
      uint32_t ppk[BWD_COLS / 2], dpk[BWD_COLS / 2];
      {
        uint32_t sv[BWD_COLS], dv[BWD_COLS];
        tmem_ld_cols<BWD_COLS>(tSt + lane_off + (it & 1) * 64 + part * BWD_COLS, sv);
        tmem_ld_cols<BWD_COLS>(tdPt + lane_off + (it & 1) * 64 + part * BWD_COLS, dv);
        float sl[BWD_COLS], sd[BWD_COLS];
#pragma unroll
        for (int c4 = 0; c4 < BWD_COLS / 4; c4++) {
          const float4 a = reinterpret_cast<const float4*>(st_lse + part * BWD_COLS)[c4];
          const float4 d = reinterpret_cast<const float4*>(st_dlt + part * BWD_COLS)[c4];
          sl[4 * c4] = a.x; sl[4 * c4 + 1] = a.y; sl[4 * c4 + 2] = a.z; sl[4 * c4 + 3] = a.w;
          sd[4 * c4] = d.x; sd[4 * c4 + 1] = d.y; sd[4 * c4 + 2] = d.z; sd[4 * c4 + 3] = d.w;
        }
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < BWD_COLS / 2; c++) {
          float pp[2], ds[2];
#pragma unroll
          for (int e = 0; e < 2; e++) {
            const int cc = 2 * c + e, qi = q0 + part * BWD_COLS + cc;
            float p = exp2f(__uint_as_float(sv[cc]) * scale_log2 - sl[cc]);
            if ((causal && kvidx > qi) || !kvalid) p = 0.f;
            pp[e] = p;
            ds[e] = p * (__uint_as_float(dv[cc]) - sd[cc]) * scale;
          }
          __nv_bfloat162 hp = __floats2bfloat162_rn(pp[0], pp[1]), hd = __floats2bfloat162_rn(ds[0], ds[1]);
          ppk[c] = *reinterpret_cast<uint32_t*>(&hp);
          dpk[c] = *reinterpret_cast<uint32_t*>(&hd);
        }
      }
      if (it > 0) {
        if (!bw_wait(dkv_done, (it - 1) & 1)) { if (lane == 0) ft_set_status(status, FT_K_FA_BWD, 16, it); ok = false; break; }
      }
      uint8_t* prow = sPt + r * 128;
      uint8_t* drow = sdSt + r * 128;
#pragma unroll
      for (int c4 = 0; c4 < BWD_COLS / 8; c4++) {
        const int sw = ((part * (BWD_COLS / 8) + c4) ^ (r & 7)) << 4;
        *reinterpret_cast<uint4*>(prow + sw) = make_uint4(ppk[4 * c4], ppk[4 * c4 + 1], ppk[4 * c4 + 2], ppk[4 * c4 + 3]);
        *reinterpret_cast<uint4*>(drow + sw) = make_uint4(dpk[4 * c4], dpk[4 * c4 + 1], dpk[4 * c4 + 2], dpk[4 * c4 + 3]);
      }
      if (tid < 128 && it + 1 < n_it) sStat[((it + 1) & 1) * 128 + tid] = next_stat;
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(pds_ready);
    }
    if (ok && !bw_wait(dkv_done, (n_it - 1) & 1)) { if (lane == 0) ft_set_status(status, FT_K_FA_BWD, 17, 0); ok = false; }
    if (ok) {
      tc_fence_after();
      // dV -> sV region, dK -> sK region (both operands are dead: every MMA has retired)
#pragma unroll 1
      for (int which = 0; which < 2; which++) {
        const uint32_t tsrc = which == 0 ? tdV : tdK;
        uint8_t* sdst = which == 0 ? sV : sK;
#pragma unroll 1
        for (int c = part * (4 / BWD_PARTS); c < (part + 1) * (4 / BWD_PARTS); c++) {   // 128 output columns = 4 chunks of 32
          uint32_t ov[32];
          tmem_ld_32x32b_x32(tsrc + lane_off + c * 32, ov);
          tmem_ld_wait();
          uint8_t* orow = sdst + (c >> 1) * 16384 + r * 128;
#pragma unroll
          for (int c8 = 0; c8 < 4; c8++) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
              __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(ov[8 * c8 + 2 * e]), __uint_as_float(ov[8 * c8 + 2 * e + 1]));
              w[e] = *reinterpret_cast<uint32_t*>(&hh);
            }
            const int chunk = (c & 1) * 4 + c8;
            *reinterpret_cast<uint4*>(orow + ((chunk ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      fence_proxy_async_smem();
      asm volatile("bar.sync 1, %0;" ::"n"(BWD_ARITH) : "memory");
      if (threadIdx.x == 64) {
        tma_store_3d(&tmdKV, sV, vcol, kv0, b);
        tma_store_3d(&tmdKV, sV + 16384, vcol + 64, kv0, b);
        tma_store_3d(&tmdKV, sK, kcol, kv0, b);
        tma_store_3d(&tmdKV, sK + 16384, kcol + 64, kv0, b);
        tma_store_commit();
        tma_store_wait<0>();
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

}  // namespace

// qkv, dqkv: bf16 [B*S, ld]; out, dout: bf16 [B*S, Hq*128]; lse: f32 [B,Hq,S]; delta: f32 scratch [B,Hq,S].
FT_EXPORT int ft_flash_bwd_ws(const void* qkv, const void* out, const float* lse, const void* dout, void* dqkv, float* delta, int B,
                              int S, int Hq, int Hkv, int D, int64_t ld, int causal, float scale, cudaStream_t stream) {
  if (D != BD || B <= 0 || S <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv || (ld & 7)) return FT_ERR_ARG;
  int dev = 0;
  FT_CUDA_TRY(cudaGetDevice(&dev));
  FT_CUDA_TRY(ft_bind_context(dev));
  const uint64_t ldq = (uint64_t)ld, ldo = (uint64_t)Hq * BD;
  CUtensorMap tQ128, tQ64, tdO128, tdO64, tdQKV128;
  int r;
  if ((r = ft_make_tmap_3d(&tQ128, qkv, 2, true, ldq, S, B, ldq * 2, (uint64_t)S * ldq * 2, 64, 128, 1, CU_TENSOR_MAP_SWIZZLE_128B))) return r;
  if ((r = ft_make_tmap_3d(&tQ64, qkv, 2, true, ldq, S, B, ldq * 2, (uint64_t)S * ldq * 2, 64, 64, 1, CU_TENSOR_MAP_SWIZZLE_128B))) return r;
  if ((r = ft_make_tmap_3d(&tdO128, dout, 2, true, ldo, S, B, ldo * 2, (uint64_t)S * ldo * 2, 64, 128, 1, CU_TENSOR_MAP_SWIZZLE_128B))) return r;
  if ((r = ft_make_tmap_3d(&tdO64, dout, 2, true, ldo, S, B, ldo * 2, (uint64_t)S * ldo * 2, 64, 64, 1, CU_TENSOR_MAP_SWIZZLE_128B))) return r;
  if ((r = ft_make_tmap_3d(&tdQKV128, dqkv, 2, true, ldq, S, B, ldq * 2, (uint64_t)S * ldq * 2, 64, 128, 1, CU_TENSOR_MAP_SWIZZLE_128B))) return r;
  static bool configured = false;
  if (!configured) {
    FT_CUDA_TRY(cudaFuncSetAttribute(flash_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DQ_SMEM));
    FT_CUDA_TRY(cudaFuncSetAttribute(flash_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DKV_SMEM));
    configured = true;
  }
  uint32_t* status = ft_status_ptr();
  const int total_warps = B * S * Hq;
  flash_delta_kernel<<<(total_warps * 32 + 255) / 256, 256, 0, stream>>>((const __nv_bfloat16*)out, (const __nv_bfloat16*)dout, delta, B, S, Hq);
  dim3 gq((S + DQ_BM - 1) / DQ_BM, Hq, B);
  flash_bwd_dq_kernel<<<gq, BWD_THREADS, DQ_SMEM, stream>>>(tQ128, tQ64, tdO128, tdQKV128, lse, delta, S, Hq, Hkv, causal, scale, status);
  dim3 gk((S + DKV_BN - 1) / DKV_BN, Hkv, B);
  flash_bwd_dkv_kernel<<<gk, BWD_THREADS, DKV_SMEM, stream>>>(tQ128, tQ64, tdO64, tdQKV128, lse, delta, S, Hq, Hkv, causal, scale, status);
  return (int)cudaGetLastError();
}
