// FlashAttention forward for sm_100a: causal / full, grouped-query, head_dim 128, bf16, on the packed QKV layout
// qkv[B*S, ld] (query heads, then key heads, then value heads along a row), output out[B*S, Hq*128], lse[B,Hq,S].
//
// One CTA per (128-query block, head, batch); two CTAs fit on an SM (112 KiB smem, 256 TMEM columns each), so one
// CTA's softmax overlaps the other's tensor-core work. Roles (192 threads):
//   warp 0      TMA producer: Q once, then K/V blocks of 64 keys into a 2-stage ring (3-D tensor map, so rows past
//               the end of a sequence are zero-filled and never belong to the next batch entry)
//   warp 1      TMEM allocation; one lane issues S = Q.K^T (128x64x128) and O += P.V (128x128x64) with tcgen05.mma;
//               S is double-buffered in TMEM so S(j+1) is computed while softmax works on S(j)
//   warps 2..5  one thread per query row: tcgen05.ld of the S row, mask, online softmax in the log2 domain,
//               P (bf16) written to swizzled smem as the next MMA's A operand, O rescaled in TMEM only when the
//               running maximum grew by more than 2^8 (otherwise the stale maximum is kept; the final 1/l
//               normalisation makes the result identical), final O/l -> bf16 -> smem -> TMA store, LSE store
// V is consumed straight from its [keys, 128] row-major tile as an MN-major B operand: no transposes anywhere.
//
// Capability parity: FLASH_ATTENTION_PTX (ferrotorch-gpu/src/flash_attention.rs:90, one thread per query row, f32,
// no GQA) and the materialised-score attention of ferrotorch-llama/src/gpu.rs:609-628.
#include "common.cuh"
#include "host_common.h"

namespace {

constexpr int FA_BM = 128, FA_BN = 64, FA_D = 128;
constexpr int FA_THREADS = 192;
constexpr int FA_Q_BYTES = FA_BM * FA_D * 2;           // 32 KiB (two 64-column sub-tiles)
constexpr int FA_KV_BYTES = FA_BN * FA_D * 2;          // 16 KiB per K or V block
constexpr int FA_P_BYTES = FA_BM * FA_BN * 2;          // 16 KiB
// two CTAs per SM: 2 * (FA_SMEM + 1 KiB reserved) must stay within the SM's 228 KiB
constexpr int FA_SMEM_DATA = FA_Q_BYTES + 4 * FA_KV_BYTES + FA_P_BYTES;
constexpr int FA_SMEM = FA_SMEM_DATA + 128 + 896;
constexpr int FA_TMEM_COLS = 256;                      // S0 [0,64) S1 [64,128) O [128,256)

FT_DEVICE bool fa_wait(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = globaltimer_ns();
  for (uint32_t i = 1;; i++) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 0xff) == 0 && globaltimer_ns() - t0 > 2000000000ull) return false;
  }
}

__global__ void __launch_bounds__(FA_THREADS, 2)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV,
                 const __grid_constant__ CUtensorMap tmO, float* __restrict__ lse, int S, int Hq, int Hkv, int causal,
                 float scale_log2, uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  if (smem - smem_raw > 896) {               // the carve-out below would not fit: refuse instead of overrunning
    if (threadIdx.x == 0) ft_set_status(status, FT_K_FA_FWD, 15, (uint32_t)(smem - smem_raw));
    return;
  }
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + FA_Q_BYTES;            // 2 stages
  uint8_t* sV = sK + 2 * FA_KV_BYTES;       // 2 stages
  uint8_t* sP = sV + 2 * FA_KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + FA_P_BYTES);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* v_full = bars + 3;    // [2]
  uint64_t* kv_empty = bars + 5;  // [2]
  uint64_t* s_full = bars + 7;    // [2]
  uint64_t* p_ready = bars + 9;
  uint64_t* pv_done = bars + 10;
  uint64_t* k_empty = bars + 11;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mblk = gridDim.x - 1 - blockIdx.x;   // heaviest (latest) query blocks first
  const int h = blockIdx.y, b = blockIdx.z;
  const int g = h / (Hq / Hkv);
  const int m0 = mblk * FA_BM;
  int kv_end = causal ? min(S, m0 + FA_BM) : S;
  const int nblk = (kv_end + FA_BN - 1) / FA_BN;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; i++) { mbar_init(&k_full[i], 1); mbar_init(&v_full[i], 1); mbar_init(&kv_empty[i], 1); mbar_init(&s_full[i], 1); mbar_init(&k_empty[i], 1); }
    mbar_init(p_ready, 128);
    mbar_init(pv_done, 1);
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmKV); tma_prefetch_desc(&tmO); }
  if (warp == 1) { tmem_alloc(tmem_slot, FA_TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tO = tmem_base + 128;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, FA_Q_BYTES);
      tma_load_3d(sQ, &tmQ, q_full, h * FA_D, m0, b);
      tma_load_3d(sQ + 16384, &tmQ, q_full, h * FA_D + 64, m0, b);
      const int kcol = (Hq + g) * FA_D, vcol = (Hq + Hkv + g) * FA_D;
      // load order K(0), K(1), V(0), K(2), V(1), ...: K's slot is free as soon as S of two blocks ago has retired, V's only
      // after O += P.V of two blocks ago, so issuing K one block ahead of V keeps the single producer thread from stalling
      // the next S behind a V slot
      auto load_k = [&](int j) -> bool {
        const int s = j & 1;
        if (!fa_wait(&k_empty[s], ((j >> 1) & 1) ^ 1)) { ft_set_status(status, FT_K_FA_FWD, 1, j); return false; }
        mbar_expect_tx(&k_full[s], FA_KV_BYTES);
        tma_load_3d(sK + s * FA_KV_BYTES, &tmKV, &k_full[s], kcol, j * FA_BN, b);
        tma_load_3d(sK + s * FA_KV_BYTES + 8192, &tmKV, &k_full[s], kcol + 64, j * FA_BN, b);
        return true;
      };
      bool ok = load_k(0);
      for (int j = 0; j < nblk && ok; j++) {
        if (j + 1 < nblk) ok = load_k(j + 1);
        if (!ok) break;
        const int s = j & 1;
        if (!fa_wait(&kv_empty[s], ((j >> 1) & 1) ^ 1)) { ft_set_status(status, FT_K_FA_FWD, 9, j); break; }
        mbar_expect_tx(&v_full[s], FA_KV_BYTES);
        tma_load_3d(sV + s * FA_KV_BYTES, &tmKV, &v_full[s], vcol, j * FA_BN, b);
        tma_load_3d(sV + s * FA_KV_BYTES + 8192, &tmKV, &v_full[s], vcol + 64, j * FA_BN, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_f16(FA_BM, FA_BN, 1, 0, 0);
      constexpr uint32_t idesc_o = make_idesc_f16(FA_BM, FA_D, 1, 0, 1);
      const uint32_t q_base = smem_u32(sQ), p_base = smem_u32(sP);
      auto issue_s = [&](int j) {
        const uint32_t k_base = smem_u32(sK + (j & 1) * FA_KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < FA_D / 16; kk++) {
          const uint64_t ad = make_smem_desc(q_base + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024, FT_SWZ_128B);
          const uint64_t bd = make_smem_desc(k_base + (kk >> 2) * 8192 + (kk & 3) * 32, 16, 1024, FT_SWZ_128B);
          umma_f16_ss(tS + (j & 1) * FA_BN, ad, bd, idesc_s, kk != 0);
        }
        umma_commit(&s_full[j & 1]);
        umma_commit(&k_empty[j & 1]);
      };
      bool ok = fa_wait(q_full, 0);
      if (ok) ok = fa_wait(&k_full[0], 0);
      if (!ok) ft_set_status(status, FT_K_FA_FWD, 2, 0);
      if (ok) {
        tc_fence_after();
        issue_s(0);
        for (int j = 0; j < nblk; j++) {
          if (j + 1 < nblk) {
            if (!fa_wait(&k_full[(j + 1) & 1], ((j + 1) >> 1) & 1)) { ft_set_status(status, FT_K_FA_FWD, 3, j); break; }
            tc_fence_after();
            issue_s(j + 1);
          }
          if (!fa_wait(p_ready, j & 1)) { ft_set_status(status, FT_K_FA_FWD, 4, j); break; }
          if (!fa_wait(&v_full[j & 1], (j >> 1) & 1)) { ft_set_status(status, FT_K_FA_FWD, 5, j); break; }
          tc_fence_after();
          const uint32_t v_base = smem_u32(sV + (j & 1) * FA_KV_BYTES);
#pragma unroll
          for (int kk = 0; kk < FA_BN / 16; kk++) {
            const uint64_t ad = make_smem_desc(p_base + kk * 32, 16, 1024, FT_SWZ_128B);
            const uint64_t bd = make_smem_desc(v_base + kk * 2048, 8192, 1024, FT_SWZ_128B);
            umma_f16_ss(tO, ad, bd, idesc_o, (j | kk) != 0);
          }
          umma_commit(pv_done);
          umma_commit(&kv_empty[j & 1]);
        }
      }
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;               // row inside the query block
    const int qidx = m0 + r;                   // position inside the sequence
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nblk && ok; j++) {
      if (!fa_wait(&s_full[j & 1], (j >> 1) & 1)) { if (lane == 0) ft_set_status(status, FT_K_FA_FWD, 6, j); ok = false; break; }
      tc_fence_after();
      uint32_t sv[64];
      tmem_ld_32x32b_x32(tS + lane_off + (j & 1) * FA_BN, sv);
      tmem_ld_32x32b_x32(tS + lane_off + (j & 1) * FA_BN + 32, sv + 32);
      tmem_ld_wait();
      const int kv0 = j * FA_BN;
      const bool need_mask = (causal && kv0 + FA_BN - 1 > m0) || (kv0 + FA_BN > S);
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 64; c++) {
          const int kv = kv0 + c;
          if ((causal && kv > qidx) || kv >= S) sv[c] = __float_as_uint(-INFINITY);
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four independent chains instead of one of length 64
#pragma unroll
      for (int c = 0; c < 64; c++) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sv[c]));
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      float m_new = fmaxf(m_used, mx);
      if (m_new == -INFINITY) m_new = 0.f;
      const bool grow = (m_new - m_used) * scale_log2 > 8.f;     // also true on the first block (m_used = -inf)
      const bool rescale = __any_sync(0xffffffffu, grow);
      float alpha = 1.f;
      if (rescale) {
        alpha = exp2f((m_used - m_new) * scale_log2);            // 0 on the first block
        m_used = m_new;
      }
      const float moff = m_used * scale_log2;
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 32; c++) {
        const float p0 = exp2f(__uint_as_float(sv[2 * c]) * scale_log2 - moff);
        const float p1 = exp2f(__uint_as_float(sv[2 * c + 1]) * scale_log2 - moff);
        rs4[c & 3] += p0 + p1;
        __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
        pk[c] = *reinterpret_cast<uint32_t*>(&hh);
      }
      l = l * alpha + ((rs4[0] + rs4[1]) + (rs4[2] + rs4[3]));
      if (j > 0) {
        if (!fa_wait(pv_done, (j - 1) & 1)) { if (lane == 0) ft_set_status(status, FT_K_FA_FWD, 7, j); ok = false; break; }
        tc_fence_after();
        if (rescale) {
#pragma unroll 1
          for (int c = 0; c < 4; c++) {
            uint32_t ov[32];
            tmem_ld_32x32b_x32(tO + lane_off + c * 32, ov);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; e++) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * alpha);
            tmem_st_32x32b_x32(tO + lane_off + c * 32, ov);
          }
          tmem_st_wait();
        }
      }
      uint8_t* prow = sP + r * 128;
#pragma unroll
      for (int c8 = 0; c8 < 8; c8++)
        *reinterpret_cast<uint4*>(prow + ((c8 ^ (r & 7)) << 4)) = make_uint4(pk[4 * c8], pk[4 * c8 + 1], pk[4 * c8 + 2], pk[4 * c8 + 3]);
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_ready);
    }
    if (ok) {
      if (!fa_wait(pv_done, (nblk - 1) & 1)) { if (lane == 0) ft_set_status(status, FT_K_FA_FWD, 8, 0); ok = false; }
    }
    if (ok) {
      tc_fence_after();
      const float inv_l = 1.f / l;
#pragma unroll 1
      for (int c = 0; c < 4; c++) {
        uint32_t ov[32];
        tmem_ld_32x32b_x32(tO + lane_off + c * 32, ov);
        tmem_ld_wait();
        uint8_t* orow = sQ + (c >> 1) * 16384 + r * 128;      // Q's smem is free: every S MMA has retired
#pragma unroll
        for (int c8 = 0; c8 < 4; c8++) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; e++) {
            __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(ov[8 * c8 + 2 * e]) * inv_l, __uint_as_float(ov[8 * c8 + 2 * e + 1]) * inv_l);
            w[e] = *reinterpret_cast<uint32_t*>(&hh);
          }
          const int chunk = (c & 1) * 4 + c8;
          *reinterpret_cast<uint4*>(orow + ((chunk ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      if (qidx < S) lse[((size_t)b * Hq + h) * S + qidx] = (m_used * scale_log2 + log2f(l)) * 0.6931471805599453f;
      fence_proxy_async_smem();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 64) {
        tma_store_3d(&tmO, sQ, h * FA_D, m0, b);
        tma_store_3d(&tmO, sQ + 16384, h * FA_D + 64, m0, b);
        tma_store_commit();
        tma_store_wait<0>();
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, FA_TMEM_COLS);
  }
}

}  // namespace

// qkv: bf16 [B*S, ld]; out: bf16 [B*S, Hq*128]; lse: f32 [B, Hq, S]. D must be 128.
FT_EXPORT int ft_flash_fwd(const void* qkv, void* out, float* lse, int B, int S, int Hq, int Hkv, int D, int64_t ld, int causal,
                           float scale, cudaStream_t stream) {
  if (D != FA_D || B <= 0 || S <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv || (ld & 7)) return FT_ERR_ARG;
  int dev = 0;
  FT_CUDA_TRY(cudaGetDevice(&dev));
  FT_CUDA_TRY(ft_bind_context(dev));
  CUtensorMap tQ, tKV, tO;
  int r = ft_make_tmap_3d(&tQ, qkv, 2, true, (uint64_t)ld, (uint64_t)S, (uint64_t)B, (uint64_t)ld * 2, (uint64_t)S * ld * 2, 64, FA_BM, 1,
                          CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r;
  r = ft_make_tmap_3d(&tKV, qkv, 2, true, (uint64_t)ld, (uint64_t)S, (uint64_t)B, (uint64_t)ld * 2, (uint64_t)S * ld * 2, 64, FA_BN, 1,
                      CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r;
  const uint64_t ldo = (uint64_t)Hq * FA_D;
  r = ft_make_tmap_3d(&tO, out, 2, true, ldo, (uint64_t)S, (uint64_t)B, ldo * 2, (uint64_t)S * ldo * 2, 64, FA_BM, 1,
                      CU_TENSOR_MAP_SWIZZLE_128B);
  if (r) return r;
  static bool configured = false;
  if (!configured) {
    FT_CUDA_TRY(cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_SMEM));
    configured = true;
  }
  dim3 grid((S + FA_BM - 1) / FA_BM, Hq, B);
  flash_fwd_kernel<<<grid, FA_THREADS, FA_SMEM, stream>>>(tQ, tKV, tO, lse, S, Hq, Hkv, causal, scale * 1.4426950408889634f,
                                                          ft_status_ptr());
  return (int)cudaGetLastError();
}
