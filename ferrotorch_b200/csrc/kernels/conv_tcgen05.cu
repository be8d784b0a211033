// 3x3 convolution (stride 1, padding 1, dilation 1), channels-last bf16, as an implicit GEMM on tcgen05.
//
//   Y[n, h, w, :] = sum_{r, s} X[n, h + r - 1, w + s - 1, :] . W[:, r, s, :]^T        X: [N, H, W, Cin], W: [Cout, 3, 3, Cin], Y: [N, H, W, Cout]
//
// GEMM view: M = output pixels, N = Cout, K = 9 * Cin. An M tile is a 16 (rows) x 8 (columns) patch of one image; for filter tap (r, s)
// and a 64-channel slice, the A operand is that patch shifted by (r - 1, s - 1), fetched by ONE 4-D TMA box load {64 ch, 8, 16, 1} whose
// out-of-range rows / columns (the padding halo, and the ragged edge of patches that overhang the image) arrive as zeros. The box lands in
// shared memory as 128 pixel rows x 128 bytes with the 128-byte swizzle, which is exactly the K-major operand layout of the dense GEMM, so the
// im2col matrix never exists. The weights are a plain K-major [Cout, 9 * Cin] matrix. The output tile leaves through 4-D TMA stores
// {64 ch, 8, 4, 1} per epilogue warp, which clip the overhang.
//
// The same kernel computes the data gradient: dX = conv3x3(dY, W') with W'[ci, r, s, co] = W[co, 2 - r, 2 - s, ci].
// Structure (producer / MMA / 4 epilogue warps, two TMEM accumulators, bounded waits) follows gemm_tcgen05.cu.
//
// Capability parity: ferrotorch-gpu/src/conv.rs:218,381,504 (im2col kernel + SGEMM + bias add, forward only); the reference has no device
// convolution backward (ferrotorch-nn/src/conv.rs:888-903 computes it on the host).
#include "common.cuh"
#include "host_common.h"

namespace {

constexpr int BM = 128, BK = 64, UMMA_K = 16, PH = 16, PW = 8;     // M tile = PH x PW pixels
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int EPI_WARPS = 4, EPI_BUF_BYTES = 32 * 128;
constexpr int NUM_THREADS = 32 * (2 + EPI_WARPS);
constexpr uint32_t FT_K_CONV3 = 8;

template <int BN>
struct Cfg {
  static constexpr int B_STAGE_BYTES = BN * BK * 2;
  static constexpr int SMEM = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + EPI_WARPS * EPI_BUF_BYTES + 256 + 1024;
  static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;        // 128, 256 or 512: powers of two
};

FT_DEVICE bool mbar_wait_deadline(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = globaltimer_ns();
  for (uint32_t i = 1;; i++) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 0xff) == 0 && globaltimer_ns() - t0 > 2000000000ull) return false;
  }
}

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
conv3x3_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmY, int Nimg, int H, int W,
               int Cin, int Cout, int relu, uint32_t* status) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + STAGES * A_STAGE_BYTES;
  uint8_t* sEpi = sB + STAGES * C::B_STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sEpi + EPI_WARPS * EPI_BUF_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int th = (H + PH - 1) / PH, tw = (W + PW - 1) / PW, tn = (Cout + BN - 1) / BN;
  const int num_tiles = Nimg * th * tw * tn;
  const int kc = Cin / BK, num_kb = 9 * kc;

  // tile -> (image, patch row, patch column, channel tile); channel tiles of one patch are adjacent so the shifted input boxes are re-used from L2
  auto coords = [&](int tile, int& n, int& h0, int& w0, int& c0) {
    c0 = (tile % tn) * BN;
    int t = tile / tn;
    w0 = (t % tw) * PW;
    t /= tw;
    h0 = (t % th) * PH;
    n = t / th;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; a++) { mbar_init(&tfull_bar[a], 1); mbar_init(&tempty_bar[a], EPI_WARPS); }
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tmX); tma_prefetch_desc(&tmW); tma_prefetch_desc(&tmY); }
  if (warp == 1) { tmem_alloc(tmem_slot, C::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t s = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int n, h0, w0, c0;
        coords(tile, n, h0, w0, c0);
        for (int kb = 0; kb < num_kb; kb++) {
          const int tap = kb / kc, ch = (kb % kc) * BK, r = tap / 3, sx = tap % 3;
          if (!mbar_wait_deadline(&empty_bar[s], phase ^ 1)) { ft_set_status(status, FT_K_CONV3, 1, s); ok = false; break; }
          mbar_expect_tx(&full_bar[s], A_STAGE_BYTES + C::B_STAGE_BYTES);
          tma_load_4d(sA + s * A_STAGE_BYTES, &tmX, &full_bar[s], ch, w0 + sx - 1, h0 + r - 1, n);          // x = channel offset: a multiple of 64
          tma_load_2d(sB + s * C::B_STAGE_BYTES, &tmW, &full_bar[s], tap * Cin + ch, c0);
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
      }
      if (!ok) for (int i = 0; i < 64; i++) __nanosleep(1000);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(BM, BN, 1, 0, 0);
      uint32_t s = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait_deadline(&tempty_bar[acc], acc_phase ^ 1)) { ft_set_status(status, FT_K_CONV3, 2, acc); ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait_deadline(&full_bar[s], phase)) { ft_set_status(status, FT_K_CONV3, 3, s); ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = smem_u32(sA + s * A_STAGE_BYTES), b_base = smem_u32(sB + s * C::B_STAGE_BYTES);
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
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int n, h0, w0, c0;
      coords(tile, n, h0, w0, c0);
      if (!mbar_wait_deadline(&tfull_bar[acc], acc_phase)) { if (lane == 0) ft_set_status(status, FT_K_CONV3, 4, acc); ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < CHUNKS; c++) {
        uint32_t v[64];
        tmem_ld_32x32b_x32(t_row + c * 64, v);
        tmem_ld_32x32b_x32(t_row + c * 64 + 32, v + 32);
        if (lane == 0) tma_store_wait_read<0>();
        __syncwarp();
        tmem_ld_wait();
        uint8_t* row = buf + lane * 128;
#pragma unroll
        for (int j = 0; j < 8; j++) {
          uint32_t pk[4];
#pragma unroll
          for (int e = 0; e < 4; e++) {
            float f0 = __uint_as_float(v[8 * j + 2 * e]), f1 = __uint_as_float(v[8 * j + 2 * e + 1]);
            if (relu) { f0 = fmaxf(f0, 0.f); f1 = fmaxf(f1, 0.f); }
            __nv_bfloat162 h2 = __floats2bfloat162_rn(f0, f1);
            pk[e] = *reinterpret_cast<uint32_t*>(&h2);
          }
          *reinterpret_cast<uint4*>(row + ((j ^ (lane & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
        fence_proxy_async_smem();
        __syncwarp();
        // this warp's 32 accumulator rows are patch rows 4q .. 4q+3 (8 pixels each); the store clips whatever overhangs the image
        if (lane == 0 && c0 + c * 64 < Cout && h0 + 4 * q < H) tma_store_4d(&tmY, buf, c0 + c * 64, w0, h0 + 4 * q, n);
        if (lane == 0) tma_store_commit();
      }
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
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

int g_sms[64] = {0};

template <int BN>
int launch_conv(const void* x, const void* w, void* y, int N, int H, int W, int Cin, int Cout, int relu, int sms, cudaStream_t st) {
  using C = Cfg<BN>;
  CUtensorMap tX, tW, tY;
  const uint64_t xd[4] = {(uint64_t)Cin, (uint64_t)W, (uint64_t)H, (uint64_t)N};
  const uint64_t xp[3] = {(uint64_t)Cin * 2, (uint64_t)W * Cin * 2, (uint64_t)H * W * Cin * 2};
  const uint32_t xb[4] = {BK, PW, PH, 1};
  int r;
  if ((r = ft_make_tmap_4d(&tX, x, 2, true, xd, xp, xb, CU_TENSOR_MAP_SWIZZLE_128B))) return r;
  if ((r = ft_make_tmap_2d(&tW, w, 2, true, (uint64_t)9 * Cin, (uint64_t)Cout, (uint64_t)9 * Cin * 2, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B))) return r;
  const uint64_t yd[4] = {(uint64_t)Cout, (uint64_t)W, (uint64_t)H, (uint64_t)N};
  const uint64_t yp[3] = {(uint64_t)Cout * 2, (uint64_t)W * Cout * 2, (uint64_t)H * W * Cout * 2};
  const uint32_t yb[4] = {64, PW, 4, 1};
  if ((r = ft_make_tmap_4d(&tY, y, 2, true, yd, yp, yb, CU_TENSOR_MAP_SWIZZLE_128B))) return r;
  static bool configured = false;
  if (!configured) {
    FT_CUDA_TRY(cudaFuncSetAttribute(conv3x3_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
    configured = true;
  }
  const long long tiles = (long long)N * ((H + PH - 1) / PH) * ((W + PW - 1) / PW) * ((Cout + BN - 1) / BN);
  if (tiles > 2147483647LL) return FT_ERR_TOO_LARGE;
  const int grid = tiles < sms ? (int)tiles : sms;
  conv3x3_kernel<BN><<<grid, NUM_THREADS, C::SMEM, st>>>(tX, tW, tY, N, H, W, Cin, Cout, relu, ft_status_ptr());
  return (int)cudaGetLastError();
}

}  // namespace

// y[N, H, W, Cout] = conv3x3(x[N, H, W, Cin], w[Cout, 3, 3, Cin]), stride 1, zero padding 1, all bf16 and dense (16-byte aligned bases).
// Cin must be a multiple of 64, Cout of 8. relu = 1 clamps the output at zero.
FT_EXPORT int ft_conv3x3_nhwc(const void* x, const void* w, void* y, int N, int H, int W, int Cin, int Cout, int relu, cudaStream_t st) {
  if (N < 1 || H < 1 || W < 1 || Cin < 64 || (Cin % 64) || Cout < 8 || (Cout % 8)) return FT_ERR_ARG;
  int dev = 0;
  FT_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return FT_ERR_ARG;
  FT_CUDA_TRY(ft_bind_context(dev));
  if (!g_sms[dev]) FT_CUDA_TRY(cudaDeviceGetAttribute(&g_sms[dev], cudaDevAttrMultiProcessorCount, dev));
  if (Cout <= 64) return launch_conv<64>(x, w, y, N, H, W, Cin, Cout, relu, g_sms[dev], st);
  if (Cout <= 128) return launch_conv<128>(x, w, y, N, H, W, Cin, Cout, relu, g_sms[dev], st);
  return launch_conv<256>(x, w, y, N, H, W, Cin, Cout, relu, g_sms[dev], st);
}
