// RMSNorm / LayerNorm forward and backward, bf16 storage with f32 math.
// One CTA per row (grid-stride over rows), 128-bit loads, row kept in registers
// between the reduction and the normalisation so x is read from HBM once.
//
// Capability parity: RMSNORM_PTX / RMSNORM_BACKWARD_PTX (ferrotorch-gpu/src/kernels.rs:7910,8057),
// RMSNORM_BF16_PTX (ferrotorch-gpu/src/bf16.rs:926), LAYERNORM* (kernels.rs:7394,7593).
#include "common.cuh"
#include "host_common.h"
#include <mutex>

#define FT_VPT_DISPATCH(d, ...)                              \
  do {                                                      \
    if ((d) <= 512 * 8) { constexpr int V = 1; constexpr int R = 1; (void)R; __VA_ARGS__; } \
    else if ((d) <= 512 * 16) { constexpr int V = 2; constexpr int R = 1; (void)R; __VA_ARGS__; } \
    else { constexpr int V = 4; constexpr int R = 1; (void)R; __VA_ARGS__; } \
  } while (0)

namespace {

constexpr int NT = 512;          // threads per CTA
constexpr int MAXV_LIMIT = 4;    // 16-byte vectors per thread  => d <= 512*4*8 = 16384

// R block-wide sums at once (one pair of barriers for all of them); every sum is formed in the order block_sum uses.
template <int R>
FT_DEVICE void block_sum_n(float (&v)[R], float* red) {
#pragma unroll
  for (int r = 0; r < R; r++) v[r] = warp_sum(v[r]);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) {
#pragma unroll
    for (int r = 0; r < R; r++) red[r * 32 + w] = v[r];
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < R; r++) v[r] = warp_sum(l < nw ? red[r * 32 + l] : 0.f);
}

// The kernels can take rows in groups of R consecutive rows (all loads of a group issued before one block-wide reduction). Measured on a
// B200 at 4096 x 4096 bf16 with R = 4: forward 30.7 us against 24.6 us with R = 1, backward 50.2 us against 42.0 us (the larger groups leave
// 296 resident CTAs instead of 592 and lengthen each CTA's dependent chain), so every width runs with R = 1.
inline int norm_rows_per_iter(int) { return 1; }

// y = (x [+ res]) * rstd * w ;  optionally writes the summed residual stream back to `xout`.
template <int MAXV, bool HAS_RES, int R, int NTT = NT, int MINB = 1>
__global__ void __launch_bounds__(NTT, MINB) rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                                                         const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                                         __nv_bfloat16* __restrict__ xout, float* __restrict__ rstd_out,
                                                         int rows, int d, float eps) {
  __shared__ float red[32 * R];
  const int nvec = d >> 3;
  for (int row0 = blockIdx.x * R; row0 < rows; row0 += gridDim.x * R) {
    float v[R][MAXV][8];
    float ss[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
      const int row = row0 + r;
      ss[r] = 0.f;
      if (row < rows) {
        const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + (size_t)row * d);
        const bf16x8* rr = HAS_RES ? reinterpret_cast<const bf16x8*>(res + (size_t)row * d) : nullptr;
#pragma unroll
        for (int i = 0; i < MAXV; i++) {
          int c = threadIdx.x + i * NTT;
          if (c < nvec) {
            bf16x8_to_float(xr[c], v[r][i]);
            if (HAS_RES) {
              float t[8];
              bf16x8_to_float(rr[c], t);
#pragma unroll
              for (int e = 0; e < 8; e++) v[r][i][e] += t[e];
              bf16x8 o = float_to_bf16x8(v[r][i]);
              reinterpret_cast<bf16x8*>(xout + (size_t)row * d)[c] = o;
              bf16x8_to_float(o, v[r][i]);  // normalise exactly what the residual stream stores
            }
#pragma unroll
            for (int e = 0; e < 8; e++) ss[r] += v[r][i][e] * v[r][i][e];
          }
        }
      }
    }
    block_sum_n<R>(ss, red);
#pragma unroll
    for (int r = 0; r < R; r++) {
      const int row = row0 + r;
      if (row < rows) {
        const float rstd = rsqrtf(ss[r] / (float)d + eps);
        if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
        for (int i = 0; i < MAXV; i++) {
          int c = threadIdx.x + i * NTT;
          if (c < nvec) {
            float wv[8], o[8];
            bf16x8_to_float(reinterpret_cast<const bf16x8*>(w)[c], wv);
#pragma unroll
            for (int e = 0; e < 8; e++) o[e] = v[r][i][e] * rstd * wv[e];
            reinterpret_cast<bf16x8*>(y + (size_t)row * d)[c] = float_to_bf16x8(o);
          }
        }
      }
    }
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) [+ dres]; dw partial per CTA in f32. Groups of R rows as in the forward kernel.
template <int MAXV, bool HAS_DRES, int R, int NTT = NT, int MINB = 1>
__global__ void __launch_bounds__(NTT, MINB) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                         const __nv_bfloat16* __restrict__ dy, const float* __restrict__ rstd_in,
                                                         const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                                                         float* __restrict__ dw_partial, int rows, int d) {
  __shared__ float red[32 * R];
  const int nvec = d >> 3;
  float dwacc[MAXV][8];
#pragma unroll
  for (int i = 0; i < MAXV; i++)
#pragma unroll
    for (int e = 0; e < 8; e++) dwacc[i][e] = 0.f;
  float wv[MAXV][8];
#pragma unroll
  for (int i = 0; i < MAXV; i++) {
    int c = threadIdx.x + i * NTT;
    if (c < nvec) bf16x8_to_float(reinterpret_cast<const bf16x8*>(w)[c], wv[i]);
  }
  for (int row0 = blockIdx.x * R; row0 < rows; row0 += gridDim.x * R) {
    float xh[R][MAXV][8], g[R][MAXV][8];
    float dot[R], rstd[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
      const int row = row0 + r;
      dot[r] = 0.f;
      rstd[r] = row < rows ? rstd_in[row] : 0.f;
      if (row < rows) {
#pragma unroll
        for (int i = 0; i < MAXV; i++) {
          int c = threadIdx.x + i * NTT;
          if (c < nvec) {
            float xv[8], dyv[8];
            bf16x8_to_float(reinterpret_cast<const bf16x8*>(x + (size_t)row * d)[c], xv);
            bf16x8_to_float(reinterpret_cast<const bf16x8*>(dy + (size_t)row * d)[c], dyv);
#pragma unroll
            for (int e = 0; e < 8; e++) {
              xh[r][i][e] = xv[e] * rstd[r];
              g[r][i][e] = dyv[e] * wv[i][e];
              dot[r] += g[r][i][e] * xh[r][i][e];
              dwacc[i][e] += dyv[e] * xh[r][i][e];
            }
          }
        }
      }
    }
    block_sum_n<R>(dot, red);
#pragma unroll
    for (int r = 0; r < R; r++) {
      const int row = row0 + r;
      if (row < rows) {
        const float dm = dot[r] / (float)d;
#pragma unroll
        for (int i = 0; i < MAXV; i++) {
          int c = threadIdx.x + i * NTT;
          if (c < nvec) {
            float o[8];
#pragma unroll
            for (int e = 0; e < 8; e++) o[e] = rstd[r] * (g[r][i][e] - xh[r][i][e] * dm);
            if (HAS_DRES) {
              float t[8];
              bf16x8_to_float(reinterpret_cast<const bf16x8*>(dres + (size_t)row * d)[c], t);
#pragma unroll
              for (int e = 0; e < 8; e++) o[e] += t[e];
            }
            reinterpret_cast<bf16x8*>(dx + (size_t)row * d)[c] = float_to_bf16x8(o);
          }
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MAXV; i++) {
    int c = threadIdx.x + i * NTT;
    if (c < nvec) {
      float4* p = reinterpret_cast<float4*>(dw_partial + (size_t)blockIdx.x * d + (size_t)c * 8);
      p[0] = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
      p[1] = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
    }
  }
}

// dw[c] (+)= sum_p partial[p][c]. A CTA of 32x8 threads owns 32 columns; the 8 thread rows each add every 8th partial row and
// are then combined in a fixed order, so the result is bit-stable run to run.
__global__ void colsum_partials_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ dw_bf16,
                                       float* __restrict__ dw_f32, int nparts, int d, int accumulate) {
  __shared__ float sm[8][33];
  const int c = blockIdx.x * 32 + threadIdx.x, ry = threadIdx.y;
  float s = 0.f;
  if (c < d)
    for (int p = ry; p < nparts; p += 8) s += partial[(size_t)p * d + c];
  sm[ry][threadIdx.x] = s;
  __syncthreads();
  if (ry == 0 && c < d) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) t += sm[i][threadIdx.x];
    if (dw_f32) dw_f32[c] = accumulate ? dw_f32[c] + t : t;
    if (dw_bf16) dw_bf16[c] = __float2bfloat16(accumulate ? __bfloat162float(dw_bf16[c]) + t : t);
  }
}

// LayerNorm forward: y = (x-mean)*rstd*w + b
template <int MAXV>
__global__ void __launch_bounds__(NT) layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                           const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y,
                                                           float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows,
                                                           int d, float eps) {
  __shared__ float red[32];
  const int nvec = d >> 3;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    float v[MAXV][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; i++) {
      int c = threadIdx.x + i * NT;
      if (c < nvec) {
        bf16x8_to_float(reinterpret_cast<const bf16x8*>(x + (size_t)row * d)[c], v[i]);
#pragma unroll
        for (int e = 0; e < 8; e++) s += v[i][e];
      }
    }
    const float mean = block_sum(s, red) / (float)d;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; i++) {
      int c = threadIdx.x + i * NT;
      if (c < nvec)
#pragma unroll
        for (int e = 0; e < 8; e++) { float t = v[i][e] - mean; ss += t * t; }
    }
    const float rstd = rsqrtf(block_sum(ss, red) / (float)d + eps);
    if (threadIdx.x == 0) { if (mean_out) mean_out[row] = mean; if (rstd_out) rstd_out[row] = rstd; }
#pragma unroll
    for (int i = 0; i < MAXV; i++) {
      int c = threadIdx.x + i * NT;
      if (c < nvec) {
        float wv[8], bv[8], o[8];
        bf16x8_to_float(reinterpret_cast<const bf16x8*>(w)[c], wv);
        if (b) bf16x8_to_float(reinterpret_cast<const bf16x8*>(b)[c], bv);
#pragma unroll
        for (int e = 0; e < 8; e++) o[e] = (v[i][e] - mean) * rstd * wv[e] + (b ? bv[e] : 0.f);
        reinterpret_cast<bf16x8*>(y + (size_t)row * d)[c] = float_to_bf16x8(o);
      }
    }
  }
}

// LayerNorm backward: dx, and per-CTA partials of dw and db.
template <int MAXV>
__global__ void __launch_bounds__(NT) layernorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                           const __nv_bfloat16* __restrict__ dy, const float* __restrict__ mean_in,
                                                           const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                                                           float* __restrict__ dw_partial, float* __restrict__ db_partial,
                                                           int rows, int d) {
  __shared__ float red[32];
  const int nvec = d >> 3;
  float dwacc[MAXV][8], dbacc[MAXV][8], wv[MAXV][8];
#pragma unroll
  for (int i = 0; i < MAXV; i++) {
    int c = threadIdx.x + i * NT;
#pragma unroll
    for (int e = 0; e < 8; e++) { dwacc[i][e] = 0.f; dbacc[i][e] = 0.f; }
    if (c < nvec) bf16x8_to_float(reinterpret_cast<const bf16x8*>(w)[c], wv[i]);
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float mean = mean_in[row], rstd = rstd_in[row];
    float xh[MAXV][8], g[MAXV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; i++) {
      int c = threadIdx.x + i * NT;
      if (c < nvec) {
        float xv[8], dyv[8];
        bf16x8_to_float(reinterpret_cast<const bf16x8*>(x + (size_t)row * d)[c], xv);
        bf16x8_to_float(reinterpret_cast<const bf16x8*>(dy + (size_t)row * d)[c], dyv);
#pragma unroll
        for (int e = 0; e < 8; e++) {
          xh[i][e] = (xv[e] - mean) * rstd;
          g[i][e] = dyv[e] * wv[i][e];
          s1 += g[i][e];
          s2 += g[i][e] * xh[i][e];
          dwacc[i][e] += dyv[e] * xh[i][e];
          dbacc[i][e] += dyv[e];
        }
      }
    }
    s1 = block_sum(s1, red) / (float)d;
    s2 = block_sum(s2, red) / (float)d;
#pragma unroll
    for (int i = 0; i < MAXV; i++) {
      int c = threadIdx.x + i * NT;
      if (c < nvec) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; e++) o[e] = rstd * (g[i][e] - s1 - xh[i][e] * s2);
        reinterpret_cast<bf16x8*>(dx + (size_t)row * d)[c] = float_to_bf16x8(o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MAXV; i++) {
    int c = threadIdx.x + i * NT;
    if (c < nvec)
#pragma unroll
      for (int e = 0; e < 8; e++) {
        dw_partial[(size_t)blockIdx.x * d + (size_t)c * 8 + e] = dwacc[i][e];
        db_partial[(size_t)blockIdx.x * d + (size_t)c * 8 + e] = dbacc[i][e];
      }
  }
}

}  // namespace

// Number of per-CTA partial rows the backward kernels write for `rows` rows.
FT_EXPORT int ft_norm_bwd_parts(int rows) { return rows < 592 ? rows : 592; }

// Thread / vector shape of the RMSNorm kernels for rows of at most 4096 elements (4096 x 4096 bf16 on a B200, CUDA events):
//   0  512 threads x 1 vector                    forward 26.6 us (3 CTAs per SM at 38 registers)   backward 42.0 us (2 CTAs per SM, 296 CTAs)
//   1  forward 512 x 1 held to 32 registers        forward 24.6 us (4 CTAs per SM)
//   2  256 threads x 2 vectors                    forward 22.5 us (twice the bytes in flight)       backward 46.1 us (up to 444 CTAs)
// Defaults: forward 2, backward 0. FT_NORM_VARIANT (read once) forces one number for both directions (A/B switch).
static int norm_variant(int dflt) {
  static int v = -2;
  if (v == -2) {
    const char* e = getenv("FT_NORM_VARIANT");
    v = e ? atoi(e) : -1;
  }
  return v >= 0 ? v : dflt;
}

FT_EXPORT int ft_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* xout, float* rstd, int rows, int d,
                             float eps, cudaStream_t st) {
  if (d % 8 || d > NT * MAXV_LIMIT * 8 || rows <= 0) return FT_ERR_ARG;
  const int groups = (rows + norm_rows_per_iter(d) - 1) / norm_rows_per_iter(d);
  int grid = groups < 148 * 8 ? groups : 148 * 8;
  const __nv_bfloat16 *xp = (const __nv_bfloat16*)x, *rp = (const __nv_bfloat16*)res, *wp = (const __nv_bfloat16*)w;
  __nv_bfloat16 *yp = (__nv_bfloat16*)y, *xo = (__nv_bfloat16*)xout;
  if (d <= 512 * 8 && norm_variant(2) == 1) {
    if (res) rmsnorm_fwd_kernel<1, true, 1, 512, 4><<<grid, 512, 0, st>>>(xp, rp, wp, yp, xo, rstd, rows, d, eps);
    else rmsnorm_fwd_kernel<1, false, 1, 512, 4><<<grid, 512, 0, st>>>(xp, nullptr, wp, yp, nullptr, rstd, rows, d, eps);
    return (int)cudaGetLastError();
  }
  if (d <= 512 * 8 && norm_variant(2) == 2) {
    grid = groups < 148 * 12 ? groups : 148 * 12;
    if (res) rmsnorm_fwd_kernel<2, true, 1, 256, 6><<<grid, 256, 0, st>>>(xp, rp, wp, yp, xo, rstd, rows, d, eps);
    else rmsnorm_fwd_kernel<2, false, 1, 256, 6><<<grid, 256, 0, st>>>(xp, nullptr, wp, yp, nullptr, rstd, rows, d, eps);
    return (int)cudaGetLastError();
  }
  if (res)
    FT_VPT_DISPATCH(d, rmsnorm_fwd_kernel<V, true, R><<<grid, NT, 0, st>>>(xp, rp, wp, yp, xo, rstd, rows, d, eps));
  else
    FT_VPT_DISPATCH(d, rmsnorm_fwd_kernel<V, false, R><<<grid, NT, 0, st>>>(xp, nullptr, wp, yp, nullptr, rstd, rows, d, eps));
  return (int)cudaGetLastError();
}

// dw_partial: f32 scratch of ft_norm_bwd_parts(rows) * d elements. dw_bf16 / dw_f32: either may be null.
FT_EXPORT int ft_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd, const void* dres, void* dx,
                             float* dw_partial, void* dw_bf16, float* dw_f32, int accumulate, int rows, int d, cudaStream_t st) {
  if (d % 8 || d > NT * MAXV_LIMIT * 8 || rows <= 0) return FT_ERR_ARG;
  const int groups = (rows + norm_rows_per_iter(d) - 1) / norm_rows_per_iter(d);
  int grid = groups < 296 ? groups : 296;      // never more partial rows than ft_norm_bwd_parts(rows), which sizes the caller's scratch
  const __nv_bfloat16 *xp = (const __nv_bfloat16*)x, *wp = (const __nv_bfloat16*)w, *dyp = (const __nv_bfloat16*)dy, *drp = (const __nv_bfloat16*)dres;
  __nv_bfloat16* dxp = (__nv_bfloat16*)dx;
  if (d <= 512 * 8 && norm_variant(0) == 2) {
    grid = groups < 444 ? groups : 444;
    if (dres) rmsnorm_bwd_kernel<2, true, 1, 256, 3><<<grid, 256, 0, st>>>(xp, wp, dyp, rstd, drp, dxp, dw_partial, rows, d);
    else rmsnorm_bwd_kernel<2, false, 1, 256, 3><<<grid, 256, 0, st>>>(xp, wp, dyp, rstd, nullptr, dxp, dw_partial, rows, d);
  } else if (dres) {
    FT_VPT_DISPATCH(d, rmsnorm_bwd_kernel<V, true, R><<<grid, NT, 0, st>>>(xp, wp, dyp, rstd, drp, dxp, dw_partial, rows, d));
  } else {
    FT_VPT_DISPATCH(d, rmsnorm_bwd_kernel<V, false, R><<<grid, NT, 0, st>>>(xp, wp, dyp, rstd, nullptr, dxp, dw_partial, rows, d));
  }
  colsum_partials_kernel<<<(d + 31) / 32, dim3(32, 8), 0, st>>>(dw_partial, (__nv_bfloat16*)dw_bf16, dw_f32, grid, d, accumulate);
  return (int)cudaGetLastError();
}

FT_EXPORT int ft_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int rows, int d,
                               float eps, cudaStream_t st) {
  if (d % 8 || d > NT * MAXV_LIMIT * 8 || rows <= 0) return FT_ERR_ARG;
  int grid = rows < 148 * 8 ? rows : 148 * 8;
  FT_VPT_DISPATCH(d, layernorm_fwd_kernel<V><<<grid, NT, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)b,
                                            (__nv_bfloat16*)y, mean, rstd, rows, d, eps));
  return (int)cudaGetLastError();
}

FT_EXPORT int ft_layernorm_bwd(const void* x, const void* w, const void* dy, const float* mean, const float* rstd, void* dx,
                               float* dw_partial, float* db_partial, void* dw_bf16, void* db_bf16, int rows, int d,
                               cudaStream_t st) {
  if (d % 8 || d > NT * MAXV_LIMIT * 8 || rows <= 0) return FT_ERR_ARG;
  int grid = ft_norm_bwd_parts(rows);
  FT_VPT_DISPATCH(d, layernorm_bwd_kernel<V><<<grid, NT, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)dy, mean, rstd,
                                            (__nv_bfloat16*)dx, dw_partial, db_partial, rows, d));
  colsum_partials_kernel<<<(d + 31) / 32, dim3(32, 8), 0, st>>>(dw_partial, (__nv_bfloat16*)dw_bf16, nullptr, grid, d, 0);
  colsum_partials_kernel<<<(d + 31) / 32, dim3(32, 8), 0, st>>>(db_partial, (__nv_bfloat16*)db_bf16, nullptr, grid, d, 0);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------------------
// Allocation-free RMSNorm backward (declared in include/ferrotorch/noalloc.h).
//
// Some callers cannot allocate device memory at the point where they need this kernel: code running inside a
// region where cudaMalloc is forbidden or would synchronise the device (a latency-critical serving loop, a
// plug-in that was handed fixed buffers by its host application, a process whose memory pool is owned by
// another runtime). ft_rmsnorm_bwd needs a scratch buffer for the per-CTA partial sums of dw; this variant keeps
// that scratch in a fixed array that lives inside the loaded library image on every GPU, so the call itself
// performs no cudaMalloc / cudaFree and calls no allocating library routine.
// ---------------------------------------------------------------------------------------------------------
namespace {
constexpr int NOALLOC_PARTS = 148;        // one partial row per SM
constexpr int NOALLOC_MAX_D = 8192;       // largest hidden size accepted
static __device__ __align__(256) float g_rmsnorm_bwd_scratch[NOALLOC_PARTS * NOALLOC_MAX_D];   // 4.6 MiB per GPU

float* g_noalloc_scratch_ptr[64] = {nullptr};
std::mutex g_noalloc_mu;

// The array's name is only a host-side handle; the device address has to be asked for, once per device,
// with that device current.
int noalloc_scratch(float** out) {
  int dev = 0;
  FT_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return FT_ERR_ARG;
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  if (!g_noalloc_scratch_ptr[dev]) {
    float* p = nullptr;
    FT_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_rmsnorm_bwd_scratch));
    if (!p) return FT_ERR_DRIVER;
    g_noalloc_scratch_ptr[dev] = p;
  }
  *out = g_noalloc_scratch_ptr[dev];
  return FT_OK;
}
}  // namespace

FT_EXPORT int ft_rmsnorm_bwd_noalloc_max_d() { return NOALLOC_MAX_D; }

FT_EXPORT int ft_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* dy, const float* rstd, const void* dres, void* dx,
                                     void* dw_bf16, float* dw_f32, int accumulate, int rows, int d, cudaStream_t st) {
  if (d % 8 || rows <= 0 || d <= 0) return FT_ERR_ARG;
  if (d > NOALLOC_MAX_D) {
    fprintf(stderr, "[ferrotorch_b200] ft_rmsnorm_bwd_noalloc: hidden size %d exceeds the built-in scratch (max %d); "
                    "use ft_rmsnorm_bwd with caller-provided scratch\n", d, NOALLOC_MAX_D);
    return FT_ERR_TOO_LARGE;
  }
  // the scratch array that is used is the current device's: a stream of another device would run the kernels there, on an address of this one
  if (st != nullptr && st != cudaStreamLegacy && st != cudaStreamPerThread) {
    int cur = -1, sdev = -1;
    FT_CUDA_TRY(cudaGetDevice(&cur));
    if (cudaStreamGetDevice(st, &sdev) == cudaSuccess && sdev != cur) return FT_ERR_ARG;
    cudaGetLastError();
  }
  float* scratch = nullptr;
  int r = noalloc_scratch(&scratch);
  if (r) return r;
  const int grid = rows < NOALLOC_PARTS ? rows : NOALLOC_PARTS;
  // every partial row in [0, grid) is fully overwritten by its CTA, so nothing has to be cleared between calls
  if (dres)
    FT_VPT_DISPATCH(d, rmsnorm_bwd_kernel<V, true, R><<<grid, NT, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)dy,
                                                                      rstd, (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, scratch, rows, d));
  else
    FT_VPT_DISPATCH(d, rmsnorm_bwd_kernel<V, false, R><<<grid, NT, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)dy,
                                                                       rstd, nullptr, (__nv_bfloat16*)dx, scratch, rows, d));
  colsum_partials_kernel<<<(d + 31) / 32, dim3(32, 8), 0, st>>>(scratch, (__nv_bfloat16*)dw_bf16, dw_f32, grid, d, accumulate);
  return (int)cudaGetLastError();
}
