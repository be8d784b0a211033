// Normalisation over channels-last activations, pooling, group norm and recurrent cells.
//
//  * BatchNorm on [M = N*H*W, C] (NHWC): column statistics in two stages (per-CTA partial sums -> finalize with running-stat update), so the
//    [2, C] sums can be all-reduced across ranks between the stages (SyncBatchNorm); apply with optional residual add and ReLU; backward with the
//    ReLU mask recomputed from the output, producing dx (and the residual gradient) in one pass.
//  * MaxPool2d NHWC forward / backward (argmax recomputed, deterministic, no atomics).
//  * GroupNorm NCHW forward / backward, one CTA per (sample, group).
//  * LSTM / GRU cell pointwise forward / backward on pre-computed gate GEMM outputs.
//
// Replaces ferrotorch-gpu/src/kernels.rs BATCHNORM_FORWARD 8324, MAXPOOL2D 8599, AVGPOOL2D 8744, FUSED_GRU_FORWARD 12032 and
// ferrotorch-gpu/src/group_norm.rs:56; the backward kernels have no device counterpart in the reference (its module path falls back to the host).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include "common.cuh"
#include "host_common.h"

namespace {

template <typename T> struct VecT;
template <> struct VecT<float> { static constexpr int N = 4; };
template <> struct VecT<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T, int N> FT_DEVICE void load_vec(const T* p, float* out);
template <> FT_DEVICE void load_vec<float, 4>(const float* p, float* out) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
template <> FT_DEVICE void load_vec<__nv_bfloat16, 8>(const __nv_bfloat16* p, float* out) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const float2 f = __bfloat1622float2(h[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}
template <typename T, int N> FT_DEVICE void store_vec(T* p, const float* in);
template <> FT_DEVICE void store_vec<float, 4>(float* p, const float* in) { *reinterpret_cast<float4*>(p) = make_float4(in[0], in[1], in[2], in[3]); }
template <> FT_DEVICE void store_vec<__nv_bfloat16, 8>(__nv_bfloat16* p, const float* in) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; i++) h[i] = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = v;
}

// ---- column sums over [M, C]: MODE 0: (sum x, sum x^2); MODE 1: (sum dy', sum dy' * xhat) with dy' = relu-masked dy ---------------------
// block = 256 threads = TXW column-groups x (256 / TXW) row lanes; grid = (C / VEC / TXW, row blocks). partial: [gridDim.y][2][C].
// The last CTA of every column block (arrival counter, self-resetting) adds the partials in block order and writes sums[2][C], so the result is
// bit-stable and no second launch is needed. The counters are one static array per device: statistics launches on one device must not overlap.
__device__ unsigned int g_col_counters[512];

template <typename T, int MODE>
__global__ void __launch_bounds__(256) col_stats_kernel(const T* __restrict__ a, const T* __restrict__ x, const T* __restrict__ y, const float* __restrict__ mean,
                                                        const float* __restrict__ invstd, size_t M, int C, int txw, float* __restrict__ partial,
                                                        float* __restrict__ sums) {
  constexpr int N = VecT<T>::N;
  extern __shared__ float sm[];                        // [2][rows_lanes][txw * N]
  __shared__ int is_last;
  const int tx = threadIdx.x % txw, ty = threadIdx.x / txw, tyn = 256 / txw;
  const int c0 = (blockIdx.x * txw + tx) * N;
  float s0[N], s1[N], mu[N], is[N];
#pragma unroll
  for (int e = 0; e < N; e++) {
    s0[e] = s1[e] = 0.f;
    mu[e] = (MODE == 1) ? mean[c0 + e] : 0.f;
    is[e] = (MODE == 1) ? invstd[c0 + e] : 0.f;
  }
  for (size_t r = (size_t)blockIdx.y * tyn + ty; r < M; r += (size_t)gridDim.y * tyn) {
    float v[N];
    load_vec<T, N>(a + r * C + c0, v);
    if (MODE == 0) {
#pragma unroll
      for (int e = 0; e < N; e++) { s0[e] += v[e]; s1[e] += v[e] * v[e]; }
    } else {
      float xv[N];
      load_vec<T, N>(x + r * C + c0, xv);
      if (y) {
        float yv[N];
        load_vec<T, N>(y + r * C + c0, yv);
#pragma unroll
        for (int e = 0; e < N; e++) if (!(yv[e] > 0.f)) v[e] = 0.f;
      }
#pragma unroll
      for (int e = 0; e < N; e++) { s0[e] += v[e]; s1[e] += v[e] * (xv[e] - mu[e]) * is[e]; }
    }
  }
  const int W = txw * N;
  float* sm0 = sm;
  float* sm1 = sm + tyn * W;
#pragma unroll
  for (int e = 0; e < N; e++) { sm0[ty * W + tx * N + e] = s0[e]; sm1[ty * W + tx * N + e] = s1[e]; }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * W; i += 256) {
    const int which = i / W, c = i % W;
    const float* src = which ? sm1 : sm0;
    float acc = 0.f;
    for (int k = 0; k < tyn; k++) acc += src[k * W + c];
    partial[((size_t)blockIdx.y * 2 + which) * C + blockIdx.x * W + c] = acc;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(&g_col_counters[blockIdx.x], 1u);
    is_last = prev == gridDim.y - 1;
    if (is_last) g_col_counters[blockIdx.x] = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // 2 * W (which, column) pairs; the 256 threads split the block range of every pair into 256 / (2 W) slices (>= 1), combined in slice order
  const int pairs = 2 * W, slices = pairs >= 256 ? 1 : 256 / pairs, nblk = gridDim.y;
  float* red = sm;                                     // [slices][pairs] (fits: slices * pairs <= 256 floats, or pairs when slices == 1)
  for (int i = threadIdx.x; i < pairs * slices; i += 256) {
    const int pr = i % pairs, sl = i / pairs, which = pr / W, c = pr % W;
    const int k0 = (int)((long long)nblk * sl / slices), k1 = (int)((long long)nblk * (sl + 1) / slices);
    float acc = 0.f;
#pragma unroll 8
    for (int k = k0; k < k1; k++) acc += __ldcg(partial + ((size_t)k * 2 + which) * C + blockIdx.x * W + c);
    red[sl * pairs + pr] = acc;
  }
  __syncthreads();
  for (int pr = threadIdx.x; pr < pairs; pr += 256) {
    float acc = 0.f;
    for (int sl = 0; sl < slices; sl++) acc += red[sl * pairs + pr];
    sums[(pr / W) * C + blockIdx.x * W + (pr % W)] = acc;
  }
}

// mean / invstd from (sum, sumsq) over `count` elements per channel; running stats updated with the unbiased variance
__global__ void __launch_bounds__(256) bn_finalize_kernel(const float* __restrict__ sums, int C, float count, float eps, float momentum, float* __restrict__ mean,
                                                          float* __restrict__ invstd, float* __restrict__ running_mean, float* __restrict__ running_var) {
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= C) return;
  const float m = sums[c] / count;
  const float var = fmaxf(sums[C + c] / count - m * m, 0.f);
  mean[c] = m;
  invstd[c] = rsqrtf(var + eps);
  if (running_mean) running_mean[c] = (1.f - momentum) * running_mean[c] + momentum * m;
  if (running_var) running_var[c] = (1.f - momentum) * running_var[c] + momentum * var * (count > 1.f ? count / (count - 1.f) : 1.f);
}

// y = relu?(x * a + b (+ residual)) with a = invstd * gamma, b = beta - mean * a held in registers: a thread owns one 16-byte channel group and walks
// down the rows (block = TXW groups x 256 / TXW row lanes, as in the statistics kernel), so the per-channel constants are read once per thread.
template <typename T>
__global__ void __launch_bounds__(256) bn_apply_kernel(const T* __restrict__ x, const float* __restrict__ mean, const float* __restrict__ invstd,
                                                       const float* __restrict__ gamma, const float* __restrict__ beta, const T* __restrict__ residual, int relu,
                                                       size_t M, int C, int txw, T* __restrict__ y) {
  constexpr int N = VecT<T>::N;
  const int tx = threadIdx.x % txw, ty = threadIdx.x / txw, tyn = 256 / txw;
  const int c0 = (blockIdx.x * txw + tx) * N;
  float a[N], b[N];
#pragma unroll
  for (int e = 0; e < N; e++) {
    a[e] = invstd[c0 + e] * (gamma ? gamma[c0 + e] : 1.f);
    b[e] = (beta ? beta[c0 + e] : 0.f) - mean[c0 + e] * a[e];
  }
  for (size_t r = (size_t)blockIdx.y * tyn + ty; r < M; r += (size_t)gridDim.y * tyn) {
    float v[N], rs[N];
    load_vec<T, N>(x + r * C + c0, v);
    if (residual) load_vec<T, N>(residual + r * C + c0, rs);
#pragma unroll
    for (int e = 0; e < N; e++) {
      float o = v[e] * a[e] + b[e];
      if (residual) o += rs[e];
      v[e] = relu ? fmaxf(o, 0.f) : o;
    }
    store_vec<T, N>(y + r * C + c0, v);
  }
}

// dx = gamma * invstd * (dy' - sum_dy / count - xhat * sum_dy_xhat / count); dres = dy' (the residual branch's gradient), both optional ReLU-masked
template <typename T>
__global__ void __launch_bounds__(256) bn_bwd_apply_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ y, const float* __restrict__ mean,
                                                           const float* __restrict__ invstd, const float* __restrict__ gamma, const float* __restrict__ sums, float count,
                                                           size_t M, int C, int txw, T* __restrict__ dx, T* __restrict__ dres) {
  constexpr int N = VecT<T>::N;
  const int tx = threadIdx.x % txw, ty = threadIdx.x / txw, tyn = 256 / txw;
  const int c0 = (blockIdx.x * txw + tx) * N;
  const float inv_count = 1.f / count;
  float k1[N], k2[N], k3[N], mu[N], is[N];
#pragma unroll
  for (int e = 0; e < N; e++) {
    const int c = c0 + e;
    mu[e] = mean[c];
    is[e] = invstd[c];
    k1[e] = (gamma ? gamma[c] : 1.f) * is[e];
    k2[e] = sums[c] * inv_count;
    k3[e] = sums[C + c] * inv_count;
  }
  for (size_t r = (size_t)blockIdx.y * tyn + ty; r < M; r += (size_t)gridDim.y * tyn) {
    float g[N], xv[N], yv[N], o[N];
    load_vec<T, N>(dy + r * C + c0, g);
    load_vec<T, N>(x + r * C + c0, xv);
    if (y) {
      load_vec<T, N>(y + r * C + c0, yv);
#pragma unroll
      for (int e = 0; e < N; e++) if (!(yv[e] > 0.f)) g[e] = 0.f;
    }
#pragma unroll
    for (int e = 0; e < N; e++) o[e] = k1[e] * (g[e] - k2[e] - (xv[e] - mu[e]) * is[e] * k3[e]);
    store_vec<T, N>(dx + r * C + c0, o);
    if (dres) store_vec<T, N>(dres + r * C + c0, g);
  }
}

// ---- max pooling, NHWC -----------------------------------------------------------------------------------------------------------------
// forward: a thread handles one 16-byte channel group of one output pixel; it also records, per channel, which window position (dh * k + dw, first
// maximum in row-major order) won, so the backward never re-reads the input.
template <typename T>
__global__ void __launch_bounds__(256) maxpool_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, uint8_t* __restrict__ idx, int Nb, int H, int W, int C, int Ho, int Wo,
                                                          int k, int s, int p) {
  constexpr int N = VecT<T>::N;
  const size_t total = (size_t)Nb * Ho * Wo * (C / N);
  for (size_t i = blockIdx.x * (size_t)256 + threadIdx.x; i < total; i += (size_t)gridDim.x * 256) {
    const int cg = (int)(i % (C / N));
    size_t r = i / (C / N);
    const int wo = (int)(r % Wo);
    r /= Wo;
    const int ho = (int)(r % Ho), n = (int)(r / Ho);
    float m[N];
    uint8_t am[N];
#pragma unroll
    for (int e = 0; e < N; e++) { m[e] = -CUDART_INF_F; am[e] = 0; }
    for (int dh = 0; dh < k; dh++) {
      const int h = ho * s - p + dh;
      if (h < 0 || h >= H) continue;
      for (int dw = 0; dw < k; dw++) {
        const int w = wo * s - p + dw;
        if (w < 0 || w >= W) continue;
        float v[N];
        load_vec<T, N>(x + (((size_t)n * H + h) * W + w) * C + cg * N, v);
#pragma unroll
        for (int e = 0; e < N; e++)
          if (v[e] > m[e] || (v[e] != v[e] && m[e] == m[e])) { m[e] = v[e]; am[e] = (uint8_t)(dh * k + dw); }
      }
    }
    store_vec<T, N>(y + i * N, m);
    if (idx) {
#pragma unroll
      for (int e = 0; e < N; e++) idx[i * N + e] = am[e];
    }
  }
}

// backward from the recorded positions: a thread owns one channel group of one INPUT pixel and visits the (at most ceil(k/s)^2) windows that contain it
template <typename T>
__global__ void __launch_bounds__(256) maxpool_bwd_kernel(const uint8_t* __restrict__ idx, const T* __restrict__ dy, T* __restrict__ dx, int Nb, int H, int W, int C, int Ho,
                                                          int Wo, int k, int s, int p) {
  constexpr int N = VecT<T>::N;
  const size_t total = (size_t)Nb * H * W * (C / N);
  for (size_t i = blockIdx.x * (size_t)256 + threadIdx.x; i < total; i += (size_t)gridDim.x * 256) {
    const int cg = (int)(i % (C / N));
    size_t r = i / (C / N);
    const int w = (int)(r % W);
    r /= W;
    const int h = (int)(r % H), n = (int)(r / H);
    float acc[N];
#pragma unroll
    for (int e = 0; e < N; e++) acc[e] = 0.f;
    const int ho_lo = max(0, (h + p - k + s) / s), ho_hi = min(Ho - 1, (h + p) / s);
    const int wo_lo = max(0, (w + p - k + s) / s), wo_hi = min(Wo - 1, (w + p) / s);
    for (int ho = ho_lo; ho <= ho_hi; ho++)
      for (int wo = wo_lo; wo <= wo_hi; wo++) {
        const int want = (h - (ho * s - p)) * k + (w - (wo * s - p));
        const size_t o = (((size_t)n * Ho + ho) * Wo + wo) * C + cg * N;
        uint8_t am[N];
        if (N == 8) *reinterpret_cast<uint2*>(am) = *reinterpret_cast<const uint2*>(idx + o);
        else *reinterpret_cast<uint32_t*>(am) = *reinterpret_cast<const uint32_t*>(idx + o);
        float g[N];
        load_vec<T, N>(dy + o, g);
#pragma unroll
        for (int e = 0; e < N; e++)
          if (am[e] == want) acc[e] += g[e];
      }
    store_vec<T, N>(dx + i * N, acc);
  }
}

// ---- group norm, NCHW: one CTA per (n, g); the group's (C/G) * HW elements are contiguous -------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) group_norm_fwd_kernel(const T* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta, T* __restrict__ y,
                                                             float* __restrict__ mean_out, float* __restrict__ rstd_out, int C, int G, size_t HW, float eps) {
  __shared__ float red[8];
  const int n = blockIdx.x / G, g = blockIdx.x % G, cpg = C / G;
  const size_t len = (size_t)cpg * HW, base = ((size_t)n * C + (size_t)g * cpg) * HW;
  float s = 0.f, ss = 0.f;
  for (size_t i = threadIdx.x; i < len; i += 256) {
    const float v = (float)x[base + i];
    s += v;
    ss += v * v;
  }
  s = block_sum(s, red);
  ss = block_sum(ss, red);
  const float mu = s / (float)len, rstd = rsqrtf(fmaxf(ss / (float)len - mu * mu, 0.f) + eps);
  if (threadIdx.x == 0) { mean_out[blockIdx.x] = mu; rstd_out[blockIdx.x] = rstd; }
  for (size_t i = threadIdx.x; i < len; i += 256) {
    const int c = g * cpg + (int)(i / HW);
    y[base + i] = (T)(((float)x[base + i] - mu) * rstd * (gamma ? gamma[c] : 1.f) + (beta ? beta[c] : 0.f));
  }
}

// dx for one (n, g); dgamma / dbeta partials accumulate with atomics into f32 [C] (zeroed by the caller)
template <typename T>
__global__ void __launch_bounds__(256) group_norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ mean,
                                                             const float* __restrict__ rstd, T* __restrict__ dx, float* __restrict__ dgamma, float* __restrict__ dbeta,
                                                             int C, int G, size_t HW) {
  __shared__ float red[8];
  const int n = blockIdx.x / G, g = blockIdx.x % G, cpg = C / G;
  const size_t len = (size_t)cpg * HW, base = ((size_t)n * C + (size_t)g * cpg) * HW;
  const float mu = mean[blockIdx.x], rs = rstd[blockIdx.x];
  float s1 = 0.f, s2 = 0.f;                                                   // sum dy*gamma, sum dy*gamma*xhat
  for (int cc = 0; cc < cpg; cc++) {
    const int c = g * cpg + cc;
    const float gm = gamma ? gamma[c] : 1.f;
    float a = 0.f, b = 0.f;
    for (size_t i = threadIdx.x; i < HW; i += 256) {
      const float d = (float)dy[base + cc * HW + i], xh = ((float)x[base + cc * HW + i] - mu) * rs;
      a += d;
      b += d * xh;
    }
    a = block_sum(a, red);
    b = block_sum(b, red);
    if (threadIdx.x == 0) {
      if (dbeta) atomicAdd(dbeta + c, a);
      if (dgamma) atomicAdd(dgamma + c, b);
    }
    s1 += a * gm;
    s2 += b * gm;
  }
  const float inv = 1.f / (float)len;
  for (size_t i = threadIdx.x; i < len; i += 256) {
    const int c = g * cpg + (int)(i / HW);
    const float gm = gamma ? gamma[c] : 1.f;
    const float xh = ((float)x[base + i] - mu) * rs;
    dx[base + i] = (T)(rs * ((float)dy[base + i] * gm - s1 * inv - xh * s2 * inv));
  }
}

// ---- recurrent cells ----------------------------------------------------------------------------------------------------------------------
FT_DEVICE float sigm(float v) { return 1.f / (1.f + __expf(-v)); }

// gates [B, 4H] = W x + U h + b in order (i, f, g, o); writes h, c and the activated gates (for the backward)
__global__ void __launch_bounds__(256) lstm_cell_fwd_kernel(const float* __restrict__ gates, const float* __restrict__ c_prev, float* __restrict__ h, float* __restrict__ c,
                                                            float* __restrict__ act, int B, int H) {
  const size_t i = blockIdx.x * (size_t)256 + threadIdx.x;
  if (i >= (size_t)B * H) return;
  const size_t b = i / H, j = i % H;
  const float* gp = gates + b * 4 * H;
  const float ig = sigm(gp[j]), fg = sigm(gp[H + j]), gg = tanhf(gp[2 * H + j]), og = sigm(gp[3 * H + j]);
  const float cn = fg * c_prev[i] + ig * gg;
  c[i] = cn;
  h[i] = og * tanhf(cn);
  if (act) {
    float* ap = act + b * 4 * H;
    ap[j] = ig; ap[H + j] = fg; ap[2 * H + j] = gg; ap[3 * H + j] = og;
  }
}
__global__ void __launch_bounds__(256) lstm_cell_bwd_kernel(const float* __restrict__ dh, const float* __restrict__ dc, const float* __restrict__ act,
                                                            const float* __restrict__ c_prev, const float* __restrict__ c, float* __restrict__ dgates,
                                                            float* __restrict__ dc_prev, int B, int H) {
  const size_t i = blockIdx.x * (size_t)256 + threadIdx.x;
  if (i >= (size_t)B * H) return;
  const size_t b = i / H, j = i % H;
  const float* ap = act + b * 4 * H;
  const float ig = ap[j], fg = ap[H + j], gg = ap[2 * H + j], og = ap[3 * H + j];
  const float tc = tanhf(c[i]);
  const float dcn = (dc ? dc[i] : 0.f) + (dh ? dh[i] : 0.f) * og * (1.f - tc * tc);
  float* dg = dgates + b * 4 * H;
  dg[j] = dcn * gg * ig * (1.f - ig);
  dg[H + j] = dcn * c_prev[i] * fg * (1.f - fg);
  dg[2 * H + j] = dcn * ig * (1.f - gg * gg);
  dg[3 * H + j] = (dh ? dh[i] : 0.f) * tc * og * (1.f - og);
  dc_prev[i] = dcn * fg;
}

// gi = W x + b_i, gh = U h + b_h, both [B, 3H] in order (r, z, n): h' = (1 - z) * n + z * h, n = tanh(gi_n + r * gh_n)
__global__ void __launch_bounds__(256) gru_cell_fwd_kernel(const float* __restrict__ gi, const float* __restrict__ gh, const float* __restrict__ h_prev, float* __restrict__ h,
                                                           float* __restrict__ act, int B, int H) {
  const size_t i = blockIdx.x * (size_t)256 + threadIdx.x;
  if (i >= (size_t)B * H) return;
  const size_t b = i / H, j = i % H;
  const float* a = gi + b * 3 * H;
  const float* u = gh + b * 3 * H;
  const float r = sigm(a[j] + u[j]), z = sigm(a[H + j] + u[H + j]);
  const float hn = u[2 * H + j], nn = tanhf(a[2 * H + j] + r * hn);
  h[i] = (1.f - z) * nn + z * h_prev[i];
  if (act) {
    float* ap = act + b * 4 * H;
    ap[j] = r; ap[H + j] = z; ap[2 * H + j] = nn; ap[3 * H + j] = hn;
  }
}
__global__ void __launch_bounds__(256) gru_cell_bwd_kernel(const float* __restrict__ dh, const float* __restrict__ act, const float* __restrict__ h_prev, float* __restrict__ dgi,
                                                           float* __restrict__ dgh, float* __restrict__ dh_prev, int B, int H) {
  const size_t i = blockIdx.x * (size_t)256 + threadIdx.x;
  if (i >= (size_t)B * H) return;
  const size_t b = i / H, j = i % H;
  const float* ap = act + b * 4 * H;
  const float r = ap[j], z = ap[H + j], nn = ap[2 * H + j], hn = ap[3 * H + j], g = dh[i];
  const float dn = g * (1.f - z) * (1.f - nn * nn);
  const float dz = g * (h_prev[i] - nn) * z * (1.f - z);
  const float dr = dn * hn * r * (1.f - r);
  float* a = dgi + b * 3 * H;
  float* u = dgh + b * 3 * H;
  a[j] = dr; a[H + j] = dz; a[2 * H + j] = dn;
  u[j] = dr; u[H + j] = dz; u[2 * H + j] = dn * r;
  dh_prev[i] = g * z;
}

inline int grid_for(size_t work) {
  const size_t g = (work + 255) / 256;
  return (int)(g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g));
}

// grid of the column-resident apply kernels: x = column-group blocks, y = row blocks (about 16 CTAs per SM in total, bounded by the rows)
inline dim3 apply_grid(int64_t M, int C, int vec, int& txw) {
  const int groups = C / vec;
  txw = 32;
  while (txw > 1 && groups % txw) txw >>= 1;
  const int gx = groups / txw, tyn = 256 / txw;
  int64_t gy = (148 * 16 + gx - 1) / gx;
  const int64_t maxy = (M + tyn - 1) / tyn;
  gy = gy > maxy ? maxy : gy;
  if (gy > 65535) gy = 65535;
  return dim3((unsigned)gx, (unsigned)(gy < 1 ? 1 : gy));
}

template <typename T, int MODE>
int col_stats_launch(const T* a, const T* x, const T* y, const float* mean, const float* invstd, size_t M, int C, float* partial, float* sums, int nblk, cudaStream_t st) {
  constexpr int N = VecT<T>::N;
  if (C % N) return FT_ERR_ARG;
  const int groups = C / N;
  int txw = 32;
  while (txw > 1 && groups % txw) txw >>= 1;
  const size_t smem = 2 * (size_t)(256 / txw) * txw * N * sizeof(float);
  if (groups / txw > 512) return FT_ERR_TOO_LARGE;
  size_t smem_need = smem < 256 * sizeof(float) ? 256 * sizeof(float) : smem;
  col_stats_kernel<T, MODE><<<dim3(groups / txw, nblk), 256, smem_need, st>>>(a, x, y, mean, invstd, M, C, txw, partial, sums);
  return (int)cudaGetLastError();
}

}  // namespace

// Row blocks the statistics kernels use for an [M, C] activation: partial buffers hold nblk * 2 * C floats.
FT_EXPORT int ft_bn_num_blocks(int64_t M, int C, int elem_bytes) {
  const int vec = elem_bytes == 2 ? 8 : 4;
  int txw = 32;
  while (txw > 1 && (C / vec) % txw) txw >>= 1;
  const int gx = C / vec / txw;
  int64_t nb = (148 * 2 + gx - 1) / (gx < 1 ? 1 : gx);
  const int64_t rows_per = 256 / txw;
  const int64_t maxb = (M + rows_per - 1) / rows_per;
  nb = nb > maxb ? maxb : nb;
  return (int)(nb < 1 ? 1 : nb);
}

// sums[2][C] = (sum x, sum x^2) over the M rows. bf16: is_bf16 = 1, else f32. partial: ft_bn_num_blocks(...) * 2 * C floats of scratch.
FT_EXPORT int ft_bn_stats(int is_bf16, const void* x, int64_t M, int C, float* partial, float* sums, cudaStream_t st) {
  if (M < 1 || C < 1) return FT_ERR_ARG;
  const int nblk = ft_bn_num_blocks(M, C, is_bf16 ? 2 : 4);
  return is_bf16 ? col_stats_launch<__nv_bfloat16, 0>((const __nv_bfloat16*)x, nullptr, nullptr, nullptr, nullptr, (size_t)M, C, partial, sums, nblk, st)
                 : col_stats_launch<float, 0>((const float*)x, nullptr, nullptr, nullptr, nullptr, (size_t)M, C, partial, sums, nblk, st);
}

// mean / invstd from sums over `count` elements per channel (count = M * world for SyncBatchNorm after the sums were all-reduced).
FT_EXPORT int ft_bn_finalize(const float* sums, int C, double count, float eps, float momentum, float* mean, float* invstd, float* running_mean, float* running_var,
                             cudaStream_t st) {
  bn_finalize_kernel<<<(C + 255) / 256, 256, 0, st>>>(sums, C, (float)count, eps, momentum, mean, invstd, running_mean, running_var);
  return (int)cudaGetLastError();
}

// y = relu?((x - mean) * invstd * gamma + beta (+ residual)); gamma / beta / residual may be null.
FT_EXPORT int ft_bn_apply(int is_bf16, const void* x, const float* mean, const float* invstd, const float* gamma, const float* beta, const void* residual, int relu,
                          int64_t M, int C, void* y, cudaStream_t st) {
  if (C % (is_bf16 ? 8 : 4)) return FT_ERR_ARG;
  int txw;
  const dim3 grid = apply_grid(M, C, is_bf16 ? 8 : 4, txw);
  if (is_bf16) bn_apply_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, mean, invstd, gamma, beta, (const __nv_bfloat16*)residual, relu, (size_t)M, C, txw, (__nv_bfloat16*)y);
  else bn_apply_kernel<float><<<grid, 256, 0, st>>>((const float*)x, mean, invstd, gamma, beta, (const float*)residual, relu, (size_t)M, C, txw, (float*)y);
  return (int)cudaGetLastError();
}

// sums[2][C] = (sum dy', sum dy' * xhat), dy' = dy masked by (y > 0) when y is given (fused ReLU). These are also dbeta and dgamma.
FT_EXPORT int ft_bn_bwd_stats(int is_bf16, const void* dy, const void* x, const void* y, const float* mean, const float* invstd, int64_t M, int C, float* partial,
                              float* sums, cudaStream_t st) {
  const int nblk = ft_bn_num_blocks(M, C, is_bf16 ? 2 : 4);
  return is_bf16 ? col_stats_launch<__nv_bfloat16, 1>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)y, mean, invstd, (size_t)M, C, partial, sums, nblk, st)
                 : col_stats_launch<float, 1>((const float*)dy, (const float*)x, (const float*)y, mean, invstd, (size_t)M, C, partial, sums, nblk, st);
}

FT_EXPORT int ft_bn_bwd_apply(int is_bf16, const void* dy, const void* x, const void* y, const float* mean, const float* invstd, const float* gamma, const float* sums,
                              double count, int64_t M, int C, void* dx, void* dres, cudaStream_t st) {
  if (C % (is_bf16 ? 8 : 4)) return FT_ERR_ARG;
  int txw;
  const dim3 grid = apply_grid(M, C, is_bf16 ? 8 : 4, txw);
  if (is_bf16) bn_bwd_apply_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)y, mean, invstd, gamma, sums, (float)count, (size_t)M, C, txw, (__nv_bfloat16*)dx, (__nv_bfloat16*)dres);
  else bn_bwd_apply_kernel<float><<<grid, 256, 0, st>>>((const float*)dy, (const float*)x, (const float*)y, mean, invstd, gamma, sums, (float)count, (size_t)M, C, txw, (float*)dx, (float*)dres);
  return (int)cudaGetLastError();
}

// idx (optional, u8 [N, Ho, Wo, C]): winning window position of every output element, consumed by ft_maxpool2d_nhwc_bwd. k * k <= 255.
FT_EXPORT int ft_maxpool2d_nhwc(int is_bf16, const void* x, void* y, void* idx, int N, int H, int W, int C, int k, int s, int p, cudaStream_t st) {
  const int Ho = (H + 2 * p - k) / s + 1, Wo = (W + 2 * p - k) / s + 1;
  if (C % (is_bf16 ? 8 : 4) || Ho < 1 || Wo < 1 || p >= k || k * k > 255) return FT_ERR_ARG;
  const size_t total = (size_t)N * Ho * Wo * (C / (is_bf16 ? 8 : 4));
  if (is_bf16) maxpool_fwd_kernel<__nv_bfloat16><<<grid_for(total), 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, (uint8_t*)idx, N, H, W, C, Ho, Wo, k, s, p);
  else maxpool_fwd_kernel<float><<<grid_for(total), 256, 0, st>>>((const float*)x, (float*)y, (uint8_t*)idx, N, H, W, C, Ho, Wo, k, s, p);
  return (int)cudaGetLastError();
}

FT_EXPORT int ft_maxpool2d_nhwc_bwd(int is_bf16, const void* idx, const void* dy, void* dx, int N, int H, int W, int C, int k, int s, int p, cudaStream_t st) {
  const int Ho = (H + 2 * p - k) / s + 1, Wo = (W + 2 * p - k) / s + 1;
  if (C % (is_bf16 ? 8 : 4) || Ho < 1 || Wo < 1 || p >= k || !idx) return FT_ERR_ARG;
  const size_t total = (size_t)N * H * W * (C / (is_bf16 ? 8 : 4));
  if (is_bf16) maxpool_bwd_kernel<__nv_bfloat16><<<grid_for(total), 256, 0, st>>>((const uint8_t*)idx, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dx, N, H, W, C, Ho, Wo, k, s, p);
  else maxpool_bwd_kernel<float><<<grid_for(total), 256, 0, st>>>((const uint8_t*)idx, (const float*)dy, (float*)dx, N, H, W, C, Ho, Wo, k, s, p);
  return (int)cudaGetLastError();
}

FT_EXPORT int ft_group_norm_fwd(int is_bf16, const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd, int N, int C, int G, int64_t HW,
                                float eps, cudaStream_t st) {
  if (G < 1 || C % G) return FT_ERR_ARG;
  if (is_bf16) group_norm_fwd_kernel<__nv_bfloat16><<<N * G, 256, 0, st>>>((const __nv_bfloat16*)x, gamma, beta, (__nv_bfloat16*)y, mean, rstd, C, G, (size_t)HW, eps);
  else group_norm_fwd_kernel<float><<<N * G, 256, 0, st>>>((const float*)x, gamma, beta, (float*)y, mean, rstd, C, G, (size_t)HW, eps);
  return (int)cudaGetLastError();
}

// dgamma / dbeta: f32 [C], zeroed by the caller (accumulated with atomics across samples).
FT_EXPORT int ft_group_norm_bwd(int is_bf16, const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd, void* dx, float* dgamma,
                                float* dbeta, int N, int C, int G, int64_t HW, cudaStream_t st) {
  if (G < 1 || C % G) return FT_ERR_ARG;
  if (is_bf16) group_norm_bwd_kernel<__nv_bfloat16><<<N * G, 256, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, gamma, mean, rstd, (__nv_bfloat16*)dx, dgamma, dbeta, C, G, (size_t)HW);
  else group_norm_bwd_kernel<float><<<N * G, 256, 0, st>>>((const float*)dy, (const float*)x, gamma, mean, rstd, (float*)dx, dgamma, dbeta, C, G, (size_t)HW);
  return (int)cudaGetLastError();
}

FT_EXPORT int ft_lstm_cell_fwd(const float* gates, const float* c_prev, float* h, float* c, float* act, int B, int H, cudaStream_t st) {
  lstm_cell_fwd_kernel<<<(unsigned)(((size_t)B * H + 255) / 256), 256, 0, st>>>(gates, c_prev, h, c, act, B, H);
  return (int)cudaGetLastError();
}
FT_EXPORT int ft_lstm_cell_bwd(const float* dh, const float* dc, const float* act, const float* c_prev, const float* c, float* dgates, float* dc_prev, int B, int H,
                               cudaStream_t st) {
  lstm_cell_bwd_kernel<<<(unsigned)(((size_t)B * H + 255) / 256), 256, 0, st>>>(dh, dc, act, c_prev, c, dgates, dc_prev, B, H);
  return (int)cudaGetLastError();
}
FT_EXPORT int ft_gru_cell_fwd(const float* gi, const float* gh, const float* h_prev, float* h, float* act, int B, int H, cudaStream_t st) {
  gru_cell_fwd_kernel<<<(unsigned)(((size_t)B * H + 255) / 256), 256, 0, st>>>(gi, gh, h_prev, h, act, B, H);
  return (int)cudaGetLastError();
}
FT_EXPORT int ft_gru_cell_bwd(const float* dh, const float* act, const float* h_prev, float* dgi, float* dgh, float* dh_prev, int B, int H, cudaStream_t st) {
  gru_cell_bwd_kernel<<<(unsigned)(((size_t)B * H + 255) / 256), 256, 0, st>>>(dh, act, h_prev, dgi, dgh, dh_prev, B, H);
  return (int)cudaGetLastError();
}
