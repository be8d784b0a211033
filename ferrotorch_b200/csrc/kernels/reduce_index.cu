// Reductions, scans, indexing, random numbers, GGUF block dequantisation and vocabulary masks.
//
// Tensors are viewed as [outer, len, inner]: a reduction / scan runs along `len`; index ops select along `len`.
// Replaces ferrotorch-gpu/src/kernels.rs REDUCE_SUM 5678 / PROD 5784 / MIN 5988 / MAX 6090 / SUM_AXIS 6700 / MASKED_REDUCE 6255,6365,
// CUMSUM 6786 / CUMPROD 6864 / CUMMAX 6942 / CUMMIN 7026 / LOGCUMSUMEXP 7114, INDEX_SELECT 4302-4510 / SCATTER_ADD 4596 / SCATTER_ADD_ROWS 1218,
// DROPOUT 9985 and ferrotorch-gpu/src/rng.rs:557,872 (Philox4x32-10 uniform / Box-Muller normal), HAS_INF_NAN 6205, and restates the dequantisers
// and the token mask of ferrotorch-cubecl/src/quant.rs:330-483,1399 as CUDA kernels.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include "common.cuh"
#include "host_common.h"

namespace {

enum DType : int { DT_F32 = 0, DT_BF16 = 1, DT_F16 = 2, DT_F64 = 3 };
enum RedOp : int { R_SUM = 0, R_PROD, R_MIN, R_MAX, R_MEAN, R_SUMSQ, R_ABSMAX, R_LOGSUMEXP };
enum ScanOp : int { S_SUM = 0, S_PROD, S_MAX, S_MIN, S_LOGSUMEXP };

FT_DEVICE float ldf(const float* p, size_t i) { return p[i]; }
FT_DEVICE float ldf(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }
FT_DEVICE float ldf(const __half* p, size_t i) { return __half2float(p[i]); }
FT_DEVICE double ldf(const double* p, size_t i) { return p[i]; }
FT_DEVICE void stf(float* p, size_t i, float v) { p[i] = v; }
FT_DEVICE void stf(__nv_bfloat16* p, size_t i, float v) { p[i] = __float2bfloat16(v); }
FT_DEVICE void stf(__half* p, size_t i, float v) { p[i] = __float2half(v); }
FT_DEVICE void stf(double* p, size_t i, double v) { p[i] = v; }

template <typename A> FT_DEVICE A red_identity(int op) {
  switch (op) {
    case R_PROD: return (A)1;
    case R_MIN: return (A)CUDART_INF;
    case R_MAX: case R_LOGSUMEXP: return (A)-CUDART_INF;
    default: return (A)0;
  }
}
template <typename A> FT_DEVICE A red_pre(int op, A v) { return op == R_SUMSQ ? v * v : (op == R_ABSMAX ? fabs(v) : v); }
template <typename A> FT_DEVICE A red_combine(int op, A a, A b) {
  switch (op) {
    case R_PROD: return a * b;
    case R_MIN: return (b < a || b != b) ? b : a;
    case R_MAX: case R_ABSMAX: return (b > a || b != b) ? b : a;
    case R_LOGSUMEXP: {
      const A m = a > b ? a : b;
      return m == (A)-CUDART_INF ? m : m + log(exp(a - m) + exp(b - m));
    }
    default: return a + b;
  }
}

template <typename A> FT_DEVICE A warp_reduce(int op, A v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = red_combine<A>(op, v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// inner == 1: one CTA per output row, 128-bit-free generic loads, warp shuffles + smem across warps.
template <typename T, typename A>
__global__ void __launch_bounds__(256) reduce_rows_kernel(int op, const T* __restrict__ x, T* __restrict__ out, size_t len) {
  __shared__ A red[8];
  const T* row = x + (size_t)blockIdx.x * len;
  A acc = red_identity<A>(op);
  for (size_t i = threadIdx.x; i < len; i += 256) acc = red_combine<A>(op, acc, red_pre<A>(op, (A)ldf(row, i)));
  acc = warp_reduce<A>(op, acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    A v = threadIdx.x < 8 ? red[threadIdx.x] : red_identity<A>(op);
    v = warp_reduce<A>(op, v);
    if (threadIdx.x == 0) stf(out, blockIdx.x, op == R_MEAN ? v / (A)len : v);
  }
}

// inner > 1: thread per (outer, inner) column chunk, coalesced along inner; len split across blockDim.y with an smem combine.
template <typename T, typename A>
__global__ void __launch_bounds__(256) reduce_axis_kernel(int op, const T* __restrict__ x, T* __restrict__ out, size_t len, size_t inner) {
  __shared__ A red[8][33];
  const size_t col = blockIdx.x * 32 + threadIdx.x;
  const size_t o = blockIdx.y;
  A acc = red_identity<A>(op);
  if (col < inner)
    for (size_t i = threadIdx.y; i < len; i += 8) acc = red_combine<A>(op, acc, red_pre<A>(op, (A)ldf(x, (o * len + i) * inner + col)));
  red[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && col < inner) {
#pragma unroll
    for (int k = 1; k < 8; k++) acc = red_combine<A>(op, acc, red[k][threadIdx.x]);
    stf(out, o * inner + col, op == R_MEAN ? acc / (A)len : acc);
  }
}

// full reduction of a long vector: stage 1 = per-CTA partials (f32/f64), stage 2 = reduce_rows over the partials
template <typename T, typename A>
__global__ void __launch_bounds__(256) reduce_partial_kernel(int op, const T* __restrict__ x, A* __restrict__ partial, size_t n) {
  __shared__ A red[8];
  A acc = red_identity<A>(op);
  for (size_t i = blockIdx.x * (size_t)256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256) acc = red_combine<A>(op, acc, red_pre<A>(op, (A)ldf(x, i)));
  acc = warp_reduce<A>(op, acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    A v = threadIdx.x < 8 ? red[threadIdx.x] : red_identity<A>(op);
    v = warp_reduce<A>(op, v);
    if (threadIdx.x == 0) partial[blockIdx.x] = v;
  }
}
template <typename T, typename A>
__global__ void __launch_bounds__(256) reduce_final_kernel(int op, const A* __restrict__ partial, int np, T* __restrict__ out, size_t n) {
  __shared__ A red[8];
  const int cop = (op == R_SUMSQ || op == R_MEAN) ? R_SUM : (op == R_ABSMAX ? R_MAX : op);
  A acc = red_identity<A>(cop);
  for (int i = threadIdx.x; i < np; i += 256) acc = red_combine<A>(cop, acc, partial[i]);
  acc = warp_reduce<A>(cop, acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    A v = threadIdx.x < 8 ? red[threadIdx.x] : red_identity<A>(cop);
    v = warp_reduce<A>(cop, v);
    if (threadIdx.x == 0) stf(out, 0, op == R_MEAN ? v / (A)n : v);
  }
}

// ---- scans: one warp per line when inner == 1 (chunked warp scan with carry), thread per column otherwise ------------------------
template <typename A> FT_DEVICE A scan_identity(int op) {
  return op == S_PROD ? (A)1 : (op == S_MAX || op == S_LOGSUMEXP ? (A)-CUDART_INF : (op == S_MIN ? (A)CUDART_INF : (A)0));
}
template <typename A> FT_DEVICE A scan_combine(int op, A a, A b) {
  switch (op) {
    case S_PROD: return a * b;
    case S_MAX: return (b > a || b != b) ? b : a;
    case S_MIN: return (b < a || b != b) ? b : a;
    case S_LOGSUMEXP: {
      const A m = a > b ? a : b;
      return m == (A)-CUDART_INF ? m : m + log(exp(a - m) + exp(b - m));
    }
    default: return a + b;
  }
}

template <typename T, typename A>
__global__ void __launch_bounds__(128) scan_rows_kernel(int op, const T* __restrict__ x, T* __restrict__ out, size_t rows, size_t len, int reverse) {
  const size_t r = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
  const T* src = x + r * len;
  T* dst = out + r * len;
  A carry = scan_identity<A>(op);
  for (size_t base = 0; base < len; base += 32) {
    const size_t i = base + lane;
    const size_t pos = reverse ? len - 1 - i : i;
    A v = i < len ? (A)ldf(src, pos) : scan_identity<A>(op);
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const A u = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v = scan_combine<A>(op, u, v);
    }
    v = scan_combine<A>(op, carry, v);
    if (i < len) stf(dst, pos, v);
    carry = __shfl_sync(0xffffffffu, v, 31);
  }
}

template <typename T, typename A>
__global__ void __launch_bounds__(256) scan_axis_kernel(int op, const T* __restrict__ x, T* __restrict__ out, size_t outer, size_t len, size_t inner, int reverse) {
  const size_t id = blockIdx.x * (size_t)256 + threadIdx.x;
  if (id >= outer * inner) return;
  const size_t o = id / inner, c = id % inner;
  A acc = scan_identity<A>(op);
  for (size_t k = 0; k < len; k++) {
    const size_t i = reverse ? len - 1 - k : k;
    const size_t off = (o * len + i) * inner + c;
    acc = scan_combine<A>(op, acc, (A)ldf(x, off));
    stf(out, off, acc);
  }
}

// ---- indexing ----------------------------------------------------------------------------------------------------------------------
// out[o, j, :] = src[o, idx[j], :]   (index_select / embedding lookup); 16-byte row copies when inner bytes allow
template <typename T>
__global__ void __launch_bounds__(256) index_select_kernel(const T* __restrict__ src, const int64_t* __restrict__ idx, T* __restrict__ out, size_t outer,
                                                           size_t src_len, size_t n_idx, size_t inner, uint32_t* status) {
  const size_t total = outer * n_idx * inner;
  for (size_t i = blockIdx.x * (size_t)256 + threadIdx.x; i < total; i += (size_t)gridDim.x * 256) {
    const size_t c = i % inner, j = (i / inner) % n_idx, o = i / (inner * n_idx);
    int64_t s = idx[j];
    if (s < 0) s += (int64_t)src_len;
    if (s < 0 || s >= (int64_t)src_len) {
      ft_set_status(status, 0x21, 1, (uint32_t)j);
      out[i] = T(0);
      continue;
    }
    out[i] = src[(o * src_len + (size_t)s) * inner + c];
  }
}

// dst[o, idx[j], :] += src[o, j, :]  (f32 atomics; the embedding / index_select backward)
__global__ void __launch_bounds__(256) index_add_kernel(float* __restrict__ dst, const int64_t* __restrict__ idx, const float* __restrict__ src, size_t outer,
                                                        size_t dst_len, size_t n_idx, size_t inner, uint32_t* status) {
  const size_t total = outer * n_idx * inner;
  for (size_t i = blockIdx.x * (size_t)256 + threadIdx.x; i < total; i += (size_t)gridDim.x * 256) {
    const size_t c = i % inner, j = (i / inner) % n_idx, o = i / (inner * n_idx);
    int64_t s = idx[j];
    if (s < 0) s += (int64_t)dst_len;
    if (s < 0 || s >= (int64_t)dst_len) {
      ft_set_status(status, 0x22, 1, (uint32_t)j);
      continue;
    }
    atomicAdd(dst + (o * dst_len + (size_t)s) * inner + c, src[i]);
  }
}

// gather along len: out[o, j, c] = src[o, idx[o, j, c], c]; scatter_add is the transpose
template <typename T, bool SCATTER>
__global__ void __launch_bounds__(256) gather_scatter_kernel(T* __restrict__ a, const int64_t* __restrict__ idx, T* __restrict__ b, size_t outer, size_t a_len,
                                                             size_t n_idx, size_t inner, uint32_t* status) {
  const size_t total = outer * n_idx * inner;
  for (size_t i = blockIdx.x * (size_t)256 + threadIdx.x; i < total; i += (size_t)gridDim.x * 256) {
    const size_t c = i % inner, o = i / (inner * n_idx);
    int64_t s = idx[i];
    if (s < 0) s += (int64_t)a_len;
    if (s < 0 || s >= (int64_t)a_len) {
      ft_set_status(status, 0x23, 1, (uint32_t)i);
      continue;
    }
    const size_t off = (o * a_len + (size_t)s) * inner + c;
    if (SCATTER) atomicAdd(reinterpret_cast<float*>(a) + off, reinterpret_cast<const float*>(b)[i]);
    else b[i] = a[off];
  }
}

// ---- Philox4x32-10 -------------------------------------------------------------------------------------------------------------------
struct Philox {
  uint32_t key[2];
  FT_DEVICE static void mulhilo(uint32_t a, uint32_t b, uint32_t& hi, uint32_t& lo) {
    const uint64_t p = (uint64_t)a * b;
    hi = (uint32_t)(p >> 32);
    lo = (uint32_t)p;
  }
  FT_DEVICE uint4 operator()(uint64_t counter, uint64_t subsequence) const {
    uint32_t c0 = (uint32_t)counter, c1 = (uint32_t)(counter >> 32), c2 = (uint32_t)subsequence, c3 = (uint32_t)(subsequence >> 32);
    uint32_t k0 = key[0], k1 = key[1];
#pragma unroll
    for (int r = 0; r < 10; r++) {
      uint32_t h0, l0, h1, l1;
      mulhilo(0xD2511F53u, c0, h0, l0);
      mulhilo(0xCD9E8D57u, c2, h1, l1);
      const uint32_t n0 = h1 ^ c1 ^ k0, n1 = l1, n2 = h0 ^ c3 ^ k1, n3 = l0;
      c0 = n0; c1 = n1; c2 = n2; c3 = n3;
      k0 += 0x9E3779B9u;
      k1 += 0xBB67AE85u;
    }
    return make_uint4(c0, c1, c2, c3);
  }
};
FT_DEVICE float u01(uint32_t r) { return ((float)(r >> 8) + 0.5f) * (1.0f / 16777216.0f); }     // (0, 1)

// element i uses counter = offset + i / 4, lane i % 4: the stream is a pure function of (seed, offset, i), so replay after a checkpoint matches
template <typename T, int MODE>   // 0 uniform[lo, hi), 1 normal(mean, std), 2 dropout(x, p) with mask out
__global__ void __launch_bounds__(256) philox_kernel(T* __restrict__ out, const T* __restrict__ x, uint8_t* __restrict__ mask, size_t n, uint64_t seed,
                                                     uint64_t offset, float a, float b) {
  Philox ph;
  ph.key[0] = (uint32_t)seed;
  ph.key[1] = (uint32_t)(seed >> 32);
  const size_t ngroups = (n + 3) / 4;
  for (size_t gidx = blockIdx.x * (size_t)256 + threadIdx.x; gidx < ngroups; gidx += (size_t)gridDim.x * 256) {
    const uint4 r = ph(offset + gidx, 0);
    const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
    float v[4];
    if (MODE == 1) {
#pragma unroll
      for (int k = 0; k < 4; k += 2) {
        const float u1 = u01(rr[k]), u2 = u01(rr[k + 1]);
        const float rad = sqrtf(-2.f * logf(u1));
        v[k] = rad * cosf(6.283185307179586f * u2) * b + a;
        v[k + 1] = rad * sinf(6.283185307179586f * u2) * b + a;
      }
    } else {
#pragma unroll
      for (int k = 0; k < 4; k++) v[k] = u01(rr[k]);
    }
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const size_t i = gidx * 4 + k;
      if (i >= n) break;
      if (MODE == 0) stf(out, i, a + (b - a) * v[k]);
      else if (MODE == 1) stf(out, i, v[k]);
      else {
        const bool keep = v[k] >= a;                     // a = drop probability
        if (mask) mask[i] = keep;
        stf(out, i, keep ? (float)ldf(x, i) * b : 0.f);  // b = 1 / (1 - p)
      }
    }
  }
}

// ---- non-finite check + unscale over a list of tensors --------------------------------------------------------------------------------
struct TensorList {
  static constexpr int MAX = 96;
  float* ptr[MAX];
  int64_t numel[MAX];
  int count;
};
__global__ void __launch_bounds__(256) multi_unscale_kernel(TensorList tl, float inv_scale, float* __restrict__ found_inf, float* __restrict__ sqnorm) {
  __shared__ float red[8];
  const int t = blockIdx.y;
  float* p = tl.ptr[t];
  const int64_t n = tl.numel[t];
  float ss = 0.f;
  bool bad = false;
  for (int64_t i = blockIdx.x * (int64_t)256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) {
    const float v = p[i] * inv_scale;
    bad |= !isfinite(v);
    p[i] = v;
    ss += v * v;
  }
  if (__syncthreads_or(bad) && threadIdx.x == 0) *found_inf = 1.f;
  ss = block_sum(ss, red);
  if (threadIdx.x == 0 && sqnorm) atomicAdd(sqnorm, ss);
}

// ---- GGUF block dequantisation ----------------------------------------------------------------------------------------------------------
enum GgufType : int { Q4_0 = 2, Q4_1 = 3, Q5_0 = 6, Q5_1 = 7, Q8_0 = 8, Q8_1 = 9 };
FT_DEVICE float h2f(const uint8_t* p) { return __half2float(*reinterpret_cast<const __half*>(p)); }

// one thread per block of 32 weights
__global__ void __launch_bounds__(256) gguf_dequant_kernel(int type, const uint8_t* __restrict__ blocks, float* __restrict__ out, size_t nblocks) {
  const size_t b = blockIdx.x * (size_t)256 + threadIdx.x;
  if (b >= nblocks) return;
  float* o = out + b * 32;
  switch (type) {
    case Q4_0: {
      const uint8_t* p = blocks + b * 18;
      const float d = h2f(p);
      for (int j = 0; j < 16; j++) {
        o[j] = ((int)(p[2 + j] & 0xF) - 8) * d;
        o[j + 16] = ((int)(p[2 + j] >> 4) - 8) * d;
      }
      break;
    }
    case Q4_1: {
      const uint8_t* p = blocks + b * 20;
      const float d = h2f(p), m = h2f(p + 2);
      for (int j = 0; j < 16; j++) {
        o[j] = (p[4 + j] & 0xF) * d + m;
        o[j + 16] = (p[4 + j] >> 4) * d + m;
      }
      break;
    }
    case Q5_0: {
      const uint8_t* p = blocks + b * 22;
      const float d = h2f(p);
      uint32_t qh;
      memcpy(&qh, p + 2, 4);
      for (int j = 0; j < 16; j++) {
        const int x0 = (p[6 + j] & 0xF) | (((qh >> j) & 1) << 4), x1 = (p[6 + j] >> 4) | (((qh >> (j + 16)) & 1) << 4);
        o[j] = (x0 - 16) * d;
        o[j + 16] = (x1 - 16) * d;
      }
      break;
    }
    case Q5_1: {
      const uint8_t* p = blocks + b * 24;
      const float d = h2f(p), m = h2f(p + 2);
      uint32_t qh;
      memcpy(&qh, p + 4, 4);
      for (int j = 0; j < 16; j++) {
        const int x0 = (p[8 + j] & 0xF) | (((qh >> j) & 1) << 4), x1 = (p[8 + j] >> 4) | (((qh >> (j + 16)) & 1) << 4);
        o[j] = x0 * d + m;
        o[j + 16] = x1 * d + m;
      }
      break;
    }
    case Q8_0: {
      const uint8_t* p = blocks + b * 34;
      const float d = h2f(p);
      for (int j = 0; j < 32; j++) o[j] = (int8_t)p[2 + j] * d;
      break;
    }
    case Q8_1: {
      const uint8_t* p = blocks + b * 36;
      const float d = h2f(p);
      for (int j = 0; j < 32; j++) o[j] = (int8_t)p[4 + j] * d;
      break;
    }
    default: break;
  }
}

// logits[r, v] = -inf where bit v of the row's allow-mask is clear (mask: u32 words, shared by all rows when mask_rows == 1)
template <typename T>
__global__ void __launch_bounds__(256) token_mask_kernel(T* __restrict__ logits, const uint32_t* __restrict__ mask, size_t rows, size_t vocab, size_t mask_rows) {
  const size_t total = rows * vocab, words = (vocab + 31) / 32;
  for (size_t i = blockIdx.x * (size_t)256 + threadIdx.x; i < total; i += (size_t)gridDim.x * 256) {
    const size_t r = i / vocab, v = i % vocab;
    const uint32_t w = mask[(mask_rows == 1 ? 0 : r) * words + v / 32];
    if (!((w >> (v % 32)) & 1u)) stf(logits, i, -CUDART_INF_F);
  }
}

inline int grid_for(size_t work) {
  const size_t g = (work + 255) / 256;
  return (int)(g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g));
}

template <typename T, typename A>
int reduce_launch(int op, const T* x, T* out, size_t outer, size_t len, size_t inner, void* scratch, size_t scratch_bytes, cudaStream_t st) {
  if (inner == 1) {
    if (outer == 1 && len > (1u << 16)) {
      const int np = 148 * 4;
      if (scratch_bytes < np * sizeof(A) || !scratch) return FT_ERR_ARG;
      reduce_partial_kernel<T, A><<<np, 256, 0, st>>>(op, x, (A*)scratch, len);
      reduce_final_kernel<T, A><<<1, 256, 0, st>>>(op, (const A*)scratch, np, out, len);
    } else {
      reduce_rows_kernel<T, A><<<(unsigned)outer, 256, 0, st>>>(op, x, out, len);
    }
  } else {
    if (outer > 65535) return FT_ERR_ARG;
    reduce_axis_kernel<T, A><<<dim3((unsigned)((inner + 31) / 32), (unsigned)outer), dim3(32, 8), 0, st>>>(op, x, out, len, inner);
  }
  return (int)cudaGetLastError();
}

}  // namespace

// x viewed as [outer, len, inner] -> out [outer, inner]. scratch: >= 148*4*8 bytes of device memory, used only for long full reductions.
FT_EXPORT int ft_reduce(int dtype, int op, const void* x, void* out, int64_t outer, int64_t len, int64_t inner, void* scratch, int64_t scratch_bytes,
                        cudaStream_t st) {
  if (outer < 1 || len < 1 || inner < 1 || outer > 2147483647LL) return FT_ERR_ARG;
  switch (dtype) {
    case DT_F32: return reduce_launch<float, float>(op, (const float*)x, (float*)out, outer, len, inner, scratch, scratch_bytes, st);
    case DT_BF16: return reduce_launch<__nv_bfloat16, float>(op, (const __nv_bfloat16*)x, (__nv_bfloat16*)out, outer, len, inner, scratch, scratch_bytes, st);
    case DT_F16: return reduce_launch<__half, float>(op, (const __half*)x, (__half*)out, outer, len, inner, scratch, scratch_bytes, st);
    case DT_F64: return reduce_launch<double, double>(op, (const double*)x, (double*)out, outer, len, inner, scratch, scratch_bytes, st);
    default: return FT_ERR_ARG;
  }
}

FT_EXPORT int ft_scan(int dtype, int op, const void* x, void* out, int64_t outer, int64_t len, int64_t inner, int reverse, cudaStream_t st) {
  if (outer < 1 || len < 1 || inner < 1) return FT_ERR_ARG;
#define FT_SCAN(T, A)                                                                                                                  \
  if (inner == 1) scan_rows_kernel<T, A><<<(unsigned)((outer + 3) / 4), 128, 0, st>>>(op, (const T*)x, (T*)out, outer, len, reverse);  \
  else scan_axis_kernel<T, A><<<(unsigned)((outer * inner + 255) / 256), 256, 0, st>>>(op, (const T*)x, (T*)out, outer, len, inner, reverse);
  switch (dtype) {
    case DT_F32: FT_SCAN(float, float) break;
    case DT_BF16: FT_SCAN(__nv_bfloat16, float) break;
    case DT_F16: FT_SCAN(__half, float) break;
    case DT_F64: FT_SCAN(double, double) break;
    default: return FT_ERR_ARG;
  }
#undef FT_SCAN
  return (int)cudaGetLastError();
}

FT_EXPORT int ft_index_select(int elem_bytes, const void* src, const int64_t* idx, void* out, int64_t outer, int64_t src_len, int64_t n_idx, int64_t inner,
                              cudaStream_t st) {
  const size_t total = (size_t)outer * n_idx * inner;
  if (total == 0) return 0;
  uint32_t* status = ft_status_ptr();
  switch (elem_bytes) {
    case 2: index_select_kernel<uint16_t><<<grid_for(total), 256, 0, st>>>((const uint16_t*)src, idx, (uint16_t*)out, outer, src_len, n_idx, inner, status); break;
    case 4: index_select_kernel<uint32_t><<<grid_for(total), 256, 0, st>>>((const uint32_t*)src, idx, (uint32_t*)out, outer, src_len, n_idx, inner, status); break;
    case 8: index_select_kernel<uint64_t><<<grid_for(total), 256, 0, st>>>((const uint64_t*)src, idx, (uint64_t*)out, outer, src_len, n_idx, inner, status); break;
    default: return FT_ERR_ARG;
  }
  return (int)cudaGetLastError();
}

FT_EXPORT int ft_index_add_f32(float* dst, const int64_t* idx, const float* src, int64_t outer, int64_t dst_len, int64_t n_idx, int64_t inner, cudaStream_t st) {
  const size_t total = (size_t)outer * n_idx * inner;
  if (total == 0) return 0;
  index_add_kernel<<<grid_for(total), 256, 0, st>>>(dst, idx, src, outer, dst_len, n_idx, inner, ft_status_ptr());
  return (int)cudaGetLastError();
}

FT_EXPORT int ft_gather(int elem_bytes, const void* src, const int64_t* idx, void* out, int64_t outer, int64_t src_len, int64_t n_idx, int64_t inner,
                        cudaStream_t st) {
  const size_t total = (size_t)outer * n_idx * inner;
  if (total == 0) return 0;
  uint32_t* status = ft_status_ptr();
  switch (elem_bytes) {
    case 2: gather_scatter_kernel<uint16_t, false><<<grid_for(total), 256, 0, st>>>((uint16_t*)src, idx, (uint16_t*)out, outer, src_len, n_idx, inner, status); break;
    case 4: gather_scatter_kernel<uint32_t, false><<<grid_for(total), 256, 0, st>>>((uint32_t*)src, idx, (uint32_t*)out, outer, src_len, n_idx, inner, status); break;
    case 8: gather_scatter_kernel<uint64_t, false><<<grid_for(total), 256, 0, st>>>((uint64_t*)src, idx, (uint64_t*)out, outer, src_len, n_idx, inner, status); break;
    default: return FT_ERR_ARG;
  }
  return (int)cudaGetLastError();
}

FT_EXPORT int ft_scatter_add_f32(float* dst, const int64_t* idx, const float* src, int64_t outer, int64_t dst_len, int64_t n_idx, int64_t inner, cudaStream_t st) {
  const size_t total = (size_t)outer * n_idx * inner;
  if (total == 0) return 0;
  gather_scatter_kernel<float, true><<<grid_for(total), 256, 0, st>>>(dst, idx, const_cast<float*>(src), outer, dst_len, n_idx, inner, ft_status_ptr());
  return (int)cudaGetLastError();
}

// mode 0: uniform in [a, b); 1: normal(mean a, std b); element i depends only on (seed, offset, i). The caller advances offset by ceil(n/4).
FT_EXPORT int ft_philox_fill(int dtype, int mode, void* out, int64_t n, int64_t seed, int64_t offset, float a, float b, cudaStream_t st) {
  if (n == 0) return 0;
  if (mode != 0 && mode != 1) return FT_ERR_ARG;
  const int g = grid_for((size_t)(n + 3) / 4);
#define FT_PH(T)                                                                                                                      \
  if (mode == 0) philox_kernel<T, 0><<<g, 256, 0, st>>>((T*)out, nullptr, nullptr, (size_t)n, (uint64_t)seed, (uint64_t)offset, a, b); \
  else philox_kernel<T, 1><<<g, 256, 0, st>>>((T*)out, nullptr, nullptr, (size_t)n, (uint64_t)seed, (uint64_t)offset, a, b);
  switch (dtype) {
    case DT_F32: FT_PH(float) break;
    case DT_BF16: FT_PH(__nv_bfloat16) break;
    case DT_F16: FT_PH(__half) break;
    default: return FT_ERR_ARG;
  }
#undef FT_PH
  return (int)cudaGetLastError();
}

// out = keep ? x / (1 - p) : 0 with keep ~ Bernoulli(1 - p) from the Philox stream; mask (u8, optional) records keep for the backward.
FT_EXPORT int ft_philox_dropout(int dtype, const void* x, void* out, void* mask_u8, int64_t n, float p, int64_t seed, int64_t offset, cudaStream_t st) {
  if (n == 0) return 0;
  if (!(p >= 0.f && p < 1.f)) return FT_ERR_ARG;
  const int g = grid_for((size_t)(n + 3) / 4);
  const float inv = 1.f / (1.f - p);
  switch (dtype) {
    case DT_F32: philox_kernel<float, 2><<<g, 256, 0, st>>>((float*)out, (const float*)x, (uint8_t*)mask_u8, (size_t)n, (uint64_t)seed, (uint64_t)offset, p, inv); break;
    case DT_BF16: philox_kernel<__nv_bfloat16, 2><<<g, 256, 0, st>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)x, (uint8_t*)mask_u8, (size_t)n, (uint64_t)seed, (uint64_t)offset, p, inv); break;
    case DT_F16: philox_kernel<__half, 2><<<g, 256, 0, st>>>((__half*)out, (const __half*)x, (uint8_t*)mask_u8, (size_t)n, (uint64_t)seed, (uint64_t)offset, p, inv); break;
    default: return FT_ERR_ARG;
  }
  return (int)cudaGetLastError();
}

// In-place g *= inv_scale over up to 96 f32 tensors in one launch; *found_inf = 1 if any result is non-finite; *sqnorm += sum of squares.
FT_EXPORT int ft_multi_unscale(const void* const* ptrs, const int64_t* numels, int count, float inv_scale, float* found_inf, float* sqnorm, cudaStream_t st) {
  if (count < 1 || count > TensorList::MAX) return FT_ERR_ARG;
  TensorList tl;
  tl.count = count;
  int64_t mx = 0;
  for (int i = 0; i < count; i++) {
    tl.ptr[i] = (float*)ptrs[i];
    tl.numel[i] = numels[i];
    mx = numels[i] > mx ? numels[i] : mx;
  }
  int gx = (int)((mx + 256 * 8 - 1) / (256 * 8));
  gx = gx < 1 ? 1 : (gx > 64 ? 64 : gx);
  multi_unscale_kernel<<<dim3(gx, count), 256, 0, st>>>(tl, inv_scale, found_inf, sqnorm);
  return (int)cudaGetLastError();
}

FT_EXPORT int ft_gguf_dequant(int type, const void* blocks, float* out, int64_t nblocks, cudaStream_t st) {
  if (nblocks < 1) return nblocks == 0 ? 0 : FT_ERR_ARG;
  if (type != Q4_0 && type != Q4_1 && type != Q5_0 && type != Q5_1 && type != Q8_0 && type != Q8_1) return FT_ERR_ARG;
  gguf_dequant_kernel<<<(unsigned)((nblocks + 255) / 256), 256, 0, st>>>(type, (const uint8_t*)blocks, out, (size_t)nblocks);
  return (int)cudaGetLastError();
}

FT_EXPORT int ft_token_mask(int dtype, void* logits, const void* mask_words, int64_t rows, int64_t vocab, int64_t mask_rows, cudaStream_t st) {
  if (rows < 1 || vocab < 1 || (mask_rows != 1 && mask_rows != rows)) return FT_ERR_ARG;
  const size_t total = (size_t)rows * vocab;
  switch (dtype) {
    case DT_F32: token_mask_kernel<float><<<grid_for(total), 256, 0, st>>>((float*)logits, (const uint32_t*)mask_words, rows, vocab, mask_rows); break;
    case DT_BF16: token_mask_kernel<__nv_bfloat16><<<grid_for(total), 256, 0, st>>>((__nv_bfloat16*)logits, (const uint32_t*)mask_words, rows, vocab, mask_rows); break;
    case DT_F16: token_mask_kernel<__half><<<grid_for(total), 256, 0, st>>>((__half*)logits, (const uint32_t*)mask_words, rows, vocab, mask_rows); break;
    default: return FT_ERR_ARG;
  }
  return (int)cudaGetLastError();
}
