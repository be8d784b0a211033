// Generic elementwise family: one vectorised iterator for contiguous operands (16 bytes per thread per operand) and one strided /
// broadcasting iterator (up to 6 dims, element strides, 0 on broadcast dims). Storage dtypes f32 / f64 / bf16 / f16; arithmetic in f32
// (f64 for double). The operation is a run-time code so that one instantiation per dtype serves the whole family.
//
// Replaces the reference's one-PTX-string-per-op kernels (ferrotorch-gpu/src/kernels.rs: ADD 188 .. TANH 11771, BROADCAST_* 10068-10352,
// GELU/SILU/ELU/MISH forward and backward 1363-4022, CLAMP 3509/6553, FILL 3565, F32_TO_F16 719, F32_TO_BF16 774, STRIDED_COPY 10615,
// TRANSPOSE_2D 578, PERMUTE_0213 639) and their bf16 variants (ferrotorch-gpu/src/bf16.rs:43-283).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "common.cuh"
#include "host_common.h"

namespace {

enum DType : int { DT_F32 = 0, DT_BF16 = 1, DT_F16 = 2, DT_F64 = 3, DT_I64 = 4, DT_I32 = 5, DT_U8 = 6 };

enum UnaryOp : int {
  U_NEG = 0, U_ABS, U_EXP, U_LOG, U_SQRT, U_RSQRT, U_RECIP, U_SIN, U_COS, U_TANH, U_SIGMOID, U_RELU, U_GELU, U_GELU_TANH, U_SILU, U_ELU,
  U_MISH, U_ERF, U_FLOOR, U_CEIL, U_ROUND, U_SIGN, U_SQUARE, U_SOFTPLUS, U_SCALE, U_ADD_SCALAR, U_POW_SCALAR, U_CLAMP, U_LEAKY_RELU,
  U_HARDSWISH, U_HARDSIGMOID, U_EXP2, U_LOG2, U_LOG1P, U_EXPM1, U_COPY, U_FATRELU
};
// backward codes: grad_in = g * f'(.) where "v" is the saved forward INPUT (x) unless noted
enum UnaryBwd : int {
  UB_RELU = 0, UB_ABS, UB_SIGMOID_Y /* v = output */, UB_TANH_Y /* v = output */, UB_GELU, UB_GELU_TANH, UB_SILU, UB_ELU, UB_MISH, UB_CLAMP,
  UB_LEAKY_RELU, UB_EXP_Y /* v = output */, UB_LOG, UB_SQRT_Y /* v = output */, UB_SOFTPLUS, UB_HARDSWISH, UB_HARDTANH
};
enum BinaryOp : int { B_ADD = 0, B_SUB, B_MUL, B_DIV, B_POW, B_MAX, B_MIN, B_EQ, B_NE, B_LT, B_LE, B_GT, B_GE, B_ATAN2, B_FMOD };

template <typename T> struct Acc { using type = float; };
template <> struct Acc<double> { using type = double; };

template <typename A> FT_DEVICE A to_acc(float v) { return (A)v; }
FT_DEVICE float ld(const float* p, size_t i) { return p[i]; }
FT_DEVICE double ld(const double* p, size_t i) { return p[i]; }
FT_DEVICE float ld(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }
FT_DEVICE float ld(const __half* p, size_t i) { return __half2float(p[i]); }
FT_DEVICE void st(float* p, size_t i, float v) { p[i] = v; }
FT_DEVICE void st(double* p, size_t i, double v) { p[i] = v; }
FT_DEVICE void st(__nv_bfloat16* p, size_t i, float v) { p[i] = __float2bfloat16(v); }
FT_DEVICE void st(__half* p, size_t i, float v) { p[i] = __float2half(v); }

template <typename A>
FT_DEVICE A unary_apply(int op, A x, A a, A b) {
  switch (op) {
    case U_NEG: return -x;
    case U_ABS: return fabs(x);
    case U_EXP: return exp(x);
    case U_LOG: return log(x);
    case U_SQRT: return sqrt(x);
    case U_RSQRT: return (A)1 / sqrt(x);
    case U_RECIP: return (A)1 / x;
    case U_SIN: return sin(x);
    case U_COS: return cos(x);
    case U_TANH: return tanh(x);
    case U_SIGMOID: return (A)1 / ((A)1 + exp(-x));
    case U_RELU: return x > (A)0 ? x : (A)0;
    case U_GELU: return (A)0.5 * x * ((A)1 + erf(x * (A)0.7071067811865476));
    case U_GELU_TANH: return (A)0.5 * x * ((A)1 + tanh((A)0.7978845608028654 * (x + (A)0.044715 * x * x * x)));
    case U_SILU: return x / ((A)1 + exp(-x));
    case U_ELU: return x > (A)0 ? x : a * (exp(x) - (A)1);
    case U_MISH: return x * tanh(x > (A)20 ? x : log1p(exp(x)));
    case U_ERF: return erf(x);
    case U_FLOOR: return floor(x);
    case U_CEIL: return ceil(x);
    case U_ROUND: return nearbyint(x);
    case U_SIGN: return (A)((x > (A)0) - (x < (A)0));
    case U_SQUARE: return x * x;
    case U_SOFTPLUS: return x * a > b ? x : log1p(exp(x * a)) / a;          // a = beta, b = threshold
    case U_SCALE: return x * a + b;
    case U_ADD_SCALAR: return x + a;
    case U_POW_SCALAR: return pow(x, a);
    case U_CLAMP: return x != x ? x : (x < a ? a : (x > b ? b : x));
    case U_LEAKY_RELU: return x > (A)0 ? x : a * x;
    case U_HARDSWISH: return x * fmin(fmax(x + (A)3, (A)0), (A)6) / (A)6;
    case U_HARDSIGMOID: return fmin(fmax(x + (A)3, (A)0), (A)6) / (A)6;
    case U_EXP2: return exp2(x);
    case U_LOG2: return log2(x);
    case U_LOG1P: return log1p(x);
    case U_EXPM1: return expm1(x);
    case U_FATRELU: return x > a ? x : (A)0;
    default: return x;
  }
}

template <typename A>
FT_DEVICE A unary_bwd_apply(int op, A g, A v, A a, A b) {
  switch (op) {
    case UB_RELU: return v > (A)0 ? g : (A)0;
    case UB_ABS: return g * (A)((v > (A)0) - (v < (A)0));
    case UB_SIGMOID_Y: return g * v * ((A)1 - v);
    case UB_TANH_Y: return g * ((A)1 - v * v);
    case UB_GELU: {
      const A cdf = (A)0.5 * ((A)1 + erf(v * (A)0.7071067811865476));
      const A pdf = (A)0.3989422804014327 * exp((A)-0.5 * v * v);
      return g * (cdf + v * pdf);
    }
    case UB_GELU_TANH: {
      const A k = (A)0.7978845608028654, c = (A)0.044715;
      const A t = tanh(k * (v + c * v * v * v));
      return g * ((A)0.5 * ((A)1 + t) + (A)0.5 * v * ((A)1 - t * t) * k * ((A)1 + (A)3 * c * v * v));
    }
    case UB_SILU: {
      const A s = (A)1 / ((A)1 + exp(-v));
      return g * s * ((A)1 + v * ((A)1 - s));
    }
    case UB_ELU: return v > (A)0 ? g : g * a * exp(v);
    case UB_MISH: {
      const A sp = v > (A)20 ? v : log1p(exp(v));
      const A t = tanh(sp), s = (A)1 / ((A)1 + exp(-v));
      return g * (t + v * ((A)1 - t * t) * s);
    }
    case UB_CLAMP: return (v >= a && v <= b) ? g : (A)0;
    case UB_LEAKY_RELU: return v > (A)0 ? g : g * a;
    case UB_EXP_Y: return g * v;
    case UB_LOG: return g / v;
    case UB_SQRT_Y: return g / ((A)2 * v);
    case UB_SOFTPLUS: return v * a > b ? g : g / ((A)1 + exp(-v * a));
    // at the kinks x = -3 and x = 3 the outer pieces' derivatives are taken (0 and 1), as PyTorch does
    case UB_HARDSWISH: return v <= (A)-3 ? (A)0 : (v >= (A)3 ? g : g * ((A)2 * v + (A)3) / (A)6);
    case UB_HARDTANH: return (v > a && v < b) ? g : (A)0;      // open interval: no gradient at the two bounds (clamp keeps it there)
    default: return g;
  }
}

template <typename A>
FT_DEVICE A binary_apply(int op, A x, A y) {
  switch (op) {
    case B_ADD: return x + y;
    case B_SUB: return x - y;
    case B_MUL: return x * y;
    case B_DIV: return x / y;
    case B_POW: return pow(x, y);
    case B_MAX: return (x > y || x != x) ? x : y;
    case B_MIN: return (x < y || x != x) ? x : y;
    case B_EQ: return (A)(x == y);
    case B_NE: return (A)(x != y);
    case B_LT: return (A)(x < y);
    case B_LE: return (A)(x <= y);
    case B_GT: return (A)(x > y);
    case B_GE: return (A)(x >= y);
    case B_ATAN2: return atan2(x, y);
    case B_FMOD: return fmod(x, y);
    default: return x;
  }
}

template <typename T>
struct alignas(16) Vec16 {
  static constexpr int N = 16 / sizeof(T);
  T v[N];
};

// ---- contiguous, vectorised -------------------------------------------------------------------------------------------------
template <typename T, int MODE>   // MODE 0: unary(x); 1: unary_bwd(g, v); 2: binary(x, y)
__global__ void __launch_bounds__(256) ew_contig_kernel(int op, const T* __restrict__ x, const T* __restrict__ y, T* __restrict__ out, size_t n,
                                                        double a_, double b_) {
  using A = typename Acc<T>::type;
  constexpr int N = Vec16<T>::N;
  const A a = (A)a_, b = (A)b_;
  const size_t nvec = n / N;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += stride) {
    Vec16<T> vx = reinterpret_cast<const Vec16<T>*>(x)[i], vy, vo;
    if (MODE != 0) vy = reinterpret_cast<const Vec16<T>*>(y)[i];
#pragma unroll
    for (int e = 0; e < N; e++) {
      const A xe = (A)ld(vx.v, e);
      A r;
      if (MODE == 0) r = unary_apply<A>(op, xe, a, b);
      else if (MODE == 1) r = unary_bwd_apply<A>(op, xe, (A)ld(vy.v, e), a, b);
      else r = binary_apply<A>(op, xe, (A)ld(vy.v, e));
      st(vo.v, e, r);
    }
    reinterpret_cast<Vec16<T>*>(out)[i] = vo;
  }
  for (size_t i = nvec * N + blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += stride) {
    const A xe = (A)ld(x, i);
    A r;
    if (MODE == 0) r = unary_apply<A>(op, xe, a, b);
    else if (MODE == 1) r = unary_bwd_apply<A>(op, xe, (A)ld(y, i), a, b);
    else r = binary_apply<A>(op, xe, (A)ld(y, i));
    st(out, i, r);
  }
}

// ---- strided / broadcast -----------------------------------------------------------------------------------------------------
constexpr int MAXD = 6;
struct IterDesc {
  int ndim;
  int64_t shape[MAXD];
  int64_t sa[MAXD], sb[MAXD], sc[MAXD];     // element strides of up to three inputs (0 = broadcast)
};

FT_DEVICE void iter_offsets(const IterDesc& d, size_t i, int64_t& oa, int64_t& ob, int64_t& oc) {
  oa = ob = oc = 0;
#pragma unroll
  for (int k = MAXD - 1; k >= 0; k--) {
    if (k < d.ndim) {
      const int64_t c = (int64_t)(i % (size_t)d.shape[k]);
      i /= (size_t)d.shape[k];
      oa += c * d.sa[k];
      ob += c * d.sb[k];
      oc += c * d.sc[k];
    }
  }
}

template <typename T, int MODE>   // 0: unary copy/op of strided x -> dense out; 2: binary; 3: where(cond u8, x, y)
__global__ void __launch_bounds__(256) ew_strided_kernel(int op, const void* __restrict__ p0, const T* __restrict__ p1, const T* __restrict__ p2,
                                                         T* __restrict__ out, size_t n, IterDesc d, double a_, double b_) {
  using A = typename Acc<T>::type;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += stride) {
    int64_t oa, ob, oc;
    iter_offsets(d, i, oa, ob, oc);
    A r;
    if (MODE == 0) r = unary_apply<A>(op, (A)ld(reinterpret_cast<const T*>(p0), oa), (A)a_, (A)b_);
    else if (MODE == 2) r = binary_apply<A>(op, (A)ld(reinterpret_cast<const T*>(p0), oa), (A)ld(p1, ob));
    else r = reinterpret_cast<const uint8_t*>(p0)[oa] ? (A)ld(p1, ob) : (A)ld(p2, oc);
    st(out, i, r);
  }
}

// dense in -> strided out (scatter form of the copy; used for slice writes / cat)
template <typename T>
__global__ void __launch_bounds__(256) ew_scatter_copy_kernel(const T* __restrict__ in, T* __restrict__ out, size_t n, IterDesc d) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += stride) {
    int64_t oa, ob, oc;
    iter_offsets(d, i, oa, ob, oc);
    out[oa] = in[i];
  }
}

// ---- casts / fill --------------------------------------------------------------------------------------------------------------
template <typename S, typename D>
__global__ void __launch_bounds__(256) cast_kernel(const S* __restrict__ in, D* __restrict__ out, size_t n) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  constexpr int N = 8;
  const size_t nvec = n / N;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += stride) {
    S s[N];
    D o[N];
#pragma unroll
    for (int e = 0; e < N; e++) s[e] = in[i * N + e];
#pragma unroll
    for (int e = 0; e < N; e++) st(o, e, (typename Acc<D>::type)ld(s, e));
#pragma unroll
    for (int e = 0; e < N; e++) out[i * N + e] = o[e];
  }
  for (size_t i = nvec * N + blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += stride) st(out, i, (typename Acc<D>::type)ld(in, i));
}

template <typename T>
__global__ void __launch_bounds__(256) fill_kernel(T* __restrict__ out, size_t n, double v) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += stride) st(out, i, (typename Acc<T>::type)v);
}

// masked_fill on a dense tensor with a dense u8 mask
template <typename T>
__global__ void __launch_bounds__(256) masked_fill_kernel(T* __restrict__ x, const uint8_t* __restrict__ mask, size_t n, double v) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += stride)
    if (mask[i]) st(x, i, (typename Acc<T>::type)v);
}

inline int grid_for(size_t work) {
  const size_t g = (work + 255) / 256;
  return (int)(g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g));
}

template <int MODE>
int launch_contig(int dtype, int op, const void* x, const void* y, void* out, size_t n, double a, double b, cudaStream_t st_) {
  if (n == 0) return 0;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) | (MODE ? reinterpret_cast<uintptr_t>(y) : 0)) & 15) return FT_ERR_ARG;
  switch (dtype) {
    case DT_F32: ew_contig_kernel<float, MODE><<<grid_for(n / 4 + 1), 256, 0, st_>>>(op, (const float*)x, (const float*)y, (float*)out, n, a, b); break;
    case DT_BF16: ew_contig_kernel<__nv_bfloat16, MODE><<<grid_for(n / 8 + 1), 256, 0, st_>>>(op, (const __nv_bfloat16*)x, (const __nv_bfloat16*)y, (__nv_bfloat16*)out, n, a, b); break;
    case DT_F16: ew_contig_kernel<__half, MODE><<<grid_for(n / 8 + 1), 256, 0, st_>>>(op, (const __half*)x, (const __half*)y, (__half*)out, n, a, b); break;
    case DT_F64: ew_contig_kernel<double, MODE><<<grid_for(n / 2 + 1), 256, 0, st_>>>(op, (const double*)x, (const double*)y, (double*)out, n, a, b); break;
    default: return FT_ERR_ARG;
  }
  return (int)cudaGetLastError();
}

int fill_desc(IterDesc& d, int ndim, const int64_t* shape, const int64_t* sa, const int64_t* sb, const int64_t* sc) {
  if (ndim < 1 || ndim > MAXD) return FT_ERR_ARG;
  d.ndim = ndim;
  for (int k = 0; k < MAXD; k++) {
    d.shape[k] = k < ndim ? shape[k] : 1;
    d.sa[k] = (k < ndim && sa) ? sa[k] : 0;
    d.sb[k] = (k < ndim && sb) ? sb[k] : 0;
    d.sc[k] = (k < ndim && sc) ? sc[k] : 0;
    if (d.shape[k] < 1) return FT_ERR_ARG;
  }
  return 0;
}

}  // namespace

// out = op(x) elementwise over n contiguous elements (all pointers 16-byte aligned). a, b: op parameters (ELU alpha, clamp bounds, scale/shift...).
FT_EXPORT int ft_ew_unary(int dtype, int op, const void* x, void* out, int64_t n, double a, double b, cudaStream_t st_) {
  return launch_contig<0>(dtype, op, x, nullptr, out, (size_t)n, a, b, st_);
}
// grad_in = grad * f'(saved); `saved` is the forward input or output as the op code states.
FT_EXPORT int ft_ew_unary_bwd(int dtype, int op, const void* grad, const void* saved, void* out, int64_t n, double a, double b, cudaStream_t st_) {
  return launch_contig<1>(dtype, op, grad, saved, out, (size_t)n, a, b, st_);
}
FT_EXPORT int ft_ew_binary(int dtype, int op, const void* x, const void* y, void* out, int64_t n, cudaStream_t st_) {
  return launch_contig<2>(dtype, op, x, y, out, (size_t)n, 0, 0, st_);
}

// Broadcasting / strided binary: out (dense, row-major over `shape`) = op(x[strides sx], y[strides sy]); strides in elements, 0 on broadcast dims.
FT_EXPORT int ft_ew_binary_strided(int dtype, int op, const void* x, const void* y, void* out, int ndim, const int64_t* shape, const int64_t* sx,
                                   const int64_t* sy, cudaStream_t st_) {
  IterDesc d;
  if (int e = fill_desc(d, ndim, shape, sx, sy, nullptr)) return e;
  size_t n = 1;
  for (int k = 0; k < ndim; k++) n *= (size_t)shape[k];
  switch (dtype) {
    case DT_F32: ew_strided_kernel<float, 2><<<grid_for(n), 256, 0, st_>>>(op, x, (const float*)y, nullptr, (float*)out, n, d, 0, 0); break;
    case DT_BF16: ew_strided_kernel<__nv_bfloat16, 2><<<grid_for(n), 256, 0, st_>>>(op, x, (const __nv_bfloat16*)y, nullptr, (__nv_bfloat16*)out, n, d, 0, 0); break;
    case DT_F16: ew_strided_kernel<__half, 2><<<grid_for(n), 256, 0, st_>>>(op, x, (const __half*)y, nullptr, (__half*)out, n, d, 0, 0); break;
    case DT_F64: ew_strided_kernel<double, 2><<<grid_for(n), 256, 0, st_>>>(op, x, (const double*)y, nullptr, (double*)out, n, d, 0, 0); break;
    default: return FT_ERR_ARG;
  }
  return (int)cudaGetLastError();
}

// Strided gather-copy with an optional unary op: out (dense) = op(x[strides]). Covers transpose / permute / expand / slice reads.
FT_EXPORT int ft_ew_unary_strided(int dtype, int op, const void* x, void* out, int ndim, const int64_t* shape, const int64_t* sx, double a, double b,
                                  cudaStream_t st_) {
  IterDesc d;
  if (int e = fill_desc(d, ndim, shape, sx, nullptr, nullptr)) return e;
  size_t n = 1;
  for (int k = 0; k < ndim; k++) n *= (size_t)shape[k];
  switch (dtype) {
    case DT_F32: ew_strided_kernel<float, 0><<<grid_for(n), 256, 0, st_>>>(op, x, nullptr, nullptr, (float*)out, n, d, a, b); break;
    case DT_BF16: ew_strided_kernel<__nv_bfloat16, 0><<<grid_for(n), 256, 0, st_>>>(op, x, nullptr, nullptr, (__nv_bfloat16*)out, n, d, a, b); break;
    case DT_F16: ew_strided_kernel<__half, 0><<<grid_for(n), 256, 0, st_>>>(op, x, nullptr, nullptr, (__half*)out, n, d, a, b); break;
    case DT_F64: ew_strided_kernel<double, 0><<<grid_for(n), 256, 0, st_>>>(op, x, nullptr, nullptr, (double*)out, n, d, a, b); break;
    default: return FT_ERR_ARG;
  }
  return (int)cudaGetLastError();
}

// out (dense) = cond ? x : y with broadcasting; cond is u8.
FT_EXPORT int ft_ew_where(int dtype, const void* cond, const void* x, const void* y, void* out, int ndim, const int64_t* shape, const int64_t* sc,
                          const int64_t* sx, const int64_t* sy, cudaStream_t st_) {
  IterDesc d;
  if (int e = fill_desc(d, ndim, shape, sc, sx, sy)) return e;
  size_t n = 1;
  for (int k = 0; k < ndim; k++) n *= (size_t)shape[k];
  switch (dtype) {
    case DT_F32: ew_strided_kernel<float, 3><<<grid_for(n), 256, 0, st_>>>(0, cond, (const float*)x, (const float*)y, (float*)out, n, d, 0, 0); break;
    case DT_BF16: ew_strided_kernel<__nv_bfloat16, 3><<<grid_for(n), 256, 0, st_>>>(0, cond, (const __nv_bfloat16*)x, (const __nv_bfloat16*)y, (__nv_bfloat16*)out, n, d, 0, 0); break;
    case DT_F16: ew_strided_kernel<__half, 3><<<grid_for(n), 256, 0, st_>>>(0, cond, (const __half*)x, (const __half*)y, (__half*)out, n, d, 0, 0); break;
    case DT_F64: ew_strided_kernel<double, 3><<<grid_for(n), 256, 0, st_>>>(0, cond, (const double*)x, (const double*)y, (double*)out, n, d, 0, 0); break;
    default: return FT_ERR_ARG;
  }
  return (int)cudaGetLastError();
}

// Dense `in` written into a strided destination view (slice write, cat, scatter of a block).
FT_EXPORT int ft_ew_scatter_copy(int elem_bytes, const void* in, void* out, int ndim, const int64_t* shape, const int64_t* so, cudaStream_t st_) {
  IterDesc d;
  if (int e = fill_desc(d, ndim, shape, so, nullptr, nullptr)) return e;
  size_t n = 1;
  for (int k = 0; k < ndim; k++) n *= (size_t)shape[k];
  switch (elem_bytes) {
    case 1: ew_scatter_copy_kernel<uint8_t><<<grid_for(n), 256, 0, st_>>>((const uint8_t*)in, (uint8_t*)out, n, d); break;
    case 2: ew_scatter_copy_kernel<uint16_t><<<grid_for(n), 256, 0, st_>>>((const uint16_t*)in, (uint16_t*)out, n, d); break;
    case 4: ew_scatter_copy_kernel<uint32_t><<<grid_for(n), 256, 0, st_>>>((const uint32_t*)in, (uint32_t*)out, n, d); break;
    case 8: ew_scatter_copy_kernel<uint64_t><<<grid_for(n), 256, 0, st_>>>((const uint64_t*)in, (uint64_t*)out, n, d); break;
    default: return FT_ERR_ARG;
  }
  return (int)cudaGetLastError();
}

FT_EXPORT int ft_ew_cast(int src_dtype, int dst_dtype, const void* in, void* out, int64_t n_, cudaStream_t st_) {
  const size_t n = (size_t)n_;
  if (n == 0) return 0;
  const int g = grid_for(n / 8 + 1);
#define FT_CAST(SD, ST, DD, DT_)                                                                         \
  if (src_dtype == SD && dst_dtype == DD) {                                                              \
    cast_kernel<ST, DT_><<<g, 256, 0, st_>>>((const ST*)in, (DT_*)out, n);                               \
    return (int)cudaGetLastError();                                                                      \
  }
  FT_CAST(DT_F32, float, DT_BF16, __nv_bfloat16) FT_CAST(DT_F32, float, DT_F16, __half) FT_CAST(DT_F32, float, DT_F64, double)
  FT_CAST(DT_BF16, __nv_bfloat16, DT_F32, float) FT_CAST(DT_F16, __half, DT_F32, float) FT_CAST(DT_F64, double, DT_F32, float)
  FT_CAST(DT_BF16, __nv_bfloat16, DT_F16, __half) FT_CAST(DT_F16, __half, DT_BF16, __nv_bfloat16)
#undef FT_CAST
  return FT_ERR_ARG;
}

FT_EXPORT int ft_ew_fill(int dtype, void* out, int64_t n, double v, cudaStream_t st_) {
  if (n == 0) return 0;
  switch (dtype) {
    case DT_F32: fill_kernel<float><<<grid_for((size_t)n), 256, 0, st_>>>((float*)out, (size_t)n, v); break;
    case DT_BF16: fill_kernel<__nv_bfloat16><<<grid_for((size_t)n), 256, 0, st_>>>((__nv_bfloat16*)out, (size_t)n, v); break;
    case DT_F16: fill_kernel<__half><<<grid_for((size_t)n), 256, 0, st_>>>((__half*)out, (size_t)n, v); break;
    case DT_F64: fill_kernel<double><<<grid_for((size_t)n), 256, 0, st_>>>((double*)out, (size_t)n, v); break;
    default: return FT_ERR_ARG;
  }
  return (int)cudaGetLastError();
}

FT_EXPORT int ft_ew_masked_fill(int dtype, void* x, const void* mask_u8, int64_t n, double v, cudaStream_t st_) {
  if (n == 0) return 0;
  switch (dtype) {
    case DT_F32: masked_fill_kernel<float><<<grid_for((size_t)n), 256, 0, st_>>>((float*)x, (const uint8_t*)mask_u8, (size_t)n, v); break;
    case DT_BF16: masked_fill_kernel<__nv_bfloat16><<<grid_for((size_t)n), 256, 0, st_>>>((__nv_bfloat16*)x, (const uint8_t*)mask_u8, (size_t)n, v); break;
    case DT_F16: masked_fill_kernel<__half><<<grid_for((size_t)n), 256, 0, st_>>>((__half*)x, (const uint8_t*)mask_u8, (size_t)n, v); break;
    case DT_F64: masked_fill_kernel<double><<<grid_for((size_t)n), 256, 0, st_>>>((double*)x, (const uint8_t*)mask_u8, (size_t)n, v); break;
    default: return FT_ERR_ARG;
  }
  return (int)cudaGetLastError();
}
