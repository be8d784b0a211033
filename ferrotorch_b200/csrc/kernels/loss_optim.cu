// Fused cross-entropy (online logsumexp over the vocabulary, loss and in-place
// gradient in one launch) and the flat multi-tensor optimizer kernels
// (AdamW with bf16 params + f32 master/moments, SGD with momentum, squared-norm
// reduction and unscale/found-inf for loss scaling).
//
// Capability parity: the host cross-entropy loop of ferrotorch-nn/src/loss.rs:187-330 (backward is
// NotImplementedOnCuda there), LOG_SOFTMAX/SOFTMAX kernels (ferrotorch-gpu/src/kernels.rs:5008-5547),
// FUSED_ADAM_PTX (kernels.rs:11918), foreach AdamW/SGD chains (ferrotorch-optim/src/adamw.rs:226-373,
// sgd.rs:210), GradScaler::unscale_ (ferrotorch-optim/src/grad_scaler.rs:200-240), HAS_INF_NAN (kernels.rs:6205).
#include "common.cuh"
#include "host_common.h"

namespace {

constexpr int CE_THREADS = 1024;

// One CTA per row. loss[row] = lse - logit[target] (+ label smoothing term); when dlogits != null
// writes (softmax - target distribution) * (*grad_scale_ptr or grad_scale) in place or out of place.
// Rows whose target == ignore_index get loss 0 and zero gradient.
template <typename T>
__global__ void __launch_bounds__(CE_THREADS) cross_entropy_kernel(const T* __restrict__ logits, const int64_t* __restrict__ targets,
                                                                   float* __restrict__ loss, float* __restrict__ lse_out,
                                                                   T* dlogits, int V, int64_t ld, int64_t ignore_index,
                                                                   float label_smoothing, float grad_scale,
                                                                   const float* __restrict__ grad_scale_ptr) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  const T* x = logits + (size_t)row * ld;
  const int64_t tgt = targets[row];
  constexpr int VEC = 16 / sizeof(T);
  const int nvec = V / VEC;  // V % VEC handled by the scalar tail

  float m = -INFINITY, s = 0.f, sumx = 0.f;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    float f[VEC];
    if constexpr (sizeof(T) == 2) bf16x8_to_float(reinterpret_cast<const bf16x8*>(x)[i], f);
    else { float4 t = reinterpret_cast<const float4*>(x)[i]; f[0] = t.x; f[1] = t.y; f[2] = t.z; f[3] = t.w; }
    float lm = f[0];
#pragma unroll
    for (int e = 1; e < VEC; e++) lm = fmaxf(lm, f[e]);
    const float nm = fmaxf(m, lm);
    float acc = 0.f;
#pragma unroll
    for (int e = 0; e < VEC; e++) { acc += __expf(f[e] - nm); sumx += f[e]; }
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  for (int i = nvec * VEC + threadIdx.x; i < V; i += CE_THREADS) {
    float f = (float)x[i];
    const float nm = fmaxf(m, f);
    s = s * __expf(m - nm) + __expf(f - nm);
    m = nm;
    sumx += f;
  }
  const float gm = block_max(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  const float gs = block_sum(s, red);
  const float gsumx = block_sum(sumx, red);
  const float lse = gm + __logf(gs);
  const bool valid = (tgt != ignore_index) && tgt >= 0 && tgt < V;
  if (threadIdx.x == 0) {
    float l = 0.f;
    if (valid) {
      const float xt = (float)x[tgt];
      l = (1.f - label_smoothing) * (lse - xt) + label_smoothing * (lse - gsumx / (float)V);
    }
    loss[row] = l;
    if (lse_out) lse_out[row] = lse;
  }
  if (dlogits == nullptr) return;
  const float gsc = valid ? (grad_scale_ptr ? grad_scale * (*grad_scale_ptr) : grad_scale) : 0.f;
  const float smooth = label_smoothing / (float)V;
  T* dx = dlogits + (size_t)row * ld;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    float f[VEC];
    if constexpr (sizeof(T) == 2) bf16x8_to_float(reinterpret_cast<const bf16x8*>(x)[i], f);
    else { float4 t = reinterpret_cast<const float4*>(x)[i]; f[0] = t.x; f[1] = t.y; f[2] = t.z; f[3] = t.w; }
#pragma unroll
    for (int e = 0; e < VEC; e++) {
      float p = __expf(f[e] - lse) - smooth;
      if ((int64_t)(i * VEC + e) == tgt) p -= (1.f - label_smoothing);
      f[e] = p * gsc;
    }
    if constexpr (sizeof(T) == 2) reinterpret_cast<bf16x8*>(dx)[i] = float_to_bf16x8(f);
    else reinterpret_cast<float4*>(dx)[i] = make_float4(f[0], f[1], f[2], f[3]);
  }
  for (int i = nvec * VEC + threadIdx.x; i < V; i += CE_THREADS) {
    float p = __expf((float)x[i] - lse) - smooth;
    if ((int64_t)i == tgt) p -= (1.f - label_smoothing);
    dx[i] = (T)(p * gsc);
  }
}

// Deterministic mean of the per-row losses over valid rows; also writes the count of valid rows.
__global__ void loss_mean_kernel(const float* __restrict__ loss, const int64_t* __restrict__ targets, int rows, int64_t ignore_index,
                                 float* __restrict__ out_mean, float* __restrict__ out_count) {
  __shared__ float red[32];
  float s = 0.f, c = 0.f;
  for (int i = threadIdx.x; i < rows; i += blockDim.x) {
    if (targets[i] != ignore_index) { s += loss[i]; c += 1.f; }
  }
  s = block_sum(s, red);
  c = block_sum(c, red);
  if (threadIdx.x == 0) { *out_mean = c > 0.f ? s / c : 0.f; if (out_count) *out_count = c; }
}

struct AdamWArgs {
  float lr, beta1, beta2, eps, weight_decay, bias_c1, bias_c2;  // bias_c = 1 - beta^t
  int maximize;
};

// Flat AdamW: decoupled decay p *= (1 - lr*wd); f32 master + moments; optional bf16 shadow of the params.
// GradT is bf16 or f32. grad_scale_ptr (optional, device) multiplies every gradient (clip coefficient / loss-scale inverse);
// skip_ptr (optional, device) != 0 skips the whole update (found-inf).
template <typename GradT>
__global__ void adamw_kernel(float* __restrict__ master, __nv_bfloat16* __restrict__ p_bf16, float* __restrict__ m, float* __restrict__ v,
                             const GradT* __restrict__ grad, size_t n, AdamWArgs a, const float* __restrict__ grad_scale_ptr,
                             const int* __restrict__ skip_ptr) {
  if (skip_ptr && *skip_ptr) return;
  const float gs = grad_scale_ptr ? *grad_scale_ptr : 1.f;
  const float decay = 1.f - a.lr * a.weight_decay;
  const float step = a.lr / a.bias_c1;
  const float inv_c2 = rsqrtf(a.bias_c2);
  const size_t nvec = n >> 2;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
    float4 pw = reinterpret_cast<float4*>(master)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float g[4];
    if constexpr (sizeof(GradT) == 2) {
      uint2 raw = reinterpret_cast<const uint2*>(grad)[i];
      float2 a0 = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&raw.x));
      float2 a1 = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&raw.y));
      g[0] = a0.x; g[1] = a0.y; g[2] = a1.x; g[3] = a1.y;
    } else {
      float4 t = reinterpret_cast<const float4*>(grad)[i];
      g[0] = t.x; g[1] = t.y; g[2] = t.z; g[3] = t.w;
    }
    float p[4] = {pw.x, pw.y, pw.z, pw.w}, m1[4] = {mm.x, mm.y, mm.z, mm.w}, v1[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
    for (int e = 0; e < 4; e++) {
      float gg = g[e] * gs;
      if (a.maximize) gg = -gg;
      p[e] *= decay;
      m1[e] = a.beta1 * m1[e] + (1.f - a.beta1) * gg;
      v1[e] = a.beta2 * v1[e] + (1.f - a.beta2) * gg * gg;
      const float denom = sqrtf(v1[e]) * inv_c2 + a.eps;
      p[e] -= step * m1[e] / denom;
    }
    reinterpret_cast<float4*>(master)[i] = make_float4(p[0], p[1], p[2], p[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(m1[0], m1[1], m1[2], m1[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(v1[0], v1[1], v1[2], v1[3]);
    if (p_bf16) {
      __nv_bfloat162 h0 = __floats2bfloat162_rn(p[0], p[1]), h1 = __floats2bfloat162_rn(p[2], p[3]);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&h0);
      o.y = *reinterpret_cast<uint32_t*>(&h1);
      reinterpret_cast<uint2*>(p_bf16)[i] = o;
    }
  }
  // scalar tail
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    size_t i = (nvec << 2) + threadIdx.x;
    float gg = (float)grad[i] * gs;
    if (a.maximize) gg = -gg;
    float p = master[i] * decay;
    float m1 = a.beta1 * m[i] + (1.f - a.beta1) * gg;
    float v1 = a.beta2 * v[i] + (1.f - a.beta2) * gg * gg;
    p -= step * m1 / (sqrtf(v1) * inv_c2 + a.eps);
    master[i] = p; m[i] = m1; v[i] = v1;
    if (p_bf16) p_bf16[i] = __float2bfloat16(p);
  }
}

struct SgdArgs { float lr, momentum, dampening, weight_decay; int nesterov, first_step, maximize; };

// Flat SGD with the reference's semantics: weight decay folded into the gradient, momentum buffer seeded with the
// first gradient, dampening and Nesterov as in PyTorch (ferrotorch-optim/src/sgd.rs:324-440).
template <typename GradT>
__global__ void sgd_kernel(float* __restrict__ master, __nv_bfloat16* __restrict__ p_bf16, float* __restrict__ buf,
                           const GradT* __restrict__ grad, size_t n, SgdArgs a, const float* __restrict__ grad_scale_ptr) {
  const float gs = grad_scale_ptr ? *grad_scale_ptr : 1.f;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float g = (float)grad[i] * gs;
    if (a.maximize) g = -g;
    float p = master[i];
    if (a.weight_decay != 0.f) g += a.weight_decay * p;
    if (a.momentum != 0.f) {
      float b = a.first_step ? g : a.momentum * buf[i] + (1.f - a.dampening) * g;
      buf[i] = b;
      g = a.nesterov ? g + a.momentum * b : b;
    }
    p -= a.lr * g;
    master[i] = p;
    if (p_bf16) p_bf16[i] = __float2bfloat16(p);
  }
}

// partial[blockIdx] = sum x^2 over this CTA's grid-stride range; non-finite values raise *found_inf.
template <typename T>
__global__ void sqnorm_partial_kernel(const T* __restrict__ x, size_t n, float* __restrict__ partial, int* __restrict__ found_inf) {
  __shared__ float red[32];
  float s = 0.f;
  bool bad = false;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float f = (float)x[i];
    bad |= !isfinite(f);
    s += f * f;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
  if (bad && found_inf) *found_inf = 1;
}

// total_sq (+)= sum partial; then, when finalize: norm = sqrt(total), clip_coef = min(1, max_norm/(norm+1e-6)).
__global__ void sqnorm_finish_kernel(const float* __restrict__ partial, int nparts, float* __restrict__ total_sq, int accumulate,
                                     int finalize, float max_norm, float* __restrict__ norm_out, float* __restrict__ clip_coef) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) s += partial[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) {
    float t = accumulate ? *total_sq + s : s;
    *total_sq = t;
    if (finalize) {
      float nrm = sqrtf(t);
      if (norm_out) *norm_out = nrm;
      if (clip_coef) *clip_coef = (max_norm > 0.f) ? fminf(1.f, max_norm / (nrm + 1e-6f)) : 1.f;
    }
  }
}

template <typename T>
__global__ void scale_inplace_kernel(T* __restrict__ x, size_t n, float scale, const float* __restrict__ scale_ptr) {
  const float s = scale_ptr ? scale * (*scale_ptr) : scale;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    x[i] = (T)((float)x[i] * s);
}

inline int flat_grid(size_t n, int block) {
  size_t g = (n + block - 1) / block;
  size_t cap = 148 * 8;
  return (int)(g < cap ? (g ? g : 1) : cap);
}

}  // namespace

// dtype: 0 = bf16 logits, 1 = f32 logits. dlogits may alias logits (in place) or be null (loss only).
FT_EXPORT int ft_cross_entropy(const void* logits, const int64_t* targets, float* loss_rows, float* lse_rows, void* dlogits, int rows,
                               int V, int64_t ld, int64_t ignore_index, float label_smoothing, float grad_scale,
                               const float* grad_scale_ptr, int dtype, cudaStream_t st) {
  if (rows <= 0 || V <= 0) return FT_ERR_ARG;
  if (dtype == 0) {
    if (ld % 8) return FT_ERR_ARG;
    cross_entropy_kernel<__nv_bfloat16><<<rows, CE_THREADS, 0, st>>>((const __nv_bfloat16*)logits, targets, loss_rows, lse_rows,
                                                                     (__nv_bfloat16*)dlogits, V, ld, ignore_index, label_smoothing,
                                                                     grad_scale, grad_scale_ptr);
  } else {
    if (ld % 4) return FT_ERR_ARG;
    cross_entropy_kernel<float><<<rows, CE_THREADS, 0, st>>>((const float*)logits, targets, loss_rows, lse_rows, (float*)dlogits, V, ld,
                                                             ignore_index, label_smoothing, grad_scale, grad_scale_ptr);
  }
  return (int)cudaGetLastError();
}

FT_EXPORT int ft_loss_mean(const float* loss_rows, const int64_t* targets, int rows, int64_t ignore_index, float* out_mean,
                           float* out_count, cudaStream_t st) {
  loss_mean_kernel<<<1, 1024, 0, st>>>(loss_rows, targets, rows, ignore_index, out_mean, out_count);
  return (int)cudaGetLastError();
}

// grad_dtype: 0 = bf16, 1 = f32. p_bf16 may be null. step >= 1.
// max_ctas > 0 caps the grid: a small grid (two CTAs per SM) keeps the kernel's register/thread footprint low enough that a
// persistent GEMM launched on another stream can always become resident beside it, which is what lets the optimizer run
// concurrently with backward instead of delaying it.
FT_EXPORT int ft_adamw_flat(float* master, void* p_bf16, float* m, float* v, const void* grad, int64_t n, int grad_dtype, float lr,
                            float beta1, float beta2, float eps, float weight_decay, int step, int maximize,
                            const float* grad_scale_ptr, const int* skip_ptr, int max_ctas, cudaStream_t st) {
  if (n <= 0 || step < 1) return FT_ERR_ARG;
  AdamWArgs a{lr, beta1, beta2, eps, weight_decay, 1.f - powf(beta1, (float)step), 1.f - powf(beta2, (float)step), maximize};
  int grid = flat_grid(((size_t)n + 3) / 4, 256);
  static bool configured = false;
  static int resident[2] = {8, 8};          // CTAs of each instantiation that fit one SM
  if (!configured) {
    ft_prefer_max_shared(adamw_kernel<__nv_bfloat16>);
    ft_prefer_max_shared(adamw_kernel<float>);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident[0], adamw_kernel<__nv_bfloat16>, 256, 0) != cudaSuccess || resident[0] < 1) resident[0] = 8;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident[1], adamw_kernel<float>, 256, 0) != cudaSuccess || resident[1] < 1) resident[1] = 8;
    cudaGetLastError();
    configured = true;
  }
  // one wave: with the grid-stride loop a partial second wave (1184 CTAs against 888 resident at 40 registers) ran its last third of the
  // data at a third of the memory parallelism (0.78 of the copy bandwidth in the profile of the 64 M parameter case)
  const int wave = 148 * resident[grad_dtype == 0 ? 0 : 1];
  if (grid > wave) grid = wave;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  if (grad_dtype == 0)
    adamw_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(master, (__nv_bfloat16*)p_bf16, m, v, (const __nv_bfloat16*)grad, (size_t)n, a,
                                                      grad_scale_ptr, skip_ptr);
  else
    adamw_kernel<float><<<grid, 256, 0, st>>>(master, (__nv_bfloat16*)p_bf16, m, v, (const float*)grad, (size_t)n, a, grad_scale_ptr,
                                              skip_ptr);
  return (int)cudaGetLastError();
}

FT_EXPORT int ft_sgd_flat(float* master, void* p_bf16, float* buf, const void* grad, int64_t n, int grad_dtype, float lr, float momentum,
                          float dampening, float weight_decay, int nesterov, int first_step, int maximize,
                          const float* grad_scale_ptr, cudaStream_t st) {
  if (n <= 0) return FT_ERR_ARG;
  SgdArgs a{lr, momentum, dampening, weight_decay, nesterov, first_step, maximize};
  int grid = flat_grid((size_t)n, 256);
  if (grad_dtype == 0)
    sgd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(master, (__nv_bfloat16*)p_bf16, buf, (const __nv_bfloat16*)grad, (size_t)n, a,
                                                    grad_scale_ptr);
  else
    sgd_kernel<float><<<grid, 256, 0, st>>>(master, (__nv_bfloat16*)p_bf16, buf, (const float*)grad, (size_t)n, a, grad_scale_ptr);
  return (int)cudaGetLastError();
}

// Squared L2 norm of a flat buffer into *total_sq (device). `partial` is scratch of >= 1184 floats.
// accumulate != 0 adds to the value already in *total_sq (multi-buffer norms); finalize != 0 also writes
// norm_out = sqrt(total) and clip_coef = min(1, max_norm/(norm+1e-6)).
FT_EXPORT int ft_sqnorm(const void* x, int64_t n, int dtype, float* partial, float* total_sq, int accumulate, int finalize,
                        float max_norm, float* norm_out, float* clip_coef, int* found_inf, cudaStream_t st) {
  if (n <= 0) return FT_ERR_ARG;
  int grid = flat_grid((size_t)n, 512);
  if (dtype == 0) sqnorm_partial_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>((const __nv_bfloat16*)x, (size_t)n, partial, found_inf);
  else sqnorm_partial_kernel<float><<<grid, 512, 0, st>>>((const float*)x, (size_t)n, partial, found_inf);
  sqnorm_finish_kernel<<<1, 1024, 0, st>>>(partial, grid, total_sq, accumulate, finalize, max_norm, norm_out, clip_coef);
  return (int)cudaGetLastError();
}

FT_EXPORT int ft_scale_inplace(void* x, int64_t n, int dtype, float scale, const float* scale_ptr, cudaStream_t st) {
  if (n <= 0) return FT_ERR_ARG;
  int grid = flat_grid((size_t)n, 256);
  if (dtype == 0) scale_inplace_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((__nv_bfloat16*)x, (size_t)n, scale, scale_ptr);
  else scale_inplace_kernel<float><<<grid, 256, 0, st>>>((float*)x, (size_t)n, scale, scale_ptr);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------------------
// One element-wise kernel for the optimizers that are a per-element recurrence over up to three state buffers:
// Adagrad, RMSprop, Adadelta, Adamax, NAdam, RAdam, Rprop, ASGD (ferrotorch-optim/src/{adagrad,rmsprop,adadelta,adamax,nadam,radam,rprop,
// asgd}.rs run these as chains of tensor operations, a dozen launches per parameter). The step-dependent scalars (bias corrections,
// decayed learning rates, the NAdam momentum products, the RAdam rectification) are computed on the host and arrive in `h`.
// ---------------------------------------------------------------------------------------------------------
namespace {
struct OptHp { float v[12]; };
enum OptAlgo : int { OPT_ADAGRAD = 0, OPT_RMSPROP = 1, OPT_ADADELTA = 2, OPT_ADAMAX = 3, OPT_NADAM = 4, OPT_RADAM = 5, OPT_RPROP = 6, OPT_ASGD = 7 };

template <int ALGO>
__global__ void foreach_opt_kernel(float* __restrict__ p, const float* __restrict__ grad, float* __restrict__ s0, float* __restrict__ s1,
                                   float* __restrict__ s2, size_t n, OptHp h, float gsign) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float w = p[i], g = grad[i] * gsign;
    if constexpr (ALGO == OPT_ADAGRAD) {            // h: clr, wd, eps
      g += h.v[1] * w;
      const float s = s0[i] + g * g;
      s0[i] = s;
      w -= h.v[0] * g / (sqrtf(s) + h.v[2]);
    } else if constexpr (ALGO == OPT_RMSPROP) {     // h: lr, alpha, eps, wd, momentum, centered
      g += h.v[3] * w;
      const float sq = h.v[1] * s0[i] + (1.f - h.v[1]) * g * g;
      s0[i] = sq;
      float avg;
      if (h.v[5] != 0.f) {
        const float ga = h.v[1] * s2[i] + (1.f - h.v[1]) * g;
        s2[i] = ga;
        avg = sqrtf(sq - ga * ga) + h.v[2];
      } else {
        avg = sqrtf(sq) + h.v[2];
      }
      if (h.v[4] > 0.f) {
        const float b = h.v[4] * s1[i] + g / avg;
        s1[i] = b;
        w -= h.v[0] * b;
      } else {
        w -= h.v[0] * g / avg;
      }
    } else if constexpr (ALGO == OPT_ADADELTA) {    // h: lr, rho, eps, wd
      g += h.v[3] * w;
      const float sq = h.v[1] * s0[i] + (1.f - h.v[1]) * g * g;
      s0[i] = sq;
      const float delta = sqrtf(s1[i] + h.v[2]) / sqrtf(sq + h.v[2]) * g;
      s1[i] = h.v[1] * s1[i] + (1.f - h.v[1]) * delta * delta;
      w -= h.v[0] * delta;
    } else if constexpr (ALGO == OPT_ADAMAX) {      // h: clr = lr / (1 - b1^t), b1, b2, eps, wd
      g += h.v[4] * w;
      const float m = h.v[1] * s0[i] + (1.f - h.v[1]) * g;
      const float u = fmaxf(h.v[2] * s1[i], fabsf(g) + h.v[3]);
      s0[i] = m;
      s1[i] = u;
      w -= h.v[0] * m / u;
    } else if constexpr (ALGO == OPT_NADAM) {       // h: c_grad, c_mom, b1, b2, eps, wd (coupled), bc2, decay factor (decoupled)
      w *= h.v[7];
      g += h.v[5] * w;
      const float m = h.v[2] * s0[i] + (1.f - h.v[2]) * g;
      const float v = h.v[3] * s1[i] + (1.f - h.v[3]) * g * g;
      s0[i] = m;
      s1[i] = v;
      const float den = sqrtf(v / h.v[6]) + h.v[4];
      w -= h.v[0] * g / den;
      w -= h.v[1] * m / den;
    } else if constexpr (ALGO == OPT_RADAM) {       // h: lr, b1, b2, eps, wd (coupled), bc1, bc2, rect (0: not rectified), decay factor (decoupled)
      w *= h.v[8];
      g += h.v[4] * w;
      const float m = h.v[1] * s0[i] + (1.f - h.v[1]) * g;
      const float v = h.v[2] * s1[i] + (1.f - h.v[2]) * g * g;
      s0[i] = m;
      s1[i] = v;
      const float mh = m / h.v[5];
      if (h.v[7] != 0.f) w -= h.v[0] * mh * h.v[7] * sqrtf(h.v[6]) / (sqrtf(v) + h.v[3]);
      else w -= h.v[0] * mh;
    } else if constexpr (ALGO == OPT_RPROP) {       // h: eta-, eta+, step min, step max
      const float sgn = g * s0[i];
      float st = s1[i];
      if (sgn > 0.f) st = fminf(st * h.v[1], h.v[3]);
      else if (sgn < 0.f) { st = fmaxf(st * h.v[0], h.v[2]); g = 0.f; }
      s1[i] = st;
      s0[i] = g;
      w -= (g > 0.f ? st : (g < 0.f ? -st : 0.f));
    } else {                                        // ASGD; h: eta, lambd, wd, mu
      g += h.v[2] * w;
      w *= 1.f - h.v[1] * h.v[0];
      w -= h.v[0] * g;
      s0[i] = h.v[3] != 1.f ? s0[i] + (w - s0[i]) * h.v[3] : w;
    }
    p[i] = w;
  }
}
}  // namespace

// algo: 0 Adagrad, 1 RMSprop, 2 Adadelta, 3 Adamax, 4 NAdam, 5 RAdam, 6 Rprop, 7 ASGD. p, grad: f32 [n]; s0..s2: the algorithm's state buffers
// (unused ones may be null); hp: HOST array of 12 floats, the per-step scalars in the order documented beside each branch of the kernel;
// maximize != 0 negates the gradient.
FT_EXPORT int ft_foreach_opt(int algo, float* p, const float* grad, float* s0, float* s1, float* s2, int64_t n, const float* hp, int maximize,
                             cudaStream_t st) {
  if (n <= 0 || hp == nullptr || algo < 0 || algo > 7) return FT_ERR_ARG;
  OptHp h;
  for (int i = 0; i < 12; i++) h.v[i] = hp[i];
  const int grid = flat_grid((size_t)n, 256);
  const float gs = maximize ? -1.f : 1.f;
#define FT_OPT_CASE(A) case A: foreach_opt_kernel<A><<<grid, 256, 0, st>>>(p, grad, s0, s1, s2, (size_t)n, h, gs); break;
  switch (algo) {
    FT_OPT_CASE(0) FT_OPT_CASE(1) FT_OPT_CASE(2) FT_OPT_CASE(3) FT_OPT_CASE(4) FT_OPT_CASE(5) FT_OPT_CASE(6) FT_OPT_CASE(7)
  }
#undef FT_OPT_CASE
  return (int)cudaGetLastError();
}
