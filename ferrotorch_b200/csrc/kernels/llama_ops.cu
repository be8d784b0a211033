// Bandwidth-bound transformer pieces: half-rotation RoPE (in place, forward and
// inverse), fused SwiGLU forward/backward on the [gate|up] GEMM output,
// embedding gather and its scatter-add backward, residual add.
//
// Capability parity: ROPE_HALF_BF16_PTX (ferrotorch-gpu/src/bf16.rs:1438) and RoPEBackward
// (ferrotorch-nn/src/transformer.rs:503); SILU/MUL_BF16 (bf16.rs:43,165); EMBEDDING_GATHER (bf16.rs:606,763),
// SCATTER_ADD_ROWS (ferrotorch-gpu/src/kernels.rs:1218); ADD (kernels.rs:188,239).
#include "common.cuh"
#include "host_common.h"

namespace {

// x: [tokens, row_stride] bf16; heads [head0, head0+nheads) of width D are rotated in place.
// cos/sin: [max_pos, D/2] f32. pos = positions ? positions[t] : (t % seq_len).
// sign = +1 forward, -1 inverse rotation (the backward of RoPE).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cs, const float* __restrict__ sn,
                            const int* __restrict__ positions, int tokens, int seq_len, int row_stride, int nheads, int D,
                            float sign) {
  const int half = D >> 1;
  const int vec_per_head = half >> 3;  // 8 bf16 per vector on each half
  const size_t total = (size_t)tokens * nheads * vec_per_head;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int v = (int)(i % vec_per_head);
    const int h = (int)((i / vec_per_head) % nheads);
    const int t = (int)(i / ((size_t)vec_per_head * nheads));
    const int pos = positions ? positions[t] : (t % seq_len);
    __nv_bfloat16* base = x + (size_t)t * row_stride + (size_t)h * D + v * 8;
    bf16x8 lo = *reinterpret_cast<bf16x8*>(base);
    bf16x8 hi = *reinterpret_cast<bf16x8*>(base + half);
    float a[8], b[8], c[8], s[8];
    bf16x8_to_float(lo, a);
    bf16x8_to_float(hi, b);
    const float4* cp = reinterpret_cast<const float4*>(cs + (size_t)pos * half + v * 8);
    const float4* sp = reinterpret_cast<const float4*>(sn + (size_t)pos * half + v * 8);
    float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
    c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
    s[0] = s0.x; s[1] = s0.y; s[2] = s0.z; s[3] = s0.w; s[4] = s1.x; s[5] = s1.y; s[6] = s1.z; s[7] = s1.w;
    float o1[8], o2[8];
#pragma unroll
    for (int e = 0; e < 8; e++) {
      float sg = sign * s[e];
      o1[e] = a[e] * c[e] - b[e] * sg;
      o2[e] = b[e] * c[e] + a[e] * sg;
    }
    *reinterpret_cast<bf16x8*>(base) = float_to_bf16x8(o1);
    *reinterpret_cast<bf16x8*>(base + half) = float_to_bf16x8(o2);
  }
}

// gu: [rows, 2F] (gate = cols [0,F), up = cols [F,2F)); out[r,c] = silu(gate)*up
// IDX is the type of the flat (row, vector) index: 32-bit whenever rows * F / 8 fits (a 64-bit divide per element costs as much as the math).
// The sigmoid uses the fast reciprocal (2 ulp): the result is rounded to bf16 anyway, and the kernel is close to issue-bound otherwise.
template <typename IDX>
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int rows, int F) {
  const IDX vecs = (IDX)(F >> 3);
  const IDX total = (IDX)rows * vecs;
  for (IDX i = (IDX)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (IDX)gridDim.x * blockDim.x) {
    const IDX r = i / vecs;
    const int c = (int)(i - r * vecs) * 8;
    const __nv_bfloat16* row = gu + (size_t)r * 2 * F;
    float g[8], u[8], o[8];
    bf16x8_to_float(*reinterpret_cast<const bf16x8*>(row + c), g);
    bf16x8_to_float(*reinterpret_cast<const bf16x8*>(row + F + c), u);
#pragma unroll
    for (int e = 0; e < 8; e++) o[e] = __fdividef(g[e], 1.f + __expf(-g[e])) * u[e];
    *reinterpret_cast<bf16x8*>(out + (size_t)r * F + c) = float_to_bf16x8(o);
  }
}

// dgu[r, :F] = dout * up * dsilu(gate) ; dgu[r, F:] = dout * silu(gate). May run in place (dgu == gu).
template <typename IDX>
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* gu, const __nv_bfloat16* __restrict__ dout, __nv_bfloat16* dgu, int rows,
                                  int F) {
  const IDX vecs = (IDX)(F >> 3);
  const IDX total = (IDX)rows * vecs;
  for (IDX i = (IDX)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (IDX)gridDim.x * blockDim.x) {
    const IDX r = i / vecs;
    const int c = (int)(i - r * vecs) * 8;
    const size_t ro = (size_t)r * 2 * F;
    float g[8], u[8], d[8], dg[8], du[8];
    bf16x8_to_float(*reinterpret_cast<const bf16x8*>(gu + ro + c), g);
    bf16x8_to_float(*reinterpret_cast<const bf16x8*>(gu + ro + F + c), u);
    bf16x8_to_float(*reinterpret_cast<const bf16x8*>(dout + (size_t)r * F + c), d);
#pragma unroll
    for (int e = 0; e < 8; e++) {
      float sg = __fdividef(1.f, 1.f + __expf(-g[e]));
      float silu = g[e] * sg;
      du[e] = d[e] * silu;
      dg[e] = d[e] * u[e] * (sg + silu * (1.f - sg));
    }
    *reinterpret_cast<bf16x8*>(dgu + ro + c) = float_to_bf16x8(dg);
    *reinterpret_cast<bf16x8*>(dgu + ro + F + c) = float_to_bf16x8(du);
  }
}

// out[t,:] = table[ids[t],:]; ids outside [0,vocab) produce zeros and set *oob (if given).
__global__ void embedding_fwd_kernel(const int64_t* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, int tokens, int d, int64_t vocab, int* oob) {
  const int vecs = d >> 3;
  const size_t total = (size_t)tokens * vecs;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / vecs;
    const int c = (int)(i % vecs) * 8;
    const int64_t id = ids[t];
    bf16x8 v;
    if (id >= 0 && id < vocab) {
      v = *reinterpret_cast<const bf16x8*>(table + (size_t)id * d + c);
    } else {
#pragma unroll
      for (int e = 0; e < 4; e++) v.v[e] = __floats2bfloat162_rn(0.f, 0.f);
      if (oob) *oob = 1;
    }
    *reinterpret_cast<bf16x8*>(out + t * d + c) = v;
  }
}

// dtable[ids[t],:] += dout[t,:]  (f32 accumulation table or bf16x2 atomics)
template <typename AccT>
__global__ void embedding_bwd_kernel(const int64_t* __restrict__ ids, const __nv_bfloat16* __restrict__ dout, AccT* __restrict__ dtable,
                                     int tokens, int d, int64_t vocab) {
  const int pairs = d >> 1;
  const size_t total = (size_t)tokens * pairs;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / pairs;
    const int c = (int)(i % pairs) * 2;
    const int64_t id = ids[t];
    if (id < 0 || id >= vocab) continue;
    __nv_bfloat162 g = *reinterpret_cast<const __nv_bfloat162*>(dout + t * d + c);
    if constexpr (sizeof(AccT) == 4) {
      float2 f = __bfloat1622float2(g);
      atomicAdd(reinterpret_cast<float*>(dtable) + (size_t)id * d + c, f.x);
      atomicAdd(reinterpret_cast<float*>(dtable) + (size_t)id * d + c + 1, f.y);
    } else {
      atomicAdd(reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(dtable) + (size_t)id * d + c), g);
    }
  }
}

// Deterministic form: the token rows are visited grouped by id (the caller sorted the ids stably and passes the permutation and the segment
// bounds), one CTA per distinct id, each output element summed in f32 in token order by one thread. No atomics: the same bits on every run.
template <typename AccT>
__global__ void __launch_bounds__(128) embedding_bwd_sorted_kernel(const int64_t* __restrict__ uniq_ids, const int64_t* __restrict__ seg_end,
                                                                   const int64_t* __restrict__ perm, const __nv_bfloat16* __restrict__ dout,
                                                                   AccT* __restrict__ dtable, int n_uniq, int d, int64_t vocab) {
  for (int u = blockIdx.x; u < n_uniq; u += gridDim.x) {
    const int64_t id = uniq_ids[u];
    if (id < 0 || id >= vocab) continue;
    const int64_t k0 = u == 0 ? 0 : seg_end[u - 1], k1 = seg_end[u];
    for (int c = threadIdx.x * 8; c < d; c += blockDim.x * 8) {
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; e++) acc[e] = (float)dtable[(size_t)id * d + c + e];        // running sum already in the table
      for (int64_t k = k0; k < k1; k++) {
        float f[8];
        bf16x8_to_float(*reinterpret_cast<const bf16x8*>(dout + (size_t)perm[k] * d + c), f);
#pragma unroll
        for (int e = 0; e < 8; e++) acc[e] += f[e];
      }
#pragma unroll
      for (int e = 0; e < 8; e++) dtable[(size_t)id * d + c + e] = (AccT)acc[e];
    }
  }
}

// out = a + b (bf16, 128-bit vectors, n % 8 == 0)
__global__ void add_bf16_kernel(const __nv_bfloat16* a, const __nv_bfloat16* b, __nv_bfloat16* out, size_t nvec) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
    float x[8], y[8];
    bf16x8_to_float(reinterpret_cast<const bf16x8*>(a)[i], x);
    bf16x8_to_float(reinterpret_cast<const bf16x8*>(b)[i], y);
#pragma unroll
    for (int e = 0; e < 8; e++) x[e] += y[e];
    reinterpret_cast<bf16x8*>(out)[i] = float_to_bf16x8(x);
  }
}

inline int grid_for(size_t work_items, int block) {
  size_t g = (work_items + block - 1) / block;
  size_t cap = 148 * 16;
  return (int)(g < cap ? (g ? g : 1) : cap);
}

}  // namespace

FT_EXPORT int ft_rope_inplace(void* x, const float* cos_t, const float* sin_t, const int* positions, int tokens, int seq_len,
                              int row_stride, int head0, int nheads, int D, int inverse, cudaStream_t st) {
  if (D % 16 || row_stride % 8 || tokens <= 0 || nheads <= 0) return FT_ERR_ARG;
  size_t total = (size_t)tokens * nheads * (D / 16);
  rope_kernel<<<grid_for(total, 256), 256, 0, st>>>((__nv_bfloat16*)x + (size_t)head0 * D, cos_t, sin_t, positions, tokens, seq_len,
                                                     row_stride, nheads, D, inverse ? -1.f : 1.f);
  return (int)cudaGetLastError();
}

FT_EXPORT int ft_swiglu_fwd(const void* gu, void* out, int rows, int F, cudaStream_t st) {
  if (F % 8 || rows <= 0) return FT_ERR_ARG;
  const size_t total = (size_t)rows * (F / 8);
  if (total + (size_t)grid_for(total, 256) * 256 < (1ull << 32))          // the loop counter may pass `total` by one grid stride
    swiglu_fwd_kernel<uint32_t><<<grid_for(total, 256), 256, 0, st>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, rows, F);
  else
    swiglu_fwd_kernel<size_t><<<grid_for(total, 256), 256, 0, st>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, rows, F);
  return (int)cudaGetLastError();
}

FT_EXPORT int ft_swiglu_bwd(const void* gu, const void* dout, void* dgu, int rows, int F, cudaStream_t st) {
  if (F % 8 || rows <= 0) return FT_ERR_ARG;
  const size_t total = (size_t)rows * (F / 8);
  if (total + (size_t)grid_for(total, 256) * 256 < (1ull << 32))
    swiglu_bwd_kernel<uint32_t><<<grid_for(total, 256), 256, 0, st>>>((const __nv_bfloat16*)gu, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dgu, rows, F);
  else
    swiglu_bwd_kernel<size_t><<<grid_for(total, 256), 256, 0, st>>>((const __nv_bfloat16*)gu, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dgu, rows, F);
  return (int)cudaGetLastError();
}

FT_EXPORT int ft_embedding_fwd(const int64_t* ids, const void* table, void* out, int tokens, int d, int64_t vocab, int* oob,
                               cudaStream_t st) {
  if (d % 8 || tokens <= 0) return FT_ERR_ARG;
  embedding_fwd_kernel<<<grid_for((size_t)tokens * (d / 8), 256), 256, 0, st>>>(ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out,
                                                                                 tokens, d, vocab, oob);
  return (int)cudaGetLastError();
}

// acc_f32 = 1: dtable is f32 [vocab,d]; 0: dtable is bf16 [vocab,d]. The caller zeroes dtable first.
FT_EXPORT int ft_embedding_bwd(const int64_t* ids, const void* dout, void* dtable, int tokens, int d, int64_t vocab, int acc_f32,
                               cudaStream_t st) {
  if (d % 2 || tokens <= 0) return FT_ERR_ARG;
  int grid = grid_for((size_t)tokens * (d / 2), 256);
  if (acc_f32)
    embedding_bwd_kernel<float><<<grid, 256, 0, st>>>(ids, (const __nv_bfloat16*)dout, (float*)dtable, tokens, d, vocab);
  else
    embedding_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(ids, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dtable, tokens, d, vocab);
  return (int)cudaGetLastError();
}

// uniq_ids [n_uniq]: the distinct ids in ascending order; seg_end [n_uniq]: inclusive prefix sums of their counts; perm [tokens]: token indices
// sorted stably by id (so perm[seg_end[u-1] .. seg_end[u]) are the tokens of uniq_ids[u] in their original order). d % 8 == 0.
FT_EXPORT int ft_embedding_bwd_sorted(const int64_t* uniq_ids, const int64_t* seg_end, const int64_t* perm, const void* dout, void* dtable, int n_uniq,
                                      int d, int64_t vocab, int acc_f32, cudaStream_t st) {
  if (d % 8 || n_uniq <= 0) return FT_ERR_ARG;
  const int grid = n_uniq < 148 * 16 ? n_uniq : 148 * 16;
  if (acc_f32)
    embedding_bwd_sorted_kernel<float><<<grid, 128, 0, st>>>(uniq_ids, seg_end, perm, (const __nv_bfloat16*)dout, (float*)dtable, n_uniq, d, vocab);
  else
    embedding_bwd_sorted_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(uniq_ids, seg_end, perm, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dtable, n_uniq, d, vocab);
  return (int)cudaGetLastError();
}

FT_EXPORT int ft_add_bf16(const void* a, const void* b, void* out, int64_t n, cudaStream_t st) {
  if (n % 8 || n <= 0) return FT_ERR_ARG;
  add_bf16_kernel<<<grid_for((size_t)n / 8, 256), 256, 0, st>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)out,
                                                                 (size_t)n / 8);
  return (int)cudaGetLastError();
}
