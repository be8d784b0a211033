// Exact-precision GEMM / GEMV on the FMA pipes for f32 and f64 (the tensor-core path rounds operands to bf16 / fp16): register-tiled
// 64 x 64 x 16 shared-memory kernel, strided-batched, either operand optionally transposed, C = alpha * op(A) op(B) + beta * C.
// Also dot / matrix-vector products (one warp per row, vector loads).
//
// Capability parity: the sgemm / dgemm, strided-batched, dot / mv / vm wrappers of ferrotorch-gpu/src/blas.rs:67-1428 and the naive small-matrix
// kernels ferrotorch-gpu/src/kernels.rs:835,16762,16846 (SMALL_MATMUL).
#include <cuda_runtime.h>

#include "common.cuh"
#include "host_common.h"

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

// op(A)[m][k]: ta == 0 -> A[m * lda + k], ta == 1 -> A[k * lda + m]; same for B with (k, n).
template <typename T>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const T* __restrict__ A, const T* __restrict__ B, T* __restrict__ C, int M, int N, int K, int64_t lda, int64_t ldb,
                                                        int64_t ldc, int64_t sA, int64_t sB, int64_t sC, int ta, int tb, T alpha, T beta) {
  __shared__ T As[TK][TM + 1], Bs[TK][TN + 1];
  const int bz = blockIdx.z;
  A += (size_t)bz * sA;
  B += (size_t)bz * sB;
  C += (size_t)bz * sC;
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;       // each thread owns a 4 x 4 patch
  T acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += TK) {
    for (int i = threadIdx.x; i < TM * TK; i += 256) {
      const int m = ta ? i % TM : i / TK, k = ta ? i / TM : i % TK;       // walk the contiguous dimension fastest
      const int gm = m0 + m, gk = k0 + k;
      As[k][m] = (gm < M && gk < K) ? (ta ? A[(size_t)gk * lda + gm] : A[(size_t)gm * lda + gk]) : T(0);
    }
    for (int i = threadIdx.x; i < TN * TK; i += 256) {
      const int n = tb ? i / TK : i % TN, k = tb ? i % TK : i / TN;
      const int gn = n0 + n, gk = k0 + k;
      Bs[k][n] = (gn < N && gk < K) ? (tb ? B[(size_t)gn * ldb + gk] : B[(size_t)gk * ldb + gn]) : T(0);
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TK; k++) {
      T a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; i++) { a[i] = As[k][ty * 4 + i]; b[i] = Bs[k][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] += a[i] * b[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int gn = n0 + tx * 4 + j;
      if (gn < N) {
        T* c = C + (size_t)gm * ldc + gn;
        *c = beta == T(0) ? alpha * acc[i][j] : alpha * acc[i][j] + beta * *c;
      }
    }
  }
}

// y[r] = alpha * dot(A[r, :], x) + beta * y[r]; one warp per row
template <typename T>
__global__ void __launch_bounds__(256) gemv_kernel(const T* __restrict__ A, const T* __restrict__ x, T* __restrict__ y, int rows, int cols, int64_t lda, T alpha, T beta) {
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= rows) return;
  const T* a = A + (size_t)r * lda;
  T acc = T(0);
  for (int c = lane; c < cols; c += 32) acc += a[c] * x[c];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) y[r] = beta == T(0) ? alpha * acc : alpha * acc + beta * y[r];
}

// y[c] = alpha * sum_r x[r] * A[r, c] + beta * y[c] (vector-matrix): thread per column, coalesced over c
template <typename T>
__global__ void __launch_bounds__(256) gevm_kernel(const T* __restrict__ A, const T* __restrict__ x, T* __restrict__ y, int rows, int cols, int64_t lda, T alpha, T beta) {
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= cols) return;
  T acc = T(0);
  for (int r = 0; r < rows; r++) acc += x[r] * A[(size_t)r * lda + c];
  y[c] = beta == T(0) ? alpha * acc : alpha * acc + beta * y[c];
}

}  // namespace

// dtype 0 = f32, 3 = f64. C[b] = alpha * op(A[b]) op(B[b]) + beta * C[b]; strides between batches in elements (0 broadcasts an operand).
FT_EXPORT int ft_gemm_simt(int dtype, const void* A, const void* B, void* C, int batch, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int64_t sA,
                           int64_t sB, int64_t sC, int ta, int tb, double alpha, double beta, cudaStream_t st) {
  if (batch < 1 || M < 1 || N < 1 || K < 1 || batch > 65535) return FT_ERR_ARG;
  const dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM, batch);
  if (grid.y > 65535) return FT_ERR_ARG;
  if (dtype == 0) gemm_simt_kernel<float><<<grid, 256, 0, st>>>((const float*)A, (const float*)B, (float*)C, M, N, K, lda, ldb, ldc, sA, sB, sC, ta, tb, (float)alpha, (float)beta);
  else if (dtype == 3) gemm_simt_kernel<double><<<grid, 256, 0, st>>>((const double*)A, (const double*)B, (double*)C, M, N, K, lda, ldb, ldc, sA, sB, sC, ta, tb, alpha, beta);
  else return FT_ERR_ARG;
  return (int)cudaGetLastError();
}

// trans == 0: y[rows] = alpha * A x + beta * y; trans == 1: y[cols] = alpha * A^T x + beta * y. A is [rows, cols] row-major with pitch lda.
FT_EXPORT int ft_gemv(int dtype, const void* A, const void* x, void* y, int rows, int cols, int64_t lda, int trans, double alpha, double beta, cudaStream_t st) {
  if (rows < 1 || cols < 1) return FT_ERR_ARG;
#define FT_GEMV(T)                                                                                                                             \
  if (!trans) gemv_kernel<T><<<(rows + 7) / 8, 256, 0, st>>>((const T*)A, (const T*)x, (T*)y, rows, cols, lda, (T)alpha, (T)beta);             \
  else gevm_kernel<T><<<(cols + 255) / 256, 256, 0, st>>>((const T*)A, (const T*)x, (T*)y, rows, cols, lda, (T)alpha, (T)beta);
  if (dtype == 0) { FT_GEMV(float) }
  else if (dtype == 3) { FT_GEMV(double) }
  else return FT_ERR_ARG;
#undef FT_GEMV
  return (int)cudaGetLastError();
}
