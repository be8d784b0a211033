// Non-maximum suppression on the device: a pairwise suppression bit-mask (64 x 64 box blocks) followed by a single-CTA sequential sweep that
// keeps the result on the device (no mask round trip through the host).
// Capability parity: ferrotorch-vision/src/ops.rs:209 (nms), restated as CUDA kernels.
#include <cuda_runtime.h>

#include <cstdint>

#include "common.cuh"
#include "host_common.h"

namespace {

// Every product, sum and the quotient are individually rounded (no fused multiply-add, no approximate division), so the value equals the host
// sweep's bit for bit and a pair sitting exactly at the threshold is classified the same way on both.
FT_DEVICE float iou_of(const float4 a, const float4 b) {
  const float w = fmaxf(fminf(a.z, b.z) - fmaxf(a.x, b.x), 0.f), h = fmaxf(fminf(a.w, b.w) - fmaxf(a.y, b.y), 0.f);
  const float inter = __fmul_rn(w, h);
  const float area_a = __fmul_rn(a.z - a.x, a.w - a.y), area_b = __fmul_rn(b.z - b.x, b.w - b.y);
  return __fdiv_rn(inter, __fsub_rn(__fadd_rn(area_a, area_b), inter));
}

// mask[i * words + w] bit b = box (w*64+b) is suppressed by box i (only j > i are set). grid (words, words), 64 threads.
__global__ void __launch_bounds__(64) nms_mask_kernel(const float4* __restrict__ boxes, int n, float thr, unsigned long long* __restrict__ mask) {
  const int row_blk = blockIdx.y, col_blk = blockIdx.x, words = gridDim.x;
  if (row_blk > col_blk) return;
  __shared__ float4 cols[64];
  const int cj = col_blk * 64 + threadIdx.x;
  if (cj < n) cols[threadIdx.x] = boxes[cj];
  __syncthreads();
  const int i = row_blk * 64 + threadIdx.x;
  if (i >= n) return;
  const float4 me = boxes[i];
  unsigned long long bits = 0;
  const int ncol = min(64, n - col_blk * 64);
  for (int b = (row_blk == col_blk) ? threadIdx.x + 1 : 0; b < ncol; b++)
    if (iou_of(me, cols[b]) > thr) bits |= 1ull << b;
  mask[(size_t)i * words + col_blk] = bits;
}

// keep[i] = 1 for survivors (boxes sorted by decreasing score); one CTA, the removed-set lives in shared memory
__global__ void __launch_bounds__(256) nms_sweep_kernel(const unsigned long long* __restrict__ mask, int n, int words, uint8_t* __restrict__ keep, int* __restrict__ num_kept) {
  extern __shared__ unsigned long long removed[];
  for (int w = threadIdx.x; w < words; w += 256) removed[w] = 0;
  __shared__ int alive;
  int kept = 0;
  __syncthreads();
  for (int i = 0; i < n; i++) {
    if (threadIdx.x == 0) alive = !((removed[i >> 6] >> (i & 63)) & 1ull);
    __syncthreads();
    const int a = alive;
    if (a) {
      for (int w = (i >> 6) + threadIdx.x; w < words; w += 256) removed[w] |= mask[(size_t)i * words + w];
      kept++;
    }
    if (threadIdx.x == 0) keep[i] = (uint8_t)a;
    __syncthreads();
  }
  if (threadIdx.x == 0 && num_kept) *num_kept = kept;
}

}  // namespace

// boxes: f32 [n, 4] sorted by decreasing score (16-byte aligned); mask scratch: n * ceil(n/64) u64; keep: u8 [n]; num_kept: optional device int.
FT_EXPORT int ft_nms_sorted(const float* boxes, int n, float iou_threshold, void* mask_scratch, void* keep, int* num_kept, cudaStream_t st) {
  if (n < 1) return n == 0 ? 0 : FT_ERR_ARG;
  const int words = (n + 63) / 64;
  if ((size_t)words * 8 > 200 * 1024) return FT_ERR_TOO_LARGE;            // the sweep keeps one bit per box in shared memory
  if (reinterpret_cast<uintptr_t>(boxes) & 15) return FT_ERR_ARG;
  FT_CUDA_TRY(cudaMemsetAsync(mask_scratch, 0, (size_t)n * words * 8, st));
  nms_mask_kernel<<<dim3(words, words), 64, 0, st>>>((const float4*)boxes, n, iou_threshold, (unsigned long long*)mask_scratch);
  static bool configured = false;
  if (!configured) {
    FT_CUDA_TRY(cudaFuncSetAttribute(nms_sweep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    configured = true;
  }
  nms_sweep_kernel<<<1, 256, (size_t)words * 8, st>>>((const unsigned long long*)mask_scratch, n, words, (uint8_t*)keep, num_kept);
  return (int)cudaGetLastError();
}
