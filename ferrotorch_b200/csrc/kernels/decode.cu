// Decode-path kernels for tensor-parallel LLM serving (small token batch, paged KV cache, block size 16).
//
// The projections run as split-K GEMMs (ft_gemm_bf16_splitk) that leave f32 partial planes P[s][token][n]; each kernel
// here consumes those planes directly, summing over s on the fly, so no stand-alone reduction pass exists:
//   ft_decode_qkv_rope_kvwrite   sum -> RoPE at each sequence's position -> q [B,Hq,D] bf16 and K/V written into their cache pages
//   ft_paged_attn_decode         one query token per sequence against the paged cache, GQA, split over the sequence; the last
//                                CTA of each (sequence, kv head) merges the splits (self-resetting counters, no extra launch)
//   ft_decode_swiglu             sum -> silu(gate)*up -> bf16
//   ft_decode_ar_residual_norm   row-parallel output: sum of planes -> one-shot all-reduce over NVLink peer memory (fixed rank
//                                order) -> + residual -> RMSNorm, in one kernel (the 128 KB-class all-reduce of TP decoding)
//   ft_splitk_reduce             generic plane sum (+bias) to bf16 or f32 (LM head logits)
//   ft_paged_kv_write            copy prefill K/V rows from the packed QKV buffer into cache pages
// Launch sequence numbers for the cross-GPU flags are read from device memory and advanced by the kernel itself, so the
// whole decode step can be captured once in a CUDA graph and replayed.
//
// Capability parity: KVPage/PagePool/PagedKVCache bookkeeping exists only on the CPU in the reference
// (ferrotorch-nn/src/paged_attention.rs:59-518); its GPU inferencer has no KV cache and re-prefills every token
// (ferrotorch-llama/examples/llama3_8b_gpu.rs:118-122, ferrotorch-llama/src/gpu.rs:518-700).
#include <cooperative_groups.h>

#include "common.cuh"
#include "host_common.h"

namespace {

constexpr int KV_BLOCK = 16;
constexpr int MAXR = 8;
constexpr uint64_t DEC_TIMEOUT_NS = 2000000000ull;

FT_DEVICE float plane_sum(const float* __restrict__ p, int splits, size_t plane_stride, size_t idx) {
  float a = 0.f;
  for (int s = 0; s < splits; s++) a += p[s * plane_stride + idx];
  return a;
}

// ------------------------------------------------------------------------------------------------------------
// generic plane sum
// ------------------------------------------------------------------------------------------------------------
template <typename OutT>
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, int splits, int rows, int N, int64_t ldp, size_t plane_stride,
                                     const __nv_bfloat16* __restrict__ bias, OutT* __restrict__ out, int64_t ldo) {
  pdl_wait();
  pdl_launch_dependents();
  const size_t total = (size_t)rows * N;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / N), n = (int)(i % N);
    float a = plane_sum(partial, splits, plane_stride, (size_t)r * ldp + n);
    if (bias) a += __bfloat162float(bias[n]);
    out[(size_t)r * ldo + n] = (OutT)a;
  }
}

// ------------------------------------------------------------------------------------------------------------
// QKV epilogue: plane sum + RoPE + q store + KV cache write
// grid (B, Hq + 2*Hkv), block D/2 threads: thread i owns the rotation pair (i, i + D/2)
// ------------------------------------------------------------------------------------------------------------
__global__ void qkv_rope_kvwrite_kernel(const float* __restrict__ partial, int splits, int64_t ldp, size_t plane_stride, int Hq, int Hkv,
                                        int D, const int* __restrict__ positions, const float* __restrict__ cos_t,
                                        const float* __restrict__ sin_t, __nv_bfloat16* __restrict__ q_out,
                                        __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                        const int* __restrict__ block_table, int max_blocks) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x, h = blockIdx.y, i = threadIdx.x, half = D >> 1;
  const int pos = positions[b];
  const size_t base = (size_t)b * ldp + (size_t)h * D;
  float lo = plane_sum(partial, splits, plane_stride, base + i);
  float hi = plane_sum(partial, splits, plane_stride, base + i + half);
  if (h < Hq + Hkv) {   // q and k heads are rotated, v heads are not
    const float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
    const float a = lo * c - hi * s, bb = hi * c + lo * s;
    lo = a;
    hi = bb;
  }
  if (h < Hq) {
    __nv_bfloat16* q = q_out + ((size_t)b * Hq + h) * D;
    q[i] = __float2bfloat16(lo);
    q[i + half] = __float2bfloat16(hi);
  } else {
    const int blk = block_table[(size_t)b * max_blocks + pos / KV_BLOCK];
    if (blk < 0) return;
    const bool is_k = h < Hq + Hkv;
    const int kvh = is_k ? h - Hq : h - Hq - Hkv;
    __nv_bfloat16* dst = (is_k ? k_cache : v_cache) + (((size_t)blk * KV_BLOCK + pos % KV_BLOCK) * Hkv + kvh) * D;
    dst[i] = __float2bfloat16(lo);
    dst[i + half] = __float2bfloat16(hi);
  }
}

// prefill: rows of the packed qkv buffer [tokens, ld] (token t of sequence b at row b*S + t) -> cache pages
__global__ void paged_kv_write_kernel(const __nv_bfloat16* __restrict__ qkv, int64_t ld, int S, int Hq, int Hkv, int D,
                                      __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                      const int* __restrict__ block_table, int max_blocks, int pos0) {
  const int t = blockIdx.x, b = blockIdx.y;
  const int vec = (Hkv * D) / 8;
  const int pos = pos0 + t;
  const int blk = block_table[(size_t)b * max_blocks + pos / KV_BLOCK];
  if (blk < 0) return;
  const __nv_bfloat16* row = qkv + ((size_t)b * S + t) * ld;
  const size_t dst = ((size_t)blk * KV_BLOCK + pos % KV_BLOCK) * Hkv * D;
  for (int i = threadIdx.x; i < vec; i += blockDim.x) {
    reinterpret_cast<bf16x8*>(k_cache + dst)[i] = reinterpret_cast<const bf16x8*>(row + (size_t)Hq * D)[i];
    reinterpret_cast<bf16x8*>(v_cache + dst)[i] = reinterpret_cast<const bf16x8*>(row + (size_t)(Hq + Hkv) * D)[i];
  }
}

// ------------------------------------------------------------------------------------------------------------
// paged decode attention (D = 128, group size G = Hq/Hkv <= 8)
// grid (nsplit, Hkv, B), 128 threads. Workspace per (b, kvh, split, g): PA_WS_ROW floats = 128 accumulators, running max, running sum, 2 pad.
// counters: int [B*Hkv], zero before the first launch (the kernel re-zeroes them).
// A CTA streams its token range through a three-stage shared-memory ring of 64-token K/V chunks filled by 16-byte cp.async copies
// (XOR-swizzled 16-byte columns), so the whole range is in flight after one page-table lookup. Each warp owns 16 tokens of a chunk:
// S = Q K^T and O += P V run on mma.sync m16n8k16 with the G query heads as the (zero-padded) M rows -- the decode shape has M = G <= 8,
// far below a tcgen05 tile, and the kernel is bound by the K/V stream, not by the tensor pipe.
// ------------------------------------------------------------------------------------------------------------
constexpr int PA_CHUNK = 64, PA_STAGES = 3;
constexpr int PA_STAGE_BYTES = PA_CHUNK * 128 * 2 * 2;       // K and V rows of one chunk
constexpr int PA_SMEM = PA_STAGES * PA_STAGE_BYTES;
constexpr int PA_WS_ROW = 132;
constexpr int PA_MAX_SPLIT = 64;

FT_DEVICE void cp_async16(uint32_t dst, const void* src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory"); }
FT_DEVICE void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
FT_DEVICE void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
FT_DEVICE void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
FT_DEVICE void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
FT_DEVICE void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
FT_DEVICE uint32_t pa_sw(int row, int chunk) { return (uint32_t)(row * 256 + ((chunk ^ (row & 7)) << 4)); }

__global__ void __launch_bounds__(128, 2) paged_attn_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                                                                const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_table,
                                                                int max_blocks, const int* __restrict__ seq_lens, int Hq, int Hkv, float scale,
                                                                float* __restrict__ ws, int* __restrict__ counters,
                                                                __nv_bfloat16* __restrict__ out) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int D = 128;
  extern __shared__ __align__(128) uint8_t pa_smem[];
  const int G = Hq / Hkv;
  const int split = blockIdx.x, nsplit = gridDim.x, kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int len = seq_lens[b];
  const int per = (((len + nsplit - 1) / nsplit) + KV_BLOCK - 1) / KV_BLOCK * KV_BLOCK;   // whole pages per split
  const int t0 = split * per, t1 = min(len, t0 + per);
  const int nchunks = t1 > t0 ? (t1 - t0 + PA_CHUNK - 1) / PA_CHUNK : 0;
  const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(pa_smem);
  const int* bt = block_table + (size_t)b * max_blocks;

  auto load_chunk = [&](int c, int stage) {
    const int c0 = t0 + c * PA_CHUNK, cnt = min(PA_CHUNK, t1 - c0);
    const uint32_t kdst = smem_base + stage * PA_STAGE_BYTES, vdst = kdst + PA_CHUNK * D * 2;
    for (int i = threadIdx.x; i < cnt * 16; i += 128) {            // 16 copies of 16 bytes per 256-byte row
      const int r = i >> 4, part = i & 15, t = c0 + r;
      const int blk = __ldg(bt + t / KV_BLOCK);
      const size_t off = (((size_t)blk * KV_BLOCK + t % KV_BLOCK) * Hkv + kvh) * D + part * 8;
      cp_async16(kdst + pa_sw(r, part), k_cache + off);
      cp_async16(vdst + pa_sw(r, part), v_cache + off);
    }
    // rows up to the next multiple of 16 feed the tensor cores with weight zero: they must hold finite values
    uint8_t* kz = pa_smem + stage * PA_STAGE_BYTES;
    for (int i = cnt * 16 + threadIdx.x; i < ((cnt + 15) & ~15) * 16; i += 128) {
      const int r = i >> 4, part = i & 15;
      *reinterpret_cast<uint4*>(kz + pa_sw(r, part)) = make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(kz + PA_CHUNK * D * 2 + pa_sw(r, part)) = make_uint4(0, 0, 0, 0);
    }
  };
#pragma unroll
  for (int s = 0; s < PA_STAGES; s++) {
    if (s < nchunks) load_chunk(s, s);
    cp_async_commit();
  }

  // A fragments of Q (rows = query heads of this KV head, rows >= G are zero): registers 0 and 2 of every k-step
  const int g_row = lane >> 2, qc = (lane & 3) * 2;
  uint32_t qf[8][2];
#pragma unroll
  for (int ks = 0; ks < 8; ks++) {
    qf[ks][0] = qf[ks][1] = 0u;
    if (g_row < G) {
      const __nv_bfloat16* qp = q + ((size_t)b * Hq + kvh * G + g_row) * D + ks * 16 + qc;
      qf[ks][0] = *reinterpret_cast<const uint32_t*>(qp);
      qf[ks][1] = *reinterpret_cast<const uint32_t*>(qp + 8);
    }
  }
  const float sl2 = scale * 1.4426950408889634f;
  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;                             // of head g_row; l_run is this thread's share of the row sum

  for (int c = 0; c < nchunks; c++) {
    cp_async_wait<PA_STAGES - 1>();
    __syncthreads();
    const int stage = c % PA_STAGES, cnt = min(PA_CHUNK, t1 - (t0 + c * PA_CHUNK));
    const uint32_t kbase = smem_base + stage * PA_STAGE_BYTES, vbase = kbase + PA_CHUNK * D * 2;
    const int r0 = warp * 16;
    if (r0 < cnt) {
      float sacc[2][4];
#pragma unroll
      for (int j = 0; j < 2; j++) sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.f;
      {
        const int row = r0 + (lane & 7) + ((lane >> 4) << 3), cb = (lane >> 3) & 1;
#pragma unroll
        for (int ks = 0; ks < 8; ks++) {
          uint32_t kb[4];
          ldmatrix_x4(kb, kbase + pa_sw(row, ks * 2 + cb));
          mma_16816(sacc[0], qf[ks][0], 0u, qf[ks][1], 0u, kb[0], kb[1]);
          mma_16816(sacc[1], qf[ks][0], 0u, qf[ks][1], 0u, kb[2], kb[3]);
        }
      }
      bool valid[2][2];
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 2; j++)
#pragma unroll
        for (int e = 0; e < 2; e++) {
          valid[j][e] = r0 + j * 8 + qc + e < cnt;
          if (valid[j][e]) mx = fmaxf(mx, sacc[j][e]);
        }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run, mx);                         // finite: the group holds at least one live token
      const float alpha = exp2f((m_run - m_new) * sl2);
      float p[2][2], psum = 0.f;
#pragma unroll
      for (int j = 0; j < 2; j++)
#pragma unroll
        for (int e = 0; e < 2; e++) {
          p[j][e] = valid[j][e] ? exp2f((sacc[j][e] - m_new) * sl2) : 0.f;
          psum += p[j][e];
        }
      l_run = l_run * alpha + psum;
      m_run = m_new;
#pragma unroll
      for (int i = 0; i < 16; i++) { o[i][0] *= alpha; o[i][1] *= alpha; }
      __nv_bfloat162 p0 = __floats2bfloat162_rn(p[0][0], p[0][1]), p1 = __floats2bfloat162_rn(p[1][0], p[1][1]);
      const uint32_t pa0 = *reinterpret_cast<uint32_t*>(&p0), pa2 = *reinterpret_cast<uint32_t*>(&p1);
      {
        const int row = r0 + (lane & 7) + (((lane >> 3) & 1) << 3), cb = lane >> 4;
#pragma unroll
        for (int dp = 0; dp < 8; dp++) {
          uint32_t vb[4];
          ldmatrix_x4_trans(vb, vbase + pa_sw(row, dp * 2 + cb));
          mma_16816(o[2 * dp], pa0, 0u, pa2, 0u, vb[0], vb[1]);
          mma_16816(o[2 * dp + 1], pa0, 0u, pa2, 0u, vb[2], vb[3]);
        }
      }
    }
    __syncthreads();                                                // the stage is free again
    if (c + PA_STAGES < nchunks) load_chunk(c + PA_STAGES, stage);
    cp_async_commit();
  }
  cp_async_wait<0>();
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  __syncthreads();
  // merge the four warps of this CTA (the ring is idle: its first bytes hold the per-warp accumulators)
  __shared__ float sm_m[4][8], sm_l[4][8];
  __shared__ int is_last;
  float (*sm_acc)[8][D] = reinterpret_cast<float (*)[8][D]>(pa_smem);
  if (g_row < G) {
    if ((lane & 3) == 0) { sm_m[warp][g_row] = m_run; sm_l[warp][g_row] = l_run; }
#pragma unroll
    for (int i = 0; i < 16; i++) *reinterpret_cast<float2*>(&sm_acc[warp][g_row][i * 8 + qc]) = make_float2(o[i][0], o[i][1]);
  }
  __syncthreads();
  float* my_ws = ws + (((size_t)b * Hkv + kvh) * nsplit + split) * G * PA_WS_ROW;
  for (int i = threadIdx.x; i < G * D; i += 128) {
    const int g = i / D, d = i % D;
    const float mm = fmaxf(fmaxf(sm_m[0][g], sm_m[1][g]), fmaxf(sm_m[2][g], sm_m[3][g]));
    float a = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < 4; w++) {
      const float f = (sm_m[w][g] == -INFINITY) ? 0.f : exp2f((sm_m[w][g] - mm) * sl2);
      a += sm_acc[w][g][d] * f;
      ll += sm_l[w][g] * f;
    }
    my_ws[g * PA_WS_ROW + d] = a;
    if (d == 0) { my_ws[g * PA_WS_ROW + D] = mm * scale; my_ws[g * PA_WS_ROW + D + 1] = ll; }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(&counters[b * Hkv + kvh], 1);
    is_last = (prev == nsplit - 1);
    if (is_last) counters[b * Hkv + kvh] = 0;     // ready for the next launch
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // the last CTA of this (sequence, KV head) combines the splits: first the weights f[s][g] and row sums, then one pass of float4 loads
  const float* base = ws + ((size_t)b * Hkv + kvh) * nsplit * G * PA_WS_ROW;
  float* sm_pm = reinterpret_cast<float*>(pa_smem + 32768);        // [nsplit * G] each, behind the warp accumulators
  float* sm_pl = sm_pm + PA_MAX_SPLIT * 8;
  float* sm_L = sm_pl + PA_MAX_SPLIT * 8;
  for (int i = threadIdx.x; i < nsplit * G; i += 128) {
    const float2 ml = __ldcg(reinterpret_cast<const float2*>(base + (size_t)i * PA_WS_ROW + D));
    sm_pm[i] = ml.x;
    sm_pl[i] = ml.y;
  }
  __syncthreads();
  if (threadIdx.x < G) {
    const int g = threadIdx.x;
    float mm = -INFINITY, ll = 0.f;
    for (int s = 0; s < nsplit; s++) mm = fmaxf(mm, sm_pm[s * G + g]);
    for (int s = 0; s < nsplit; s++) {
      const float pm = sm_pm[s * G + g];
      const float f = (pm == -INFINITY) ? 0.f : __expf(pm - mm);
      ll += sm_pl[s * G + g] * f;
      sm_pm[s * G + g] = f;
    }
    sm_L[g] = ll;
  }
  __syncthreads();
  // Each thread owns one float4 column of one query head per pass; the partials of sixteen splits are requested before any is used, with
  // the tail of the split range predicated rather than peeled, so that the pass costs ceil(nsplit / 16) memory round trips whatever
  // nsplit is (a peeled remainder loop issued its loads one after another: a round trip per leftover split).
  for (int i = threadIdx.x; i < G * (D / 4); i += 128) {
    const int g = i / (D / 4), d4 = (i % (D / 4)) * 4;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    const float* col = base + (size_t)g * PA_WS_ROW + d4;
    for (int s0 = 0; s0 < nsplit; s0 += 16) {
      float4 v[16];
#pragma unroll
      for (int j = 0; j < 16; j++)
        v[j] = (s0 + j < nsplit) ? __ldcg(reinterpret_cast<const float4*>(col + (size_t)(s0 + j) * G * PA_WS_ROW)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int j = 0; j < 16; j++) {
        const float f = (s0 + j < nsplit) ? sm_pm[(s0 + j) * G + g] : 0.f;
        a.x += v[j].x * f; a.y += v[j].y * f; a.z += v[j].z * f; a.w += v[j].w * f;
      }
    }
    const float inv = sm_L[g] > 0.f ? 1.f / sm_L[g] : 0.f;
    __nv_bfloat162 lo = __floats2bfloat162_rn(a.x * inv, a.y * inv), hi = __floats2bfloat162_rn(a.z * inv, a.w * inv);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&lo);
    pk.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(out + ((size_t)b * Hq + kvh * G + g) * D + d4) = pk;
  }
}

// ------------------------------------------------------------------------------------------------------------
// SwiGLU on split-K planes: P[s][b][0:F] = gate, P[s][b][F:2F] = up
// ------------------------------------------------------------------------------------------------------------
__global__ void decode_swiglu_kernel(const float* __restrict__ partial, int splits, int64_t ldp, size_t plane_stride, int rows, int F,
                                     __nv_bfloat16* __restrict__ out) {
  pdl_wait();
  pdl_launch_dependents();
  const size_t total = (size_t)rows * F;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / F), f = (int)(i % F);
    const float g = plane_sum(partial, splits, plane_stride, (size_t)r * ldp + f);
    const float u = plane_sum(partial, splits, plane_stride, (size_t)r * ldp + F + f);
    out[i] = __float2bfloat16(g / (1.f + __expf(-g)) * u);
  }
}

// ------------------------------------------------------------------------------------------------------------
// plane sum -> all-reduce (one shot, peer loads) -> + residual -> RMSNorm
//   grid = rows * chunks CTAs (all co-resident), 256 threads, each CTA owns `cols = d/chunks` columns of one token row.
//   sync block (device ints): [0] launch sequence, [1] grid barrier A counter, [2] grid barrier B counter (monotonic).
//   sym[r] = rank r's staging buffer: 2 slots x rows_pad x d floats (slot = sequence parity).
//   flags[r] = rank r's flag block: u32[MAXR], flags[r][q] = last sequence number rank q announced.
// ------------------------------------------------------------------------------------------------------------
struct ArNormArgs {
  float* sym[MAXR];
  uint32_t* flags[MAXR];
  int rank, world;
};

FT_DEVICE bool grid_barrier(int* ctr, int target, uint32_t* status, int site) {
  __syncthreads();
  bool ok = true;
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(ctr, 1);
    uint64_t t0 = globaltimer_ns();
    while (*reinterpret_cast<volatile int*>(ctr) < target) {
      if (globaltimer_ns() - t0 > DEC_TIMEOUT_NS) { ft_set_status(status, FT_K_COMM, site, blockIdx.x); ok = false; break; }
    }
    __threadfence();
  }
  __shared__ int ok_sh;
  if (threadIdx.x == 0) ok_sh = ok;
  __syncthreads();
  return ok_sh != 0;
}

__global__ void __launch_bounds__(256) decode_ar_residual_norm_kernel(const float* __restrict__ partial, int splits, int64_t ldp, size_t plane_stride,
                                                                      ArNormArgs a, int* __restrict__ sync, __nv_bfloat16* __restrict__ x,
                                                                      const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ h,
                                                                      float* __restrict__ sumsq, int rows, int rows_pad, int d, int chunks, float eps,
                                                                      uint32_t* status) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float red[32];
  const int row = blockIdx.x / chunks, chunk = blockIdx.x % chunks;
  const int cols = d / chunks, c0 = chunk * cols;
  const int seq = sync[0] + 1;                       // every CTA reads it before any barrier; CTA 0 advances it at the very end
  const int nctas = gridDim.x;
  const size_t slot = (size_t)(seq & 1) * rows_pad * d;
  // phase A: local plane sum into this rank's staging slot
  float* mine = a.sym[a.rank] + slot + (size_t)row * d + c0;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) mine[i] = plane_sum(partial, splits, plane_stride, (size_t)row * ldp + c0 + i);
  if (a.world > 1) {
    __threadfence_system();
    if (!grid_barrier(&sync[1], seq * nctas, status, 11)) return;
    if (blockIdx.x == 0 && threadIdx.x < a.world) st_release_sys(a.flags[threadIdx.x] + a.rank, (uint32_t)seq);
    bool ok = true;
    if (threadIdx.x < a.world) {
      ok = wait_flag_ge(a.flags[a.rank] + threadIdx.x, (uint32_t)seq, DEC_TIMEOUT_NS);
      if (!ok) ft_set_status(status, FT_K_COMM, 12, threadIdx.x);
    }
    if (__syncthreads_or(!ok)) return;
  }
  // phase B: cross-rank sum in fixed rank order + residual; row-wide sum of squares
  float ss = 0.f;
  __nv_bfloat16* xr = x + (size_t)row * d + c0;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) {
    float v = 0.f;
    for (int r = 0; r < a.world; r++) v += a.sym[r][slot + (size_t)row * d + c0 + i];
    v += __bfloat162float(xr[i]);
    const __nv_bfloat16 vb = __float2bfloat16(v);
    xr[i] = vb;
    const float vf = __bfloat162float(vb);
    ss += vf * vf;
  }
  ss = block_sum(ss, red);
  float* ssq = sumsq + (size_t)(seq & 1) * rows_pad * chunks;
  if (threadIdx.x == 0) ssq[row * chunks + chunk] = ss;
  if (!grid_barrier(&sync[2], seq * nctas, status, 13)) return;
  float tot = 0.f;
  for (int c = 0; c < chunks; c++) tot += ssq[row * chunks + c];
  const float rstd = rsqrtf(tot / (float)d + eps);
  __nv_bfloat16* hr = h + (size_t)row * d + c0;
  for (int i = threadIdx.x; i < cols; i += blockDim.x)
    hr[i] = __float2bfloat16(__bfloat162float(xr[i]) * rstd * __bfloat162float(w[c0 + i]));
  if (blockIdx.x == 0 && threadIdx.x == 0) sync[0] = seq;    // everybody is past barrier B, so nobody still needs the old value
}

// ------------------------------------------------------------------------------------------------------------
// plane sum -> all-reduce -> + residual -> RMSNorm, second form: no grid-wide barrier.
//   A thread-block cluster of AR_CL CTAs owns one token row (each CTA d / AR_CL columns). The cross-rank handshake is per (row, column chunk):
//   a CTA announces its chunk to every peer and waits only for the peers' same chunk; the row-wide sum of squares for the norm is combined
//   inside the cluster through distributed shared memory. A step of this kernel costs one launch, one peer round trip and two cluster barriers,
//   where the first form paid two grid barriers on top.
//   flags[r] = rank r's flag block u32[MAXR][rows_pad * AR_CL]: flags[r][q][row * AR_CL + chunk] = last launch number rank q announced.
//   sync: int[4] zeroed once: [0] launch number, [1] finished-CTA counter (self-resetting).
// ------------------------------------------------------------------------------------------------------------
constexpr int AR_CL = 4, AR_THREADS = 512;

// PUSH = false: every rank stages its own partial rows and reads the peers' staging buffers after the handshake (one flag trip plus one remote
// load trip). PUSH = true: every rank stores its partial rows into every peer's staging buffer (slot [rank] of a [world][rows_pad][d] layout)
// before it raises the flags, so after the handshake all operands are in local memory (one trip).
template <bool PUSH>
__global__ void __cluster_dims__(AR_CL, 1, 1) __launch_bounds__(AR_THREADS)
decode_ar_residual_norm_cluster_kernel(const float* __restrict__ partial, int splits, int64_t ldp, size_t plane_stride, ArNormArgs a, int* __restrict__ sync,
                                       __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ h, int rows, int rows_pad,
                                       int d, float eps, uint32_t* status) {
  namespace cg = cooperative_groups;
  pdl_wait();
  pdl_launch_dependents();
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ float red[32];
  __shared__ float cta_ss;
  const int row = blockIdx.x / AR_CL, chunk = blockIdx.x % AR_CL;
  const int cols = d / AR_CL, c0 = chunk * cols;
  const int seq = *reinterpret_cast<volatile int*>(sync) + 1;
  const size_t slot = (size_t)(seq & 1) * rows_pad * d * (PUSH ? a.world : 1);
  const int nflag = rows_pad * AR_CL, fidx = row * AR_CL + chunk;
  // phase A: plane sum of this chunk into this rank's staging slot (float4 columns; the splits are independent loads)
  const size_t my_off = slot + (PUSH ? (size_t)a.rank * rows_pad * d : 0) + (size_t)row * d + c0;
  float* mine = a.sym[a.rank] + my_off;
  const float* prow = partial + (size_t)row * ldp + c0;
  for (int i = threadIdx.x * 4; i < cols; i += AR_THREADS * 4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int s = 0; s < splits; s++) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(prow + (size_t)s * plane_stride + i));
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if constexpr (PUSH) {
      for (int q = 0; q < a.world; q++) *reinterpret_cast<float4*>(a.sym[q] + my_off + i) = acc;
    } else {
      *reinterpret_cast<float4*>(mine + i) = acc;
    }
  }
  bool ok = true;
  if (a.world > 1) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < a.world) {
      st_release_sys(a.flags[threadIdx.x] + (size_t)a.rank * nflag + fidx, (uint32_t)seq);
      ok = wait_flag_ge(a.flags[a.rank] + (size_t)threadIdx.x * nflag + fidx, (uint32_t)seq, DEC_TIMEOUT_NS);
      if (!ok) ft_set_status(status, FT_K_COMM, 14, threadIdx.x);
    }
    ok = !__syncthreads_or(!ok);              // on a timeout the CTA still walks through the cluster barriers below (its partners wait there)
  } else {
    __syncthreads();
  }
  // phase B: cross-rank sum in fixed rank order + residual; this chunk's share of the row's sum of squares
  float ss = 0.f;
  __nv_bfloat16* xr = x + (size_t)row * d + c0;
  for (int i = threadIdx.x * 4; i < cols; i += AR_THREADS * 4) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < a.world; r++) {
      const float* src = PUSH ? a.sym[a.rank] + slot + ((size_t)r * rows_pad + row) * d + c0 + i : a.sym[r] + slot + (size_t)row * d + c0 + i;
      const float4 p = PUSH ? __ldcg(reinterpret_cast<const float4*>(src)) : *reinterpret_cast<const float4*>(src);
      v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
    }
    const uint2 raw = *reinterpret_cast<const uint2*>(xr + i);
    const float2 x0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x)), x1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    __nv_bfloat162 o0 = __floats2bfloat162_rn(v.x + x0.x, v.y + x0.y), o1 = __floats2bfloat162_rn(v.z + x1.x, v.w + x1.y);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&o0);
    pk.y = *reinterpret_cast<uint32_t*>(&o1);
    *reinterpret_cast<uint2*>(xr + i) = pk;
    const float2 f0 = __bfloat1622float2(o0), f1 = __bfloat1622float2(o1);
    ss += f0.x * f0.x + f0.y * f0.y + f1.x * f1.x + f1.y * f1.y;
  }
  ss = block_sum(ss, red);
  if (threadIdx.x == 0) cta_ss = ss;
  cluster.sync();
  float tot = 0.f;
  for (int r = 0; r < AR_CL; r++) tot += *cluster.map_shared_rank(&cta_ss, r);
  cluster.sync();                             // nobody leaves while a partner may still read its shared memory
  const float rstd = rsqrtf(tot / (float)d + eps);
  __nv_bfloat16* hr = h + (size_t)row * d + c0;
  for (int i = threadIdx.x * 4; i < cols; i += AR_THREADS * 4) {
    const uint2 raw = *reinterpret_cast<const uint2*>(xr + i), wr = *reinterpret_cast<const uint2*>(w + c0 + i);
    const float2 x0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x)), x1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    const float2 w0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wr.x)), w1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wr.y));
    __nv_bfloat162 o0 = __floats2bfloat162_rn(x0.x * rstd * w0.x, x0.y * rstd * w0.y), o1 = __floats2bfloat162_rn(x1.x * rstd * w1.x, x1.y * rstd * w1.y);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&o0);
    pk.y = *reinterpret_cast<uint32_t*>(&o1);
    *reinterpret_cast<uint2*>(hr + i) = pk;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int prev = atomicAdd(&sync[1], 1);
    if (prev == (int)gridDim.x - 1) {         // every CTA has read the launch number: advance it for the next launch (or graph replay)
      sync[1] = 0;
      __threadfence();
      sync[0] = seq;
    }
  }
}

inline int small_grid(size_t work, int block) {
  size_t g = (work + block - 1) / block;
  return (int)(g < 1 ? 1 : (g > 592 ? 592 : g));
}

}  // namespace

// out[r][n] = sum_s partial[s][r][n] (+bias[n]); partial planes are rows x ldp floats, plane_stride = elements between planes.
FT_EXPORT int ft_splitk_reduce(const float* partial, int splits, int rows, int N, int64_t ldp, int64_t plane_stride, const void* bias, void* out,
                               int64_t ldo, int out_f32, cudaStream_t st) {
  if (splits < 1 || rows < 1 || N < 1) return FT_ERR_ARG;
  const int grid = small_grid((size_t)rows * N, 256);
  if (out_f32) return (int)ft_launch_pdl(splitk_reduce_kernel<float>, dim3(grid), dim3(256), 0, st, partial, splits, rows, N, ldp, (size_t)plane_stride, (const __nv_bfloat16*)bias, (float*)out, ldo);
  return (int)ft_launch_pdl(splitk_reduce_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, partial, splits, rows, N, ldp, (size_t)plane_stride, (const __nv_bfloat16*)bias, (__nv_bfloat16*)out, ldo);
}

// positions[b] = index of the token being decoded in sequence b; caches are [num_blocks, 16, Hkv, D] bf16.
FT_EXPORT int ft_decode_qkv_rope_kvwrite(const float* partial, int splits, int64_t ldp, int64_t plane_stride, int B, int Hq, int Hkv, int D,
                                         const int* positions, const float* cos_t, const float* sin_t, void* q_out, void* k_cache,
                                         void* v_cache, const int* block_table, int max_blocks, cudaStream_t st) {
  if (B < 1 || D % 2 || D / 2 > 1024) return FT_ERR_ARG;
  return (int)ft_launch_pdl(qkv_rope_kvwrite_kernel, dim3(B, Hq + 2 * Hkv), dim3(D / 2), 0, st, partial, splits, ldp, (size_t)plane_stride, Hq, Hkv, D, positions,
                            cos_t, sin_t, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, block_table, max_blocks);
}

FT_EXPORT int ft_paged_kv_write(const void* qkv, int64_t ld, int B, int S, int Hq, int Hkv, int D, void* k_cache, void* v_cache,
                                const int* block_table, int max_blocks, int pos0, cudaStream_t st) {
  if ((Hkv * D) % 8 || (ld % 8)) return FT_ERR_ARG;
  paged_kv_write_kernel<<<dim3(S, B), 128, 0, st>>>((const __nv_bfloat16*)qkv, ld, S, Hq, Hkv, D, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache,
                                                    block_table, max_blocks, pos0);
  return (int)cudaGetLastError();
}

// q, out: bf16 [B, Hq, 128]; seq_lens[b] counts the tokens already in the cache (including the one just written).
// ws: f32 scratch of B * Hkv * nsplit * (Hq/Hkv) * 132 floats (16-byte aligned); counters: int [B*Hkv], zero before the first call
// (the kernel re-zeroes them). Hq/Hkv <= 8, nsplit <= 64.
FT_EXPORT int ft_paged_attn_decode(const void* q, const void* k_cache, const void* v_cache, const int* block_table, int max_blocks,
                                   const int* seq_lens, int B, int Hq, int Hkv, int D, float scale, int nsplit, float* ws, int* counters, void* out,
                                   cudaStream_t st) {
  if (D != 128 || Hq % Hkv || Hq / Hkv > 8 || nsplit < 1 || nsplit > PA_MAX_SPLIT || (reinterpret_cast<uintptr_t>(ws) & 15)) return FT_ERR_ARG;
  int dev = 0;
  cudaGetDevice(&dev);
  static bool attr_set[64] = {};
  if (dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(paged_attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PA_SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev] = true;
  }
  return (int)ft_launch_pdl(paged_attn_decode_kernel, dim3(nsplit, Hkv, B), dim3(128), (size_t)PA_SMEM, st, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache,
                            (const __nv_bfloat16*)v_cache, block_table, max_blocks, seq_lens, Hq, Hkv, scale, ws, counters, (__nv_bfloat16*)out);
}

FT_EXPORT int ft_decode_swiglu(const float* partial, int splits, int64_t ldp, int64_t plane_stride, int rows, int F, void* out, cudaStream_t st) {
  if (rows < 1 || F < 1) return FT_ERR_ARG;
  return (int)ft_launch_pdl(decode_swiglu_kernel, dim3(small_grid((size_t)rows * F, 256)), dim3(256), 0, st, partial, splits, ldp, (size_t)plane_stride, rows, F,
                            (__nv_bfloat16*)out);
}

// sym_ptrs / flag_ptrs: `world` mappings of every rank's staging buffer (2 * rows_pad * d floats) and flag block (u32[8], zeroed once).
// sync: int[4] device memory, zeroed once. sumsq: float[2 * rows_pad * chunks]. x: residual stream [rows, d] bf16, updated in place;
// h: normalised output [rows, d] bf16. d % chunks == 0; rows * chunks CTAs must all be resident (<= number of SMs).
FT_EXPORT int ft_decode_ar_residual_norm(const float* partial, int splits, int64_t ldp, int64_t plane_stride, void* const* sym_ptrs,
                                         void* const* flag_ptrs, int rank, int world, int* sync, void* x, const void* w, void* h, float* sumsq,
                                         int rows, int rows_pad, int d, int chunks, float eps, cudaStream_t st) {
  if (world < 1 || world > MAXR || rows < 1 || chunks < 1 || d % chunks || rows * chunks > 148) return FT_ERR_ARG;
  ArNormArgs a;
  for (int i = 0; i < MAXR; i++) { a.sym[i] = i < world ? (float*)sym_ptrs[i] : nullptr; a.flags[i] = i < world ? (uint32_t*)flag_ptrs[i] : nullptr; }
  a.rank = rank;
  a.world = world;
  return (int)ft_launch_pdl(decode_ar_residual_norm_kernel, dim3(rows * chunks), dim3(256), 0, st, partial, splits, ldp, (size_t)plane_stride, a, sync,
                            (__nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)h, sumsq, rows, rows_pad, d, chunks, eps, ft_status_ptr());
}

// Cluster form of ft_decode_ar_residual_norm (no grid barriers). flag blocks: u32[8][rows_pad * 4] per rank, zeroed once; sync: int[4] zeroed once.
// d must be a multiple of 16. Launch numbers live in sync[0], so a captured launch advances on every graph replay.
// push = 0: staging buffers hold 2 * rows_pad * d floats per rank and peers are read after the handshake;
// push = 1: staging buffers hold 2 * world * rows_pad * d floats per rank and every rank stores its rows into all of them before the handshake.
FT_EXPORT int ft_decode_ar_residual_norm_cluster(const float* partial, int splits, int64_t ldp, int64_t plane_stride, void* const* sym_ptrs, void* const* flag_ptrs,
                                                 int rank, int world, int* sync, void* x, const void* w, void* h, int rows, int rows_pad, int d, float eps,
                                                 int push, cudaStream_t st) {
  if (world < 1 || world > MAXR || rows < 1 || rows > rows_pad || d % (AR_CL * 4) || (ldp & 3) || (plane_stride & 3)) return FT_ERR_ARG;
  ArNormArgs a;
  for (int i = 0; i < MAXR; i++) { a.sym[i] = i < world ? (float*)sym_ptrs[i] : nullptr; a.flags[i] = i < world ? (uint32_t*)flag_ptrs[i] : nullptr; }
  a.rank = rank;
  a.world = world;
  if (push)
    return (int)ft_launch_pdl(decode_ar_residual_norm_cluster_kernel<true>, dim3(rows * AR_CL), dim3(AR_THREADS), 0, st, partial, splits, ldp, (size_t)plane_stride, a,
                              sync, (__nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)h, rows, rows_pad, d, eps, ft_status_ptr());
  return (int)ft_launch_pdl(decode_ar_residual_norm_cluster_kernel<false>, dim3(rows * AR_CL), dim3(AR_THREADS), 0, st, partial, splits, ldp, (size_t)plane_stride, a, sync,
                            (__nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)h, rows, rows_pad, d, eps, ft_status_ptr());
}
