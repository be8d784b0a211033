// Launcher of the two-SM (tcgen05 cta_group::2) GEMM, shared between gemm_2sm.cu (definition) and gemm_tcgen05.cu (dispatch).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

struct Gemm2Epi {
  int act;                 // 0 none, 1 relu, 2 gelu (erf), 3 gelu (tanh), 4 silu
  const void* residual;    // [M, N] in the output dtype, rows ldr elements apart, or null
  int64_t ldr;
  int in_f16;              // operands are fp16 instead of bf16
};

// Arrival gate of the B operand: B lies inside a gather slot that peers fill piece by piece (fsdp_gather.cu). The TMA producer waits (bounded) until
// the arrival counters of the pieces it is about to read have reached `expected`. counters == null: no gate.
struct Gemm2Gate {
  const uint32_t* counters;   // arrival counters of the slot (this GPU's memory, written by the peers)
  uint32_t expected;
  int mode;                   // 1: per N tile (B is [N, K], K contiguous, rows ldb apart: a tile's rows are one byte range);
                              // 2: the whole operand before the first load (any layout)
  long long b_byte_off;       // offset of B's first element from the start of the slot
  long long b_bytes;          // extent of the operand in the slot
  long long piece_bytes;
  // operand = 1 gates the A operand instead (an activation whose row blocks are pushed by the peers, tensor-parallel all-gather -> GEMM): A is
  // [M, K] with K contiguous, piece_bytes then counts ROWS per piece, b_byte_off the row of A's first row inside the gathered buffer and b_bytes
  // the number of rows; mode 1 waits per 128-row tile, mode 2 for all rows.
  int operand = 0;
  int m_rot = 0;              // the 256-row tile order starts at this tile row and wraps (each rank starts on the rows it already has)
};

// True when the pair kernel should take the problem: enabled, M large enough for 256-row tiles, the device can co-schedule CTA pairs.
bool ft_gemm2_wanted(int M, int N, int K, int k_splits);

// Same contract as the one-SM launcher: D[splits][M][N] = A (x) B restricted to each K slice (+ bias, activation, residual when k_splits == 1).
// Returns FT_OK / FT_ERR_* / a CUDA error code.
int ft_gemm2_launch(const void* A, const void* B, void* D, const void* bias, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldd, int a_mn,
                    int b_mn, int out_f32, int k_splits, cudaStream_t stream, const Gemm2Epi& epi, const Gemm2Gate& gate = Gemm2Gate{nullptr, 0, 0, 0, 0, 1, 0, 0});
