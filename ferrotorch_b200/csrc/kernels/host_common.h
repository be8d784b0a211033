// Host-side helpers shared by the kernel launchers: error codes, the driver
// entry point for tensor-map encoding (looked up at run time so the library
// has no link-time dependency on libcuda and imports on a machine with no
// driver), and a per-device status word that kernels write instead of trapping.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define FT_EXPORT extern "C" __attribute__((visibility("default")))

// Return codes of every exported launcher. 0 = launched; negative = refused
// before any launch (bad argument); positive = a CUDA runtime error code.
enum FtError : int {
  FT_OK = 0,
  FT_ERR_ARG = -1,         // unsupported shape / alignment
  FT_ERR_DRIVER = -2,      // driver entry point unavailable
  FT_ERR_TMAP = -3,        // cuTensorMapEncodeTiled refused the descriptor
  FT_ERR_TOO_LARGE = -4,   // request exceeds a compiled-in maximum
  FT_ERR_CORRUPT = -5,     // a guard region was overwritten (allocator debug mode)
};

#define FT_CUDA_TRY(expr)                                  \
  do {                                                     \
    cudaError_t _e = (expr);                               \
    if (_e != cudaSuccess) return (int)_e;                 \
  } while (0)

typedef CUresult (*PFN_ftTensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                               CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                               CUtensorMapFloatOOBfill);

PFN_ftTensorMapEncodeTiled ft_get_tmap_encoder();

// Encode a 2-D row-major tensor map (dims given innermost first).
//   elem_bytes 2 (bf16) or 4 (f32). ld_bytes = row pitch in bytes (multiple of 16).
int ft_make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, bool is_bf16, uint64_t inner, uint64_t outer,
                    uint64_t ld_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swz);
// 3-D variant: dims (inner, mid, outer) with pitches for mid and outer.
int ft_make_tmap_3d(CUtensorMap* out, const void* base, int elem_bytes, bool is_bf16, uint64_t d0, uint64_t d1,
                    uint64_t d2, uint64_t pitch1_bytes, uint64_t pitch2_bytes, uint32_t b0, uint32_t b1, uint32_t b2,
                    CUtensorMapSwizzle swz);
int ft_make_tmap_4d(CUtensorMap* out, const void* base, int elem_bytes, bool is_bf16, const uint64_t dims[4],
                    const uint64_t pitches_bytes[3], const uint32_t box[4], CUtensorMapSwizzle swz);

// Make the device's primary context current in the calling thread. A thread that has only ever called
// cudaGetDevice (an autograd worker, say) has no current context, and the driver-level tensor-map encoder then
// fails with CUDA_ERROR_INVALID_CONTEXT.
cudaError_t ft_bind_context(int dev);

// Per-device status word in device memory (lazily allocated, zeroed).
uint32_t* ft_status_ptr();

// Kernels meant to run BESIDE the persistent GEMM (optimizer, collectives, parameter pushes, all on side streams) ask for the same shared-memory
// carveout as the GEMM. An SM runs with one L1 / shared-memory split at a time: a kernel that prefers another split is not co-scheduled onto an SM
// the GEMM occupies and would only get SMs at kernel boundaries, which serialises the "overlapped" work behind the GEMMs.
#ifdef __CUDACC__
template <typename K>
inline void ft_prefer_max_shared(K kernel) {
  cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
}
#endif

// Launch with the programmatic-stream-serialization attribute when programmatic dependent launch is switched on (ft_set_pdl), else an ordinary
// launch. Only kernels that call pdl_wait() before touching memory a predecessor may still be writing (or reading) go through this.
bool ft_pdl_enabled();
#ifdef __CUDACC__
template <typename... KArgs, typename... Args>
inline cudaError_t ft_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ft_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#endif
