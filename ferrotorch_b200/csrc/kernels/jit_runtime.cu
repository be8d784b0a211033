// Loader and launcher for kernels generated at run time: a compiled sm_100a image (cubin) is loaded as a CUDA library, kernels are looked
// up by name and launched on the caller's stream with a parameter array. The code generator lives in ferrotorch_b200/jit/codegen_cuda.py.
#include <cuda_runtime.h>

#include <cstdint>

#include "host_common.h"

FT_EXPORT int ft_jit_load(const void* image, void** library_out) {
  if (!image || !library_out) return FT_ERR_ARG;
  cudaLibrary_t lib = nullptr;
  cudaError_t e = cudaLibraryLoadData(&lib, image, nullptr, nullptr, 0, nullptr, nullptr, 0);
  if (e != cudaSuccess) return (int)e;
  *library_out = (void*)lib;
  return 0;
}

FT_EXPORT int ft_jit_get_kernel(void* library, const char* name, void** kernel_out) {
  if (!library || !name || !kernel_out) return FT_ERR_ARG;
  cudaKernel_t k = nullptr;
  cudaError_t e = cudaLibraryGetKernel(&k, (cudaLibrary_t)library, name);
  if (e != cudaSuccess) return (int)e;
  *kernel_out = (void*)k;
  return 0;
}

// params: array of pointers to the individual kernel arguments, in declaration order.
FT_EXPORT int ft_jit_launch(void* kernel, int64_t grid_x, int block_x, int smem_bytes, void** params, cudaStream_t st) {
  if (!kernel || grid_x < 1 || grid_x > 2147483647LL || block_x < 1 || block_x > 1024) return FT_ERR_ARG;
  cudaError_t e = cudaLaunchKernel((const void*)kernel, dim3((unsigned)grid_x), dim3((unsigned)block_x), params, (size_t)smem_bytes, st);
  return (int)e;
}

FT_EXPORT int ft_jit_unload(void* library) {
  if (!library) return FT_ERR_ARG;
  return (int)cudaLibraryUnload((cudaLibrary_t)library);
}
