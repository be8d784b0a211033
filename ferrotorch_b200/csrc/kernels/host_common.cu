#include "host_common.h"
#include <mutex>

static PFN_ftTensorMapEncodeTiled g_encode = nullptr;
static std::once_flag g_encode_once;

PFN_ftTensorMapEncodeTiled ft_get_tmap_encoder() {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) g_encode = (PFN_ftTensorMapEncodeTiled)fn;
  });
  return g_encode;
}

cudaError_t ft_bind_context(int dev) {
  static thread_local int bound = -1;
  if (bound == dev) return cudaSuccess;
  cudaError_t e = cudaSetDevice(dev);
  if (e == cudaSuccess) e = cudaFree(0);
  if (e == cudaSuccess) bound = dev;
  return e;
}

static int encode(CUtensorMap* out, const void* base, bool is_bf16, int elem_bytes, int rank, const cuuint64_t* dims,
                  const cuuint64_t* strides, const cuuint32_t* box, CUtensorMapSwizzle swz) {
  PFN_ftTensorMapEncodeTiled enc = ft_get_tmap_encoder();
  if (!enc) return FT_ERR_DRIVER;
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUtensorMapDataType dt = is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                   : (elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                                      : (elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8));
  CUresult r = enc(out, dt, rank, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[ferrotorch_b200] cuTensorMapEncodeTiled failed: %d (rank %d, base %p, dims %llu %llu, box %u %u)\n",
            (int)r, rank, base, (unsigned long long)dims[0], (unsigned long long)dims[1], box[0], box[1]);
    return FT_ERR_TMAP;
  }
  return FT_OK;
}

int ft_make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, bool is_bf16, uint64_t inner, uint64_t outer,
                    uint64_t ld_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swz) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld_bytes & 15)) return FT_ERR_ARG;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  return encode(out, base, is_bf16, elem_bytes, 2, dims, strides, box, swz);
}

int ft_make_tmap_3d(CUtensorMap* out, const void* base, int elem_bytes, bool is_bf16, uint64_t d0, uint64_t d1,
                    uint64_t d2, uint64_t pitch1_bytes, uint64_t pitch2_bytes, uint32_t b0, uint32_t b1, uint32_t b2,
                    CUtensorMapSwizzle swz) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (pitch1_bytes & 15) || (pitch2_bytes & 15)) return FT_ERR_ARG;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {pitch1_bytes, pitch2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  return encode(out, base, is_bf16, elem_bytes, 3, dims, strides, box, swz);
}

int ft_make_tmap_4d(CUtensorMap* out, const void* base, int elem_bytes, bool is_bf16, const uint64_t dims_[4],
                    const uint64_t pitches_bytes[3], const uint32_t box_[4], CUtensorMapSwizzle swz) {
  if (reinterpret_cast<uintptr_t>(base) & 15) return FT_ERR_ARG;
  cuuint64_t dims[4], strides[3];
  cuuint32_t box[4];
  for (int i = 0; i < 4; i++) { dims[i] = dims_[i]; box[i] = box_[i]; }
  for (int i = 0; i < 3; i++) { if (pitches_bytes[i] & 15) return FT_ERR_ARG; strides[i] = pitches_bytes[i]; }
  return encode(out, base, is_bf16, elem_bytes, 4, dims, strides, box, swz);
}

// ---------------------------------------------------------------------------
// status word, one per device
// ---------------------------------------------------------------------------
static uint32_t* g_status[64] = {nullptr};
static std::mutex g_status_mu;

uint32_t* ft_status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_status_mu);
  if (!g_status[dev]) {
    uint32_t* p = nullptr;
    if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 256);
    g_status[dev] = p;
  }
  return g_status[dev];
}

// Read the status word of the current device (synchronises the device) and
// clear it. 0 = every bounded wait since the last read completed normally.
FT_EXPORT int ft_status_read_clear(uint32_t* out) {
  uint32_t* p = ft_status_ptr();
  if (!p) return FT_ERR_DRIVER;
  FT_CUDA_TRY(cudaDeviceSynchronize());
  FT_CUDA_TRY(cudaMemcpy(out, p, 4, cudaMemcpyDeviceToHost));
  if (*out) FT_CUDA_TRY(cudaMemset(p, 0, 4));
  return FT_OK;
}

FT_EXPORT int ft_abi_version() { return 1; }

static bool g_pdl = false;
bool ft_pdl_enabled() { return g_pdl; }
// Switch programmatic dependent launch on or off for the kernels that support it (the decode path). Returns the previous setting.
FT_EXPORT int ft_set_pdl(int enabled) {
  const int prev = g_pdl ? 1 : 0;
  g_pdl = enabled != 0;
  return prev;
}
