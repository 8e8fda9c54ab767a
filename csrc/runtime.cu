// Host-side runtime of the kernel library: error word, device properties, TMA tensor-map
// encoding through the driver entry point (no link-time dependency on libcuda).
#include <mutex>
#include <stdio.h>

#include <cstdlib>
#include "common.cuh"

namespace {
std::mutex g_mu;
int* g_err_host = nullptr;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

EncodeTiledFn get_encode() {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_encode) return g_encode;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || fn == nullptr) return nullptr;
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return g_encode;
}
}  // namespace

int* cs_error_word() {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_err_host == nullptr) {
    if (cudaHostAlloc(reinterpret_cast<void**>(&g_err_host), 64,
                      cudaHostAllocPortable | cudaHostAllocMapped) != cudaSuccess) {
      g_err_host = nullptr;
      return nullptr;
    }
    for (int i = 0; i < 16; ++i) g_err_host[i] = 0;
  }
  return g_err_host;  // unified addressing: the same address is valid on every device
}

int cs_num_sms() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

// 2-D tiled map over a row-major [outer, inner] view.  Out-of-range reads return zero.
int cs_encode_tmap_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                      uint64_t outer_stride_bytes, uint32_t box_inner, uint32_t box_outer,
                      int elem_bytes, int swizzle128) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (outer_stride_bytes & 15) != 0) return -2;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {outer_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                             : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = enc(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

// 3-D tiled bf16 map, 128-byte swizzle; strides of dims 1 and 2 in bytes.
int cs_encode_tmap_3d(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                      uint64_t s1_bytes, uint64_t s2_bytes, uint32_t b0, uint32_t b1, uint32_t b2) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (s1_bytes & 15) != 0 || (s2_bytes & 15) != 0) return -2;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {s1_bytes, s2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

// ---- exported C API ---------------------------------------------------------------------

// Returns the first error code recorded by any kernel since the last reset (0 = none).
CS_API int cs_last_error() {
  int* p = cs_error_word();
  return p ? *reinterpret_cast<volatile int*>(p) : -1;
}
CS_API void cs_reset_error() {
  int* p = cs_error_word();
  if (p) *reinterpret_cast<volatile int*>(p) = 0;
}
int cs_pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* v = getenv("CORNSERVE_PDL");
    on = (v != nullptr && v[0] == '0') ? 0 : 1;
  }
  return on;
}

CS_API int cs_sm_count() { return cs_num_sms(); }
CS_API int cs_abi_version() { return 1; }
