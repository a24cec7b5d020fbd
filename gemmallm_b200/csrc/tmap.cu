// Host-side TMA tensor-map encoding (cuTensorMapEncodeTiled through the runtime's
// driver entry point, so the library links against cudart only) and the
// per-expert weight maps of the plan buffer.
#include <cuda.h>
#include "common.cuh"

namespace moe {

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      (void)cudaGetLastError();
  }
  return fn;
}

}  // namespace

// [rows, cols] row-major bf16, box = box_rows x 64 columns (128 bytes), 128-byte swizzle.
int encode_tmap_2d(void* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  static_assert(sizeof(CUtensorMap) == 128, "tensor map size");
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return set_error(MOE_B200_ERR_DRIVER, "cuTensorMapEncodeTiled unavailable");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(static_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(MOE_B200_ERR_DRIVER, "cuTensorMapEncodeTiled failed");
  return 0;
}

// Plan maps per expert: W1 and W2 with 128-row boxes (large-N path), then W1
// and W2 with 64-row boxes (small-N path).
int build_weight_tensor_maps(const void* const* h_W1, const void* const* h_W2, int E, int d, int f,
                             void* h_tmaps) {
  char* maps = static_cast<char*>(h_tmaps);
  for (int e = 0; e < E; ++e) {
    int rc = encode_tmap_2d(maps + 128 * (size_t)e, h_W1[e], (uint64_t)2 * f, (uint64_t)d, 128);
    if (rc) return rc;
    rc = encode_tmap_2d(maps + 128 * (size_t)(E + e), h_W2[e], (uint64_t)d, (uint64_t)f, 128);
    if (rc) return rc;
    rc = encode_tmap_2d(maps + 128 * (size_t)(2 * E + e), h_W1[e], (uint64_t)2 * f, (uint64_t)d, 64);
    if (rc) return rc;
    rc = encode_tmap_2d(maps + 128 * (size_t)(3 * E + e), h_W2[e], (uint64_t)d, (uint64_t)f, 64);
    if (rc) return rc;
  }
  return 0;
}

// SM count of the current device (cached per device).
int sm_count(int* sms) {
  static int cached[kMaxDevices] = {};
  int dev = 0;
  MOE_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) {
    MOE_CUDA_CHECK(cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev));
    return 0;
  }
  if (cached[dev] == 0)
    MOE_CUDA_CHECK(cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev));
  *sms = cached[dev];
  return 0;
}

}  // namespace moe
