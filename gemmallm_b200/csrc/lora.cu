// LoRA branch of an expert's Linear folded into its weight (reference
// model.py:175-179 and 185-189, fine_tuning=True):
//   x W^T + b + s * (B (A x + a) + b_lora)  =  x (W + s B A)^T + (b + s (B a + b_lora))
// so the grouped GEMM kernels run unchanged on W' = W + s B A and b' = b + s (B a + b_lora).
// W [out,in], A [r,in], B [out,r]; fp32 arithmetic, one rounding to the parameter dtype.
// Memory-bound: W is read once and W' written once; A and B reach the arithmetic through shared memory.
#include "common.cuh"

namespace moe {

namespace {

constexpr int kMaxRank = 64;

constexpr int kTileRows = 32, kTileCols = 256;

// One block per 32 x 256 tile of W: the tile's slice of A [rank][256] and the scaled rows of
// B [32][rank] wait in shared memory, every thread owns 4 rows x 8 columns, so an element of A
// is read from shared memory once per four outputs and W streams through once.
template <typename T>
__global__ void __launch_bounds__(256)
lora_merge_kernel(const T* __restrict__ W, const T* __restrict__ b, const T* __restrict__ A,
                  const T* __restrict__ a_bias, const T* __restrict__ B, const T* __restrict__ b_lora,
                  float scale, int out_f, int in_f, int rank, T* __restrict__ out_W,
                  T* __restrict__ out_b) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* s_a = reinterpret_cast<T*>(smem_raw);                                        // [rank][256]
  float* s_b = reinterpret_cast<float*>(smem_raw + (size_t)rank * kTileCols * sizeof(T));   // [32][rank]
  const int c0 = blockIdx.x * kTileCols, r0 = blockIdx.y * kTileRows;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = c0 + tx * 8;
  // W first: its loads are in flight while the tables are filled
  float acc[4][8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = r0 + ty * 4 + i;
    if (row < out_f && c < in_f) {
      load8(W + (size_t)row * in_f + c, acc[i]);
    } else {
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[i][q] = 0.f;
    }
  }
  for (int i = threadIdx.x; i < rank * (kTileCols / 8); i += 256) {
    const int r = i / (kTileCols / 8), pc = i - r * (kTileCols / 8);
    float v[8];
    if (c0 + pc * 8 < in_f) {
      load8_ldg(A + (size_t)r * in_f + c0 + pc * 8, v);
    } else {
#pragma unroll
      for (int q = 0; q < 8; ++q) v[q] = 0.f;
    }
    store8(s_a + (size_t)r * kTileCols + pc * 8, v);
  }
  for (int i = threadIdx.x; i < kTileRows * rank; i += 256) {
    const int row = r0 + i / rank;
    s_b[i] = row < out_f ? scale * to_f32(B[(size_t)row * rank + (i % rank)]) : 0.f;
  }
  __syncthreads();
  for (int r = 0; r < rank; ++r) {
    float a[8];
    load8(s_a + (size_t)r * kTileCols + tx * 8, a);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float br = s_b[(ty * 4 + i) * rank + r];
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[i][q] = fmaf(br, a[q], acc[i][q]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = r0 + ty * 4 + i;
    if (row < out_f && c < in_f) store8(out_W + (size_t)row * in_f + c, acc[i]);
  }
  if (blockIdx.x == 0 && threadIdx.x < kTileRows && r0 + threadIdx.x < out_f) {
    const int row = r0 + threadIdx.x;
    float sum = 0.f;
    for (int r = 0; r < rank; ++r) sum = fmaf(s_b[threadIdx.x * rank + r], to_f32(a_bias[r]), sum);
    T v;
    from_f32(v, to_f32(b[row]) + sum + scale * to_f32(b_lora[row]));
    out_b[row] = v;
  }
}

template <typename T>
int launch_merge(const void* W, const void* b, const void* A, const void* a_bias, const void* B,
                 const void* b_lora, float scale, int out_f, int in_f, int rank, void* out_W,
                 void* out_b, cudaStream_t s) {
  const size_t smem = (size_t)rank * kTileCols * sizeof(T) + (size_t)kTileRows * rank * sizeof(float);
  static PerDeviceOnce once;
  if (smem > 48 * 1024) {
    int rc = ensure_dynamic_smem(once, lora_merge_kernel<T>, 96 * 1024);
    if (rc) return rc;
  }
  lora_merge_kernel<T><<<dim3((in_f + kTileCols - 1) / kTileCols, (out_f + kTileRows - 1) / kTileRows),
                         256, smem, s>>>(
      static_cast<const T*>(W), static_cast<const T*>(b), static_cast<const T*>(A),
      static_cast<const T*>(a_bias), static_cast<const T*>(B), static_cast<const T*>(b_lora), scale,
      out_f, in_f, rank, static_cast<T*>(out_W), static_cast<T*>(out_b));
  MOE_CUDA_CHECK(cudaGetLastError());
  return 0;
}

}  // namespace
}  // namespace moe

using namespace moe;

extern "C" int moe_b200_lora_merge(const void* W, const void* b, const void* A, const void* a_bias,
                                   const void* B, const void* b_lora, float scale, int out_features,
                                   int in_features, int rank, int dtype, void* out_W, void* out_b,
                                   void* stream) {
  if (dtype != MOE_B200_F32 && dtype != MOE_B200_BF16)
    return set_error(MOE_B200_ERR_DTYPE, "dtype must be MOE_B200_F32 or MOE_B200_BF16");
  if (out_features < 1 || in_features < 8 || (in_features & 7) || rank < 1 || rank > kMaxRank)
    return set_error(MOE_B200_ERR_SHAPE, "in_features must be a multiple of 8 and rank in [1,64]");
  if (!W || !b || !A || !a_bias || !B || !b_lora || !out_W || !out_b)
    return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (!aligned16(W) || !aligned16(A) || !aligned16(out_W))
    return set_error(MOE_B200_ERR_ALIGN, "W, A and out_W must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == MOE_B200_BF16)
    return launch_merge<__nv_bfloat16>(W, b, A, a_bias, B, b_lora, scale, out_features, in_features, rank,
                                       out_W, out_b, s);
  return launch_merge<float>(W, b, A, a_bias, B, b_lora, scale, out_features, in_features, rank, out_W,
                             out_b, s);
}
