// LoRA branch of an expert's Linear folded into its weight (reference
// model.py:175-179 and 185-189, fine_tuning=True):
//   x W^T + b + s * (B (A x + a) + b_lora)  =  x (W + s B A)^T + (b + s (B a + b_lora))
// so the grouped GEMM kernels run unchanged on W' = W + s B A and b' = b + s (B a + b_lora).
// W [out,in], A [r,in], B [out,r]; fp32 arithmetic, one rounding to the parameter dtype.
// Memory-bound (W is read once and W' written once); the r x in matrix A stays in L1/L2.
#include "common.cuh"

namespace moe {

namespace {

constexpr int kMaxRank = 64;

template <typename T>
__global__ void __launch_bounds__(256)
lora_merge_kernel(const T* __restrict__ W, const T* __restrict__ b, const T* __restrict__ A,
                  const T* __restrict__ a_bias, const T* __restrict__ B, const T* __restrict__ b_lora,
                  float scale, int out_f, int in_f, int rank, T* __restrict__ out_W,
                  T* __restrict__ out_b) {
  __shared__ float s_b[kMaxRank];
  const int row = blockIdx.x;
  for (int r = threadIdx.x; r < rank; r += 256) s_b[r] = scale * to_f32(B[(size_t)row * rank + r]);
  __syncthreads();
  for (int c = threadIdx.x * 8; c < in_f; c += 256 * 8) {
    float acc[8];
    load8(W + (size_t)row * in_f + c, acc);
    for (int r = 0; r < rank; ++r) {
      float a[8];
      load8_ldg(A + (size_t)r * in_f + c, a);
      const float br = s_b[r];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = fmaf(br, a[i], acc[i]);
    }
    store8(out_W + (size_t)row * in_f + c, acc);
  }
  if (threadIdx.x == 0) {
    float acc = 0.f;
    for (int r = 0; r < rank; ++r) acc = fmaf(s_b[r], to_f32(a_bias[r]), acc);
    T v;
    from_f32(v, to_f32(b[row]) + acc + scale * to_f32(b_lora[row]));
    out_b[row] = v;
  }
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
  if (dtype == MOE_B200_BF16) {
    using T = __nv_bfloat16;
    lora_merge_kernel<T><<<out_features, 256, 0, s>>>(
        static_cast<const T*>(W), static_cast<const T*>(b), static_cast<const T*>(A),
        static_cast<const T*>(a_bias), static_cast<const T*>(B), static_cast<const T*>(b_lora), scale,
        out_features, in_features, rank, static_cast<T*>(out_W), static_cast<T*>(out_b));
  } else {
    lora_merge_kernel<float><<<out_features, 256, 0, s>>>(
        static_cast<const float*>(W), static_cast<const float*>(b), static_cast<const float*>(A),
        static_cast<const float*>(a_bias), static_cast<const float*>(B),
        static_cast<const float*>(b_lora), scale, out_features, in_features, rank,
        static_cast<float*>(out_W), static_cast<float*>(out_b));
  }
  MOE_CUDA_CHECK(cudaGetLastError());
  return 0;
}
