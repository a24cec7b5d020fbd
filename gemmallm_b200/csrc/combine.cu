// Combine kernel: weighted un-permute of the expert outputs back to token
// order, fused with the caller's residual add.
//   out[t] = sum_j w[t,j] * y[row_of[t,j]]  (+ residual[t])
// in fp32, slots in order, rounded once. Replaces the two zero-filled fp32
// scatter buffers, the index_copy_ calls and the weighted sum of reference
// model.py:264-271, and the `tensor += skip_connection` of model.py:319.
//
// HBM-bound gather (no atomics, deterministic): each thread produces eight
// consecutive output elements from k 16-byte (bf16) or 32-byte (fp32) loads.
#include "common.cuh"
#include "ep_sync.cuh"

namespace moe {

namespace {

template <typename T>
__global__ void __launch_bounds__(256)
combine_kernel(const T* __restrict__ y, const int32_t* __restrict__ row_of,
               const float* __restrict__ w, const T* __restrict__ residual, int64_t N, int d,
               int k, T* __restrict__ out, const EpSync sy, int32_t* __restrict__ status) {
  const int pieces = d >> 3;
  const int64_t item = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  pdl_wait();
  // expert-parallel: y is the return buffer the expert owners store into; wait for all of them
  if (!epsync::block_wait(sy, status, 25)) return;
  if (item >= N * pieces) return;
  const int64_t t = item / pieces;
  const int c = (int)(item - t * pieces) << 3;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  for (int j = 0; j < k; ++j) {
    // row_of == nullptr: y is already in (token, slot) order (expert-parallel return buffer)
    const int row = row_of != nullptr ? __ldg(&row_of[t * k + j]) : (int)(t * k + j);
    if (row < 0) continue;
    const float wj = __ldg(&w[t * k + j]);
    float v[8];
    load8(y + (int64_t)row * d + c, v);
    // mul then add, not fma: the reference forms w0*a + w1*b from rounded products
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], __fmul_rn(wj, v[i]));
  }
  if (residual != nullptr) {
    float r[8];
    load8(residual + t * d + c, r);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], r[i]);
  }
  store8(out + t * d + c, acc);
}


// Small-N variant: the down product arrives as `ksplit` fp32 partial buffers
// part[s][M][d] without bias; sum them in order s = 0..ksplit-1, add the
// expert's down.bias, then weight and add as above.
// TWO: the call has two slots per token (the reference's k): the routing of both and all the
// partial sums of both are requested before anything is added, so that the kernel is two
// round trips to L2 long instead of one per slot and kind of load.
template <bool TWO>
__global__ void __launch_bounds__(64)
combine_decode_kernel(const float* __restrict__ part, int ksplit, int64_t part_stride,
                      const int32_t* __restrict__ row_of, const int32_t* __restrict__ idx,
                      const float* __restrict__ w, const void* const* __restrict__ b2,
                      const __nv_bfloat16* __restrict__ residual, int64_t N, int d, int k,
                      __nv_bfloat16* __restrict__ out) {
  const int pieces = d >> 3;
  const int64_t item = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  pdl_launch_dependents();   // the next kernel may become resident; it waits before it reads
  pdl_wait();
  if (item >= N * pieces) return;
  const int64_t t = item / pieces;
  const int c = (int)(item - t * pieces) << 3;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  if constexpr (TWO) {
    // (routing through L2 after the wait, as below)
    int row[2], e[2];
    float wj[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      row[j] = __ldcg(&row_of[t * 2 + j]);
      e[j] = __ldcg(&idx[t * 2 + j]);
      wj[j] = __ldcg(&w[t * 2 + j]);
    }
    float r[8];
    if (residual != nullptr) load8(residual + t * d + c, r);
    float v[2][8], pv[2][8][8];
#pragma unroll
    for (int j = 0; j < 2; ++j)
      if (row[j] >= 0) {
        load8_ldg(static_cast<const __nv_bfloat16*>(b2[e[j]]) + c, v[j]);
#pragma unroll
        for (int sp = 0; sp < 8; ++sp)
          if (sp < ksplit) load8(part + (int64_t)sp * part_stride + (int64_t)row[j] * d + c, pv[j][sp]);
      }
#pragma unroll
    for (int j = 0; j < 2; ++j)
      if (row[j] >= 0) {
        float s2[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) s2[i] = 0.f;
#pragma unroll
        for (int sp = 0; sp < 8; ++sp)
          if (sp < ksplit) {
#pragma unroll
            for (int i = 0; i < 8; ++i) s2[i] += pv[j][sp][i];
          }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float yv = __bfloat162float(__float2bfloat16_rn(s2[i] + v[j][i]));
          acc[i] = __fadd_rn(acc[i], __fmul_rn(wj[j], yv));
        }
      }
    if (residual != nullptr) {
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], r[i]);
    }
    store8(out + t * d + c, acc);
    return;
  }
  for (int j = 0; j < k; ++j) {
    // row_of, idx and w come from the routing kernel, which may still be running when this
    // kernel becomes resident: read them through L2 after the wait, never through the read-only
    // path (whose loads the compiler may move above the wait)
    const int row = __ldcg(&row_of[t * k + j]);
    if (row < 0) continue;
    const int e = __ldcg(&idx[t * k + j]);
    const float wj = __ldcg(&w[t * k + j]);
    float v[8];
    load8_ldg(static_cast<const __nv_bfloat16*>(b2[e]) + c, v);
    float s[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i] = 0.f;
    // all partial loads in flight at once; summed in order sp = 0, 1, ...
    float pv[8][8];
#pragma unroll
    for (int sp = 0; sp < 8; ++sp)
      if (sp < ksplit) load8(part + (int64_t)sp * part_stride + (int64_t)row * d + c, pv[sp]);
#pragma unroll
    for (int sp = 0; sp < 8; ++sp)
      if (sp < ksplit) {
#pragma unroll
        for (int i = 0; i < 8; ++i) s[i] += pv[sp][i];
      }
    // the expert's output is rounded to bf16 before weighting, as on the large-N path
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float yv = __bfloat162float(__float2bfloat16_rn(s[i] + v[i]));
      acc[i] = __fadd_rn(acc[i], __fmul_rn(wj, yv));
    }
  }
  if (residual != nullptr) {
    float r[8];
    load8(residual + t * d + c, r);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], r[i]);
  }
  store8(out + t * d + c, acc);
}

}  // namespace

int launch_combine_decode(const float* part, int ksplit, int64_t M, const int32_t* row_of,
                          const int32_t* idx, const float* w, const void* plan, int E,
                          const void* residual, int64_t N, int d, int k, void* out, cudaStream_t s) {
  if (N == 0) return 0;
  PlanView pv = plan_view(plan, E);
  const int64_t items = N * (d >> 3);
  const int64_t blocks = (items + 63) / 64;   // small blocks: spread few items over many SMs
  if (k == 2)
    MOE_CUDA_CHECK(launch_pdl(combine_decode_kernel<true>, dim3((unsigned)blocks), dim3(64), 0, s, part, ksplit,
                              M * (int64_t)d, row_of, idx, w, pv.b2,
                              static_cast<const __nv_bfloat16*>(residual), N, d, k,
                              static_cast<__nv_bfloat16*>(out)));
  else
    MOE_CUDA_CHECK(launch_pdl(combine_decode_kernel<false>, dim3((unsigned)blocks), dim3(64), 0, s, part, ksplit,
                              M * (int64_t)d, row_of, idx, w, pv.b2,
                              static_cast<const __nv_bfloat16*>(residual), N, d, k,
                              static_cast<__nv_bfloat16*>(out)));
  return 0;
}

int launch_combine(const void* y, const int32_t* row_of, const float* w, const void* residual,
                   int64_t N, int d, int k, int dtype, void* out, cudaStream_t s,
                   const EpSync* ep_wait, int32_t* status) {
  if (N == 0) return 0;
  const EpSync nosync = {};
  const EpSync& sy = ep_wait != nullptr ? *ep_wait : nosync;
  const int64_t items = N * (d >> 3);
  const int64_t blocks = (items + 255) / 256;
  if (dtype == MOE_B200_BF16) {
    MOE_CUDA_CHECK(launch_pdl(combine_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, s,
                              static_cast<const __nv_bfloat16*>(y), row_of, w,
                              static_cast<const __nv_bfloat16*>(residual), N, d, k,
                              static_cast<__nv_bfloat16*>(out), sy, status));
  } else {
    MOE_CUDA_CHECK(launch_pdl(combine_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, s,
                              static_cast<const float*>(y), row_of, w,
                              static_cast<const float*>(residual), N, d, k, static_cast<float*>(out),
                              sy, status));
  }
  return 0;
}

}  // namespace moe

