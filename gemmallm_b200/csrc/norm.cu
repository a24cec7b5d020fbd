// The caller's LayerNorm in front of the block (reference model.py:298,311-312:
// `tensor = self.norm2(tensor)` before `self.moe(tensor)`), folded into the block's
// first two kernels so that the normalised tensor is never written and re-read:
//
//   router:   logits[e] = LN(x) . Wg[e] + bg[e]
//                       = rstd * (x . Wn[e] - mean * c1[e]) + c2[e]
//             with Wn[e] = Wg[e] * gamma (rounded to the parameter dtype),
//             c1[e] = sum_j Wn[e][j], c2[e] = sum_j beta[j] * Wg[e][j] + bg[e].
//             The router forms x . Wn[e] and the row's mean / rstd in the same pass
//             over x (router.cu) and keeps (mean, rstd) per token for the dispatch.
//   dispatch: copies (x - mean) * rstd * gamma + beta instead of x (dispatch.cu).
//
// norm_fold_kernel computes Wn, c1 and c2 (E*d elements: microseconds).
// layernorm_rows_kernel is the plain row normalisation for calls of up to 4096
// rows, whose single-launch front end and weight-streaming kernels read x through
// TMA: there the normalised rows (at most a few MB) are written once.
#include "common.cuh"

namespace moe {

namespace {

template <typename T>
__global__ void __launch_bounds__(256)
norm_fold_kernel(const T* __restrict__ Wg, const T* __restrict__ bg, const T* __restrict__ gamma,
                 const T* __restrict__ beta, int E, int d, T* __restrict__ Wn,
                 float* __restrict__ c /* [2E]: c1, c2 */) {
  __shared__ float s1[256], s2[256];
  const int e = blockIdx.x;
  float a1 = 0.f, a2 = 0.f;
  for (int j = threadIdx.x; j < d; j += 256) {
    const float w = to_f32(Wg[(size_t)e * d + j]);
    T wn;
    from_f32(wn, w * to_f32(gamma[j]));
    Wn[(size_t)e * d + j] = wn;
    a1 += to_f32(wn);
    a2 = fmaf(to_f32(beta[j]), w, a2);
  }
  s1[threadIdx.x] = a1;
  s2[threadIdx.x] = a2;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) {
      s1[threadIdx.x] += s1[threadIdx.x + o];
      s2[threadIdx.x] += s2[threadIdx.x + o];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    c[e] = s1[0];
    c[E + e] = s2[0] + to_f32(bg[e]);
  }
}

// One warp per row: mean, biased variance around the mean, y = (x - mean) * rstd * gamma + beta,
// as torch.nn.LayerNorm. Rows of up to 2048 elements stay in the lanes' registers between the
// three steps (one pass over memory); longer rows are re-read (from L1).
template <typename T>
__global__ void __launch_bounds__(256)
layernorm_rows_kernel(const T* __restrict__ x, const T* __restrict__ gamma,
                      const T* __restrict__ beta, float eps, int64_t N, int d, T* __restrict__ out,
                      float* __restrict__ stats /* nullable [N][2] */) {
  pdl_wait();
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= N) return;
  const T* xr = x + row * d;
  constexpr int kKeep = 8;                 // 8 x 8 elements per lane = rows of up to 2048
  const bool keep = d <= kKeep * 256;
  float r[kKeep][8];
  float sum = 0.f;
  if (keep) {
#pragma unroll
    for (int i = 0; i < kKeep; ++i) {
      const int c = lane * 8 + i * 256;
      if (c < d) {
        load8(xr + c, r[i]);
#pragma unroll
        for (int q = 0; q < 8; ++q) sum += r[i][q];
      }
    }
  } else {
    for (int c = lane * 8; c < d; c += 256) {
      float v[8];
      load8(xr + c, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) sum += v[i];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float mean = sum / (float)d;
  float sq = 0.f;
  if (keep) {
#pragma unroll
    for (int i = 0; i < kKeep; ++i)
      if (lane * 8 + i * 256 < d) {
#pragma unroll
        for (int q = 0; q < 8; ++q) sq = fmaf(r[i][q] - mean, r[i][q] - mean, sq);
      }
  } else {
    for (int c = lane * 8; c < d; c += 256) {
      float v[8];
      load8(xr + c, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) sq = fmaf(v[i] - mean, v[i] - mean, sq);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  const float rstd = rsqrtf(sq / (float)d + eps);
  if (keep) {
#pragma unroll
    for (int i = 0; i < kKeep; ++i) {
      const int c = lane * 8 + i * 256;
      if (c < d) {
        float g[8], b[8], o[8];
        load8_ldg(gamma + c, g);
        load8_ldg(beta + c, b);
#pragma unroll
        for (int q = 0; q < 8; ++q) o[q] = fmaf((r[i][q] - mean) * rstd, g[q], b[q]);
        store8(out + row * d + c, o);
      }
    }
  } else {
    for (int c = lane * 8; c < d; c += 256) {
      float v[8], g[8], b[8], o[8];
      load8(xr + c, v);
      load8_ldg(gamma + c, g);
      load8_ldg(beta + c, b);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = fmaf((v[i] - mean) * rstd, g[i], b[i]);
      store8(out + row * d + c, o);
    }
  }
  if (stats != nullptr && lane == 0) {
    stats[2 * row] = mean;
    stats[2 * row + 1] = rstd;
  }
}

}  // namespace

int launch_norm_fold(const void* Wg, const void* bg, const void* gamma, const void* beta, int E,
                     int d, int dtype, void* Wn, float* c, cudaStream_t s) {
  if (dtype == MOE_B200_BF16)
    norm_fold_kernel<__nv_bfloat16><<<E, 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(Wg), static_cast<const __nv_bfloat16*>(bg),
        static_cast<const __nv_bfloat16*>(gamma), static_cast<const __nv_bfloat16*>(beta), E, d,
        static_cast<__nv_bfloat16*>(Wn), c);
  else
    norm_fold_kernel<float><<<E, 256, 0, s>>>(static_cast<const float*>(Wg),
                                              static_cast<const float*>(bg),
                                              static_cast<const float*>(gamma),
                                              static_cast<const float*>(beta), E, d,
                                              static_cast<float*>(Wn), c);
  MOE_CUDA_CHECK(cudaGetLastError());
  return 0;
}

int launch_layernorm_rows(const void* x, const void* gamma, const void* beta, float eps, int64_t N,
                          int d, int dtype, void* out, float* stats, cudaStream_t s) {
  if (N == 0) return 0;
  const unsigned blocks = (unsigned)((N + 7) / 8);
  if (dtype == MOE_B200_BF16)
    MOE_CUDA_CHECK(launch_pdl(layernorm_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, s,
                              static_cast<const __nv_bfloat16*>(x),
                              static_cast<const __nv_bfloat16*>(gamma),
                              static_cast<const __nv_bfloat16*>(beta), eps, N, d,
                              static_cast<__nv_bfloat16*>(out), stats));
  else
    MOE_CUDA_CHECK(launch_pdl(layernorm_rows_kernel<float>, dim3(blocks), dim3(256), 0, s,
                              static_cast<const float*>(x), static_cast<const float*>(gamma),
                              static_cast<const float*>(beta), eps, N, d, static_cast<float*>(out),
                              stats));
  return 0;
}

}  // namespace moe
