// Expert feed-forward on CUDA cores: the fp32 implementation of
// FeedForward.forward (reference model.py:173-190, fine_tuning=False, eval):
//   h = gelu_tanh(x W1[:f]^T + b1[:f]) * (x W1[f:]^T + b1[f:])   (model.py:174,180-182)
//   y = h W2^T + b2                                               (model.py:184)
// grouped over experts by the row offsets the dispatch kernel wrote.
//
// fp32 needs max-abs 1e-4 against the reference, which single-pass TF32
// tensor-core math does not give after two chained products, so this path is
// plain FFMA with fp32 accumulation: a 64x64x16 shared-memory tile, a 4x4
// register tile per thread. With bf16 operands it is the second implementation
// the tensor-core kernel is checked against (MOE_B200_FLAG_SIMT_EXPERTS).
#include "common.cuh"

namespace moe {

namespace {

constexpr int BM = 64, BN = 64, BK = 16;

__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
  float4 a = __ldg(reinterpret_cast<const float4*>(p));
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
  uint2 a = __ldg(reinterpret_cast<const uint2*>(p));
  v[0] = bf16_lo(a.x); v[1] = bf16_hi(a.x); v[2] = bf16_lo(a.y); v[3] = bf16_hi(a.y);
}

// A: [rows, K] activations (sorted buffer); W: per-expert [Nw, K]; out [rows, Nout].
// GEGLU: Nw = 2*Nout, gate rows [0,Nout), up rows [Nout, 2*Nout).
template <typename T, bool GEGLU>
__global__ void __launch_bounds__(256)
grouped_ffn_kernel(const T* __restrict__ A, const int32_t* __restrict__ offsets,
                   const void* const* __restrict__ Wp, const void* const* __restrict__ bp, int E,
                   int K, int Nout, T* __restrict__ out) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[GEGLU ? 2 : 1][BK][BN + 4];
  __shared__ int s_e, s_row0, s_rows;

  if (threadIdx.x == 0) {
    int tile = blockIdx.x, e = 0, found = -1, row0 = 0, rows = 0;
    for (; e < E; ++e) {
      int beg = offsets[e], cnt = offsets[e + 1] - beg;
      int tiles = (cnt + BM - 1) / BM;
      if (tile < tiles) { found = e; row0 = beg + tile * BM; rows = min(BM, cnt - tile * BM); break; }
      tile -= tiles;
    }
    s_e = found; s_row0 = row0; s_rows = rows;
  }
  __syncthreads();
  const int e = s_e;
  if (e < 0) return;
  const int row0 = s_row0, rows = s_rows;
  const int n0 = blockIdx.y * BN;
  const T* W = static_cast<const T*>(Wp[e]);
  const T* bias = static_cast<const T*>(bp[e]);

  const int tid = threadIdx.x;
  const int lr = tid >> 2;         // 0..63: tile row this thread loads
  const int lk = (tid & 3) << 2;   // 0,4,8,12
  const int tx = tid & 15, ty = tid >> 4;  // 16x16 threads, 4x4 outputs each

  float acc[GEGLU ? 2 : 1][4][4];
#pragma unroll
  for (int g = 0; g < (GEGLU ? 2 : 1); ++g)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[g][i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (lr < rows && k0 + lk < K) load4(A + (int64_t)(row0 + lr) * K + k0 + lk, v);
#pragma unroll
    for (int i = 0; i < 4; ++i) As[lk + i][lr] = v[i];
#pragma unroll
    for (int g = 0; g < (GEGLU ? 2 : 1); ++g) {
      float u[4] = {0.f, 0.f, 0.f, 0.f};
      int n = n0 + lr;
      if (n < Nout && k0 + lk < K) load4(W + (int64_t)(g * Nout + n) * K + k0 + lk, u);
#pragma unroll
      for (int i = 0; i < 4; ++i) Bs[g][lk + i][lr] = u[i];
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[GEGLU ? 2 : 1][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int g = 0; g < (GEGLU ? 2 : 1); ++g)
#pragma unroll
        for (int j = 0; j < 4; ++j) b[g][j] = Bs[g][kk][tx * 4 + j];
#pragma unroll
      for (int g = 0; g < (GEGLU ? 2 : 1); ++g)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[g][i][j] = fmaf(a[i], b[g][j], acc[g][i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int r = ty * 4 + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int n = n0 + tx * 4 + j;
      if (n >= Nout) continue;
      float val;
      if (GEGLU) {
        float g = acc[0][i][j] + to_f32(bias[n]);
        float u = acc[GEGLU ? 1 : 0][i][j] + to_f32(bias[Nout + n]);
        val = gelu_tanh_precise(g) * u;
      } else {
        val = acc[0][i][j] + to_f32(bias[n]);
      }
      from_f32(out[(int64_t)(row0 + r) * Nout + n], val);
    }
  }
}

template <typename T>
int run(const void* perm, const int32_t* offsets, const void* plan, int64_t M, int d, int f, int E,
        void* h, void* y, cudaStream_t s) {
  PlanView pv = plan_view(plan, E);
  const unsigned mtiles = (unsigned)((M + BM - 1) / BM + E);
  dim3 g1(mtiles, (unsigned)((f + BN - 1) / BN));
  grouped_ffn_kernel<T, true><<<g1, 256, 0, s>>>(static_cast<const T*>(perm), offsets, pv.W1, pv.b1,
                                                 E, d, f, static_cast<T*>(h));
  MOE_CUDA_CHECK(cudaGetLastError());
  dim3 g2(mtiles, (unsigned)((d + BN - 1) / BN));
  grouped_ffn_kernel<T, false><<<g2, 256, 0, s>>>(static_cast<const T*>(h), offsets, pv.W2, pv.b2,
                                                  E, f, d, static_cast<T*>(y));
  MOE_CUDA_CHECK(cudaGetLastError());
  return 0;
}

}  // namespace

int launch_experts_simt(const void* perm, const int32_t* offsets, const void* plan, int64_t M,
                        int d, int f, int E, int dtype, void* h, void* y, cudaStream_t s) {
  if (M == 0) return 0;
  if (dtype == MOE_B200_BF16) return run<__nv_bfloat16>(perm, offsets, plan, M, d, f, E, h, y, s);
  return run<float>(perm, offsets, plan, M, d, f, E, h, y, s);
}

}  // namespace moe
