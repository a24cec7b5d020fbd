// Router kernel: logits = x Wg^T + bg in fp32, softmax, top-k, renormalise.
// Covers reference model.py:206-223 (gate Linear, F.softmax, topk, score
// renormalisation) and the per-expert probability sums of model.py:215.
//
// HBM-bound: x [N,d] is read once; Wg [E,d] stays in L1/L2. A block of four
// warps owns 32 consecutive tokens. Each warp computes the logits of four
// tokens at a time (so every Wg register is used four times), eight experts
// per pass, with 16-byte loads and a warp-shuffle reduction, then does
// softmax/top-k for its tokens with one expert slice per lane.
#include "common.cuh"

namespace moe {

namespace {

constexpr int kWarps = 4;
constexpr int kTokPerWarp = kRouterTokensPerBlock / kWarps;  // 8
constexpr int kTokGroup = 4;
constexpr int kExpGroup = 8;

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
router_kernel(const T* __restrict__ x, const T* __restrict__ Wg, const T* __restrict__ bg,
              int64_t N, int d, int E, int k, float* __restrict__ out_logits,
              int32_t* __restrict__ out_idx, float* __restrict__ out_w,
              float* __restrict__ psum_part) {
  extern __shared__ float smem[];
  float* s_logits = smem;                                     // [32][E]
  float* s_psum = smem + (size_t)kRouterTokensPerBlock * E;   // [kWarps][E]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t tok_block0 = (int64_t)blockIdx.x * kRouterTokensPerBlock;
  const int64_t tok_warp0 = tok_block0 + warp * kTokPerWarp;

  // ---- logits ------------------------------------------------------------
  for (int g = 0; g < kTokPerWarp / kTokGroup; ++g) {
    const int64_t t0 = tok_warp0 + g * kTokGroup;
    if (t0 >= N) break;
    const T* xrow[kTokGroup];
#pragma unroll
    for (int t = 0; t < kTokGroup; ++t) {
      int64_t tt = t0 + t < N ? t0 + t : N - 1;  // clamp: duplicates are discarded below
      xrow[t] = x + tt * d;
    }
    for (int e0 = 0; e0 < E; e0 += kExpGroup) {
      float acc[kTokGroup][kExpGroup];
#pragma unroll
      for (int t = 0; t < kTokGroup; ++t)
#pragma unroll
        for (int e = 0; e < kExpGroup; ++e) acc[t][e] = 0.f;

      for (int c = lane * 8; c < d; c += 256) {
        float xv[kTokGroup][8];
#pragma unroll
        for (int t = 0; t < kTokGroup; ++t) load8(xrow[t] + c, xv[t]);
#pragma unroll
        for (int e = 0; e < kExpGroup; ++e) {
          if (e0 + e < E) {
            float wv[8];
            load8_ldg(Wg + (size_t)(e0 + e) * d + c, wv);
#pragma unroll
            for (int t = 0; t < kTokGroup; ++t)
#pragma unroll
              for (int i = 0; i < 8; ++i) acc[t][e] = fmaf(xv[t][i], wv[i], acc[t][e]);
          }
        }
      }
#pragma unroll
      for (int t = 0; t < kTokGroup; ++t)
#pragma unroll
        for (int e = 0; e < kExpGroup; ++e) {
          float v = acc[t][e];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          acc[t][e] = v;
        }
      if (lane == 0) {
#pragma unroll
        for (int t = 0; t < kTokGroup; ++t)
#pragma unroll
          for (int e = 0; e < kExpGroup; ++e)
            if (e0 + e < E)
              s_logits[(size_t)(warp * kTokPerWarp + g * kTokGroup + t) * E + e0 + e] =
                  acc[t][e] + to_f32(bg[e0 + e]);
      }
    }
  }
  __syncwarp();

  // ---- softmax, top-k, renormalise --------------------------------------
  constexpr int kPerLane = kMaxExperts / 32;  // 8
  float psum_local[kPerLane];
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) psum_local[i] = 0.f;

  for (int tl = 0; tl < kTokPerWarp; ++tl) {
    const int64_t tok = tok_warp0 + tl;
    if (tok >= N) break;
    const float* lg = s_logits + (size_t)(warp * kTokPerWarp + tl) * E;
    float l[kPerLane];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      int e = lane + 32 * i;
      l[i] = e < E ? lg[e] : -INFINITY;
      m = fmaxf(m, l[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float p[kPerLane];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      int e = lane + 32 * i;
      p[i] = e < E ? expf(l[i] - m) : 0.f;
      sum += p[i];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      p[i] = p[i] / sum;
      psum_local[i] += p[i];
    }
    if (out_logits != nullptr) {
#pragma unroll
      for (int i = 0; i < kPerLane; ++i) {
        int e = lane + 32 * i;
        if (e < E) out_logits[tok * E + e] = l[i];
      }
    }
    // k rounds of arg-max over (logit desc, index asc). Ordering by logit
    // agrees with ordering by softmax probability wherever the probabilities
    // differ, and is well defined where they collide.
    uint32_t taken = 0;  // bit i: this lane's slice i already chosen
    float total = 0.f;
    float vals[kMaxTopK];
    int sel[kMaxTopK];
    for (int j = 0; j < k; ++j) {
      float bl = -INFINITY, bp = 0.f;
      int be = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < kPerLane; ++i) {
        int e = lane + 32 * i;
        if (e < E && !((taken >> i) & 1u)) {
          if (l[i] > bl || (l[i] == bl && e < be)) { bl = l[i]; be = e; bp = p[i]; }
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        float ol = __shfl_xor_sync(0xffffffffu, bl, o);
        int oe = __shfl_xor_sync(0xffffffffu, be, o);
        float op = __shfl_xor_sync(0xffffffffu, bp, o);
        if (ol > bl || (ol == bl && oe < be)) { bl = ol; be = oe; bp = op; }
      }
      if ((be & 31) == lane && be < E) taken |= 1u << (be >> 5);
      sel[j] = be;
      vals[j] = bp;
      total += bp;  // left-to-right sum, as model.py:221
    }
    if (lane == 0) {
      for (int j = 0; j < k; ++j) {
        out_idx[tok * k + j] = sel[j];
        out_w[tok * k + j] = vals[j] / total;
      }
    }
  }

  // ---- per-block probability sums, fixed order --------------------------
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    int e = lane + 32 * i;
    if (e < E) s_psum[warp * E + e] = psum_local[i];
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) s += s_psum[w * E + e];
    psum_part[(size_t)blockIdx.x * E + e] = s;
  }
}

}  // namespace

int launch_router(const void* x, const void* Wg, const void* bg, int64_t N, int d, int E, int k,
                  int dtype, float* out_logits, int32_t* out_idx, float* out_w, float* psum_part,
                  int32_t* status, cudaStream_t s) {
  (void)status;
  if (N == 0) return 0;
  const int64_t blocks = (N + kRouterTokensPerBlock - 1) / kRouterTokensPerBlock;
  const size_t smem = sizeof(float) * (size_t)(kRouterTokensPerBlock + kWarps) * E;
  if (dtype == MOE_B200_BF16) {
    router_kernel<__nv_bfloat16><<<(unsigned)blocks, kWarps * 32, smem, s>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(Wg),
        static_cast<const __nv_bfloat16*>(bg), N, d, E, k, out_logits, out_idx, out_w, psum_part);
  } else {
    router_kernel<float><<<(unsigned)blocks, kWarps * 32, smem, s>>>(
        static_cast<const float*>(x), static_cast<const float*>(Wg), static_cast<const float*>(bg),
        N, d, E, k, out_logits, out_idx, out_w, psum_part);
  }
  MOE_CUDA_CHECK(cudaGetLastError());
  return 0;
}

}  // namespace moe
