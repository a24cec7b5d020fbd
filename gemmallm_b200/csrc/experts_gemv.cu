// Expert feed-forward for a handful of rows per call (decode with one to a few tokens):
// the same products as experts_tc2.cu (reference model.py:174,180-184), arranged as a
// weight-streaming matrix-vector product. With one or two rows per expert the work is
// 2 flops per weight byte: HBM-bound by two orders of magnitude, tensor-core shape or not,
// and what matters is how many weight bytes every SM keeps in flight. So the weights are the
// 16-row A operand of mma.sync m16n8k16 (the legacy tensor path is ample here), loaded from
// global memory straight into fragment registers with 16-byte loads (the contraction index
// inside each 32-element chunk is permuted identically for both operands), the expert's rows
// (up to 8 per pass) are the B operand, and the contraction is split over the warps of a
// block (GEGLU) and additionally over `ksplit` blocks (down product, fp32 partial sums that
// moe_b200_combine_decode adds up), so that thousands of warps stream at once even when
// only two experts are hit.
#include "common.cuh"

namespace moe {

namespace {

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The grid has one group of blocks per expert that can be hit (at most min(E, rows) of them):
// group i works on the i-th expert with rows. -1: fewer experts were hit.
__device__ __forceinline__ int nth_expert_with_rows(const int32_t* __restrict__ offsets, int E, int nth,
                                                    int* row0, int* rows) {
  int prev = __ldcg(&offsets[0]);
  for (int e = 0; e < E; ++e) {
    const int next = __ldcg(&offsets[e + 1]);
    if (next > prev && nth-- == 0) {
      *row0 = prev;
      *rows = next - prev;
      return e;
    }
    prev = next;
  }
  return -1;
}

constexpr int kWarps = 4;       // warps of a block split the contraction range of one tile
constexpr int kUnroll = 4;      // 32-element chunks in flight per lane and weight row
constexpr int kMaxPass = 2;     // n-tiles (of 8 rows) whose accumulators a warp keeps at once

// One pass over the contraction range [k_begin, k_end) (multiples of 8) for a 16-row weight
// tile `wa`/`wb` (rows g and g + 8 of this lane) against up to kMaxPass * 8 token rows.
// NW = 2 for the GEGLU product (gate tile and up tile share the token operand).
template <int NW>
__device__ __forceinline__ void stream_tile(const uint4* const (&wrow)[NW][2], const uint4* const (&trow)[kMaxPass],
                                            int piece_begin, int piece_end, int t,
                                            float (&acc)[NW][kMaxPass][4]) {
  const uint4 zero = make_uint4(0, 0, 0, 0);
  for (int p0 = piece_begin; p0 < piece_end; p0 += 4 * kUnroll) {
    uint4 A[NW][2][kUnroll], B[kMaxPass][kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int piece = p0 + 4 * u + t;
      const bool ok = piece < piece_end;
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        A[w][0][u] = ok ? __ldg(wrow[w][0] + piece) : zero;
        A[w][1][u] = ok ? __ldg(wrow[w][1] + piece) : zero;
      }
#pragma unroll
      for (int n = 0; n < kMaxPass; ++n)
        B[n][u] = (ok && trow[n] != nullptr) ? __ldcg(trow[n] + piece) : zero;
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
#pragma unroll
      for (int w = 0; w < NW; ++w)
#pragma unroll
        for (int n = 0; n < kMaxPass; ++n) {
          mma_bf16_16816(acc[w][n], A[w][0][u].x, A[w][1][u].x, A[w][0][u].y, A[w][1][u].y,
                         B[n][u].x, B[n][u].y);
          mma_bf16_16816(acc[w][n], A[w][0][u].z, A[w][1][u].z, A[w][0][u].w, A[w][1][u].w,
                         B[n][u].z, B[n][u].w);
        }
  }
}

// h[row][j] = gelu_tanh(x W1[j] + b1[j]) * (x W1[f + j] + b1[f + j]) for the rows of every
// expert; block = (expert, 16 features), its warps split d.
__global__ void __launch_bounds__(kWarps * 32)
geglu_gemv_kernel(const __nv_bfloat16* __restrict__ perm, const int32_t* __restrict__ offsets,
                  const void* const* __restrict__ W1, const void* const* __restrict__ b1, int E, int d,
                  int f, int tiles_per_expert, __nv_bfloat16* __restrict__ h) {
  __shared__ float s_red[kWarps][2][kMaxPass][4][32];
  const int slot = blockIdx.x / tiles_per_expert;
  const int j0 = (blockIdx.x - slot * tiles_per_expert) * 16;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  pdl_wait();                 // offsets and the sorted rows come from the routing kernel
  pdl_launch_dependents();
  int row0 = 0, rows = 0;
  const int e = nth_expert_with_rows(offsets, E, slot, &row0, &rows);
  if (e < 0) return;
  const int pieces = d >> 3;
  const __nv_bfloat16* W = static_cast<const __nv_bfloat16*>(W1[e]);
  const int ja = min(j0 + g, f - 1), jb = min(j0 + g + 8, f - 1);   // clamped: masked at the store
  const uint4* const wrow[2][2] = {
      {reinterpret_cast<const uint4*>(W + (size_t)ja * d), reinterpret_cast<const uint4*>(W + (size_t)jb * d)},
      {reinterpret_cast<const uint4*>(W + (size_t)(f + ja) * d), reinterpret_cast<const uint4*>(W + (size_t)(f + jb) * d)}};
  // this warp's share of the contraction: whole groups of 4 * kUnroll pieces
  const int group = 4 * kUnroll;
  const int groups = (pieces + group - 1) / group;
  const int per_warp = (groups + kWarps - 1) / kWarps;
  const int pb = min(pieces, warp * per_warp * group), pe = min(pieces, (warp + 1) * per_warp * group);
  const __nv_bfloat16* bias = static_cast<const __nv_bfloat16*>(b1[e]);
  for (int n0 = 0; n0 < rows; n0 += 8 * kMaxPass) {
    const uint4* trow[kMaxPass];
#pragma unroll
    for (int n = 0; n < kMaxPass; ++n) {
      const int r = n0 + 8 * n + g;
      trow[n] = r < rows ? reinterpret_cast<const uint4*>(perm + (size_t)(row0 + r) * d) : nullptr;
    }
    float acc[2][kMaxPass][4];
#pragma unroll
    for (int w = 0; w < 2; ++w)
#pragma unroll
      for (int n = 0; n < kMaxPass; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[w][n][i] = 0.f;
    stream_tile<2>(wrow, trow, pb, pe, t, acc);
    __syncthreads();
#pragma unroll
    for (int w = 0; w < 2; ++w)
#pragma unroll
      for (int n = 0; n < kMaxPass; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) s_red[warp][w][n][i][lane] = acc[w][n][i];
    __syncthreads();
    // accumulator layout: c0,c1 -> feature g, rows 2t, 2t+1; c2,c3 -> feature g + 8
    for (int item = threadIdx.x; item < kMaxPass * 4 * 32; item += kWarps * 32) {
      const int n = item / 128, i = (item >> 5) & 3, ln = item & 31;
      float gs = 0.f, us = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        gs += s_red[w][0][n][i][ln];
        us += s_red[w][1][n][i][ln];
      }
      const int feat = j0 + (ln >> 2) + ((i >> 1) << 3);
      const int r = n0 + 8 * n + 2 * (ln & 3) + (i & 1);
      if (feat < f && r < rows) {
        const float gv = gs + __bfloat162float(bias[feat]);
        const float uv = us + __bfloat162float(bias[f + feat]);
        h[(size_t)(row0 + r) * f + feat] = __float2bfloat16_rn(gelu_tanh_fast(gv) * uv);
      }
    }
  }
}

// part[s][row][c] = sum over the s-th range of k of h[row][k] W2[c][k] (no bias); block =
// (expert, 16 output columns, k range), its warps split the range.
__global__ void __launch_bounds__(kWarps * 32)
down_gemv_kernel(const __nv_bfloat16* __restrict__ h, const int32_t* __restrict__ offsets,
                 const void* const* __restrict__ W2, int E, int d, int f, int tiles_per_expert,
                 int ksplit, int64_t part_stride, float* __restrict__ part) {
  __shared__ float s_red[kWarps][kMaxPass][4][32];
  const int s = blockIdx.y;
  const int slot = blockIdx.x / tiles_per_expert;
  const int c0 = (blockIdx.x - slot * tiles_per_expert) * 16;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  pdl_wait();                 // h comes from the kernel before this one
  pdl_launch_dependents();
  int row0 = 0, rows = 0;
  const int e = nth_expert_with_rows(offsets, E, slot, &row0, &rows);
  if (e < 0) return;
  const int pieces = f >> 3;
  const __nv_bfloat16* W = static_cast<const __nv_bfloat16*>(W2[e]);
  const int ca = min(c0 + g, d - 1), cb = min(c0 + g + 8, d - 1);
  const uint4* const wrow[1][2] = {
      {reinterpret_cast<const uint4*>(W + (size_t)ca * f), reinterpret_cast<const uint4*>(W + (size_t)cb * f)}};
  const int group = 4 * kUnroll;
  const int groups = (pieces + group - 1) / group;
  const int per_split = (groups + ksplit - 1) / ksplit;
  const int per_warp = (per_split + kWarps - 1) / kWarps;
  const int sb = s * per_split;
  const int pb = min(pieces, min((s + 1) * per_split, sb + warp * per_warp) * group);
  const int pe = min(pieces, min((s + 1) * per_split, sb + (warp + 1) * per_warp) * group);
  for (int n0 = 0; n0 < rows; n0 += 8 * kMaxPass) {
    const uint4* trow[kMaxPass];
#pragma unroll
    for (int n = 0; n < kMaxPass; ++n) {
      const int r = n0 + 8 * n + g;
      trow[n] = r < rows ? reinterpret_cast<const uint4*>(h + (size_t)(row0 + r) * f) : nullptr;
    }
    float acc[1][kMaxPass][4];
#pragma unroll
    for (int n = 0; n < kMaxPass; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[0][n][i] = 0.f;
    stream_tile<1>(wrow, trow, pb, pe, t, acc);
    __syncthreads();
#pragma unroll
    for (int n = 0; n < kMaxPass; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) s_red[warp][n][i][lane] = acc[0][n][i];
    __syncthreads();
    for (int item = threadIdx.x; item < kMaxPass * 4 * 32; item += kWarps * 32) {
      const int n = item / 128, i = (item >> 5) & 3, ln = item & 31;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) v += s_red[w][n][i][ln];
      const int col = c0 + (ln >> 2) + ((i >> 1) << 3);
      const int r = n0 + 8 * n + 2 * (ln & 3) + (i & 1);
      if (col < d && r < rows) part[(size_t)s * part_stride + (size_t)(row0 + r) * d + col] = v;
    }
  }
}

}  // namespace

// h [M,f] and part [ksplit][M][d] (no down.bias) from the sorted rows, for calls with a few
// rows per expert. Any row count works (more than 16 rows of one expert re-read its weights).
int launch_experts_gemv(const void* perm, const int32_t* offsets, const void* plan, int64_t M, int d,
                        int f, int E, int ksplit, void* h, float* part, cudaStream_t s) {
  if (M == 0) return 0;
  PlanView pv = plan_view(plan, E);
  const int t1 = (f + 15) / 16, t2 = (d + 15) / 16;
  const int slots = (int)(M < E ? M : E);    // no more experts than rows can be hit
  MOE_CUDA_CHECK(launch_pdl(geglu_gemv_kernel, dim3((unsigned)(slots * t1)), dim3(kWarps * 32), 0, s,
                            static_cast<const __nv_bfloat16*>(perm), offsets, pv.W1, pv.b1, E, d, f, t1,
                            static_cast<__nv_bfloat16*>(h)));
  MOE_CUDA_CHECK(launch_pdl(down_gemv_kernel, dim3((unsigned)(slots * t2), (unsigned)ksplit),
                            dim3(kWarps * 32), 0, s, static_cast<const __nv_bfloat16*>(h), offsets,
                            pv.W2, E, d, f, t2, ksplit, M * (int64_t)d, part));
  return 0;
}

}  // namespace moe
