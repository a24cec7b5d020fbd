// Backward pass of the block (the reference trains through MOE.forward with torch.autograd:
// loss.backward() in train.py:140-141 reaches model.py:200-276 and 173-190). The two input
// gradients and the two weight gradients of the expert Linears are grouped products on the
// tcgen05 kernel of experts_tc2.cu; this file holds what surrounds them, all HBM-bound:
//
//   combine_bwd      dy[r] = w[pair] * dOut[token], dw[pair] = dOut[token] . y[r]   (model.py:271)
//   router_bwd       dw -> d(renormalised scores) -> d(softmax) -> dlogits, plus the gradient
//                    of the load-balancing loss through the mean probabilities
//                    (model.py:207-223; the counts of model.py:213 carry no gradient)
//   router_bwd_wx    dWg = dlogits^T x, dbg = sum dlogits, dx += dlogits Wg       (model.py:206)
//   geglu_bwd        through dropout, the product and the tanh-GELU                (model.py:180-183)
//   transposes       W -> W^T per expert (input gradients contract over the output features);
//                    activations [rows, C] -> [C, padded rows] with every expert's rows starting
//                    at a multiple of 64 and zero fill (weight gradients contract over rows)
//   colsum           bias gradients per expert
#include "common.cuh"
#include "philox.cuh"

namespace moe {

namespace {

// koff[e+1] = koff[e] + round_up(rows of e, 64)
__global__ void pad_offsets_kernel(const int32_t* __restrict__ offsets, int E, int32_t* __restrict__ koff) {
  if (threadIdx.x == 0) {
    int acc = 0;
    koff[0] = 0;
    for (int e = 0; e < E; ++e) {
      acc += (offsets[e + 1] - offsets[e] + 63) & ~63;
      koff[e + 1] = acc;
    }
  }
}

__global__ void pair_of_kernel(const int32_t* __restrict__ row_of, int64_t M, int32_t* __restrict__ pair_of) {
  const int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (p < M) {
    const int r = row_of[p];
    if (r >= 0) pair_of[r] = (int32_t)p;
  }
}

// One warp per sorted row.
__global__ void __launch_bounds__(256)
combine_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ y,
                   const int32_t* __restrict__ pair_of, const float* __restrict__ w, int64_t M, int d,
                   int k, __nv_bfloat16* __restrict__ dy, float* __restrict__ dw) {
  const int64_t r = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= M) return;
  const int p = pair_of[r];
  const int64_t t = p / k;
  const float wp = w[p];
  float dot = 0.f;
  for (int c = lane * 8; c < d; c += 256) {
    float g[8], yv[8], o[8];
    load8(dout + t * d + c, g);
    load8(y + r * d + c, yv);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      dot = fmaf(g[i], yv[i], dot);
      o[i] = wp * g[i];
    }
    store8(dy + r * d + c, o);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
  if (lane == 0) dw[p] = dot;
}

// One warp per token; lane e handles experts e, e+32, ...
//   w_j = v_j / total, v_j = p[idx_j]:  dv_j = (dw_j - sum_i dw_i w_i) / total
//   aux = E * sum_e mean_n p[n,e] * cnt0_e / N:  dp[e] += grad_aux * E * cnt0_e / N^2
//   dl[e] = p[e] * (dp[e] - sum_e' p[e'] dp[e'])
__global__ void __launch_bounds__(256)
router_bwd_kernel(const float* __restrict__ logits, const int32_t* __restrict__ idx,
                  const float* __restrict__ w, const float* __restrict__ dw,
                  const int32_t* __restrict__ cnt0, float grad_aux, int64_t N, int E, int k,
                  float* __restrict__ dl) {
  const int64_t t = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= N) return;
  constexpr int kPer = kMaxExperts / 32;
  float l[kPer], p[kPer], dp[kPer];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int e = lane + 32 * i;
    l[i] = e < E ? logits[t * E + e] : -INFINITY;
    m = fmaxf(m, l[i]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int e = lane + 32 * i;
    p[i] = e < E ? expf(l[i] - m) : 0.f;
    sum += p[i];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  // total of the chosen probabilities and sum_i dw_i w_i (every lane computes them: k <= 8)
  float total = 0.f, dww = 0.f;
  for (int j = 0; j < k; ++j) dww = fmaf(dw[t * k + j], w[t * k + j], dww);
  const float aux_c = grad_aux * (float)E / ((float)N * (float)N);
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int e = lane + 32 * i;
    p[i] = p[i] / sum;
    dp[i] = e < E ? aux_c * (float)cnt0[e] : 0.f;
  }
  for (int j = 0; j < k; ++j) {
    // p[e] lives in lane e & 31, slice e >> 5
    const int e = idx[t * k + j];
    float v = 0.f;
#pragma unroll
    for (int i = 0; i < kPer; ++i)
      if (i == (e >> 5)) v = p[i];
    total += __shfl_sync(0xffffffffu, v, e & 31);
  }
  for (int j = 0; j < k; ++j) {
    const int e = idx[t * k + j];
    const float dv = (dw[t * k + j] - dww) / total;
    if ((e & 31) == lane) {
#pragma unroll
      for (int i = 0; i < kPer; ++i)
        if (i == (e >> 5)) dp[i] += dv;
    }
  }
  float pdp = 0.f;
#pragma unroll
  for (int i = 0; i < kPer; ++i) pdp = fmaf(p[i], dp[i], pdp);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) pdp += __shfl_xor_sync(0xffffffffu, pdp, o);
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int e = lane + 32 * i;
    if (e < E) dl[t * E + e] = p[i] * (dp[i] - pdp);
  }
}

// dWg[e][c] += sum_t dl[t][e] x[t][c] (fp32 atomics into a zeroed buffer), dbg[e] += sum_t dl[t][e],
// dxr[t][c] = sum_e dl[t][e] Wg[e][c]. A block owns 256 columns and a range of tokens; experts in
// groups of 32 (E > 32 re-reads the token range from L2).
__global__ void __launch_bounds__(256)
router_bwd_wx_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ Wg,
                     const float* __restrict__ dl, int64_t N, int d, int E, int tokens_per_block,
                     float* __restrict__ dWg, float* __restrict__ dbg,
                     __nv_bfloat16* __restrict__ dxr) {
  __shared__ float s_dl[64][33];
  const int c = blockIdx.x * 256 + threadIdx.x;
  const int64_t t_begin = (int64_t)blockIdx.y * tokens_per_block;
  const int64_t t_end = t_begin + tokens_per_block < N ? t_begin + tokens_per_block : N;
  const bool col_ok = c < d;
  for (int e0 = 0; e0 < E; e0 += 32) {
    const int ne = E - e0 < 32 ? E - e0 : 32;
    float acc[32], wg[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      acc[i] = 0.f;
      wg[i] = (col_ok && i < ne) ? __bfloat162float(Wg[(size_t)(e0 + i) * d + c]) : 0.f;
    }
    float bsum = 0.f;   // thread i < ne of column block 0 sums dl[:, e0 + i]
    for (int64_t t0 = t_begin; t0 < t_end; t0 += 64) {
      const int nt = (int)(t_end - t0 < 64 ? t_end - t0 : 64);
      __syncthreads();
      for (int i = threadIdx.x; i < 64 * 32; i += 256) {
        const int tl = i >> 5, el = i & 31;
        s_dl[tl][el] = (tl < nt && el < ne) ? dl[(t0 + tl) * E + e0 + el] : 0.f;
      }
      __syncthreads();
      if (blockIdx.x == 0 && (int)threadIdx.x < ne)
        for (int tl = 0; tl < nt; ++tl) bsum += s_dl[tl][threadIdx.x];
      if (col_ok) {
        for (int tl = 0; tl < nt; ++tl) {
          const float xv = __bfloat162float(x[(t0 + tl) * d + c]);
          float dx = 0.f;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float g = s_dl[tl][i];
            acc[i] = fmaf(g, xv, acc[i]);
            dx = fmaf(g, wg[i], dx);
          }
          // more than 32 experts: the sum over expert groups passes through the bf16 buffer
          // (one extra rounding per group of 32 experts)
          float prev = e0 == 0 ? 0.f : __bfloat162float(dxr[(t0 + tl) * d + c]);
          dxr[(t0 + tl) * d + c] = __float2bfloat16_rn(prev + dx);
        }
      }
    }
    if (col_ok)
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < ne) atomicAdd(&dWg[(size_t)(e0 + i) * d + c], acc[i]);
    if (blockIdx.x == 0 && (int)threadIdx.x < ne) atomicAdd(&dbg[e0 + threadIdx.x], bsum);
  }
}

__global__ void iota_kernel(int32_t* __restrict__ p, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = (int32_t)i;
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ src, int64_t n, __nv_bfloat16* __restrict__ dst) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = __float2bfloat16_rn(src[i]);
}

__global__ void fill_f32_kernel(float* __restrict__ p, int64_t n, float v) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = v;
}

// In place over gu [M, 2f]: (g, u) -> (dg, du), given dh [M, f] (gradient of the dropped h):
//   dhe = dh * mask * scale;  du = dhe * gelu(g);  dg = dhe * u * gelu'(g)
//   gelu(g) = 0.5 g (1 + t), t = tanh(b (g + a g^3)), gelu'(g) = 0.5 (1 + t) + 0.5 g (1 - t^2) b (1 + 3 a g^2)
__global__ void __launch_bounds__(256)
geglu_bwd_kernel(const __nv_bfloat16* __restrict__ dh, __nv_bfloat16* __restrict__ gu,
                 const int32_t* __restrict__ pair_of, int64_t M, int f, uint32_t thresh, float scale,
                 uint32_t seed_lo, uint32_t seed_hi) {
  const int pieces = f >> 3;
  const int64_t item = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= M * pieces) return;
  const int64_t r = item / pieces;
  const int c = (int)(item - r * pieces) << 3;
  float dv[8], g[8], u[8], dg[8], du[8];
  load8(dh + r * f + c, dv);
  load8(gu + r * 2 * f + c, g);
  load8(gu + r * 2 * f + f + c, u);
  if (thresh != 0u) {
    const uint32_t pair = (uint32_t)pair_of[r];
#pragma unroll
    for (int b4 = 0; b4 < 2; ++b4) {
      const uint4 rn = philox4x32_10((uint32_t)(c >> 2) + b4, pair, seed_lo, seed_hi);
      const uint32_t wv[4] = {rn.x, rn.y, rn.z, rn.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) dv[b4 * 4 + i] = wv[i] >= thresh ? dv[b4 * 4 + i] * scale : 0.f;
    }
  }
  const float kB = 0.7978845608028654f, kA = 0.044715f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float x = g[i];
    const float t = tanhf(kB * (x + kA * x * x * x));
    const float gelu = 0.5f * x * (1.f + t);
    const float dgelu = 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * kB * (1.f + 3.f * kA * x * x);
    du[i] = dv[i] * gelu;
    dg[i] = dv[i] * u[i] * dgelu;
  }
  store8(gu + r * 2 * f + c, dg);
  store8(gu + r * 2 * f + f + c, du);
}

// 64 x 64 tile transpose with 16-byte global accesses on both sides: rows r < rows_valid of
// `src` (row pitch C elements, columns [c0, c0 + 64)) become columns of `dst`:
// dst[(c0 + c) * ldd + i] = src[i][c0 + c], zero where i >= rows_valid. Positions i >= k_valid of
// dst do not exist and are not written. Shared memory holds the tile as 32-bit words (two
// neighbouring columns), 33 words per row; a thread then reads one word of eight consecutive
// rows and splits them into the two columns' 16-byte pieces.
__device__ __forceinline__ void transpose_tile64(const __nv_bfloat16* __restrict__ src, int rows_valid,
                                                 int C, int c0, __nv_bfloat16* __restrict__ dst,
                                                 int64_t ldd, int k_valid, uint32_t (&tile)[64 * 33]) {
  const int tid = threadIdx.x;
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    const int p = tid + s * 256;
    const int i = p >> 3, pc = p & 7;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (i < rows_valid && c0 + pc * 8 < C)
      v = __ldg(reinterpret_cast<const uint4*>(src + (size_t)i * C + c0 + pc * 8));
    uint32_t* t4 = &tile[i * 33 + pc * 4];
    t4[0] = v.x; t4[1] = v.y; t4[2] = v.z; t4[3] = v.w;
  }
  __syncthreads();
  const int kp = tid & 7, cp = tid >> 3;     // eight rows kp*8.., columns 2cp and 2cp + 1
  uint32_t w[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) w[q] = tile[(kp * 8 + q) * 33 + cp];
  uint4 lo, hi;
  lo.x = __byte_perm(w[0], w[1], 0x5410); hi.x = __byte_perm(w[0], w[1], 0x7632);
  lo.y = __byte_perm(w[2], w[3], 0x5410); hi.y = __byte_perm(w[2], w[3], 0x7632);
  lo.z = __byte_perm(w[4], w[5], 0x5410); hi.z = __byte_perm(w[4], w[5], 0x7632);
  lo.w = __byte_perm(w[6], w[7], 0x5410); hi.w = __byte_perm(w[6], w[7], 0x7632);
  if (kp * 8 < k_valid) {
    const int c = c0 + 2 * cp;
    if (c < C) *reinterpret_cast<uint4*>(dst + (size_t)(2 * cp) * ldd + kp * 8) = lo;
    if (c + 1 < C) *reinterpret_cast<uint4*>(dst + (size_t)(2 * cp + 1) * ldd + kp * 8) = hi;
  }
}

// dst[e] [C, R] = src[e] [R, C] transposed (R, C multiples of 8); one block per 64 x 64 tile.
__global__ void __launch_bounds__(256)
transpose_weight_kernel(const void* const* __restrict__ src_ptrs, int R, int C,
                        __nv_bfloat16* __restrict__ dst) {
  __shared__ uint32_t tile[64 * 33];
  const int e = blockIdx.z;
  const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(src_ptrs[e]);
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const int rows = R - r0 < 64 ? R - r0 : 64;
  transpose_tile64(src + (size_t)r0 * C, rows, C, c0,
                   dst + (size_t)e * R * C + (size_t)c0 * R + r0, R, rows, tile);
}

// dst [C, Kpad]: column koff[e] + j holds row offsets[e] + j of src [M, C] for j < rows of e,
// zero for the padding up to koff[e+1]. One block per 64 padded columns x 64 source columns.
__global__ void __launch_bounds__(256)
transpose_pad_kernel(const __nv_bfloat16* __restrict__ src, const int32_t* __restrict__ offsets,
                     const int32_t* __restrict__ koff, int E, int C, int64_t Kpad,
                     __nv_bfloat16* __restrict__ dst) {
  __shared__ uint32_t tile[64 * 33];
  __shared__ int s_row0, s_rows;
  const int k0 = blockIdx.x * 64, c0 = blockIdx.y * 64;
  if (threadIdx.x == 0) {
    int row0 = 0, rows = 0;
    if (k0 < koff[E]) {
      int lo = 0, hi = E;   // last e with koff[e] <= k0
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (koff[mid] <= k0) lo = mid; else hi = mid;
      }
      const int within = k0 - koff[lo];
      const int n = offsets[lo + 1] - offsets[lo];
      row0 = offsets[lo] + within;
      rows = n - within < 0 ? 0 : (n - within > 64 ? 64 : n - within);
    }
    s_row0 = row0;
    s_rows = rows;
  }
  __syncthreads();
  transpose_tile64(src + (size_t)s_row0 * C, s_rows, C, c0, dst + (size_t)c0 * Kpad + k0, Kpad, 64, tile);
}

// db[e][c] = sum over the expert's rows of src[r][c] (C a multiple of 8). One block per (expert,
// 64 columns): eight threads cover a row's 128 bytes, 32 such groups take rows r, r + 32, ...
// with four 16-byte loads in flight each; the 32 partial sums of a column are added in order.
__global__ void __launch_bounds__(256)
colsum_kernel(const __nv_bfloat16* __restrict__ src, const int32_t* __restrict__ offsets, int C,
              __nv_bfloat16* __restrict__ db) {
  __shared__ float part[32][65];
  const int e = blockIdx.y;
  const int pc = threadIdx.x & 7, lane_r = threadIdx.x >> 3;
  const int c = blockIdx.x * 64 + pc * 8;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  if (c < C) {
    const int r1 = offsets[e + 1];
    int r = offsets[e] + lane_r;
    const uint4* base = reinterpret_cast<const uint4*>(src + c);
    const size_t pitch = (size_t)C >> 3;     // 16-byte pieces per row
    for (; r + 96 < r1; r += 128) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = __ldg(base + (size_t)(r + 32 * u) * pitch);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[2 * i] += bf16_lo(w[i]);
          acc[2 * i + 1] += bf16_hi(w[i]);
        }
      }
    }
    for (; r < r1; r += 32) {
      const uint4 v = __ldg(base + (size_t)r * pitch);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[2 * i] += bf16_lo(w[i]);
        acc[2 * i + 1] += bf16_hi(w[i]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) part[lane_r][pc * 8 + i] = acc[i];
  __syncthreads();
  if (threadIdx.x < 64) {
    const int col = blockIdx.x * 64 + threadIdx.x;
    if (col < C) {
      float sum = 0.f;
      for (int q = 0; q < 32; ++q) sum += part[q][threadIdx.x];
      db[(size_t)e * C + col] = __float2bfloat16_rn(sum);
    }
  }
}

unsigned blocks_for(int64_t n, int per) { return (unsigned)((n + per - 1) / per); }

}  // namespace

int launch_pair_of(const int32_t* row_of, int64_t M, int32_t* pair_of, cudaStream_t s) {
  if (M == 0) return 0;
  pair_of_kernel<<<blocks_for(M, 256), 256, 0, s>>>(row_of, M, pair_of);
  MOE_CUDA_CHECK(cudaGetLastError());
  return 0;
}

int launch_pad_offsets(const int32_t* offsets, int E, int32_t* koff, cudaStream_t s) {
  pad_offsets_kernel<<<1, 32, 0, s>>>(offsets, E, koff);
  MOE_CUDA_CHECK(cudaGetLastError());
  return 0;
}

int launch_combine_bwd(const void* dout, const void* y, const int32_t* pair_of, const float* w,
                       int64_t M, int d, int k, void* dy, float* dw, cudaStream_t s) {
  if (M == 0) return 0;
  combine_bwd_kernel<<<blocks_for(M, 8), 256, 0, s>>>(
      static_cast<const __nv_bfloat16*>(dout), static_cast<const __nv_bfloat16*>(y), pair_of, w, M, d,
      k, static_cast<__nv_bfloat16*>(dy), dw);
  MOE_CUDA_CHECK(cudaGetLastError());
  return 0;
}

int launch_router_bwd(const float* logits, const int32_t* idx, const float* w, const float* dw,
                      const int32_t* cnt0, float grad_aux, const void* x, const void* Wg, int64_t N,
                      int d, int E, int k, float* dl, float* dWg_f32, float* dbg_f32, void* dWg,
                      void* dbg, void* dxr, cudaStream_t s) {
  if (N == 0) return 0;
  router_bwd_kernel<<<blocks_for(N, 8), 256, 0, s>>>(logits, idx, w, dw, cnt0, grad_aux, N, E, k, dl);
  MOE_CUDA_CHECK(cudaGetLastError());
  MOE_CUDA_CHECK(cudaMemsetAsync(dWg_f32, 0, sizeof(float) * (size_t)E * d, s));
  MOE_CUDA_CHECK(cudaMemsetAsync(dbg_f32, 0, sizeof(float) * (size_t)E, s));
  // about two token ranges per SM column block
  int sms = 0;
  int rc = sm_count(&sms);
  if (rc) return rc;
  const int col_blocks = (d + 255) / 256;
  int64_t ranges = (2 * (int64_t)sms + col_blocks - 1) / col_blocks;
  int64_t per = (N + ranges - 1) / ranges;
  per = (per + 63) / 64 * 64;
  ranges = (N + per - 1) / per;
  router_bwd_wx_kernel<<<dim3(col_blocks, (unsigned)ranges), 256, 0, s>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(Wg), dl, N, d, E,
      (int)per, dWg_f32, dbg_f32, static_cast<__nv_bfloat16*>(dxr));
  MOE_CUDA_CHECK(cudaGetLastError());
  f32_to_bf16_kernel<<<blocks_for((int64_t)E * d, 256), 256, 0, s>>>(dWg_f32, (int64_t)E * d,
                                                                       static_cast<__nv_bfloat16*>(dWg));
  f32_to_bf16_kernel<<<blocks_for(E, 256), 256, 0, s>>>(dbg_f32, E, static_cast<__nv_bfloat16*>(dbg));
  MOE_CUDA_CHECK(cudaGetLastError());
  return 0;
}

int launch_iota(int32_t* p, int64_t n, cudaStream_t s) {
  if (n == 0) return 0;
  iota_kernel<<<blocks_for(n, 256), 256, 0, s>>>(p, n);
  MOE_CUDA_CHECK(cudaGetLastError());
  return 0;
}

int launch_fill_f32(float* p, int64_t n, float v, cudaStream_t s) {
  if (n == 0) return 0;
  fill_f32_kernel<<<blocks_for(n, 256), 256, 0, s>>>(p, n, v);
  MOE_CUDA_CHECK(cudaGetLastError());
  return 0;
}

int launch_geglu_bwd(const void* dh, void* gu, const int32_t* pair_of, int64_t M, int f,
                     uint32_t thresh, float scale, uint32_t seed_lo, uint32_t seed_hi, cudaStream_t s) {
  if (M == 0) return 0;
  geglu_bwd_kernel<<<blocks_for(M * (f >> 3), 256), 256, 0, s>>>(
      static_cast<const __nv_bfloat16*>(dh), static_cast<__nv_bfloat16*>(gu), pair_of, M, f, thresh,
      scale, seed_lo, seed_hi);
  MOE_CUDA_CHECK(cudaGetLastError());
  return 0;
}

int launch_transpose_weights(const void* const* src_ptrs, int E, int R, int C, void* dst, cudaStream_t s) {
  transpose_weight_kernel<<<dim3((C + 63) / 64, (R + 63) / 64, E), 256, 0, s>>>(
      src_ptrs, R, C, static_cast<__nv_bfloat16*>(dst));
  MOE_CUDA_CHECK(cudaGetLastError());
  return 0;
}

int launch_transpose_pad(const void* src, const int32_t* offsets, const int32_t* koff, int E, int C,
                         int64_t Kpad, void* dst, cudaStream_t s) {
  if (Kpad == 0) return 0;
  transpose_pad_kernel<<<dim3((unsigned)(Kpad / 64), (C + 63) / 64), 256, 0, s>>>(
      static_cast<const __nv_bfloat16*>(src), offsets, koff, E, C, Kpad, static_cast<__nv_bfloat16*>(dst));
  MOE_CUDA_CHECK(cudaGetLastError());
  return 0;
}

int launch_colsum(const void* src, const int32_t* offsets, int E, int C, void* db, cudaStream_t s) {
  colsum_kernel<<<dim3((C + 63) / 64, E), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(src),
                                                        offsets, C, static_cast<__nv_bfloat16*>(db));
  MOE_CUDA_CHECK(cudaGetLastError());
  return 0;
}

}  // namespace moe
