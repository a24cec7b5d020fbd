// Router kernels: logits = x Wg^T + bg in fp32, softmax, top-k, renormalise.
// Cover reference model.py:206-223 (gate Linear, F.softmax, topk, score
// renormalisation) and the per-expert probability sums of model.py:215.
//
// HBM-bound: x [N,d] is read once; Wg [E,d] stays in L1/L2. A block of four
// warps owns 64 consecutive tokens.
//   bf16: router_mma_kernel. Each warp owns 16 tokens and forms their logits
//     with mma.sync m16n8k16 (bf16 products are exact in fp32, accumulation in
//     fp32). Operands go from global memory straight into fragment registers
//     with 16-byte loads: the contraction index inside each 32-element chunk is
//     permuted the same way for x and Wg, which a dot product does not notice.
//     Eight warps per block: two warps share each group of 16 tokens and split d
//     between them (twice the loads in flight per SM; the op is latency-bound
//     otherwise), the second one's partial sums pass through shared memory.
//     Then four lanes per token do softmax / top-k over a quarter of the E logits each.
//   fp32: router_kernel. CUDA-core FMA (TF32 would perturb the logits), four
//     tokens x eight experts per warp pass, warp-shuffle reductions, softmax and
//     top-k with one expert slice per lane.
// With the caller's LayerNorm folded in (NORM, norm.cu): Wg is the folded weight
// Wn = Wg * gamma, the same pass over x also forms sum(x - x0) and sum((x - x0)^2)
// per row (x0 = the row's first element: a shift that keeps the one-pass variance
// well conditioned), and logits = rstd * (x . Wn - mean * c1) + c2. (mean, rstd)
// go to `stats` for the dispatch kernel (reference model.py:311-312, 206).
#include "common.cuh"

namespace moe {

namespace {

constexpr int kWarps = 4;
constexpr int kTokPerWarp = kRouterTokensPerBlock / kWarps;  // 16
constexpr int kTokGroup = 4;
constexpr int kExpGroup = 8;

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
router_kernel(const T* __restrict__ x, const T* __restrict__ Wg, const T* __restrict__ bg,
              int64_t N, int d, int E, int k, float* __restrict__ out_logits,
              int32_t* __restrict__ out_idx, float* __restrict__ out_w,
              float* __restrict__ psum_part, const float* __restrict__ norm_c, float eps,
              float* __restrict__ stats) {
  extern __shared__ float smem[];
  float* s_logits = smem;                                     // [64][E]
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
    // LayerNorm statistics of the four rows, formed in the first pass over them
    float shift[kTokGroup], mean[kTokGroup], rstd[kTokGroup];
#pragma unroll
    for (int t = 0; t < kTokGroup; ++t) {
      shift[t] = norm_c != nullptr ? to_f32(xrow[t][0]) : 0.f;
      mean[t] = 0.f;
      rstd[t] = 1.f;
    }
    for (int e0 = 0; e0 < E; e0 += kExpGroup) {
      float acc[kTokGroup][kExpGroup];
#pragma unroll
      for (int t = 0; t < kTokGroup; ++t)
#pragma unroll
        for (int e = 0; e < kExpGroup; ++e) acc[t][e] = 0.f;

      const bool first_pass = norm_c != nullptr && e0 == 0;
      float s1[kTokGroup], s2[kTokGroup];
#pragma unroll
      for (int t = 0; t < kTokGroup; ++t) s1[t] = s2[t] = 0.f;
      for (int c = lane * 8; c < d; c += 256) {
        float xv[kTokGroup][8];
#pragma unroll
        for (int t = 0; t < kTokGroup; ++t) load8(xrow[t] + c, xv[t]);
        if (first_pass) {
#pragma unroll
          for (int t = 0; t < kTokGroup; ++t)
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float dv = xv[t][i] - shift[t];
              s1[t] += dv;
              s2[t] = fmaf(dv, dv, s2[t]);
            }
        }
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
      if (first_pass) {
#pragma unroll
        for (int t = 0; t < kTokGroup; ++t) {
          float a = s1[t], b = s2[t];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            a += __shfl_xor_sync(0xffffffffu, a, o);
            b += __shfl_xor_sync(0xffffffffu, b, o);
          }
          const float m1 = a / (float)d;
          mean[t] = shift[t] + m1;
          rstd[t] = rsqrtf(fmaxf(b / (float)d - m1 * m1, 0.f) + eps);
          if (lane == 0 && t0 + t < N) {
            stats[2 * (t0 + t)] = mean[t];
            stats[2 * (t0 + t) + 1] = rstd[t];
          }
        }
      }
      if (lane == 0) {
#pragma unroll
        for (int t = 0; t < kTokGroup; ++t)
#pragma unroll
          for (int e = 0; e < kExpGroup; ++e)
            if (e0 + e < E)
              s_logits[(size_t)(warp * kTokPerWarp + g * kTokGroup + t) * E + e0 + e] =
                  norm_c != nullptr
                      ? rstd[t] * (acc[t][e] - mean[t] * norm_c[e0 + e]) + norm_c[E + e0 + e]
                      : acc[t][e] + to_f32(bg[e0 + e]);
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


// ---------------------------------------------------------------------------
// bf16 path
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int kMmaTokPerWarp = 16;
constexpr int kMmaWarps = 2 * kWarps;   // two warps per token group: each takes half of d

// NT = n-tiles (of 8 experts) per pass over x; E > 8*NT makes more passes.
__device__ __forceinline__ void shifted_sums(const uint4& v, float shift, float& s1, float& s2) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float a = bf16_lo(w[i]) - shift, b = bf16_hi(w[i]) - shift;
    s1 += a + b;
    s2 = fmaf(a, a, fmaf(b, b, s2));
  }
}

// STAGE: x and the block's slice of Wg go through shared memory in four cp.async stages of one
// 32-element chunk per half of d: the four token groups of a block share one read of Wg, and the
// loads of x run three steps ahead of the products without costing registers. Without it every
// warp reads its fragments straight from global memory, which is the faster way while Wg fits
// L1 (E <= 16) and few accumulators leave room for many loads in flight.
template <int NT, bool NORM, bool STAGE>
__global__ void __launch_bounds__(kMmaWarps * 32, (NT >= 4 || NORM) ? 2 : 0)
router_mma_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ Wg,
                  const __nv_bfloat16* __restrict__ bg, int64_t N, int d, int E, int k,
                  float* __restrict__ out_logits, int32_t* __restrict__ out_idx,
                  float* __restrict__ out_w, float* __restrict__ psum_part,
                  const float* __restrict__ norm_c, float eps, float* __restrict__ stats) {
  constexpr int kMmaUnroll = STAGE ? 1 : (NT <= 2 ? 8 : 4);   // 32-element chunks per lane and step
  constexpr int kStages = 4;
  constexpr int kXch = NT * 4 + 4;              // floats a lane hands over: accumulators, row sums
  extern __shared__ float smem[];
  const int ld = E + 1;                                           // row pitch: no bank conflicts
  float* s_logits = smem;                                          // [64][E+1]
  float* s_psum = smem + (size_t)kRouterTokensPerBlock * ld;       // [kWarps][E]
  float* s_xch = s_psum + (size_t)kWarps * E;                      // [kWarps][32][kXch]
  // one stage, in 16-byte pieces: Wg [2 halves of d][8*NT rows][4], then x [2 halves][64 tokens][4]
  constexpr int kStageW = 2 * 8 * NT * 4;
  constexpr int kStagePieces = kStageW + 2 * kRouterTokensPerBlock * 4;
  uint4* s_stage = reinterpret_cast<uint4*>(
      (reinterpret_cast<uintptr_t>(s_xch + (size_t)kWarps * 32 * kXch) + 15) & ~(uintptr_t)15);

  const int lane = threadIdx.x & 31;
  const int warp = (threadIdx.x >> 5) & (kWarps - 1);   // token group
  const int khalf = threadIdx.x >> 7;                   // which half of d this warp contracts
  const int g = lane >> 2, t = lane & 3;
  const int64_t tok0 = (int64_t)blockIdx.x * kRouterTokensPerBlock + warp * kMmaTokPerWarp;
  const int nvalid = (int)(N - tok0 < kMmaTokPerWarp ? (N - tok0 > 0 ? N - tok0 : 0) : kMmaTokPerWarp);
  float* my_logits = s_logits + (size_t)warp * kMmaTokPerWarp * ld;
  float* my_xch = s_xch + ((size_t)warp * 32 + lane) * kXch;

  {
    const int row_pieces = d >> 3;  // 16-byte pieces per row
    const int64_t ra = tok0 + g < N ? tok0 + g : N - 1;
    const int64_t rb = tok0 + g + 8 < N ? tok0 + g + 8 : N - 1;
    const uint4* xa = reinterpret_cast<const uint4*>(x + ra * d);
    const uint4* xb = reinterpret_cast<const uint4*>(x + rb * d);
    const uint4* w4 = reinterpret_cast<const uint4*>(Wg);
    const int nchunk = (d + 31) >> 5;
    const int half = ((nchunk + 1) / 2 + kMmaUnroll - 1) / kMmaUnroll * kMmaUnroll;
    const int c_begin = khalf ? (half < nchunk ? half : nchunk) : 0;
    const int c_end = khalf ? nchunk : (half < nchunk ? half : nchunk);
    const uint4 zero = make_uint4(0, 0, 0, 0);
    // staged mode: step = pass over experts * iters + iteration; both halves of d make `iters`
    // iterations (the shorter half pads with zeros) so that the block's barriers line up
    const int iters = half / kMmaUnroll;
    const int passes = (E + 8 * NT - 1) / (8 * NT);
    const int total_steps = passes * iters;
    const int64_t blk_tok0 = (int64_t)blockIdx.x * kRouterTokensPerBlock;
    // this thread's pieces of a stage: x piece (token, tt) of both halves of d, and one or two
    // pieces of Wg; only the chunk index changes from step to step
    const int p_tt = threadIdx.x & 3;
    const int p_tok = (threadIdx.x >> 2) & (kRouterTokensPerBlock - 1);
    const int64_t p_row = blk_tok0 + p_tok < N ? blk_tok0 + p_tok : N - 1;   // clamped: masked later
    const uint4* p_x = reinterpret_cast<const uint4*>(x) + (size_t)p_row * row_pieces + p_tt;
    constexpr int kWPer = kStageW / (kMmaWarps * 32);       // 1 (NT = 4) or 2 (NT = 8)
    static_assert(!STAGE || (kStageW % (kMmaWarps * 32) == 0 && kWPer >= 1), "stage shape");
    const int cb1 = half < nchunk ? half : nchunk;          // first chunk of the second half
    auto prefetch = [&](int step) {
      if (step < total_steps) {
        const int pass = step / iters, it = step - pass * iters;
        uint4* dst = s_stage + (size_t)(step % kStages) * kStagePieces;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int chunk = (h ? cb1 : 0) + it;
          const int piece = 4 * chunk + p_tt;
          uint4* d4 = dst + kStageW + (size_t)threadIdx.x + h * (kMmaWarps * 32);
          if (chunk < (h ? nchunk : cb1) && piece < row_pieces) {
            const uint32_t sa = (uint32_t)__cvta_generic_to_shared(d4);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(sa), "l"(p_x + 4 * chunk) : "memory");
          } else {
            *d4 = zero;
          }
        }
#pragma unroll
        for (int q = 0; q < kWPer; ++q) {
          const int i = threadIdx.x + q * (kMmaWarps * 32);
          const int r = (i >> 2) & (8 * NT - 1), h = i / (8 * NT * 4);
          const int chunk = (h ? cb1 : 0) + it;
          const int piece = 4 * chunk + p_tt;
          const int row = pass * 8 * NT + r;
          if (row < E && chunk < (h ? nchunk : cb1) && piece < row_pieces) {
            const uint32_t sa = (uint32_t)__cvta_generic_to_shared(dst + i);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
                         :: "r"(sa), "l"(w4 + (size_t)row * row_pieces + piece) : "memory");
          } else {
            dst[i] = zero;
          }
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");   // one group per step, empty or not
    };
    if (STAGE)
      for (int s0 = 0; s0 < kStages - 1; ++s0) prefetch(s0);
    // LayerNorm statistics of rows g and g+8: this lane's pieces, then the quad's four lanes
    float sha = 0.f, shb = 0.f, s1a = 0.f, s2a = 0.f, s1b = 0.f, s2b = 0.f;
    float mean_a = 0.f, rstd_a = 1.f, mean_b = 0.f, rstd_b = 1.f;
    if (NORM) {
      sha = __bfloat162float(x[ra * d]);
      shb = __bfloat162float(x[rb * d]);
    }
    for (int e_base = 0; e_base < E; e_base += 8 * NT) {
      float acc[NT][4];
#pragma unroll
      for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
      for (int c0 = c_begin, it = 0; STAGE ? it < iters : c0 < c_end; c0 += kMmaUnroll, ++it) {
        uint4 A[kMmaUnroll], B[kMmaUnroll];
        const uint4* st = nullptr;
        if (STAGE) {
          const int step = (e_base / (8 * NT)) * iters + it;
          asm volatile("cp.async.wait_group %0;" :: "n"(kStages - 2) : "memory");
          __syncthreads();   // this step's stage is complete; the stage of the step before is free
          prefetch(step + kStages - 1);
          st = s_stage + (size_t)(step % kStages) * kStagePieces;
        }
#pragma unroll
        for (int u = 0; u < kMmaUnroll; ++u) {
          const int piece = 4 * (c0 + u) + t;
          const bool ok = piece < row_pieces && c0 + u < c_end;
          if (STAGE) {
            const uint4* sx = st + kStageW + ((size_t)khalf * kRouterTokensPerBlock + warp * kMmaTokPerWarp) * 4;
            A[u] = sx[g * 4 + t];
            B[u] = sx[(g + 8) * 4 + t];
          } else {
            A[u] = ok ? xa[piece] : zero;
            B[u] = ok ? xb[piece] : zero;
          }
          if (NORM && e_base == 0 && ok) {
            shifted_sums(A[u], sha, s1a, s2a);
            shifted_sums(B[u], shb, s1b, s2b);
          }
        }
#pragma unroll
        for (int u = 0; u < kMmaUnroll; ++u) {
          const int piece = 4 * (c0 + u) + t;
#pragma unroll
          for (int j = 0; j < NT; ++j) {
            uint4 w;
            if (STAGE) {
              w = st[((size_t)khalf * 8 * NT + 8 * j + g) * 4 + t];
            } else {
              const int row = e_base + 8 * j + g;
              w = (row < E && piece < row_pieces && c0 + u < c_end)
                      ? __ldg(w4 + (size_t)row * row_pieces + piece) : zero;
            }
            mma_bf16_16816(acc[j], A[u].x, B[u].x, A[u].y, B[u].y, w.x, w.y);
            mma_bf16_16816(acc[j], A[u].z, B[u].z, A[u].w, B[u].w, w.z, w.w);
          }
        }
      }
      // the second half's partial sums join the first half's
      __syncthreads();
      if (khalf == 1) {
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
          for (int i = 0; i < 4; ++i) my_xch[j * 4 + i] = acc[j][i];
        my_xch[NT * 4 + 0] = s1a; my_xch[NT * 4 + 1] = s2a;
        my_xch[NT * 4 + 2] = s1b; my_xch[NT * 4 + 3] = s2b;
      }
      __syncthreads();
      if (khalf == 1) continue;
#pragma unroll
      for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] += my_xch[j * 4 + i];
      if (NORM && e_base == 0) {
        s1a += my_xch[NT * 4 + 0]; s2a += my_xch[NT * 4 + 1];
        s1b += my_xch[NT * 4 + 2]; s2b += my_xch[NT * 4 + 3];
#pragma unroll
        for (int o = 1; o <= 2; o <<= 1) {
          s1a += __shfl_xor_sync(0xffffffffu, s1a, o);
          s2a += __shfl_xor_sync(0xffffffffu, s2a, o);
          s1b += __shfl_xor_sync(0xffffffffu, s1b, o);
          s2b += __shfl_xor_sync(0xffffffffu, s2b, o);
        }
        const float ma = s1a / (float)d, mb = s1b / (float)d;
        mean_a = sha + ma;
        mean_b = shb + mb;
        rstd_a = rsqrtf(fmaxf(s2a / (float)d - ma * ma, 0.f) + eps);
        rstd_b = rsqrtf(fmaxf(s2b / (float)d - mb * mb, 0.f) + eps);
        if (t == 0) {
          if (tok0 + g < N) { stats[2 * (tok0 + g)] = mean_a; stats[2 * (tok0 + g) + 1] = rstd_a; }
          if (tok0 + g + 8 < N) { stats[2 * (tok0 + g + 8)] = mean_b; stats[2 * (tok0 + g + 8) + 1] = rstd_b; }
        }
      }
      // accumulator layout: c0,c1 -> token g, experts 2t,2t+1; c2,c3 -> token g+8
#pragma unroll
      for (int j = 0; j < NT; ++j) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int e = e_base + 8 * j + 2 * t + h;
          if (e < E) {
            if (NORM) {
              const float c1 = norm_c[e], c2 = norm_c[E + e];
              my_logits[g * ld + e] = rstd_a * (acc[j][h] - mean_a * c1) + c2;
              my_logits[(g + 8) * ld + e] = rstd_b * (acc[j][2 + h] - mean_b * c1) + c2;
            } else {
              const float b = __bfloat162float(bg[e]);
              my_logits[g * ld + e] = acc[j][h] + b;
              my_logits[(g + 8) * ld + e] = acc[j][2 + h] + b;
            }
          }
        }
      }
    }
  }
  __syncthreads();   // the logits of the block's 64 tokens are in shared memory
  const int64_t blk_tok0 = (int64_t)blockIdx.x * kRouterTokensPerBlock;
  const int blk_valid = (int)(N - blk_tok0 < kRouterTokensPerBlock ? N - blk_tok0 : kRouterTokensPerBlock);
  if (out_logits != nullptr) {
    for (int i = threadIdx.x; i < blk_valid * E; i += blockDim.x) {
      const int tl = i / E, e = i - tl * E;
      out_logits[blk_tok0 * E + i] = s_logits[tl * ld + e];
    }
  }
  // ---- four lanes per token (experts sub, sub + 4, ...): softmax, top-k by (logit desc,
  // index asc), renormalise; the quad's lanes are neighbours in a warp ----
  {
    const int tl = threadIdx.x >> 2, sub = threadIdx.x & 3;
    float* lg = s_logits + tl * ld;
    float m = -INFINITY;
    for (int e = sub; e < E; e += 4) m = fmaxf(m, lg[e]);
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
    float sum = 0.f;
    for (int e = sub; e < E; e += 4) sum += expf(lg[e] - m);
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    int sel[kMaxTopK];
    float sl[kMaxTopK], vals[kMaxTopK];
    float total = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxTopK; ++j) {
      if (j < k) {
        float bl = -INFINITY;
        int be = 0x7fffffff;
        for (int e = sub; e < E; e += 4) {
          const float v = lg[e];
          if (v > bl) { bl = v; be = e; }   // strict: the lowest index wins among equals
        }
#pragma unroll
        for (int o = 1; o <= 2; o <<= 1) {
          const float ol = __shfl_xor_sync(0xffffffffu, bl, o);
          const int oe = __shfl_xor_sync(0xffffffffu, be, o);
          if (ol > bl || (ol == bl && oe < be)) { bl = ol; be = oe; }
        }
        sel[j] = be;
        sl[j] = bl;
        vals[j] = expf(bl - m) / sum;
        total += vals[j];                    // left-to-right sum, as model.py:221
        if ((be & 3) == sub && be < E) lg[be] = -INFINITY;   // taken (only its owner reads it again)
      }
    }
#pragma unroll
    for (int j = 0; j < kMaxTopK; ++j) {
      if (j < k) {
        if ((sel[j] & 3) == sub && sel[j] < E) lg[sel[j]] = sl[j];
        if (sub == 0 && tl < blk_valid) {
          out_idx[(blk_tok0 + tl) * k + j] = sel[j];
          out_w[(blk_tok0 + tl) * k + j] = vals[j] / total;
        }
      }
    }
    for (int e = sub; e < E; e += 4) lg[e] = expf(lg[e] - m) / sum;  // probabilities, in place
  }
  __syncthreads();
  // per-block probability sums, tokens in order
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    float s = 0.f;
    for (int tl = 0; tl < blk_valid; ++tl) s += s_logits[tl * ld + e];
    psum_part[(size_t)blockIdx.x * E + e] = s;
  }
}

template <int NT, bool NORM, bool STAGE>
int launch_mma_variant(const void* x, const void* Wg, const void* bg, int64_t N, int d, int E, int k,
                       float* out_logits, int32_t* out_idx, float* out_w, float* psum_part,
                       const float* norm_c, float eps, float* stats, cudaStream_t s) {
  const int64_t blocks = (N + kRouterTokensPerBlock - 1) / kRouterTokensPerBlock;
  const size_t smem = sizeof(float) * ((size_t)kRouterTokensPerBlock * (E + 1) + (size_t)kWarps * E +
                                       (size_t)kWarps * 32 * (NT * 4 + 4)) +
                      (STAGE ? 16 + (size_t)4 * (2 * 8 * NT * 4 + 2 * kRouterTokensPerBlock * 4) * 16 : 0);
  static PerDeviceOnce once;
  if (smem > 48 * 1024) {
    int rc = ensure_dynamic_smem(once, router_mma_kernel<NT, NORM, STAGE>, 160 * 1024);
    if (rc) return rc;
  }
  router_mma_kernel<NT, NORM, STAGE><<<(unsigned)blocks, kMmaWarps * 32, smem, s>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(Wg),
      static_cast<const __nv_bfloat16*>(bg), N, d, E, k, out_logits, out_idx, out_w, psum_part,
      norm_c, eps, stats);
  MOE_CUDA_CHECK(cudaGetLastError());
  return 0;
}

template <int NT, bool NORM>
int launch_mma(const void* x, const void* Wg, const void* bg, int64_t N, int d, int E, int k,
               float* out_logits, int32_t* out_idx, float* out_w, float* psum_part,
               const float* norm_c, float eps, float* stats, cudaStream_t s) {
  // more than 16 experts: x and Wg staged through shared memory (also the faster of the two for
  // grids of less than one wave: 34 us against 43 us for 8192 tokens and 64 experts)
  return launch_mma_variant<NT, NORM, (NT >= 4)>(x, Wg, bg, N, d, E, k, out_logits, out_idx, out_w,
                                                  psum_part, norm_c, eps, stats, s);
}

template <bool NORM>
int launch_mma_nt(const void* x, const void* Wg, const void* bg, int64_t N, int d, int E, int k,
                  float* out_logits, int32_t* out_idx, float* out_w, float* psum_part,
                  const float* norm_c, float eps, float* stats, cudaStream_t s) {
  if (E <= 8) return launch_mma<1, NORM>(x, Wg, bg, N, d, E, k, out_logits, out_idx, out_w, psum_part, norm_c, eps, stats, s);
  if (E <= 16) return launch_mma<2, NORM>(x, Wg, bg, N, d, E, k, out_logits, out_idx, out_w, psum_part, norm_c, eps, stats, s);
  if (E <= 32) return launch_mma<4, NORM>(x, Wg, bg, N, d, E, k, out_logits, out_idx, out_w, psum_part, norm_c, eps, stats, s);
  return launch_mma<8, NORM>(x, Wg, bg, N, d, E, k, out_logits, out_idx, out_w, psum_part, norm_c, eps, stats, s);
}

}  // namespace

// norm_c == nullptr: logits = x Wg^T + bg. Otherwise Wg is the folded weight of norm.cu,
// norm_c its [2E] constants, and (mean, rstd) of every row is written to stats [N][2].
int launch_router(const void* x, const void* Wg, const void* bg, int64_t N, int d, int E, int k,
                  int dtype, float* out_logits, int32_t* out_idx, float* out_w, float* psum_part,
                  int32_t* status, cudaStream_t s, const float* norm_c, float eps, float* stats) {
  if (N == 0) return 0;
  // 17 to 64 experts without a folded LayerNorm: the tcgen05 kernel, whose epilogue has a token's
  // logits in one thread's registers (at that width router_mma_kernel spends its time in the
  // softmax/top-k of its four lanes per token, not in the product)
  if (dtype == MOE_B200_BF16 && norm_c == nullptr && status != nullptr && router_tc_supported(N, d, E, k))
    return launch_router_tc(x, Wg, bg, N, d, E, k, out_logits, out_idx, out_w, psum_part, status, s);
  const int64_t blocks = (N + kRouterTokensPerBlock - 1) / kRouterTokensPerBlock;
  const size_t smem = sizeof(float) * (size_t)(kRouterTokensPerBlock + kWarps) * E;
  if (dtype == MOE_B200_BF16) {
    if (norm_c != nullptr)
      return launch_mma_nt<true>(x, Wg, bg, N, d, E, k, out_logits, out_idx, out_w, psum_part, norm_c, eps, stats, s);
    return launch_mma_nt<false>(x, Wg, bg, N, d, E, k, out_logits, out_idx, out_w, psum_part, nullptr, 0.f, nullptr, s);
  }
  router_kernel<float><<<(unsigned)blocks, kWarps * 32, smem, s>>>(
      static_cast<const float*>(x), static_cast<const float*>(Wg), static_cast<const float*>(bg),
      N, d, E, k, out_logits, out_idx, out_w, psum_part, norm_c, eps, stats);
  MOE_CUDA_CHECK(cudaGetLastError());
  return 0;
}

}  // namespace moe
