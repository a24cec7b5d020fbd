// Router and dispatch of a small call in ONE launch: with at most a few hundred
// tokens the separate router and cooperative dispatch kernels are pure launch
// and barrier latency (13 + 19 us against a few us of work). A few blocks run;
// each one derives the complete routing by itself (the same instructions on the
// same data, so every block gets the same answer and no grid barrier is needed),
// block 0 writes the routing results, and the row copies are split over the blocks.
// Covers reference model.py:206-253 for N <= 512, N*k <= 1024, E <= 32, bf16:
//   A. logits: 32 warps = (16-token group) x (slice of K); each warp forms its
//      partial x Wg^T with mma.sync m16n8k16 exactly like router_mma_kernel
//      (router.cu), all its loads in flight at once; partials are summed over
//      the K slices in slice order, plus bias;
//   B. 8, 16 or 32 lanes per token, lane e = expert e: fp32 softmax, k passes of
//      arg-max ordered by (logit desc, index asc) with shuffle reductions
//      on order-preserving keys, renormalise;
//   C. warp 0: per-slot counts, offsets (scan over E), stable ranks in (token,
//      slot) order; then row copies into the sorted buffer with 16-byte accesses
//      (their loads were issued before B);
//   E. block 0, after its copies: probabilities summed per expert in token order; loss.
#pragma once
#include "common.cuh"

namespace moe {

constexpr int kFrontThreads = 1024;
constexpr int kFrontMaxTok = 512;
constexpr int kFrontMaxE = 32;
constexpr int kFrontMaxPairs = 1024;

namespace front_detail {

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ int ld_acquire_gpu_i32(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

}  // namespace front_detail

using front_detail::mma_bf16_16816;
using front_detail::ld_acquire_gpu_i32;

// SPLIT = false: every block derives the complete routing (fastest up to about a hundred tokens).
// SPLIT = true: block b routes tokens 16b .. 16b+15 only; the blocks then exchange their per-slot
//   expert counts and probability sums through `xch` and meet at a counter (all blocks of the grid
//   are resident: there are at most 32 of them; the wait is bounded and reports a time-out in
//   `status`), and each block places and copies its own rows. Same results as the other form
//   except for the order in which the logits' partial sums are added.
//
// A device function so that a kernel which goes on to use the routing (experts_tiny.cu) can run
// it in its own blocks: `blk` of `nblk` is the calling block's place among the blocks that run
// it, `smem` front_small_smem_bytes() of shared memory. On return (after a block barrier) the
// block's shared memory holds the routing: see FrontSmallView.
struct FrontSmallView {
  const int* idx;      // [N*k] expert of (token, slot)
  const int* row;      // [N*k] row of (token, slot) in the expert-sorted order
  const int* off;      // [E+1] first row of every expert
  const float* wgt;    // [N*k] renormalised routing weight of (token, slot)
};

__host__ __device__ inline size_t front_small_smem_bytes(int NT, int ntok, int E, int k) {
  return sizeof(float) * ((size_t)32 * 16 * 8 * NT + (size_t)ntok * (E + 1)) +
         sizeof(int) * (2 * (size_t)ntok * k + 2 * kMaxTopK * kFrontMaxE + 4 * kFrontMaxE + 1) +
         sizeof(float) * (size_t)ntok * k;
}

template <int NT, bool SPLIT>  // n-tiles of 8 experts: E <= 8*NT
__device__ __forceinline__ FrontSmallView
front_small_body(float* smem, const int blk, const int nblk,
                 const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ Wg,
                 const __nv_bfloat16* __restrict__ bg, int Ntotal, int d, int E, int k,
                 float* __restrict__ out_logits, int32_t* __restrict__ out_idx,
                 float* __restrict__ out_w, int32_t* __restrict__ cnt_slot,
                 int32_t* __restrict__ offsets, int32_t* __restrict__ row_of,
                 __nv_bfloat16* __restrict__ perm, float* __restrict__ psum,
                 float* __restrict__ aux, int* __restrict__ xch, int* __restrict__ counter,
                 int32_t* __restrict__ status) {
  constexpr int kThreads = kFrontThreads;
  constexpr int kMaxE = kFrontMaxE;
  const int ld = E + 1;
  // SPLIT: this block's 16 tokens are "the problem" for the phases A and B below
  const int tok_base = SPLIT ? 16 * blk : 0;
  const int N = SPLIT ? min(16, Ntotal - tok_base) : Ntotal;
  const bool writer = SPLIT || blk == 0;     // this block writes the per-token results
  if (SPLIT) {
    x += (size_t)tok_base * d;
    if (out_logits != nullptr) out_logits += (size_t)tok_base * E;
    out_idx += (size_t)tok_base * k;
    out_w += (size_t)tok_base * k;
    row_of += (size_t)tok_base * k;
  }
  const int ngroups = (N + 15) >> 4;                       // 16-token groups
  int gp2 = 1;
  while (gp2 < ngroups) gp2 <<= 1;                         // 1, 2, 4 or 8
  const int nslices = 32 / gp2;                            // K slices
  float* s_part = smem;                                    // [nslices][16*gp2][8*NT]
  float* s_logit = s_part + (size_t)nslices * 16 * gp2 * 8 * NT;   // [N][E+1]
  int* s_idx = reinterpret_cast<int*>(s_logit + (size_t)N * ld);   // [N*k]
  int* s_row = s_idx + N * k;                              // [N*k]
  int* s_cnt = s_row + N * k;                              // [kMaxTopK][kMaxE]
  int* s_off = s_cnt + kMaxTopK * kMaxE;                   // [kMaxE+1]
  int* s_run = s_off + kMaxE + 1;                          // [kMaxE]
  float* s_bias = reinterpret_cast<float*>(s_run + kMaxE); // [kMaxE], then s_base, s_tot (SPLIT)
  float* s_wgt = s_bias + 2 * kMaxE + kMaxTopK * kMaxE;    // [N*k]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  constexpr int ET_C = 8 * NT;
  const int ET = ET_C;
  if (tid < E) s_bias[tid] = __bfloat162float(bg[tid]);   // visible after the barrier behind part A

  // ---- A. partial logits -----------------------------------------------------
  {
    const int tg = warp % gp2, ks = warp / gp2;
    if (tg < ngroups) {
      const int tok0 = tg * 16;
      const int row_pieces = d >> 3;
      const int ra = min(tok0 + g, N - 1), rb = min(tok0 + g + 8, N - 1);
      const uint4* xa = reinterpret_cast<const uint4*>(x + (size_t)ra * d);
      const uint4* xb = reinterpret_cast<const uint4*>(x + (size_t)rb * d);
      const uint4* w4 = reinterpret_cast<const uint4*>(Wg);
      const int nchunk = (d + 31) >> 5;
      const uint4 zero = make_uint4(0, 0, 0, 0);
      float acc[NT][4];
#pragma unroll
      for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
      for (int c0 = ks; c0 < nchunk; c0 += nslices * 4) {
        uint4 A[4], B[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int c = c0 + u * nslices;
          const int piece = 4 * c + t;
          const bool ok = c < nchunk && piece < row_pieces;
          // x may be the output of the kernel before this one: through L2, not the read-only path
          A[u] = ok ? __ldcg(xa + piece) : zero;
          B[u] = ok ? __ldcg(xb + piece) : zero;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int c = c0 + u * nslices;
          const int piece = 4 * c + t;
#pragma unroll
          for (int j = 0; j < NT; ++j) {
            const int row = 8 * j + g;
            const uint4 w = (row < E && c < nchunk && piece < row_pieces)
                                ? __ldg(w4 + (size_t)row * row_pieces + piece) : zero;
            mma_bf16_16816(acc[j], A[u].x, B[u].x, A[u].y, B[u].y, w.x, w.y);
            mma_bf16_16816(acc[j], A[u].z, B[u].z, A[u].w, B[u].w, w.z, w.w);
          }
        }
      }
      float* pp = s_part + ((size_t)ks * 16 * gp2 + tok0) * ET;
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const int e = 8 * j + 2 * t;
        pp[g * ET + e] = acc[j][0];
        pp[g * ET + e + 1] = acc[j][1];
        pp[(g + 8) * ET + e] = acc[j][2];
        pp[(g + 8) * ET + e + 1] = acc[j][3];
      }
    }
  }
  for (int i = tid; i < kMaxTopK * kMaxE; i += kThreads) s_cnt[i] = 0;
  __syncthreads();
  // the first batch of row copies: the loads do not depend on the routing, so they are
  // issued now and wait in registers until the destination rows are known
  const int pieces = d >> 3;
  const int items = N * pieces;
  const uint4* src = reinterpret_cast<const uint4*>(x);
  constexpr int kInFlight = 4;
  const int first_item = (SPLIT ? 0 : blk * kThreads * kInFlight) + tid;
  const int item_stride = (SPLIT ? 1 : nblk) * kThreads * kInFlight;
  uint4 pre[kInFlight];
#pragma unroll
  for (int u = 0; u < kInFlight; ++u) {
    const int i = first_item + u * kThreads;
    if (i < items)
      asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
                   : "=r"(pre[u].x), "=r"(pre[u].y), "=r"(pre[u].z), "=r"(pre[u].w)
                   : "l"(src + i)
                   : "memory");
  }
  for (int i = tid; i < N * E; i += kThreads) {
    const int tok = i / E, e = i - tok * E;
    float s = 0.f;
    for (int ks = 0; ks < nslices; ++ks) s += s_part[((size_t)ks * 16 * gp2 + tok) * ET + e];
    s += s_bias[e];
    s_logit[tok * ld + e] = s;
    if (out_logits != nullptr && writer) out_logits[i] = s;
  }
  __syncthreads();

  // ---- B. softmax, top-k, renormalise: a group of ET lanes per token, lane e = expert e ----
  {
    constexpr int G = ET_C;                 // 8, 16 or 32 lanes
    constexpr int kTokPerWarp = 32 / G;
    const int grp = lane / G, e = lane % G;
    const unsigned gmask = G == 32 ? 0xffffffffu : (((1u << G) - 1u) << (grp * G));
    for (int tok0 = warp * kTokPerWarp; tok0 < N; tok0 += (kThreads / 32) * kTokPerWarp) {
      const int tok = tok0 + grp;
      const bool live = tok < N && e < E;
      float* lg = s_logit + (size_t)min(tok, N - 1) * ld;
      const float v = live ? lg[e] + 0.f : -INFINITY;      // + 0: no negative zero
      // order-preserving map float -> unsigned: the maximum and its first position by integer compares
      const unsigned u = __float_as_uint(v);
      unsigned key = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
      unsigned kmax = key;
#pragma unroll
      for (int o = G / 2; o > 0; o >>= 1) kmax = max(kmax, __shfl_xor_sync(gmask, kmax, o));
      const float m = __uint_as_float((kmax & 0x80000000u) ? (kmax & 0x7fffffffu) : ~kmax);
      const float p = live ? expf(v - m) : 0.f;
      float sum = p;
#pragma unroll
      for (int o = G / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(gmask, sum, o);
      const float inv_sum = __frcp_rn(sum);  // one reciprocal per token, products below: a division
                                             // is a long subroutine, and this code runs once, cold
      if (live) lg[e] = p * inv_sum;        // probabilities, for the loss below
      // k passes of arg-max ordered by (logit descending, index ascending); lane j of the group
      // keeps slot j's result. The loop is kept rolled: this code runs once per launch, from a cold
      // instruction cache, and every extra line of it costs a miss on the path to the next kernel.
      int my_sel = 0;
      float my_val = 0.f;
      float total = 0.f;
#pragma unroll 1
      for (int j = 0; j < k; ++j) {
        unsigned km = key;
#pragma unroll
        for (int o = G / 2; o > 0; o >>= 1) km = max(km, __shfl_xor_sync(gmask, km, o));
        const unsigned hit = __ballot_sync(gmask, key == km) & gmask;
        const int winner = __ffs(hit) - 1;
        const float bv = __uint_as_float((km & 0x80000000u) ? (km & 0x7fffffffu) : ~km);
        const float val = expf(bv - m) * inv_sum;
        total += val;
        if (e == j) { my_sel = winner - grp * G; my_val = val; }
        if (lane == winner) key = 0u;     // below every real key
      }
      if (e < k && tok < N) {
        if (writer) {
          out_idx[tok * k + e] = my_sel;
          out_w[tok * k + e] = my_val * __frcp_rn(total);
        }
        s_idx[tok * k + e] = my_sel;
        s_wgt[tok * k + e] = my_val * __frcp_rn(total);
        atomicAdd(&s_cnt[e * kMaxE + my_sel], 1);
      }
    }
  }
  __syncthreads();

  // ---- C. counts, offsets, ranks: warp 0 -------------------------------------------
  int* s_base = reinterpret_cast<int*>(s_bias + kMaxE);    // [kMaxE] SPLIT: rows of earlier blocks
  int* s_tot = s_base + kMaxE;                             // [kMaxTopK][kMaxE] SPLIT: grid totals
  if constexpr (SPLIT) {
    const int nb = nblk, b = blk;
    float* xps = reinterpret_cast<float*>(xch + nb * k * E);    // [nb][E] probability sums
    if (tid < k * E) xch[b * k * E + tid] = s_cnt[(tid / E) * kMaxE + tid % E];
    if (tid < E) {
      float ps = 0.f;
      for (int tok = 0; tok < N; ++tok) ps += s_logit[tok * ld + tid];
      xps[b * E + tid] = ps;
    }
    for (int i = tid; i < kMaxE + kMaxTopK * kMaxE; i += kThreads) s_base[i] = 0;   // s_base, s_tot
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      atomicAdd(counter, 1);
      unsigned long long t0 = 0;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
      for (uint32_t it = 0; ld_acquire_gpu_i32(counter) < nb; ++it) {
        if ((it & 63u) == 63u) {
          unsigned long long t1;
          asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
          if (t1 - t0 > 2000000000ull) {     // 2 s: some block of the grid never arrived
            atomicMax(&status[0], MOE_B200_DEV_TIMEOUT);
            status[1] = 41;
            status[2] = b;
            break;
          }
        }
      }
    }
    __syncthreads();
    // totals per (slot, expert) and the rows that earlier blocks put in front of this block's
    for (int i = tid; i < nb * k * E; i += kThreads) {
      const int c = __ldcg(&xch[i]);
      const int bb = i / (k * E), je = i - bb * (k * E);
      const int j = je / E, e = je - j * E;
      if (c != 0) {
        atomicAdd(&s_tot[j * kMaxE + e], c);
        if (bb < b) atomicAdd(&s_base[e], c);
      }
    }
    __syncthreads();
  }
  if (warp == 0) {
    int tot = 0;
    if (lane < E) {
      for (int j = 0; j < k; ++j) {
        const int c = SPLIT ? s_tot[j * kMaxE + lane] : s_cnt[j * kMaxE + lane];
        if (blk == 0) cnt_slot[j * E + lane] = c;
        tot += c;
      }
    }
    int incl = tot;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    if (lane < E) {
      s_off[lane] = incl - tot + (SPLIT ? s_base[lane] : 0);   // first row of this block's tokens
      s_run[lane] = 0;
      if (blk == 0) offsets[lane] = incl - tot;
    }
    if (lane == 31) {
      s_off[E] = incl;
      if (blk == 0) offsets[E] = incl;
    }
    __syncwarp();
    const int npair = N * k;
    for (int p0 = 0; p0 < npair; p0 += 32) {
      const int p = p0 + lane;
      const int e = p < npair ? s_idx[p] : -1;
      const bool ok = e >= 0;
      const unsigned grp = __match_any_sync(0xffffffffu, ok ? e : -1 - lane);
      int row = -1;
      if (ok) row = s_off[e] + s_run[e] + __popc(grp & ((1u << lane) - 1u));
      __syncwarp();
      if (ok && (grp >> lane) == 1u) s_run[e] += __popc(grp);
      __syncwarp();
      if (p < npair) {
        s_row[p] = row;
        if (writer) row_of[p] = row;
      }
    }
  }
  __syncthreads();

  // ---- D. copy the token rows into the sorted buffer (split over the blocks) -----
  for (int i0 = first_item; i0 < items; i0 += item_stride) {
    uint4 v[kInFlight];
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      const int i = i0 + u * kThreads;
      if (i0 == first_item) v[u] = pre[u];
      else if (i < items) v[u] = __ldcg(src + i);
    }
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      const int i = i0 + u * kThreads;
      if (i < items) {
        const int tok = i / pieces, pc = i - tok * pieces;
        for (int j = 0; j < k; ++j)
          reinterpret_cast<uint4*>(perm + (size_t)s_row[tok * k + j] * d)[pc] = v[u];
      }
    }
  }

  // ---- E. the loss, off the path of the kernels that wait for the rows (model.py:213-216) ----
  if (blk == 0) {
    __syncthreads();       // the partial-logit area is free again: every thread is past the reduction
    if constexpr (SPLIT) {
      // the blocks' probability sums, added in block order
      const int nb = nblk;
      const float* xps = reinterpret_cast<const float*>(xch + nb * k * E);
      if (tid < E) {
        float ps = 0.f;
        for (int bb = 0; bb < nb; ++bb) ps += __ldcg(&xps[bb * E + tid]);
        psum[tid] = ps;
        s_part[1024 + tid] = (ps / (float)Ntotal) * ((float)s_tot[tid] / (float)Ntotal);
      }
    } else {
      // probabilities summed per expert: warp w takes tokens w, w + 32, ...; the 32 partial sums
      // of an expert are then added in warp order
      if (lane < E) {
        float ps = 0.f;
        for (int tok = warp; tok < N; tok += kThreads / 32) ps += s_logit[tok * ld + lane];
        s_part[warp * 32 + lane] = ps;
      }
      __syncthreads();
      if (tid < E) {
        float ps = 0.f;
        for (int w = 0; w < kThreads / 32; ++w) ps += s_part[w * 32 + tid];
        psum[tid] = ps;
        s_part[1024 + tid] = (ps / (float)N) * ((float)s_cnt[tid] / (float)N);
      }
    }
    __syncthreads();
    if (tid == 0) {
      float a = 0.f;
      for (int e = 0; e < E; ++e) a += s_part[1024 + e];
      aux[0] = a / (float)E * (float)(E * E);
    }
  }
  if constexpr (SPLIT) {
    // the last block to leave puts the meeting counter back to zero for the next call
    __syncthreads();
    if (tid == 0 && atomicAdd(counter, 1) == 2 * nblk - 1) *counter = 0;
  }
  __syncthreads();
  return FrontSmallView{s_idx, s_row, s_off, s_wgt};
}

}  // namespace moe
