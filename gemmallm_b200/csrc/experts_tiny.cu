// The whole block for a handful of tokens (decode with one to eight tokens) in ONE
// cooperative launch: routing, GEGLU product, down product, weighted sum and residual
// (reference model.py:206-276 and the caller's model.py:319).
//
// With one or two rows per expert the call is a stream of the hit experts' weights (50 MB for
// one token at d=1024, f=4096, k=2: under 8 us at the HBM rate) and everything else is
// latency: four dependent launches cost more than the stream itself. Here one grid of one
// block per SM does it all:
//   0. every block derives the routing by itself (front_small_body: same instructions on the
//      same data in every block, so no exchange is needed); block 0 writes the routing results;
//   1. every block requests its share of the down weights into shared memory (one bulk copy
//      per weight row, completing on an mbarrier): the block owns d/gridDim output columns of
//      EVERY hit expert, and these bytes do not depend on the hidden activations, so they
//      stream while step 2 runs;
//   2. GEGLU product: tiles of 8 features (8 gate rows and 8 up rows of W1 form the 16-row A
//      operand of mma.sync m16n8k16, so a lane's accumulators hold a feature's gate and up sums
//      side by side), the expert's rows (at most 8) are the B operand, four warps split d;
//      tiles are spread evenly over the grid; h goes to global memory (it stays in L2);
//   3. one grid barrier;
//   4. down product from the weights waiting in shared memory (those that did not fit come
//      from global memory), 32 warps split f; the k experts of a token meet in the same block
//      because a block owns its columns for all experts, so the block adds the down bias,
//      rounds to bf16, weights, sums in slot order, adds the residual and writes the output:
//      no partial sums in global memory and no combine kernel.
#include <cooperative_groups.h>
#include "front_small.cuh"
#include "tc_ptx.cuh"

namespace cg = cooperative_groups;

namespace moe {

namespace {

constexpr int kThreads = kFrontThreads;     // 1024: the routing body wants 32 warps
constexpr int kWarps = kThreads / 32;
constexpr int kTinyMaxTok = 8;              // rows of one expert fit one 8-column n-tile
constexpr int kSplitB = 4;                  // warps that share one GEGLU tile (split d)
constexpr int kTilesPerIter = kWarps / kSplitB;
constexpr int kMaxPairs = kTinyMaxTok * kMaxTopK;

// bytes between two weight rows in shared memory: rows g and g + 1 of a quarter-warp's 16-byte
// reads must fall into different halves of the 128-byte bank window
__host__ __device__ inline int w2_pitch_bytes(int f) {
  const int row = f * 2;
  return row + ((64 - (row & 127)) + 128) % 128;
}

template <int NT>
__global__ void __launch_bounds__(kThreads, 1)
decode_tiny_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ Wg,
                   const __nv_bfloat16* __restrict__ bg, int N, int d, int f, int E, int k,
                   const void* const* __restrict__ W1, const void* const* __restrict__ b1,
                   const void* const* __restrict__ W2, const void* const* __restrict__ b2,
                   const __nv_bfloat16* __restrict__ residual, float* __restrict__ out_logits,
                   int32_t* __restrict__ out_idx, float* __restrict__ out_w,
                   int32_t* __restrict__ cnt_slot, int32_t* __restrict__ offsets,
                   int32_t* __restrict__ row_of, __nv_bfloat16* __restrict__ perm,
                   float* __restrict__ psum, float* __restrict__ aux,
                   __nv_bfloat16* __restrict__ h, __nv_bfloat16* __restrict__ out,
                   int32_t* __restrict__ status, int front_bytes, int w2_bytes) {
  cg::grid_group grid = cg::this_grid();
  extern __shared__ float smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int G = (int)gridDim.x, b = (int)blockIdx.x;
  // the experts' parameter pointers do not depend on the routing: fetched first, so that their
  // latency hides behind it
  const void** s_ptr = reinterpret_cast<const void**>(reinterpret_cast<char*>(smem) + front_bytes);
  const void* my_ptr = nullptr;      // requested now, stored after the routing
  if (tid < 4 * E) {
    const int which = tid / E, e = tid - which * E;
    const void* const* tab = which == 0 ? W1 : which == 1 ? b1 : which == 2 ? W2 : b2;
    my_ptr = tab[e];
  }
  uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_ptr + 4 * kFrontMaxE);   // the down weights' arrival
  int* s_abort = reinterpret_cast<int*>(s_bar + 1);
  if (tid == 0) {
    tc::mbar_init(s_bar, 1);
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_wait();                 // x may come from the kernel before this one
  pdl_launch_dependents();
  // ---- 0. routing ------------------------------------------------------------------
  const FrontSmallView rt = front_small_body<NT, false>(
      smem, b, G, x, Wg, bg, N, d, E, k, out_logits, out_idx, out_w, cnt_slot, offsets, row_of, perm,
      psum, aux, nullptr, nullptr, nullptr);
  if (tid < 4 * E) s_ptr[(tid / E) * kFrontMaxE + tid % E] = my_ptr;
  char* extra = reinterpret_cast<char*>(s_bar + 2);                // 16-byte aligned by the launcher
  int* s_hit = reinterpret_cast<int*>(extra);                      // [32] experts with rows
  int* s_tok = s_hit + 32;                                         // [kMaxPairs] token of a sorted row
  int* s_nhit = s_tok + kMaxPairs;                                 // [4]
  float* s_y = reinterpret_cast<float*>(s_nhit + 4);               // [kMaxPairs][8] down outputs
  float* s_red = s_y + kMaxPairs * 8;                              // [kWarps][32][4] partial sums
  char* s_w2 = reinterpret_cast<char*>(s_red + kWarps * 32 * 4);   // down weights waiting for h

  // this block's columns of the down weights
  const int c_lo = (int)((int64_t)d * b / G), c_hi = (int)((int64_t)d * (b + 1) / G);
  const int pieces_f = f >> 3;
  const int pitch = w2_pitch_bytes(f);
  const int ncol0 = min(8, c_hi - c_lo);
  const int M = N * k;
  for (int p = tid; p < M; p += kThreads) {
    const int r = rt.row[p];
    if (r >= 0 && r < kMaxPairs) s_tok[r] = p / k;
  }
  __syncthreads();
  if (warp == 0) {
    const bool hit = lane < E && rt.off[lane + 1] > rt.off[lane];
    const unsigned mask = __ballot_sync(0xffffffffu, hit);
    if (hit) s_hit[__popc(mask & ((1u << lane) - 1u))] = lane;
    const int nh = __popc(mask);
    if (lane == 0) s_nhit[0] = nh;
    __syncwarp();
    // ---- 1. the first group of (up to) 8 columns of as many hit experts as fit, one bulk copy
    // per weight row, on their way to shared memory ----
    const int np = ncol0 > 0 ? min(nh, w2_bytes / (8 * pitch)) : 0;
    if (np > 0) {
      if (lane == 0) tc::mbar_expect_tx(s_bar, (uint32_t)(np * ncol0) * (uint32_t)(f * 2));
      __syncwarp();
      for (int r = lane; r < np * ncol0; r += 32) {
        const int hi = r / ncol0, j = r - hi * ncol0;
        const __nv_bfloat16* W = static_cast<const __nv_bfloat16*>(s_ptr[2 * kFrontMaxE + s_hit[hi]]);
        asm volatile(
            "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
            ::"r"(tc::smem_u32(s_w2 + (size_t)(hi * 8 + j) * pitch)),
              "l"(W + (size_t)(c_lo + j) * f), "r"((uint32_t)(f * 2)), "r"(tc::smem_u32(s_bar))
            : "memory");
      }
    }
  }
  __syncthreads();
  const int nhit = s_nhit[0];
  int n_pref = ncol0 > 0 ? min(nhit, w2_bytes / (8 * pitch)) : 0;
  // ---- 2. GEGLU product ------------------------------------------------------------
  {
    const int tiles_e = (f + 7) >> 3;
    const int64_t total = (int64_t)nhit * tiles_e;
    const int T0 = (int)(total * b / G), T1 = (int)(total * (b + 1) / G);
    const int pieces_d = d >> 3;
    // this warp's share of d: whole groups of 16 pieces
    const int groups = (pieces_d + 15) >> 4;
    const int per = (groups + kSplitB - 1) / kSplitB * 16;
    const int ts = warp / kSplitB, ks = warp % kSplitB;
    const int pb = min(pieces_d, ks * per), pe = min(pieces_d, (ks + 1) * per);
    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (int base = T0; base < T1; base += kTilesPerIter) {
      const int tile = base + ts;
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      // the biases of the (tile, feature) this thread finishes below: requested with the weights
      float bias_g = 0.f, bias_u = 0.f;
      if (tid < kTilesPerIter * 64 && base + (tid >> 6) < T1) {
        const int tl = base + (tid >> 6);
        const int hi = tl / tiles_e, feat = ((tl - hi * tiles_e) << 3) + ((tid >> 3) & 7);
        if (feat < f) {
          const __nv_bfloat16* bias = static_cast<const __nv_bfloat16*>(s_ptr[kFrontMaxE + s_hit[hi]]);
          bias_g = __bfloat162float(bias[feat]);
          bias_u = __bfloat162float(bias[f + feat]);
        }
      }
      if (tile < T1) {
        const int hi = tile / tiles_e, j0 = (tile - hi * tiles_e) << 3;
        const int e = s_hit[hi];
        const int row0 = rt.off[e], rows = rt.off[e + 1] - row0;
        const __nv_bfloat16* W = static_cast<const __nv_bfloat16*>(s_ptr[e]);
        const int ja = min(j0 + g, f - 1);                      // clamped: masked at the store
        const uint4* wa = reinterpret_cast<const uint4*>(W + (size_t)ja * d);        // gate row
        const uint4* wb = reinterpret_cast<const uint4*>(W + (size_t)(f + ja) * d);  // up row
        const uint4* xr = g < rows ? reinterpret_cast<const uint4*>(x + (size_t)s_tok[row0 + g] * d)
                                   : nullptr;
        for (int p0 = pb; p0 < pe; p0 += 16) {
          uint4 A[2][4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int piece = p0 + 4 * u + t;
            const bool ok = piece < pe;
            A[0][u] = ok ? __ldg(wa + piece) : zero;
            A[1][u] = ok ? __ldg(wb + piece) : zero;
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int piece = p0 + 4 * u + t;
            const uint4 B = (xr != nullptr && piece < pe) ? xr[piece] : zero;
            mma_bf16_16816(acc, A[0][u].x, A[1][u].x, A[0][u].y, A[1][u].y, B.x, B.y);
            mma_bf16_16816(acc, A[0][u].z, A[1][u].z, A[0][u].w, A[1][u].w, B.z, B.w);
          }
        }
      }
      float* mine = s_red + ((size_t)warp * 32 + lane) * 4;
      mine[0] = acc[0]; mine[1] = acc[1]; mine[2] = acc[2]; mine[3] = acc[3];
      __syncthreads();
      // accumulators: c0,c1 -> gate sums of feature g for rows 2t, 2t+1; c2,c3 -> its up sums
      if (tid < kTilesPerIter * 64) {
        const int its = tid >> 6, ln = (tid >> 1) & 31, h2 = tid & 1;
        const int tl = base + its;
        if (tl < T1) {
          const int hi = tl / tiles_e, feat = ((tl - hi * tiles_e) << 3) + (ln >> 2);
          const int e = s_hit[hi];
          const int row0 = rt.off[e], rows = rt.off[e + 1] - row0;
          const int r = 2 * (ln & 3) + h2;
          if (feat < f && r < rows) {
            float gs = 0.f, us = 0.f;
#pragma unroll
            for (int q = 0; q < kSplitB; ++q) {
              const float* pp = s_red + ((size_t)(its * kSplitB + q) * 32 + ln) * 4;
              gs += pp[h2];
              us += pp[2 + h2];
            }
            const float gv = gs + bias_g;
            const float uv = us + bias_u;
            h[(size_t)(row0 + r) * f + feat] = __float2bfloat16_rn(gelu_tanh_fast(gv) * uv);
          }
        }
      }
      __syncthreads();
    }
  }

  // the down bias and the residual of this thread's output of the first column group: requested
  // before the barrier
  float pre_b2 = 0.f, pre_res = 0.f;
  if (tid < nhit * 64) {
    const int col = 2 * ((tid >> 1) & 3) + (tid & 1);
    if (col < ncol0)
      pre_b2 = __bfloat162float(
          static_cast<const __nv_bfloat16*>(s_ptr[3 * kFrontMaxE + s_hit[tid >> 6]])[c_lo + col]);
  }
  if (residual != nullptr && tid < N * 8 && (tid & 7) < ncol0)
    pre_res = __bfloat162float(residual[(size_t)(tid >> 3) * d + c_lo + (tid & 7)]);
  // ---- 3. every block's h is complete ------------------------------------------------
  __threadfence();
  grid.sync();
  if (n_pref > 0) {
    // every thread observes the arrival itself (the copies were written by the async proxy)
    const bool ok = tc::mbar_wait(s_bar, 0, s_abort, status, 61);
    if (!__syncthreads_and(ok)) n_pref = 0;     // reported in status; the weights come from global memory
  }

  // ---- 4. down product, weighted sum, residual ---------------------------------------
  {
    // the 32 warps are dealt to the hit experts: wpe warps per expert split f
    const int wpe = kWarps / nhit > 0 ? kWarps / nhit : 1;     // nhit <= 32
    const int hi = warp / wpe, ks = warp - hi * wpe;
    const bool live = hi < nhit;
    const int groups = (pieces_f + 15) >> 4;
    const int per = (groups + wpe - 1) / wpe * 16;
    const int pb = min(pieces_f, ks * per), pe = min(pieces_f, (ks + 1) * per);
    const uint4 zero = make_uint4(0, 0, 0, 0);
    const int e = live ? s_hit[hi] : 0;
    const int row0 = rt.off[e], rows = live ? rt.off[e + 1] - row0 : 0;
    const uint4* hr = g < rows ? reinterpret_cast<const uint4*>(h + (size_t)(row0 + g) * f) : nullptr;
    for (int c0 = c_lo; c0 < c_hi; c0 += 8) {
      const int ncol = min(8, c_hi - c0);
      const bool staged = c0 == c_lo && hi < n_pref;
      const uint4* wg = (live && g < ncol)
                            ? reinterpret_cast<const uint4*>(
                                  static_cast<const __nv_bfloat16*>(s_ptr[2 * kFrontMaxE + e]) + (size_t)(c0 + g) * f)
                            : nullptr;
      const uint4* ws = reinterpret_cast<const uint4*>(s_w2 + (size_t)(hi * 8 + g) * pitch);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      if (staged) {
        // weights from shared memory: all of h's pieces for 32 pieces of f requested at once
        for (int p0 = pb; p0 < pe; p0 += 32) {
          uint4 A[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int piece = p0 + 4 * u + t;
            A[u] = (piece < pe && hr != nullptr) ? __ldcg(hr + piece) : zero;   // written in this launch
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int piece = p0 + 4 * u + t;
            const uint4 B = (piece < pe && wg != nullptr) ? ws[piece] : zero;
            // rows 8..15 of the A tile are empty
            mma_bf16_16816(acc, A[u].x, 0u, A[u].y, 0u, B.x, B.y);
            mma_bf16_16816(acc, A[u].z, 0u, A[u].w, 0u, B.z, B.w);
          }
        }
      } else {
        for (int p0 = pb; p0 < pe; p0 += 16) {
          uint4 A[4], B[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int piece = p0 + 4 * u + t;
            const bool ok = piece < pe;
            A[u] = (ok && hr != nullptr) ? __ldcg(hr + piece) : zero;
            B[u] = (ok && wg != nullptr) ? __ldg(wg + piece) : zero;
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            mma_bf16_16816(acc, A[u].x, 0u, A[u].y, 0u, B[u].x, B[u].y);
            mma_bf16_16816(acc, A[u].z, 0u, A[u].w, 0u, B[u].z, B[u].w);
          }
        }
      }
      float* mine = s_red + ((size_t)warp * 32 + lane) * 4;
      mine[0] = acc[0]; mine[1] = acc[1];
      __syncthreads();
      // c0,c1 -> row g of the expert, columns 2t, 2t+1; one thread per (expert, row, column)
      for (int item = tid; item < nhit * 64; item += kThreads) {
        const int xh = item >> 6, ln = (item >> 1) & 31, h2 = item & 1;
        const int xe = s_hit[xh];
        const int xrow0 = rt.off[xe], xrows = rt.off[xe + 1] - xrow0;
        const int r = ln >> 2, col = 2 * (ln & 3) + h2;
        if (r < xrows && col < ncol) {
          float sum = 0.f;
          for (int w = 0; w < wpe; ++w) sum += s_red[((size_t)(xh * wpe + w) * 32 + ln) * 4 + h2];
          const float bias =
              (c0 == c_lo && item == tid)
                  ? pre_b2
                  : __bfloat162float(static_cast<const __nv_bfloat16*>(s_ptr[3 * kFrontMaxE + xe])[c0 + col]);
          // the expert's output is rounded to bf16 before weighting, as on the large-N path
          s_y[(xrow0 + r) * 8 + col] = __bfloat162float(__float2bfloat16_rn(sum + bias));
        }
      }
      __syncthreads();
      // out[token][c] = sum over the token's slots, in slot order, of w * y; then the residual
      if (tid < N * 8) {
        const int tok = tid >> 3, col = tid & 7;
        if (col < ncol) {
          float o = 0.f;
          for (int j = 0; j < k; ++j) {
            const int r = rt.row[tok * k + j];
            if (r < 0) continue;
            o = __fadd_rn(o, __fmul_rn(rt.wgt[tok * k + j], s_y[r * 8 + col]));
          }
          const size_t at = (size_t)tok * d + c0 + col;
          if (residual != nullptr)
            o = __fadd_rn(o, c0 == c_lo ? pre_res : __bfloat162float(residual[at]));
          out[at] = __float2bfloat16_rn(o);
        }
      }
      __syncthreads();
    }
  }
}

size_t tiny_extra_bytes() {
  return sizeof(void*) * 4 * kFrontMaxE + 16 + sizeof(int) * (32 + kMaxPairs + 4) +
         sizeof(float) * (kMaxPairs * 8 + kWarps * 32 * 4);
}

template <int NT>
int launch(const void* x, const void* Wg, const void* bg, int N, int d, int f, int E, int k,
           const PlanView& pv, const void* residual, float* logits, int32_t* idx, float* w,
           int32_t* cnt_slot, int32_t* offsets, int32_t* row_of, void* perm, float* psum, float* aux,
           void* h, void* out, int32_t* status, cudaStream_t s) {
  constexpr int kSmemMax = 200 * 1024;
  static PerDeviceOnce once;
  int rc = ensure_dynamic_smem(once, decode_tiny_kernel<NT>, kSmemMax);
  if (rc) return rc;
  int front_bytes = (int)((front_small_smem_bytes(NT, N, E, k) + 15) & ~(size_t)15);
  const int fixed = front_bytes + (int)tiny_extra_bytes();
  // room for the down weights: all hit experts (at most N*k of them) if they fit
  const int want = (N * k < E ? N * k : E) * 8 * w2_pitch_bytes(f);
  int w2_bytes = kSmemMax - fixed;
  if (w2_bytes > want) w2_bytes = want;
  if (w2_bytes < 0) w2_bytes = 0;
  const size_t smem = (size_t)fixed + (size_t)w2_bytes;
  int sms = 0;
  rc = sm_count(&sms);
  if (rc) return rc;
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* wgp = static_cast<const __nv_bfloat16*>(Wg);
  const __nv_bfloat16* bgp = static_cast<const __nv_bfloat16*>(bg);
  const __nv_bfloat16* resp = static_cast<const __nv_bfloat16*>(residual);
  __nv_bfloat16* permp = static_cast<__nv_bfloat16*>(perm);
  __nv_bfloat16* hp = static_cast<__nv_bfloat16*>(h);
  __nv_bfloat16* outp = static_cast<__nv_bfloat16*>(out);
  const void* const* W1 = pv.W1;
  const void* const* b1 = pv.b1;
  const void* const* W2 = pv.W2;
  const void* const* b2 = pv.b2;
  void* args[] = {(void*)&xp,     (void*)&wgp,     (void*)&bgp,  (void*)&N,       (void*)&d,
                  (void*)&f,      (void*)&E,       (void*)&k,    (void*)&W1,      (void*)&b1,
                  (void*)&W2,     (void*)&b2,      (void*)&resp, (void*)&logits,  (void*)&idx,
                  (void*)&w,      (void*)&cnt_slot, (void*)&offsets, (void*)&row_of, (void*)&permp,
                  (void*)&psum,   (void*)&aux,     (void*)&hp,   (void*)&outp,    (void*)&status,
                  (void*)&front_bytes, (void*)&w2_bytes};
  // one block per SM; a cooperative launch guarantees that they are resident together, and as a
  // programmatic dependent launch its set-up overlaps the tail of the kernel before it
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)sms);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  MOE_CUDA_CHECK(cudaLaunchKernelExC(&cfg, (const void*)decode_tiny_kernel<NT>, args));
  return 0;
}

}  // namespace

// One to eight tokens, every row of an expert in one n-tile; the routing body's limits on E and k.
bool decode_tiny_supported(int64_t N, int d, int f, int E, int k, int dtype) {
  return dtype == MOE_B200_BF16 && N >= 1 && N <= kTinyMaxTok && E <= kFrontMaxE && k <= kMaxTopK &&
         k <= E && d % 8 == 0 && f % 8 == 0 && d >= 8 && f >= 8;
}

int launch_decode_tiny(const void* x, const void* Wg, const void* bg, int64_t N, int d, int f, int E,
                       int k, const void* plan, const void* residual, float* logits, int32_t* idx,
                       float* w, int32_t* cnt_slot, int32_t* offsets, int32_t* row_of, void* perm,
                       float* psum, float* aux, void* h, void* out, int32_t* status, cudaStream_t s) {
  PlanView pv = plan_view(plan, E);
  if (E <= 8) return launch<1>(x, Wg, bg, (int)N, d, f, E, k, pv, residual, logits, idx, w, cnt_slot, offsets, row_of, perm, psum, aux, h, out, status, s);
  if (E <= 16) return launch<2>(x, Wg, bg, (int)N, d, f, E, k, pv, residual, logits, idx, w, cnt_slot, offsets, row_of, perm, psum, aux, h, out, status, s);
  return launch<4>(x, Wg, bg, (int)N, d, f, E, k, pv, residual, logits, idx, w, cnt_slot, offsets, row_of, perm, psum, aux, h, out, status, s);
}

}  // namespace moe
