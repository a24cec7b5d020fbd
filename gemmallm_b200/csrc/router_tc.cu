// Router for 17 to 64 experts on the tcgen05 path (reference model.py:206-223): logits =
// x Wg^T + bg, softmax, top-k, renormalised scores, per-block probability sums.
//
// With E = 64 the softmax and top-k over 64 logits per token, not the projection, decide the
// kernel's time (router.cu reaches 0.3 of the HBM copy rate there: four lanes share a token and
// divide, exponentiate and scan 16 experts each). Here a persistent CTA (two per SM) walks tiles of 128 tokens: x [128 x 64] and
// Wg [E x 64] tiles arrive by TMA (128-byte swizzle, three stages), one thread issues
// tcgen05.mma (M = 128, N = E padded to 32 or 64, K = 16) into one of two TMEM accumulators
// whose lane is the token, and four epilogue warps read their token's logits straight into
// registers (tcgen05.ld), where softmax and top-k need no exchange at all, while the next
// tile's loads and products already run. Results as router_mma_kernel: the same formulas in the same order, ties to
// the lowest index, psum_part rows per 64 tokens summed in token order.
#include <cuda.h>
#include "common.cuh"
#include "tc_ptx.cuh"

namespace moe {

int encode_tmap_2d(void* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);

namespace {

using namespace tc;

constexpr int kTokens = 128;          // per CTA: the accumulator's 128 lanes
constexpr int BK = 64;                // bf16 elements per stage: one 128-byte swizzle row
constexpr int kMaxStages = 6;        // three stages of 24 KB: two CTAs per SM; six when the call has no
                                      // more tiles than SMs (one tile per CTA: the loads' latency counts)
constexpr int kThreads = 192;         // warp 0: TMA, warp 1: MMA and TMEM, warps 2-5: epilogue

template <int EP>
struct Layout {
  static constexpr int kXBytes = kTokens * 128;
  static constexpr int kWBytes = EP * 128;
  static constexpr int kStageBytes = kXBytes + kWBytes;
  static constexpr int kLd = EP + 1;                                   // row pitch of the exchange buffer
  static constexpr size_t kBufBytes = sizeof(float) * kTokens * kLd;
};

struct Control {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort;
  float bias[64];
  float inv_sum[kTokens];     // 1 / softmax denominator of every token of the CTA
};

template <int EP, int kStages>
__global__ void __launch_bounds__(kThreads, kStages > 3 ? 1 : 2)
router_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                 const __nv_bfloat16* __restrict__ bg, int64_t N, int d, int E, int k,
                 float* __restrict__ out_logits, int32_t* __restrict__ out_idx,
                 float* __restrict__ out_w, float* __restrict__ psum_part,
                 int32_t* __restrict__ status) {
  using L = Layout<EP>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float* s_buf = reinterpret_cast<float*>(smem + (size_t)kStages * L::kStageBytes);   // [128][EP+1]
  Control* ctl = reinterpret_cast<Control*>(reinterpret_cast<uint8_t*>(s_buf) + L::kBufBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nkb = (d + BK - 1) / BK;
  const int num_tiles = (int)((N + kTokens - 1) / kTokens);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&ctl->acc_full[a], 1); mbar_init(&ctl->acc_empty[a], 128); }
    ctl->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_x) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_w) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&ctl->tmem_base)), "r"(2 * EP) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (threadIdx.x >= 64 && threadIdx.x - 64 < 64) {
    const int e = threadIdx.x - 64;
    ctl->bias[e] = e < E ? __bfloat162float(bg[e]) : 0.f;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctl->tmem_base);

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&ctl->empty[stage], phase ^ 1u, &ctl->abort, status, 71)) { ok = false; break; }
          uint8_t* sx = smem + (size_t)stage * L::kStageBytes;
          mbar_expect_tx(&ctl->full[stage], L::kStageBytes);
          tma_load_2d(sx, &tmap_x, &ctl->full[stage], kb * BK, tile * kTokens);
          tma_load_2d(sx + L::kXBytes, &tmap_w, &ctl->full[stage], kb * BK, 0);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t kIdesc = make_idesc(EP);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++it) {
        const int a = it & 1;
        if (!mbar_wait(&ctl->acc_empty[a], acc_phase ^ 1u, &ctl->abort, status, 74)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(a * EP);
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&ctl->full[stage], phase, &ctl->abort, status, 72)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sx = smem_u32(smem + (size_t)stage * L::kStageBytes);
          const uint64_t xdesc = make_smem_desc(sx);
          const uint64_t wdesc = make_smem_desc(sx + L::kXBytes);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk)
            tc_mma(tmem_d, xdesc + (uint64_t)(kk * 2), wdesc + (uint64_t)(kk * 2), kIdesc,
                   (kb > 0 || kk > 0) ? 1u : 0u);
          tc_commit(&ctl->empty[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) tc_commit(&ctl->acc_full[a]);
        if (a == 1) acc_phase ^= 1u;
      }
    }
  } else {
    // ---------------- epilogue: one thread per token ----------------
    const int q = warp & 3;                       // TMEM lane quadrant this warp may read
    const int tl = q * 32 + lane;                 // token within the tile
    const int et = threadIdx.x - 64;              // 0..127 among the epilogue threads
    uint32_t acc_phase = 0;
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
    const int a = it & 1;
    const int64_t tok0 = (int64_t)tile * kTokens;
    const int64_t tok = tok0 + tl;
    const int valid = (int)(N - tok0 < kTokens ? N - tok0 : kTokens);
    // warp-uniform, so that the TMEM loads below are executed by whole warps or not at all
    const bool ok = __all_sync(0xffffffffu, mbar_wait(&ctl->acc_full[a], acc_phase, &ctl->abort, status, 73));
    tc_fence_after();
    float l[EP];
    if (ok) {
#pragma unroll
      for (int c = 0; c < EP; c += 32) {
        uint32_t v[32];
        tc_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * EP + c), v);
        tc_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) l[c + i] = __uint_as_float(v[i]) + ctl->bias[c + i];
      }
    } else {
#pragma unroll
      for (int e = 0; e < EP; ++e) l[e] = 0.f;
    }
    // the accumulator is free for the tile after next
    tc_fence_before();
    mbar_arrive(&ctl->acc_empty[a]);
    if (a == 1) acc_phase ^= 1u;
    // the tile before has been summed out of the exchange buffer
    asm volatile("bar.sync 1, 128;" ::: "memory");
    // logits through shared memory: the global stores become coalesced, and the top-k below
    // can index them dynamically (entries beyond E are -inf)
    float* mine = s_buf + (size_t)tl * L::kLd;
#pragma unroll
    for (int e = 0; e < EP; ++e) {
      if (e >= E) l[e] = -INFINITY;
      mine[e] = l[e];
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (out_logits != nullptr && ok) {
      // warp w of the four writes the rows of its own 32 tokens, a lane the columns lane, lane + 32
      const int r_end = min(valid, (et >> 5) * 32 + 32);
      for (int r = (et >> 5) * 32; r < r_end; ++r)
        for (int e = lane; e < E; e += 32)
          out_logits[(tok0 + r) * E + e] = s_buf[(size_t)r * L::kLd + e];
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    // k passes of arg-max ordered by (logit descending, index ascending) over groups of eight:
    // the groups' maxima stay in registers, a pass looks into one group only
    constexpr int NG = EP / 8;
    float gm[NG];
#pragma unroll
    for (int gq = 0; gq < NG; ++gq) {
      float v = mine[gq * 8];
#pragma unroll
      for (int i = 1; i < 8; ++i) v = fmaxf(v, mine[gq * 8 + i]);
      gm[gq] = v;
    }
    float m = gm[0];
#pragma unroll
    for (int gq = 1; gq < NG; ++gq) m = fmaxf(m, gm[gq]);
    float vals[kMaxTopK];
    int sel[kMaxTopK];
    float total = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxTopK; ++j) {
      if (j < k) {
        float bv = gm[0];
        int bg = 0;
#pragma unroll
        for (int gq = 1; gq < NG; ++gq)
          if (gm[gq] > bv) { bv = gm[gq]; bg = gq; }   // strict: the lowest group wins among equals
        float* grp = mine + bg * 8;
        int bi = 7;
#pragma unroll
        for (int i = 6; i >= 0; --i)
          if (grp[i] == bv) bi = i;                    // the lowest index inside the group
        grp[bi] = -INFINITY;                           // taken
        float nm = grp[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) nm = fmaxf(nm, grp[i]);
#pragma unroll
        for (int gq = 0; gq < NG; ++gq)
          if (gq == bg) gm[gq] = nm;
        sel[j] = bg * 8 + bi;
        vals[j] = expf(bv - m);                        // the softmax denominator cancels in vals / total
        total += vals[j];                              // left-to-right sum, as model.py:221
      }
    }
    // softmax over the E real experts: the exponentials go to shared memory unscaled (they are
    // only summed per expert below, where each is multiplied by its token's 1 / denominator)
    float sum = 0.f;
#pragma unroll
    for (int e = 0; e < EP; ++e) {
      const float ex = e < E ? __expf(l[e] - m) : 0.f;
      sum += ex;
      mine[e] = ex;
    }
    ctl->inv_sum[tl] = __frcp_rn(sum);
    if (tl < valid && ok) {
#pragma unroll
      for (int j = 0; j < kMaxTopK; ++j) {
        if (j < k) {
          out_idx[tok * k + j] = sel[j];
          out_w[tok * k + j] = vals[j] / total;
        }
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    // per 64 tokens: probability sums, tokens in order
    if (ok) {
      for (int i = et; i < 2 * E; i += 128) {
        const int half = i / E, e = i - half * E;
        const int t_lo = half * 64, t_hi = min(valid, t_lo + 64);
        if (t_lo < valid) {
          float s = 0.f;
          for (int t2 = t_lo; t2 < t_hi; ++t2) s += s_buf[(size_t)t2 * L::kLd + e] * ctl->inv_sum[t2];
          psum_part[((size_t)tile * 2 + half) * E + e] = s;
        }
      }
    }
    }   // after a time-out every wait returns at once: the remaining tiles are walked without results
  }

  // ---------------- teardown ----------------
  __syncwarp();
  if (*reinterpret_cast<volatile int*>(&ctl->abort)) {
    unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 1000000ull) __nanosleep(1000);     // copies in flight
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * EP)
                 : "memory");
  }
}

template <int EP, int kStages>
int launch_stages(const CUtensorMap& tx, const CUtensorMap& tw, const void* bg, int64_t N, int d, int E,
                  int k, float* out_logits, int32_t* out_idx, float* out_w, float* psum_part,
                  int32_t* status, int64_t blocks, cudaStream_t s) {
  using L = Layout<EP>;
  const size_t smem = 1024 + (size_t)kStages * L::kStageBytes + L::kBufBytes + sizeof(Control);
  static PerDeviceOnce once;
  int rc = ensure_dynamic_smem(once, router_tc_kernel<EP, kStages>, 224 * 1024);
  if (rc) return rc;
  router_tc_kernel<EP, kStages><<<(unsigned)blocks, kThreads, smem, s>>>(
      tx, tw, static_cast<const __nv_bfloat16*>(bg), N, d, E, k, out_logits, out_idx, out_w, psum_part,
      status);
  MOE_CUDA_CHECK(cudaGetLastError());
  return 0;
}

template <int EP>
int launch(const void* x, const void* Wg, const void* bg, int64_t N, int d, int E, int k,
           float* out_logits, int32_t* out_idx, float* out_w, float* psum_part, int32_t* status,
           cudaStream_t s) {
  alignas(64) CUtensorMap tx, tw;
  int rc = encode_tmap_2d(&tx, x, (uint64_t)N, (uint64_t)d, kTokens);
  if (rc) return rc;
  rc = encode_tmap_2d(&tw, Wg, (uint64_t)E, (uint64_t)d, EP);
  if (rc) return rc;
  const int64_t tiles = (N + kTokens - 1) / kTokens;
  int sms = 0;
  rc = sm_count(&sms);
  if (rc) return rc;
  if (tiles <= sms)
    return launch_stages<EP, 6>(tx, tw, bg, N, d, E, k, out_logits, out_idx, out_w, psum_part, status,
                                tiles, s);
  // two persistent CTAs per SM
  return launch_stages<EP, 3>(tx, tw, bg, N, d, E, k, out_logits, out_idx, out_w, psum_part, status,
                              tiles < 2 * (int64_t)sms ? tiles : 2 * (int64_t)sms, s);
}

}  // namespace

// bf16, 17 to 64 experts, rows 16-byte aligned and pitched (d a multiple of 8), a token count
// TMA coordinates can hold.
bool router_tc_supported(int64_t N, int d, int E, int k) {
  return E > 16 && E <= 64 && d % 8 == 0 && d >= 64 && N >= 1 && N < (1ll << 31) && k <= kMaxTopK && k <= E;
}

int launch_router_tc(const void* x, const void* Wg, const void* bg, int64_t N, int d, int E, int k,
                     float* out_logits, int32_t* out_idx, float* out_w, float* psum_part,
                     int32_t* status, cudaStream_t s) {
  if (E <= 32)
    return launch<32>(x, Wg, bg, N, d, E, k, out_logits, out_idx, out_w, psum_part, status, s);
  return launch<64>(x, Wg, bg, N, d, E, k, out_logits, out_idx, out_w, psum_part, status, s);
}

}  // namespace moe
