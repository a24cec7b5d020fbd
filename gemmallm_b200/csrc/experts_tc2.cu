// Grouped expert GEMMs with CTA pairs (tcgen05 cta_group::2): two neighbouring
// SMs share one 256-row x 256-column output tile. Each CTA stages its own 128
// rows of the activation operand and HALF of the weight tile (for the GEGLU
// pass CTA 0 holds the 128 gate rows, CTA 1 the 128 up rows); the pair's MMA
// (M=256, N=256, K=16), issued by the even CTA, reads both halves, and each
// CTA's TMEM receives the 128x256 accumulator of its own rows. Per 128x256x64
// step a CTA therefore pulls 32 KiB from L2 and shared memory instead of the
// 48 KiB a single CTA with a 128x256 tile would need: operand delivery, not the
// tensor pipe, is what bounds a one-CTA kernel of this shape.
//
// Synchronisation inside the pair (all mbarriers, all waits bounded):
//   full[s]       lives in the even CTA; both CTAs' TMA loads complete on it
//                 (cp.async.bulk.tensor ... cta_group::2, no multicast);
//   empty[s]      one per CTA; the MMA thread commits to its own and, through
//                 the cluster-mapped address, to its peer's;
//   tmem_full[a]  one per CTA, committed the same way;
//   tmem_empty[a] in the even CTA; the 16 epilogue warps of the pair arrive on
//                 it (the odd CTA's warps through the cluster-mapped address).
// Math and epilogue (tc_epilogue.cuh): reference model.py:174,180-184.
//
// The same kernel serves the backward pass (the reference trains through this block with
// torch.autograd, train.py:140): the input gradients are two more row-grouped products
// against transposed weights; the weight gradients dW_e = dY_e^T X_e contract over an
// expert's rows, so there (COLS) a group is a range of the contraction index of two
// transposed activation buffers and every expert has the same output tiles.
#include <cuda.h>
#include "common.cuh"
#include "tc_ptx.cuh"
#include "tc_epilogue.cuh"
#include "ep_sync.cuh"

namespace moe {

namespace {

using namespace tc;

constexpr int BM = 128;           // rows per CTA = TMEM lanes
constexpr int kPairRows = 256;    // rows per tile (both CTAs)
constexpr int BK = 64;
constexpr int BN = 256;
constexpr int kStages = 6;
constexpr int kABytes = BM * BK * 2;         // 16 KiB: this CTA's rows
constexpr int kBBytes = (BN / 2) * BK * 2;   // 16 KiB: this CTA's half of the weight tile
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kThreads = 320;   // TMA warp, MMA warp, 8 epilogue warps
constexpr int kTmemCols = 2 * BN;
// M = 256 across the pair: M/16 at bit 24
constexpr uint32_t kIdesc2 = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                             ((256u >> 4) << 24);

struct Control {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort;
  int tile_start[kMaxExperts + 1];
  int offsets[kMaxExperts + 1];
  alignas(16) uint8_t stage_out[8][kStgBytes];  // one staging area per epilogue warp
};

constexpr size_t kSmemBytes = 1024 + (size_t)kStages * kStageBytes + sizeof(Control);

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `cta` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(cta));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const void* tmap, uint32_t bar_cluster,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster), "r"(c0),
      "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar_cluster) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar_cluster)
               : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster)
               : "memory");
}

// COLS = false: groups are row ranges [offsets[e], offsets[e+1]) of A; B_e = tmap_b[e]; K fixed.
// COLS = true : groups are ranges [offsets[e], offsets[e+1]) (multiples of 64) of the contraction
//               index; A has Ra rows, B (one map, tmap_bc) has Nout rows; out [E][Ra][Nout].
template <bool GEGLU, bool SCATTER, bool TRAIN, bool COLS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
grouped_gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmap_a,
                        const __grid_constant__ CUtensorMap tmap_bc,
                        const CUtensorMap* __restrict__ tmap_b,  // [E], 128-row boxes
                        const int32_t* __restrict__ offsets,
                        const void* const* __restrict__ bias_ptrs, int E, int K, int Nout,
                        __nv_bfloat16* __restrict__ out, const EpScatter sc, const TrainArgs tr,
                        const EpSync sy, int Ra, int32_t* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~(uintptr_t)1023);
  Control* ctl = reinterpret_cast<Control*>(smem + (size_t)kStages * kStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();   // 0 = even CTA: issues the MMAs, owns full/tmem_empty
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  constexpr int kTileN = GEGLU ? BN / 2 : BN;
  const int n_tiles = (Nout + kTileN - 1) / kTileN;
  const int k_blocks_rows = (K + BK - 1) / BK;
  const int m_tiles_cols = (Ra + kPairRows - 1) / kPairRows;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&ctl->tmem_full[a], 1); mbar_init(&ctl->tmem_empty[a], 16); }
    ctl->abort = 0;
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&ctl->tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  // everything above is independent of the kernels before this one in the stream
  pdl_wait();
  pdl_launch_dependents();
  // expert-parallel: the rows this kernel reads were pushed by the other ranks; wait for all of
  // them (bounded), then order those peer writes before this CTA's TMA reads
  const bool arrived = epsync::block_wait(sy, status, 24);
  if (sy.wait_flags != nullptr) asm volatile("fence.proxy.async;" ::: "memory");
  if (threadIdx.x == 0) {
    int acc = 0;
    int beg = offsets[0];
    ctl->offsets[0] = beg;
    for (int e = 0; e < E; ++e) {
      ctl->tile_start[e] = acc;
      const int end = offsets[e + 1];
      ctl->offsets[e + 1] = end;
      acc += COLS ? (end > beg ? m_tiles_cols * n_tiles : 0)
                  : ((end - beg + kPairRows - 1) / kPairRows) * n_tiles;
      beg = end;
    }
    ctl->tile_start[E] = arrived ? acc : 0;   // a peer never arrived: nothing to do
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();   // both CTAs' barriers exist before anything signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctl->tmem_base);
  const int total_tiles = ctl->tile_start[E];

  if (warp == 0) {
    // ---------------- TMA producer (each CTA loads its own rows and its half of B) -------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int e = 0;
      bool ok = true;
      for (int t = pair; ok && t < total_tiles; t += num_pairs) {
        while (t >= ctl->tile_start[e + 1]) ++e;
        const int local = t - ctl->tile_start[e];
        const int mt = local / n_tiles, nt = local - mt * n_tiles;
        const int row0 = (COLS ? 0 : ctl->offsets[e]) + mt * kPairRows + (int)cta * BM;
        const int brow = GEGLU ? (cta == 0 ? nt * kTileN : Nout + nt * kTileN)
                               : nt * kTileN + (int)cta * (BN / 2);
        const CUtensorMap* tb = COLS ? &tmap_bc : tmap_b + e;
        const int k0 = COLS ? ctl->offsets[e] : 0;
        const int k_blocks = COLS ? (ctl->offsets[e + 1] - k0) / BK : k_blocks_rows;
        for (int kb = 0; kb < k_blocks; ++kb) {
          {
            if (!mbar_wait(&ctl->empty[stage], phase ^ 1u, &ctl->abort, status, 31)) { ok = false; break; }
          }
          uint8_t* sa = smem + (size_t)stage * kStageBytes;
          const uint32_t full0 = map_to_cta(smem_u32(&ctl->full[stage]), 0);
          if (cta == 0) mbar_expect_tx(&ctl->full[stage], 2 * kStageBytes);
          tma_load_2d_pair(sa, &tmap_a, full0, k0 + kb * BK, row0);
          tma_load_2d_pair(sa + kABytes, tb, full0, k0 + kb * BK, brow);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (even CTA only) ----------------
    if (lane == 0 && cta == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase = 0;
      int it = 0;
      int e = 0;
      bool ok = true;
      for (int t = pair; ok && t < total_tiles; t += num_pairs, ++it) {
        const int a = it & 1;
        int k_blocks = k_blocks_rows;
        if (COLS) {
          while (t >= ctl->tile_start[e + 1]) ++e;
          k_blocks = (ctl->offsets[e + 1] - ctl->offsets[e]) / BK;
        }
        {
          if (!mbar_wait(&ctl->tmem_empty[a], acc_phase ^ 1u, &ctl->abort, status, 32)) { ok = false; break; }
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(a * BN);
        for (int kb = 0; kb < k_blocks; ++kb) {
          {
            if (!mbar_wait(&ctl->full[stage], phase, &ctl->abort, status, 33)) { ok = false; break; }
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + (size_t)stage * kStageBytes);
          const uint64_t adesc = make_smem_desc(sa);
          const uint64_t bdesc = make_smem_desc(sa + kABytes);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk)
            tc_mma_pair(tmem_d, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), kIdesc2,
                        (kb | kk) != 0 ? 1u : 0u);
          // the stage is free in both CTAs once these MMAs have read it
          const uint32_t e_local = smem_u32(&ctl->empty[stage]);
          tc_commit_pair(map_to_cta(e_local, 0));
          tc_commit_pair(map_to_cta(e_local, 1));
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        const uint32_t f_local = smem_u32(&ctl->tmem_full[a]);
        tc_commit_pair(map_to_cta(f_local, 0));
        tc_commit_pair(map_to_cta(f_local, 1));
        if (a == 1) acc_phase ^= 1u;
      }
    }
  } else {
    // ---------------- epilogue: 8 warps per CTA, one accumulator row per thread ----------------
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;  // two warps per TMEM lane quadrant split the columns
    const int r = quad * 32 + lane;
    uint32_t acc_phase = 0;
    int it = 0;
    int e = 0;
    bool ok = true;
    for (int t = pair; ok && t < total_tiles; t += num_pairs, ++it) {
      while (t >= ctl->tile_start[e + 1]) ++e;
      const int local = t - ctl->tile_start[e];
      const int mt = local / n_tiles, nt = local - mt * n_tiles;
      const int row = (COLS ? 0 : ctl->offsets[e]) + mt * kPairRows + (int)cta * BM + r;
      const bool row_ok = COLS ? row < Ra : row < ctl->offsets[e + 1];
      const int n0 = nt * kTileN;
      const __nv_bfloat16* bias =
          bias_ptrs != nullptr ? static_cast<const __nv_bfloat16*>(bias_ptrs[e]) : nullptr;
      __nv_bfloat16* out_e = COLS ? out + (size_t)e * Ra * Nout : out;
      const int a = it & 1;
      {
        if (!mbar_wait(&ctl->tmem_full[a], acc_phase, &ctl->abort, status, 34)) { ok = false; break; }
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(a * BN);
      store_tile<GEGLU, SCATTER, TRAIN>(taddr, row, row_ok, n0, Nout, bias, out_e, sc, tr,
                                        ctl->stage_out[warp - 2], lane, half);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&ctl->tmem_empty[a]), 0));
      if (a == 1) acc_phase ^= 1u;
    }
    if (SCATTER) __threadfence_system();
  }
  // expert-parallel down pass: the last CTA to get here tells every rank that this rank's
  // outputs have been stored
  epsync::grid_signal(sy);

  // ---------------- teardown ----------------
  __syncwarp();
  if (*reinterpret_cast<volatile int*>(&ctl->abort)) {
    unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 1000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();   // the peer may still signal this CTA's barriers or read its shared memory
  tc_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols)
                 : "memory");
  }
}

template <bool GEGLU, bool SCATTER, bool TRAIN, bool COLS>
int launch_pair(const CUtensorMap& tm_a, const CUtensorMap& tm_bc, const void* tmap_b, const int32_t* offsets,
                const void* const* bias, int E, int K, int Nout, void* out, const EpScatter& sc,
                const TrainArgs& tr, const EpSync& sy, int Ra, int32_t* status, int sms, cudaStream_t s) {
  static PerDeviceOnce once;
  auto fn = grouped_gemm_tc2_kernel<GEGLU, SCATTER, TRAIN, COLS>;
  int rc = ensure_dynamic_smem(once, fn, kSmemBytes);
  if (rc) return rc;
  MOE_CUDA_CHECK(launch_pdl(fn, dim3(sms & ~1), dim3(kThreads), kSmemBytes, s, tm_a, tm_bc,
                            static_cast<const CUtensorMap*>(tmap_b), offsets, bias, E, K, Nout,
                            static_cast<__nv_bfloat16*>(out), sc, tr, sy, Ra, status));
  return 0;
}

}  // namespace

int launch_experts_tc2(const void* perm, const int32_t* offsets, const void* plan, int64_t M, int d,
                       int f, int E, void* h, void* y, const EpScatter* sc, int32_t* status,
                       cudaStream_t s, const TrainArgs* train, const EpSync* ep_wait,
                       const EpSync* ep_signal) {
  // expert-parallel ranks take part in the hand-shakes even when they own no rows
  if ((M == 0 || E == 0) && ep_wait == nullptr && ep_signal == nullptr) return 0;
  PlanView pv = plan_view(plan, E);
  alignas(64) CUtensorMap tm_x, tm_h;
  const uint64_t rows = M > 0 ? (uint64_t)M : 1;   // a rank without rows still launches (hand-shakes)
  int rc = encode_tmap_2d(&tm_x, perm, rows, (uint64_t)d, BM);
  if (rc) return rc;
  rc = encode_tmap_2d(&tm_h, h, rows, (uint64_t)f, BM);
  if (rc) return rc;
  int sms = 0;
  rc = sm_count(&sms);
  if (rc) return rc;
  const EpScatter none = {};
  const TrainArgs eval = {};
  const EpSync nosync = {};
  const EpSync& sy1 = ep_wait != nullptr ? *ep_wait : nosync;
  const EpSync& sy2 = ep_signal != nullptr ? *ep_signal : nosync;
  if (train != nullptr)
    rc = launch_pair<true, false, true, false>(tm_x, tm_x, pv.tmap_W1, offsets, pv.b1, E, d, f, h, none, *train,
                                               sy1, 0, status, sms, s);
  else
    rc = launch_pair<true, false, false, false>(tm_x, tm_x, pv.tmap_W1, offsets, pv.b1, E, d, f, h, none, eval,
                                                sy1, 0, status, sms, s);
  if (rc) return rc;
  if (sc != nullptr)
    return launch_pair<false, true, false, false>(tm_h, tm_h, pv.tmap_W2, offsets, pv.b2, E, f, d, nullptr, *sc,
                                                  eval, sy2, 0, status, sms, s);
  return launch_pair<false, false, false, false>(tm_h, tm_h, pv.tmap_W2, offsets, pv.b2, E, f, d, y, none, eval,
                                                 sy2, 0, status, sms, s);
}

int launch_grouped_rows(const void* A, int64_t M, int K, const void* tmaps_b, const int32_t* offsets,
                        const void* const* bias, int E, int Nout, void* out, int32_t* status,
                        cudaStream_t s) {
  if (M == 0 || E == 0) return 0;
  alignas(64) CUtensorMap tm_a;
  int rc = encode_tmap_2d(&tm_a, A, (uint64_t)M, (uint64_t)K, BM);
  if (rc) return rc;
  int sms = 0;
  rc = sm_count(&sms);
  if (rc) return rc;
  const EpScatter none = {};
  const TrainArgs eval = {};
  const EpSync nosync = {};
  return launch_pair<false, false, false, false>(tm_a, tm_a, tmaps_b, offsets, bias, E, K, Nout, out, none,
                                                 eval, nosync, 0, status, sms, s);
}

int launch_grouped_cols(const void* At, const void* Bt, int64_t Kpad, int Ra, int Rb,
                        const int32_t* koff, void* out, int E, int32_t* status, cudaStream_t s) {
  if (Kpad == 0 || E == 0) return 0;
  alignas(64) CUtensorMap tm_a, tm_b;
  int rc = encode_tmap_2d(&tm_a, At, (uint64_t)Ra, (uint64_t)Kpad, BM);
  if (rc) return rc;
  rc = encode_tmap_2d(&tm_b, Bt, (uint64_t)Rb, (uint64_t)Kpad, BM);
  if (rc) return rc;
  int sms = 0;
  rc = sm_count(&sms);
  if (rc) return rc;
  const EpScatter none = {};
  const TrainArgs eval = {};
  const EpSync nosync = {};
  return launch_pair<false, false, false, true>(tm_a, tm_b, nullptr, koff, nullptr, E, 0, Rb, out,
                                                none, eval, nosync, Ra, status, sms, s);
}

}  // namespace moe
