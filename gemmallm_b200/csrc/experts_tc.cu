// Expert feed-forward on the 5th-generation tensor cores (tcgen05 + TMEM),
// bf16 operands, fp32 accumulation. Two launches of one persistent kernel:
//   GEGLU pass : h = gelu_tanh(x W1[:f]^T + b1[:f]) * (x W1[f:]^T + b1[f:])
//                (reference model.py:174,180-182), gate and up tiles side by
//                side in one 128x256 accumulator, activation in the epilogue;
//   plain pass : y = h W2^T + b2 (model.py:184).
// Experts are grouped by the row offsets the dispatch kernel wrote; nothing is
// read back to the host, every CTA derives the tile list from the offsets.
//
// One CTA per SM, 320 threads:
//   warp 0   : TMA producer  (cp.async.bulk.tensor, 128-byte swizzle, 4 stages)
//   warp 1   : MMA issuer    (tcgen05.mma cta_group::1 kind::f16, M=128 N=256 K=16)
//   warps 2-9: epilogue      (tcgen05.ld 32 lanes x 32 columns, bias, GeGLU, store);
//              two warps per TMEM lane quadrant, each taking half of the columns
// The 512 TMEM columns hold two 128x256 fp32 accumulators, so the epilogue of
// one tile runs under the main loop of the next.
//
// No TMA load uses cluster multicast. Every wait is bounded: when one runs out
// the CTA records MOE_B200_DEV_TIMEOUT in the status word, stops issuing, frees
// its TMEM and returns.
//
// The small-N ("decode") arrangement of the same products is in
// experts_decode.cu.
#include <cuda.h>
#include "common.cuh"
#include "tc_ptx.cuh"
#include "tc_epilogue.cuh"

namespace moe {

namespace {

using namespace tc;

constexpr int BM = 128;          // rows of the sorted buffer per tile = TMEM lanes
constexpr int BK = 64;           // bf16 elements = one 128-byte swizzle row
constexpr int BN = 256;          // weight rows per tile (gate 128 + up 128, or 256 plain)
constexpr int kStages = 4;
constexpr int kABytes = BM * BK * 2;          // 16 KiB
constexpr int kBHalfBytes = (BN / 2) * BK * 2;  // 16 KiB
constexpr int kStageBytes = kABytes + 2 * kBHalfBytes;
constexpr int kThreads = 320;   // TMA warp, MMA warp, 8 epilogue warps
constexpr int kTmemCols = 2 * BN;             // two accumulators
constexpr uint32_t kIdesc = make_idesc(BN);

struct Control {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort;
  int tile_start[kMaxExperts + 1];
  int offsets[kMaxExperts + 1];  // copy of the row offsets: no global loads in the tile loops
  alignas(16) uint8_t stage_out[8][kStgBytes];  // one staging area per epilogue warp
};

constexpr size_t kSmemBytes = 1024 + (size_t)kStages * kStageBytes + sizeof(Control);

// GEGLU : B = gate rows [n0, n0+128) and up rows [Nout+n0, ...) of W [2*Nout, K];
//         out[row, n0..n0+128) = gelu_tanh(gate + bg) * (up + bu).
// plain : B = rows [n0, n0+256) of W [Nout, K]; out[row, n0..n0+256) = acc + bias.
// SCATTER (plain only, expert-parallel): row i goes to the buffer of the rank
//         that owns its token, sc.ret_y[meta >> 24] + (meta & 0xffffff) * Nout,
//         with plain stores through the peer mapping.
template <bool GEGLU, bool SCATTER>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a,
                       const CUtensorMap* __restrict__ tmap_b,  // [E], global memory
                       const int32_t* __restrict__ offsets,
                       const void* const* __restrict__ bias_ptrs, int E, int K, int Nout,
                       __nv_bfloat16* __restrict__ out, const EpScatter sc,
                       int32_t* __restrict__ status) {
#ifdef MOE_TC_PROFILE
  const long long prof_entry = clock64();
  constexpr int kProfBase = GEGLU ? 0 : 8;
#endif
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~(uintptr_t)1023);
  Control* ctl = reinterpret_cast<Control*>(smem + (size_t)kStages * kStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr int kTileN = GEGLU ? BN / 2 : BN;  // output columns per tile
  const int n_tiles = (Nout + kTileN - 1) / kTileN;
  const int k_blocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&ctl->tmem_full[a], 1); mbar_init(&ctl->tmem_empty[a], 256); }
    ctl->abort = 0;
    int acc = 0;
    int beg = offsets[0];
    ctl->offsets[0] = beg;
    for (int e = 0; e < E; ++e) {
      ctl->tile_start[e] = acc;
      const int end = offsets[e + 1];
      ctl->offsets[e + 1] = end;
      acc += ((end - beg + BM - 1) / BM) * n_tiles;
      beg = end;
    }
    ctl->tile_start[E] = acc;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&ctl->tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctl->tmem_base);
  const int total_tiles = ctl->tile_start[E];
#ifdef MOE_TC_PROFILE
  const long long prof_kernel_t0 = clock64();
  if (blockIdx.x == 0 && threadIdx.x == 0) g_prof[6 + kProfBase] = prof_kernel_t0 - prof_entry;
#endif

  // tile t of expert e: local = mt * n_tiles + nt
  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int e = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        while (t >= ctl->tile_start[e + 1]) ++e;
        const int local = t - ctl->tile_start[e];
        const int mt = local / n_tiles, nt = local - mt * n_tiles;
        const int row0 = ctl->offsets[e] + mt * BM;
        const int b0 = nt * kTileN;
        const int b1 = GEGLU ? Nout + nt * kTileN : nt * kTileN + BN / 2;
        const CUtensorMap* tb = tmap_b + e;
        for (int kb = 0; kb < k_blocks; ++kb) {
          {
            PROF_T0();
            if (!mbar_wait(&ctl->empty[stage], phase ^ 1u, &ctl->abort, status, 1)) { ok = false; break; }
            PROF_ADD(0);
          }
          uint8_t* sa = smem + (size_t)stage * kStageBytes;
          mbar_expect_tx(&ctl->full[stage], kStageBytes);
          tma_load_2d(sa, &tmap_a, &ctl->full[stage], kb * BK, row0);
          tma_load_2d(sa + kABytes, tb, &ctl->full[stage], kb * BK, b0);
          tma_load_2d(sa + kABytes + kBHalfBytes, tb, &ctl->full[stage], kb * BK, b1);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x, ++it) {
        const int a = it & 1;
        {
          PROF_T0();
          if (!mbar_wait(&ctl->tmem_empty[a], acc_phase ^ 1u, &ctl->abort, status, 2)) { ok = false; break; }
          PROF_ADD(1);
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(a * BN);
        for (int kb = 0; kb < k_blocks; ++kb) {
          {
            PROF_T0();
            if (!mbar_wait(&ctl->full[stage], phase, &ctl->abort, status, 3)) { ok = false; break; }
            PROF_ADD(2);
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + (size_t)stage * kStageBytes);
          const uint64_t adesc = make_smem_desc(sa);
          const uint64_t bdesc = make_smem_desc(sa + kABytes);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            // 16 bf16 = 32 bytes further along K inside the swizzled row
            tc_mma(tmem_d, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), kIdesc,
                   (kb | kk) != 0 ? 1u : 0u);
          }
          tc_commit(&ctl->empty[stage]);  // frees the stage once these MMAs have read it
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(&ctl->tmem_full[a]);
        if (a == 1) acc_phase ^= 1u;
      }
    }
  } else {
    // ---------------- epilogue: 4 warps, one accumulator row per thread ----------------
    const int quad = warp & 3;  // TMEM lanes [32*quad, 32*quad+32) belong to this warp
    const int half = (warp - 2) >> 2;  // which half of the tile's columns
    const int r = quad * 32 + lane;
    uint32_t acc_phase = 0;
    int it = 0;
    int e = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x, ++it) {
      while (t >= ctl->tile_start[e + 1]) ++e;
      const int local = t - ctl->tile_start[e];
      const int mt = local / n_tiles, nt = local - mt * n_tiles;
      const int row = ctl->offsets[e] + mt * BM + r;
      const bool row_ok = row < ctl->offsets[e + 1];
      const int n0 = nt * kTileN;
      const __nv_bfloat16* bias = static_cast<const __nv_bfloat16*>(bias_ptrs[e]);
      const int a = it & 1;
      {
        PROF_T0();
        if (!mbar_wait(&ctl->tmem_full[a], acc_phase, &ctl->abort, status, 4)) { ok = false; break; }
        if (threadIdx.x == 64) PROF_ADD(3);
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(a * BN);
      store_tile<GEGLU, SCATTER>(taddr, row, row_ok, n0, Nout, bias, out, sc, ctl->stage_out[warp - 2], lane, half);
      tc_fence_before();
      mbar_arrive(&ctl->tmem_empty[a]);
      if (a == 1) acc_phase ^= 1u;
    }
    if (SCATTER) __threadfence_system();  // peer stores performed before the kernel ends
  }

#ifdef MOE_TC_PROFILE
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    g_prof[4 + kProfBase] = clock64() - prof_kernel_t0;
    g_prof[5 + kProfBase] = total_tiles;
  }
#endif
  // ---------------- teardown ----------------
  __syncwarp();
  if (*reinterpret_cast<volatile int*>(&ctl->abort)) {
    // give copies still in flight time to land before shared memory is released
    unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 1000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols)
                 : "memory");
  }
}

template <bool GEGLU, bool SCATTER>
int launch_one(const CUtensorMap& tm_a, const void* tmap_b, const int32_t* offsets,
               const void* const* bias, int E, int K, int Nout, void* out, const EpScatter& sc,
               int32_t* status, int sms, cudaStream_t s) {
  static bool attr_set = false;
  auto fn = grouped_gemm_tc_kernel<GEGLU, SCATTER>;
  if (!attr_set) {
    MOE_CUDA_CHECK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)kSmemBytes));
    attr_set = true;
  }
  fn<<<sms, kThreads, kSmemBytes, s>>>(tm_a, static_cast<const CUtensorMap*>(tmap_b), offsets, bias,
                                       E, K, Nout, static_cast<__nv_bfloat16*>(out), sc, status);
  MOE_CUDA_CHECK(cudaGetLastError());
  return 0;
}

}  // namespace

int launch_experts_tc(const void* perm, const int32_t* offsets, const void* plan, int64_t M, int d,
                      int f, int E, void* h, void* y, int32_t* status, cudaStream_t s) {
  if (M == 0) return 0;
  PlanView pv = plan_view(plan, E);
  alignas(64) CUtensorMap tm_x, tm_h;
  int rc = encode_tmap_2d(&tm_x, perm, (uint64_t)M, (uint64_t)d, BM);
  if (rc) return rc;
  rc = encode_tmap_2d(&tm_h, h, (uint64_t)M, (uint64_t)f, BM);
  if (rc) return rc;
  int sms = 0;
  rc = sm_count(&sms);
  if (rc) return rc;
  const EpScatter none = {};
  rc = launch_one<true, false>(tm_x, pv.tmap_W1, offsets, pv.b1, E, d, f, h, none, status, sms, s);
  if (rc) return rc;
  return launch_one<false, false>(tm_h, pv.tmap_W2, offsets, pv.b2, E, f, d, y, none, status, sms, s);
}

// Expert-parallel: the sorted buffer is this rank's receive buffer (capacity
// `cap` rows, filled up to offsets[E_local]); the down pass scatters its rows
// to the token owners.
int launch_experts_tc_ep(const void* recv_x, const int32_t* offsets, const void* plan, int64_t cap,
                         int d, int f, int E_local, void* h, const EpScatter& sc, int32_t* status,
                         cudaStream_t s) {
  if (cap == 0 || E_local == 0) return 0;
  PlanView pv = plan_view(plan, E_local);
  alignas(64) CUtensorMap tm_x, tm_h;
  int rc = encode_tmap_2d(&tm_x, recv_x, (uint64_t)cap, (uint64_t)d, BM);
  if (rc) return rc;
  rc = encode_tmap_2d(&tm_h, h, (uint64_t)cap, (uint64_t)f, BM);
  if (rc) return rc;
  int sms = 0;
  rc = sm_count(&sms);
  if (rc) return rc;
  const EpScatter none = {};
  rc = launch_one<true, false>(tm_x, pv.tmap_W1, offsets, pv.b1, E_local, d, f, h, none, status,
                               sms, s);
  if (rc) return rc;
  return launch_one<false, true>(tm_h, pv.tmap_W2, offsets, pv.b2, E_local, f, d, nullptr, sc,
                                 status, sms, s);
}

#ifdef MOE_TC_PROFILE
extern "C" void moe_b200_prof_read(long long* out, int reset) {
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(out, tc::g_prof, sizeof(long long) * 16);
  if (reset) {
    long long z[16] = {0};
    cudaMemcpyToSymbol(tc::g_prof, z, sizeof(z));
  }
}
#endif

}  // namespace moe
