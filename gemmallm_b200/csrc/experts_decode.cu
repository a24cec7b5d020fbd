// Expert feed-forward for a few rows per expert ("decode" shapes): the work is
// streaming every hit expert's weights from HBM once, so the roles of the two
// MMA operands are swapped with respect to experts_tc.cu. The weights are the
// 128-row A operand (every byte staged in shared memory is a weight byte the
// tensor core has to read anyway), the expert's tokens are the narrow B operand
// (32 rows), and the accumulator is [128 weight rows x 32 tokens] in TMEM.
//   GEGLU pass : A = 64 gate rows + 64 up rows of gate_and_up.weight; the
//                epilogue pairs accumulator lane j (gate) with lane 64+j (up)
//                through shared memory: h = gelu_tanh(g + bg) * (u + bu)
//                (reference model.py:174,180-182).
//   down pass  : A = 128 rows of down.weight, K split into `ksplit` ranges so
//                that there are enough tiles for every SM; each range writes
//                fp32 partial sums part[ks][row][d] without bias; the combine
//                kernel adds them in a fixed order (model.py:184).
// Same machinery as experts_tc.cu: one persistent CTA per SM, TMA producer
// warp, MMA warp, four epilogue warps, two accumulators, bounded waits, no
// cluster multicast. Nine stages of 20 KiB (16 KiB weights + 4 KiB tokens).
#include <cuda.h>
#include "common.cuh"
#include "tc_ptx.cuh"

namespace moe {

namespace {

using namespace tc;

constexpr int BK = 64;                     // bf16 per 128-byte swizzle row
constexpr int kWRows = 128;                // weight rows per tile = TMEM lanes
constexpr int kTok = 32;                   // token rows per tile = accumulator columns
constexpr int kStages = 9;
constexpr int kWBytes = kWRows * BK * 2;   // 16 KiB, loaded as two 64-row boxes
constexpr int kWHalf = kWBytes / 2;
constexpr int kTBytes = kTok * BK * 2;     // 4 KiB
constexpr int kStageBytes = kWBytes + kTBytes;
constexpr int kThreads = 192;
constexpr int kTmemCols = 64;              // two accumulators of 32 columns
constexpr uint32_t kIdesc = make_idesc(kTok);
constexpr int kUpPitch = kTok + 1;

struct Control {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t up_ready[2];  // the 64 "up" lanes have written their half to shared memory
  uint32_t tmem_base;
  int abort;
  int tile_start[kMaxExperts + 1];
  int offsets[kMaxExperts + 1];
  float up[2][64 * kUpPitch];  // up half of the accumulator, per accumulator buffer
};

constexpr size_t kSmemBytes = 1024 + (size_t)kStages * kStageBytes + sizeof(Control);

// GEGLU: W = gate_and_up.weight [2*Nout, K]; out = h [M, Nout] bf16.
// plain: W = down.weight [Nout, K]; out = part [ksplit][M][Nout] fp32.
template <bool GEGLU>
__global__ void __launch_bounds__(kThreads, 1)
decode_gemm_kernel(const __grid_constant__ CUtensorMap tmap_tok,
                   const CUtensorMap* __restrict__ tmap_w,  // [E], 64-row boxes, global memory
                   const int32_t* __restrict__ offsets, const void* const* __restrict__ bias_ptrs,
                   int E, int K, int Nout, int ksplit, int64_t part_stride,
                   void* __restrict__ out_raw, int32_t* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~(uintptr_t)1023);
  Control* ctl = reinterpret_cast<Control*>(smem + (size_t)kStages * kStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr int kTileN = GEGLU ? 64 : 128;  // output features per tile
  const int n_tiles = (Nout + kTileN - 1) / kTileN;
  const int k_blocks_all = (K + BK - 1) / BK;
  const int kb_per_split = (k_blocks_all + ksplit - 1) / ksplit;
  const int per_tb = n_tiles * ksplit;  // tiles per 32-token block of an expert

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], 1); }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&ctl->tmem_full[a], 1);
      mbar_init(&ctl->tmem_empty[a], 128);
      mbar_init(&ctl->up_ready[a], 64);
    }
    ctl->abort = 0;
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&ctl->tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // everything above is independent of the kernels before this one in the stream
  pdl_wait();
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    int acc = 0;
    int beg = offsets[0];
    ctl->offsets[0] = beg;
    for (int e = 0; e < E; ++e) {
      ctl->tile_start[e] = acc;
      const int end = offsets[e + 1];
      ctl->offsets[e + 1] = end;
      acc += ((end - beg + kTok - 1) / kTok) * per_tb;
      beg = end;
    }
    ctl->tile_start[E] = acc;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctl->tmem_base);
  const int total_tiles = ctl->tile_start[E];

  // tile t of expert e: local = (tb * n_tiles + nt) * ksplit + ks
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
        const int ks = local % ksplit;
        const int rest = local / ksplit;
        const int tb = rest / n_tiles, nt = rest - tb * n_tiles;
        const int row0 = ctl->offsets[e] + tb * kTok;
        const int w0 = nt * kTileN;
        const int w1 = GEGLU ? Nout + nt * kTileN : nt * kTileN + 64;
        const CUtensorMap* tw = tmap_w + e;
        const int kb0 = ks * kb_per_split;
        const int kb1 = min(k_blocks_all, kb0 + kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&ctl->empty[stage], phase ^ 1u, &ctl->abort, status, 11)) { ok = false; break; }
          uint8_t* sw = smem + (size_t)stage * kStageBytes;
          mbar_expect_tx(&ctl->full[stage], kStageBytes);
          tma_load_2d(sw, tw, &ctl->full[stage], kb * BK, w0);
          tma_load_2d(sw + kWHalf, tw, &ctl->full[stage], kb * BK, w1);
          tma_load_2d(sw + kWBytes, &tmap_tok, &ctl->full[stage], kb * BK, row0);
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
      int e = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x, ++it) {
        while (t >= ctl->tile_start[e + 1]) ++e;
        const int ks = (t - ctl->tile_start[e]) % ksplit;
        const int kb0 = ks * kb_per_split;
        const int kb1 = min(k_blocks_all, kb0 + kb_per_split);
        const int a = it & 1;
        if (!mbar_wait(&ctl->tmem_empty[a], acc_phase ^ 1u, &ctl->abort, status, 12)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(a * kTok);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&ctl->full[stage], phase, &ctl->abort, status, 13)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sw = smem_u32(smem + (size_t)stage * kStageBytes);
          const uint64_t wdesc = make_smem_desc(sw);
          const uint64_t tdesc = make_smem_desc(sw + kWBytes);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk)
            tc_mma(tmem_d, wdesc + (uint64_t)(kk * 2), tdesc + (uint64_t)(kk * 2), kIdesc,
                   (kb > kb0 || kk > 0) ? 1u : 0u);
          tc_commit(&ctl->empty[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(&ctl->tmem_full[a]);
        if (a == 1) acc_phase ^= 1u;
      }
    }
  } else {
    // ---------------- epilogue: thread r owns weight row r of the tile ----------------
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    uint32_t acc_phase = 0;
    int it = 0;
    int e = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x, ++it) {
      while (t >= ctl->tile_start[e + 1]) ++e;
      const int local = t - ctl->tile_start[e];
      const int ks = local % ksplit;
      const int rest = local / ksplit;
      const int tb = rest / n_tiles, nt = rest - tb * n_tiles;
      const int row0 = ctl->offsets[e] + tb * kTok;
      const int ntok = min(kTok, ctl->offsets[e + 1] - row0);
      const int a = it & 1;
      // feature this thread produces, and its bias (loaded before the wait)
      const int feat = GEGLU ? nt * 64 + (r & 63) : nt * 128 + r;
      const bool feat_ok = feat < Nout;
      float bias = 0.f;
      if (GEGLU && feat_ok) {
        const __nv_bfloat16* b = static_cast<const __nv_bfloat16*>(bias_ptrs[e]);
        bias = __bfloat162float(b[r < 64 ? feat : Nout + feat]);
      }
      if (!mbar_wait(&ctl->tmem_full[a], acc_phase, &ctl->abort, status, 14)) { ok = false; break; }
      tc_fence_after();
      uint32_t v[32];
      tc_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(a * kTok), v);
      tc_ld_wait();
      if (GEGLU) {
        float* up = ctl->up[a];
        if (r >= 64) {
#pragma unroll
          for (int c = 0; c < kTok; ++c) up[(r - 64) * kUpPitch + c] = __uint_as_float(v[c]) + bias;
          mbar_arrive(&ctl->up_ready[a]);
        } else if (!mbar_wait(&ctl->up_ready[a], acc_phase, &ctl->abort, status, 15)) {
          ok = false;
          break;
        }
        if (r < 64 && feat_ok) {
          __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out_raw) + (int64_t)row0 * Nout + feat;
#pragma unroll
          for (int c = 0; c < kTok; ++c) {
            if (c < ntok) {
              const float g = __uint_as_float(v[c]) + bias;
              o[(int64_t)c * Nout] = __float2bfloat16_rn(gelu_tanh_fast(g) * up[r * kUpPitch + c]);
            }
          }
        }
      } else if (feat_ok) {
        float* o = static_cast<float*>(out_raw) + (int64_t)ks * part_stride +
                   (int64_t)row0 * Nout + feat;
#pragma unroll
        for (int c = 0; c < kTok; ++c)
          if (c < ntok) o[(int64_t)c * Nout] = __uint_as_float(v[c]);
      }
      tc_fence_before();
      mbar_arrive(&ctl->tmem_empty[a]);
      if (a == 1) acc_phase ^= 1u;
    }
  }

  // ---------------- teardown ----------------
  __syncwarp();
  if (*reinterpret_cast<volatile int*>(&ctl->abort)) {
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

template <bool GEGLU>
int launch_one(const CUtensorMap& tm_tok, const void* tmap_w, const int32_t* offsets,
               const void* const* bias, int E, int K, int Nout, int ksplit, int64_t part_stride,
               void* out, int32_t* status, int sms, cudaStream_t s) {
  static bool attr_set = false;
  auto fn = decode_gemm_kernel<GEGLU>;
  if (!attr_set) {
    MOE_CUDA_CHECK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)kSmemBytes));
    attr_set = true;
  }
  MOE_CUDA_CHECK(launch_pdl(fn, dim3(sms), dim3(kThreads), kSmemBytes, s, tm_tok,
                            static_cast<const CUtensorMap*>(tmap_w), offsets, bias, E, K, Nout, ksplit,
                            part_stride, out, status));
  return 0;
}

}  // namespace

// K of the down product is cut into this many ranges (each at least 8 blocks of 64).
int decode_splits(int f) {
  const int kb = (f + BK - 1) / BK;
  int s = kb / 8;
  return s < 1 ? 1 : (s > 8 ? 8 : s);
}

int launch_experts_tc_decode(const void* perm, const int32_t* offsets, const void* plan, int64_t M,
                             int d, int f, int E, void* h, float* part, int32_t* status,
                             cudaStream_t s) {
  if (M == 0) return 0;
  PlanView pv = plan_view(plan, E);
  alignas(64) CUtensorMap tm_x, tm_h;
  int rc = encode_tmap_2d(&tm_x, perm, (uint64_t)M, (uint64_t)d, kTok);
  if (rc) return rc;
  rc = encode_tmap_2d(&tm_h, h, (uint64_t)M, (uint64_t)f, kTok);
  if (rc) return rc;
  int sms = 0;
  rc = sm_count(&sms);
  if (rc) return rc;
  rc = launch_one<true>(tm_x, pv.tmap_W1_dec, offsets, pv.b1, E, d, f, 1, 0, h, status, sms, s);
  if (rc) return rc;
  return launch_one<false>(tm_h, pv.tmap_W2_dec, offsets, pv.b2, E, f, d, decode_splits(f),
                           M * (int64_t)d, part, status, sms, s);
}

}  // namespace moe
