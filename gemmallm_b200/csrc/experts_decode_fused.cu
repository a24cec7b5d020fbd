// Small-N expert feed-forward, both products in ONE launch: the GEGLU tiles (128 weight
// rows = 64 gate + 64 up, as the A operand, against a block of up to 32 tokens as the B
// operand) and the split-K down tiles walked as one tile list by one persistent
// grid, so that the down pass's weight stream starts the moment a CTA runs out of
// GEGLU tiles instead of after a kernel boundary (launch, ramp, tail). A down tile
// needs the h rows of its 32-token block complete: every GEGLU tile, after its
// stores, adds one to ready[token block]; the producer of a down tile waits
// (bounded) until the count reaches the number of GEGLU tiles of that block, then
// orders those writes before its TMA reads with a proxy fence. GEGLU tiles wait
// for nothing and every CTA finishes its GEGLU tiles before its first down tile,
// so the waits always end provided the grid's CTAs are resident together (one CTA
// per SM, grid = SM count); if they are not, the bounded waits report
// MOE_B200_DEV_TIMEOUT instead of hanging (reference model.py:174,180-184).
#include <cuda.h>
#include "common.cuh"
#include "tc_ptx.cuh"

namespace moe {

namespace {

using namespace tc;

constexpr int BK = 64;
constexpr int kWRows = 128;
constexpr int kTok = 32;
constexpr int kStages = 9;
constexpr int kWBytes = kWRows * BK * 2;
constexpr int kWHalf = kWBytes / 2;
constexpr int kTBytes = kTok * BK * 2;
constexpr int kStageBytes = kWBytes + kTBytes;
constexpr int kThreads = 192;
constexpr int kTmemCols = 64;
constexpr uint32_t kIdesc = make_idesc(kTok);
constexpr int kUpPitch = kTok + 1;

struct Control {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t up_ready[2];
  uint64_t h_done[2];    // the 128 epilogue threads have stored (and fenced) a GEGLU tile
  uint32_t tmem_base;
  int abort;
  int tb_start[kMaxExperts + 1];   // prefix of 32-token blocks per expert
  int offsets[kMaxExperts + 1];
  float up[2][64 * kUpPitch];
};

constexpr size_t kSmemBytes = 1024 + (size_t)kStages * kStageBytes + sizeof(Control);

struct Tile {
  int e, row0, ntok, nt, ks, tbg;
  bool down;
};

// tile t: GEGLU tiles first, (token block, n tile) with n fastest; then down tiles,
// (token block, n tile, k range) with the k range fastest
__device__ __forceinline__ Tile decode_tile(const Control* ctl, int t, int E, int g1, int n1, int n2,
                                            int ksplit) {
  Tile ti;
  ti.down = t >= g1;
  int rest;
  if (!ti.down) {
    ti.ks = 0;
    ti.tbg = t / n1;
    ti.nt = t - ti.tbg * n1;
  } else {
    const int g = t - g1;
    ti.ks = g % ksplit;
    rest = g / ksplit;
    ti.tbg = rest / n2;
    ti.nt = rest - ti.tbg * n2;
  }
  int e = 0;
  while (e + 1 < E && ti.tbg >= ctl->tb_start[e + 1]) ++e;
  ti.e = e;
  ti.row0 = ctl->offsets[e] + (ti.tbg - ctl->tb_start[e]) * kTok;
  ti.ntok = min(kTok, ctl->offsets[e + 1] - ti.row0);
  return ti;
}

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(kThreads, 1)
decode_fused_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_h,
                    const CUtensorMap* __restrict__ tmap_w1, const CUtensorMap* __restrict__ tmap_w2,
                    const int32_t* __restrict__ offsets, const void* const* __restrict__ b1_ptrs,
                    const void* const* __restrict__ w1_ptrs, int spec_waves,
                    int E, int d, int f, int ksplit, int64_t part_stride,
                    __nv_bfloat16* __restrict__ h, float* __restrict__ part, int* __restrict__ ready,
                    int32_t* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~(uintptr_t)1023);
  Control* ctl = reinterpret_cast<Control*>(smem + (size_t)kStages * kStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n1 = (f + 63) / 64;        // GEGLU tiles per token block (64 features each)
  const int n2 = (d + 127) / 128;      // down n tiles per token block (128 features each)
  const int kb_all1 = (d + BK - 1) / BK;
  const int kb_all2 = (f + BK - 1) / BK;
  const int kb_per_split = (kb_all2 + ksplit - 1) / ksplit;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], 1); }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&ctl->tmem_full[a], 1);
      mbar_init(&ctl->tmem_empty[a], 128);
      mbar_init(&ctl->up_ready[a], 64);
      mbar_init(&ctl->h_done[a], 128);
    }
    ctl->abort = 0;
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
  // tensor maps into the descriptor cache: the plan is not written by earlier kernels
  if (warp == 2) {
    for (int e = lane; e < E; e += 32) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(tmap_w1 + e) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(tmap_w2 + e) : "memory");
    }
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_x) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_h) : "memory");
    }
  }
  // Speculation while the kernels before this one still run: if every expert gets
  // exactly one 32-row block, tile t is (expert t / n1, n tile t % n1), so this CTA's
  // first `spec_waves` GEGLU tiles are known before the routing is. Pull their weight
  // rows (two runs of 64 consecutive rows) into L2. A wrong guess costs bandwidth only.
  if (threadIdx.x == 96) {
    const size_t row_bytes = (size_t)d * 2;
    for (int w = 0; w < spec_waves; ++w) {
      const int t = (int)blockIdx.x + w * (int)gridDim.x;
      const int e = t / n1, nt = t - e * n1;
      if (e >= E) break;
      const char* W = static_cast<const char*>(w1_ptrs[e]);
      const int rows = min(64, f - nt * 64);
      for (int half = 0; half < 2; ++half) {
        const char* p = W + (size_t)(half * f + nt * 64) * row_bytes;
        const size_t bytes = (size_t)rows * row_bytes;
        for (size_t o = 0; o < bytes; o += 16384) {
          const uint32_t n = (uint32_t)min((size_t)16384, bytes - o);
          asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p + o), "r"(n) : "memory");
        }
      }
    }
  }
  // everything above is independent of the kernels before this one in the stream
  pdl_wait();
  pdl_launch_dependents();
  for (int e = threadIdx.x; e <= E; e += kThreads) ctl->offsets[e] = offsets[e];
  __syncthreads();
  if (warp == 0) {
    // 32-row blocks per expert, exclusive scan over the experts
    int carry = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + lane;
      const int nb = e < E ? (ctl->offsets[e + 1] - ctl->offsets[e] + kTok - 1) / kTok : 0;
      int incl = nb;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      if (e < E) ctl->tb_start[e] = carry + incl - nb;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) ctl->tb_start[E] = carry;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctl->tmem_base);
  const int token_blocks = ctl->tb_start[E];
  const int g1 = token_blocks * n1;
  const int total_tiles = g1 + token_blocks * n2 * ksplit;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        const Tile ti = decode_tile(ctl, t, E, g1, n1, n2, ksplit);
        const CUtensorMap* tw = (ti.down ? tmap_w2 : tmap_w1) + ti.e;
        const CUtensorMap* tt = ti.down ? &tmap_h : &tmap_x;
        const int w0 = ti.down ? ti.nt * 128 : ti.nt * 64;
        const int w1 = ti.down ? ti.nt * 128 + 64 : f + ti.nt * 64;
        const int kb0 = ti.down ? ti.ks * kb_per_split : 0;
        const int kb1 = ti.down ? min(kb_all2, kb0 + kb_per_split) : kb_all1;
        if (ti.down) {
          // the h rows of this token block must be complete (bounded wait), and visible to TMA
          const unsigned long long t0 = global_ns();
          for (uint32_t it = 0; ld_acquire_gpu(&ready[ti.tbg]) < n1; ++it) {
            if ((it & 63u) == 63u) {
              if (*reinterpret_cast<volatile int*>(&ctl->abort)) { ok = false; break; }
              if (global_ns() - t0 > kWaitLimitNs) {
                *reinterpret_cast<volatile int*>(&ctl->abort) = 1;
                atomicMax(&status[0], MOE_B200_DEV_TIMEOUT);
                status[1] = 16;
                ok = false;
                break;
              }
            }
          }
          if (!ok) break;
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&ctl->empty[stage], phase ^ 1u, &ctl->abort, status, 11)) { ok = false; break; }
          uint8_t* sw = smem + (size_t)stage * kStageBytes;
          mbar_expect_tx(&ctl->full[stage], kStageBytes);
          tma_load_2d(sw, tw, &ctl->full[stage], kb * BK, w0);
          tma_load_2d(sw + kWHalf, tw, &ctl->full[stage], kb * BK, w1);
          tma_load_2d(sw + kWBytes, tt, &ctl->full[stage], kb * BK, ti.row0);
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
        const bool down = t >= g1;
        const int ks = down ? (t - g1) % ksplit : 0;
        const int kb0 = down ? ks * kb_per_split : 0;
        const int kb1 = down ? min(kb_all2, kb0 + kb_per_split) : kb_all1;
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
    bool ok = true;
    for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x, ++it) {
      const Tile ti = decode_tile(ctl, t, E, g1, n1, n2, ksplit);
      const int a = it & 1;
      const int Nout = ti.down ? d : f;
      const int feat = ti.down ? ti.nt * 128 + r : ti.nt * 64 + (r & 63);
      const bool feat_ok = feat < Nout;
      float bias = 0.f;
      if (!ti.down && feat_ok) {
        const __nv_bfloat16* b = static_cast<const __nv_bfloat16*>(b1_ptrs[ti.e]);
        bias = __bfloat162float(b[r < 64 ? feat : f + feat]);
      }
      if (!mbar_wait(&ctl->tmem_full[a], acc_phase, &ctl->abort, status, 14)) { ok = false; break; }
      tc_fence_after();
      uint32_t v[32];
      tc_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(a * kTok), v);
      tc_ld_wait();
      if (!ti.down) {
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
          __nv_bfloat16* o = h + (int64_t)ti.row0 * f + feat;
#pragma unroll
          for (int c = 0; c < kTok; ++c) {
            if (c < ti.ntok) {
              const float g = __uint_as_float(v[c]) + bias;
              o[(int64_t)c * f] = __float2bfloat16_rn(gelu_tanh_fast(g) * up[r * kUpPitch + c]);
            }
          }
        }
        // publish: all 128 threads have stored and fenced, then one adds to the block's count
        __threadfence();
        mbar_arrive(&ctl->h_done[a]);
        if (r == 0) {
          if (!mbar_wait(&ctl->h_done[a], acc_phase, &ctl->abort, status, 17)) { ok = false; break; }
          __threadfence();
          atomicAdd(&ready[ti.tbg], 1);
        }
      } else if (feat_ok) {
        float* o = part + (int64_t)ti.ks * part_stride + (int64_t)ti.row0 * d + feat;
#pragma unroll
        for (int c = 0; c < kTok; ++c)
          if (c < ti.ntok) o[(int64_t)c * d] = __uint_as_float(v[c]);
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
  // The last CTA to get here leaves the counters zero for the next call on this workspace:
  // by then every CTA has read its last completion count.
  // A CTA that gave up on a wait counts too: the status word keeps the failure, the counters
  // are clean again for the next call.
  if (threadIdx.x == 0) {
    int* exit_count = ready + (MOE_B200_READY_INTS - 2);
    __threadfence();
    if (atomicAdd(exit_count, 1) == (int)gridDim.x - 1) {
      for (int i = 0; i < token_blocks; ++i) ready[i] = 0;
      *exit_count = 0;
    }
  }
}

}  // namespace

// K of the down product is cut into this many ranges (each at least 8 blocks of 64).
int decode_splits(int f) {
  const int kb = (f + BK - 1) / BK;
  int s = kb / 8;
  return s < 1 ? 1 : (s > 8 ? 8 : s);
}

// `ready`: int32 [MOE_B200_READY_INTS], zeroed by the caller before this launch.
int launch_experts_tc_decode_fused(const void* perm, const int32_t* offsets, const void* plan,
                                   int64_t M, int d, int f, int E, void* h, float* part, int* ready,
                                   int32_t* status, cudaStream_t s, int spec) {
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
  // weight rows pulled into L2 ahead of the routing: only when most experts are hit
  const int spec_waves = spec < 0 ? (M >= 4 * (int64_t)E ? 2 : (M >= E ? 1 : 0)) : spec;
  static PerDeviceOnce once;
  rc = ensure_dynamic_smem(once, decode_fused_kernel, kSmemBytes);
  if (rc) return rc;
  MOE_CUDA_CHECK(launch_pdl(decode_fused_kernel, dim3(sms), dim3(kThreads), kSmemBytes, s, tm_x, tm_h,
                            static_cast<const CUtensorMap*>(pv.tmap_W1_dec),
                            static_cast<const CUtensorMap*>(pv.tmap_W2_dec), offsets, pv.b1, pv.W1,
                            spec_waves, E, d, f,
                            decode_splits(f), M * (int64_t)d, static_cast<__nv_bfloat16*>(h), part,
                            ready, status));
  return 0;
}

}  // namespace moe
