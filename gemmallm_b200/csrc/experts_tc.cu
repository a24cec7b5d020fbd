// Expert feed-forward on the 5th-generation tensor cores (tcgen05 + TMEM),
// bf16 operands, fp32 accumulation. Two launches of one persistent kernel:
//   GEGLU pass : h = gelu_tanh(x W1[:f]^T + b1[:f]) * (x W1[f:]^T + b1[f:])
//                (reference model.py:174,180-182), gate and up tiles side by
//                side in one 128x256 accumulator, activation in the epilogue;
//   plain pass : y = h W2^T + b2 (model.py:184).
// Experts are grouped by the row offsets the dispatch kernel wrote; nothing is
// read back to the host, every CTA derives the tile list from the offsets.
//
// One CTA per SM, 192 threads:
//   warp 0   : TMA producer  (cp.async.bulk.tensor, 128-byte swizzle, 4 stages)
//   warp 1   : MMA issuer    (tcgen05.mma cta_group::1 kind::f16, M=128 N=256 K=16)
//   warps 2-5: epilogue      (tcgen05.ld 32 lanes x 32 columns, bias, GeGLU, store)
// The 512 TMEM columns hold two 128x256 fp32 accumulators, so the epilogue of
// one tile runs under the main loop of the next. No TMA load uses cluster
// multicast. Every wait is bounded: when one runs out the CTA records
// MOE_B200_DEV_TIMEOUT in the status word, stops issuing, frees its TMEM and
// returns.
#include <cuda.h>
#include "common.cuh"

namespace moe {

namespace {

constexpr int BM = 128;          // rows of the sorted buffer per tile
constexpr int BK = 64;           // bf16 elements = one 128-byte swizzle row
constexpr int BNB = 256;         // B rows per tile (gate 128 + up 128, or 256 plain)
constexpr int kStages = 4;
constexpr int kABytes = BM * BK * 2;          // 16 KiB
constexpr int kBHalfBytes = 128 * BK * 2;     // 16 KiB
constexpr int kStageBytes = kABytes + 2 * kBHalfBytes;
constexpr int kThreads = 192;
constexpr int kTmemCols = 512;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s

struct Control {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort;
  int tile_start[kMaxExperts + 1];
};

constexpr size_t kSmemBytes = 1024 + (size_t)kStages * kStageBytes + sizeof(Control);

// ---- PTX wrappers ---------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait. False when the limit passed or another role gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, Control* ctl,
                                          int32_t* status, int where) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0 = global_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 0) {
      if (*reinterpret_cast<volatile int*>(&ctl->abort)) return false;
      if (global_ns() - t0 > kWaitLimitNs) {
        *reinterpret_cast<volatile int*>(&ctl->abort) = 1;
        atomicMax(&status[0], MOE_B200_DEV_TIMEOUT);
        status[1] = where;
        status[2] = (int)blockIdx.x;
        return false;
      }
    }
  }
}
__device__ __forceinline__ void tma_load_2d(void* dst, const void* tmap, uint64_t* bar, int c0,
                                            int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0),
      "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, one 128 x 256 x 16 step
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32"
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15,"
      " %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31},"
      " [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tc_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows 128
// bytes apart, 8-row groups 1024 bytes apart (SBO), version 1.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t desc = 0;
  desc |= (uint64_t)((saddr & 0x3ffffu) >> 4);   // bits [0,14)  start address / 16
  desc |= (uint64_t)1 << 16;                     // bits [16,30) leading byte offset / 16 (unused)
  desc |= (uint64_t)(1024 >> 4) << 32;           // bits [32,46) stride byte offset / 16
  desc |= (uint64_t)1 << 46;                     // bits [46,48) descriptor version
  desc |= (uint64_t)2 << 61;                     // bits [61,64) SWIZZLE_128B
  return desc;
}
// Instruction descriptor: fp32 accumulate, bf16 x bf16, both K-major, M=128, N=256.
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((256u >> 3) << 17) |
                            ((128u >> 4) << 24);

template <bool GEGLU>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a,
                       const CUtensorMap* __restrict__ tmap_b,  // [E], global memory
                       const int32_t* __restrict__ offsets,
                       const void* const* __restrict__ bias_ptrs, int E, int K, int Nout,
                       __nv_bfloat16* __restrict__ out, int32_t* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~(uintptr_t)1023);
  Control* ctl = reinterpret_cast<Control*>(smem + (size_t)kStages * kStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr int kTileN = GEGLU ? 128 : 256;  // output columns per tile
  const int n_tiles = (Nout + kTileN - 1) / kTileN;
  const int k_blocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&ctl->tmem_full[a], 1); mbar_init(&ctl->tmem_empty[a], 128); }
    ctl->abort = 0;
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      ctl->tile_start[e] = acc;
      int cnt = offsets[e + 1] - offsets[e];
      acc += ((cnt + BM - 1) / BM) * n_tiles;
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
        const int row0 = offsets[e] + mt * BM;
        const int b0 = nt * kTileN;
        const int b1 = GEGLU ? Nout + nt * kTileN : nt * kTileN + 128;
        const CUtensorMap* tb = tmap_b + e;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&ctl->empty[stage], phase ^ 1u, ctl, status, 1)) { ok = false; break; }
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
        if (!mbar_wait(&ctl->tmem_empty[a], acc_phase ^ 1u, ctl, status, 2)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)a * 256u;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&ctl->full[stage], phase, ctl, status, 3)) { ok = false; break; }
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
    const int r = quad * 32 + lane;
    uint32_t acc_phase = 0;
    int it = 0;
    int e = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x, ++it) {
      while (t >= ctl->tile_start[e + 1]) ++e;
      const int local = t - ctl->tile_start[e];
      const int mt = local / n_tiles, nt = local - mt * n_tiles;
      const int seg_beg = offsets[e], seg_end = offsets[e + 1];
      const int row = seg_beg + mt * BM + r;
      const bool row_ok = row < seg_end;
      const int n0 = nt * kTileN;
      const __nv_bfloat16* bias = static_cast<const __nv_bfloat16*>(bias_ptrs[e]);
      const int a = it & 1;
      if (!mbar_wait(&ctl->tmem_full[a], acc_phase, ctl, status, 4)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)a * 256u;
      __nv_bfloat16* orow = out + (int64_t)row * Nout + n0;
      if (GEGLU) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t g[32], u[32];
          tc_ld32(taddr + c * 32, g);
          tc_ld32(taddr + 128 + c * 32, u);
          tc_ld_wait();
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int n = n0 + c * 32 + q * 8;
            if (n < Nout) {
              float bg[8], bu[8], o[8];
              load8_ldg(bias + n, bg);
              load8_ldg(bias + Nout + n, bu);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                float gv = __uint_as_float(g[q * 8 + i]) + bg[i];
                float uv = __uint_as_float(u[q * 8 + i]) + bu[i];
                o[i] = gelu_tanh_fast(gv) * uv;
              }
              if (row_ok) store8(orow + c * 32 + q * 8, o);
            }
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          uint32_t v[32];
          tc_ld32(taddr + c * 32, v);
          tc_ld_wait();
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int n = n0 + c * 32 + q * 8;
            if (n < Nout) {
              float b[8], o[8];
              load8_ldg(bias + n, b);
#pragma unroll
              for (int i = 0; i < 8; ++i) o[i] = __uint_as_float(v[q * 8 + i]) + b[i];
              if (row_ok) store8(orow + c * 32 + q * 8, o);
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&ctl->tmem_empty[a]);
      if (a == 1) acc_phase ^= 1u;
    }
  }

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

// ---- host side --------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      (void)cudaGetLastError();
  }
  return fn;
}

// [rows, cols] row-major bf16, box = 128 rows x 64 columns, 128-byte swizzle.
int encode_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return set_error(MOE_B200_ERR_DRIVER, "cuTensorMapEncodeTiled unavailable");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {BK, 128};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                   strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(MOE_B200_ERR_DRIVER, "cuTensorMapEncodeTiled failed");
  return 0;
}

bool g_attr_set = false;

}  // namespace

int build_weight_tensor_maps(const void* const* h_W1, const void* const* h_W2, int E, int d, int f,
                             void* h_tmaps) {
  static_assert(sizeof(CUtensorMap) == 128, "tensor map size");
  CUtensorMap* maps = static_cast<CUtensorMap*>(h_tmaps);
  for (int e = 0; e < E; ++e) {
    int rc = encode_2d(&maps[e], h_W1[e], (uint64_t)2 * f, (uint64_t)d);
    if (rc) return rc;
    rc = encode_2d(&maps[E + e], h_W2[e], (uint64_t)d, (uint64_t)f);
    if (rc) return rc;
  }
  return 0;
}

int launch_experts_tc(const void* perm, const int32_t* offsets, const void* plan, int64_t M, int d,
                      int f, int E, void* h, void* y, int32_t* status, cudaStream_t s) {
  if (M == 0) return 0;
  if (!g_attr_set) {
    MOE_CUDA_CHECK(cudaFuncSetAttribute(grouped_gemm_tc_kernel<true>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)kSmemBytes));
    MOE_CUDA_CHECK(cudaFuncSetAttribute(grouped_gemm_tc_kernel<false>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)kSmemBytes));
    g_attr_set = true;
  }
  PlanView pv = plan_view(plan, E);
  alignas(64) CUtensorMap tm_x, tm_h;
  int rc = encode_2d(&tm_x, perm, (uint64_t)M, (uint64_t)d);
  if (rc) return rc;
  rc = encode_2d(&tm_h, h, (uint64_t)M, (uint64_t)f);
  if (rc) return rc;
  int dev = 0, sms = 0;
  MOE_CUDA_CHECK(cudaGetDevice(&dev));
  MOE_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  grouped_gemm_tc_kernel<true><<<sms, kThreads, kSmemBytes, s>>>(
      tm_x, static_cast<const CUtensorMap*>(pv.tmap_W1), offsets, pv.b1, E, d, f,
      static_cast<__nv_bfloat16*>(h), status);
  MOE_CUDA_CHECK(cudaGetLastError());
  grouped_gemm_tc_kernel<false><<<sms, kThreads, kSmemBytes, s>>>(
      tm_h, static_cast<const CUtensorMap*>(pv.tmap_W2), offsets, pv.b2, E, f, d,
      static_cast<__nv_bfloat16*>(y), status);
  MOE_CUDA_CHECK(cudaGetLastError());
  return 0;
}

}  // namespace moe
