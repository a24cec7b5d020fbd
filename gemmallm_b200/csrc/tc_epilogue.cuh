// Epilogue of one CTA's 128-row x 256-column accumulator tile in the CTA-pair
// grouped GEMM kernel: TMEM -> registers (one row per thread) ->
// bias (+ GeGLU, + dropout in training mode) -> bf16 -> shared-memory staging ->
// global memory in 128-byte runs per row.
#pragma once
#include "common.cuh"
#include "tc_ptx.cuh"
#include "philox.cuh"

namespace moe {
namespace tc {

constexpr int kStgPitch = 144;               // bytes per staged row: 64 bf16 + 16 bytes pad
constexpr int kStgRows = 16;                 // half a warp's rows are staged at a time
constexpr int kStgBytes = kStgRows * kStgPitch;

// 64 output columns of this thread's row, as 8 x 16 bytes, go through this warp's staging
// area 16 rows at a time and leave as 128-byte runs (8 lanes per row, 4 rows per store
// instruction): an eighth of the memory requests a one-row-per-thread store would make,
// which compete with the TMA loads for the SM's path to L2, and the run length NVLink wants
// for the expert-parallel scatter. dst = this thread's row (nullptr: nothing to store),
// n = first column, Nlimit = number of valid columns of the row.
__device__ __forceinline__ void flush64(const uint4 (&packed)[8], __nv_bfloat16* dst, int n,
                                        int Nlimit, uint8_t* stg, int lane) {
#pragma unroll
  for (int hr = 0; hr < 2; ++hr) {
    if ((lane >> 4) == hr) {
#pragma unroll
      for (int q = 0; q < 8; ++q)
        *reinterpret_cast<uint4*>(stg + (lane & 15) * kStgPitch + q * 16) = packed[q];
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int rr = i * 4 + (lane >> 3), piece = lane & 7;
      __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(
          __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(dst), hr * 16 + rr));
      const int nn = n + piece * 8;
      if (d != nullptr && nn < Nlimit)
        *reinterpret_cast<uint4*>(d + nn) =
            *reinterpret_cast<const uint4*>(stg + rr * kStgPitch + piece * 16);
    }
    __syncwarp();
  }
}

__device__ __forceinline__ uint4 pack8(const float (&o)[8]) {
  return make_uint4(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]), pack_bf16x2(o[4], o[5]),
                    pack_bf16x2(o[6], o[7]));
}

//   taddr  : TMEM address of this warp's 32 lanes, column 0 of the accumulator
//   row    : sorted-buffer row this thread owns; row_ok: inside the expert's segment
//   half   : two warps share each TMEM lane quadrant and split the tile's columns
//   GEGLU  : columns [0,128) gate, [128,256) up; 128 outputs per row, 64 per warp
//   TRAIN  : GEGLU in training mode (see TrainArgs in common.cuh): gate/up pre-activations
//            are kept for the backward pass and h gets its dropout mask
//   plain  : 256 outputs per row, 128 per warp (two passes); bias may be nullptr (none)
//   SCATTER: plain, but the row goes to sc.ret_y[meta >> 24] + (meta & 0xffffff) * Nout
//            (the token owner's buffer, possibly on another GPU)
template <bool GEGLU, bool SCATTER, bool TRAIN>
__device__ __forceinline__ void store_tile(uint32_t taddr, int row, bool row_ok, int n0, int Nout,
                                           const __nv_bfloat16* __restrict__ bias,
                                           __nv_bfloat16* __restrict__ out, const EpScatter& sc,
                                           const TrainArgs& tr, uint8_t* stg, int lane, int half) {
  static_assert(!TRAIN || GEGLU, "training extras belong to the GEGLU pass");
  constexpr int BN = 256;
  constexpr int kTileN = GEGLU ? BN / 2 : BN;
  constexpr int kPasses = kTileN / 128;        // 64-column passes per warp
  // destination of this thread's row (nullptr: nothing to store)
  __nv_bfloat16* dst = nullptr;
  __nv_bfloat16* dst_gu = nullptr;
  uint32_t pair = 0;
  if (row_ok) {
    if (SCATTER) {
      const int meta = __ldg(&sc.meta[row]);
      dst = static_cast<__nv_bfloat16*>(sc.ret_y[(meta >> 24) & 7]) + (int64_t)(meta & 0xffffff) * Nout;
    } else {
      dst = out + (int64_t)row * Nout;
    }
    if (TRAIN) {
      dst_gu = tr.gu + (int64_t)row * 2 * Nout;
      pair = (uint32_t)__ldg(&tr.pair_of[row]);
    }
  }
#pragma unroll 1
  for (int p = 0; p < kPasses; ++p) {
    const int col0 = (half * kPasses + p) * 64;   // first output column of this pass inside the tile
    uint4 packed[8];
    uint4 packed_g[8], packed_u[8];   // training mode only (dead otherwise)
#pragma unroll
    for (int hc = 0; hc < 2; ++hc) {              // two 32-column chunks
      const int c = col0 / 32 + hc;
      uint32_t g[32];
      tc_ld32(taddr + c * 32, g);
      if (GEGLU) {
        uint32_t u[32];
        tc_ld32(taddr + BN / 2 + c * 32, u);
        tc_ld_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int n = n0 + c * 32 + q * 8;
          float bg[8], bu[8], o[8], gv[8], uv[8];
          if (n < Nout) {
            load8_ldg(bias + n, bg);
            load8_ldg(bias + Nout + n, bu);
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) bg[i] = bu[i] = 0.f;
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            gv[i] = __uint_as_float(g[q * 8 + i]) + bg[i];
            uv[i] = __uint_as_float(u[q * 8 + i]) + bu[i];
            o[i] = gelu_tanh_fast(gv[i]) * uv[i];
          }
          if (TRAIN) {
            packed_g[hc * 4 + q] = pack8(gv);
            packed_u[hc * 4 + q] = pack8(uv);
            if (tr.thresh != 0u) {
              // columns n .. n+7 of this pair: two Philox blocks of four words
#pragma unroll
              for (int b4 = 0; b4 < 2; ++b4) {
                const uint4 r = philox4x32_10((uint32_t)(n >> 2) + b4, pair, tr.seed_lo, tr.seed_hi);
                const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
                for (int i = 0; i < 4; ++i)
                  o[b4 * 4 + i] = w[i] >= tr.thresh ? o[b4 * 4 + i] * tr.scale : 0.f;
              }
            }
          }
          packed[hc * 4 + q] = pack8(o);
        }
      } else {
        tc_ld_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int n = n0 + c * 32 + q * 8;
          float b[8], o[8];
          if (bias != nullptr && n < Nout) {
            load8_ldg(bias + n, b);
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) b[i] = 0.f;
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = __uint_as_float(g[q * 8 + i]) + b[i];
          packed[hc * 4 + q] = pack8(o);
        }
      }
    }
    flush64(packed, dst, n0 + col0, Nout, stg, lane);
    if constexpr (TRAIN) {
      flush64(packed_g, dst_gu, n0 + col0, Nout, stg, lane);
      flush64(packed_u, dst_gu != nullptr ? dst_gu + Nout : nullptr, n0 + col0, Nout, stg, lane);
    }
  }
}

}  // namespace tc
}  // namespace moe
