// Epilogue of the 128-row x 256-column accumulator tile shared by the one-CTA and
// the CTA-pair grouped GEMM kernels: TMEM -> registers (one row per thread) ->
// bias (+ GeGLU) -> bf16 -> global memory.
#pragma once
#include "common.cuh"
#include "tc_ptx.cuh"

namespace moe {
namespace tc {

constexpr int kStgPitch = 144;  // bytes per staged row: 64 bf16 + 16 bytes pad

// taddr: TMEM address of this warp's 32 lanes, column 0 of the accumulator.
// row/row_ok: the sorted-buffer row this thread owns. stg: this warp's staging
// area (32 * kStgPitch bytes), used by SCATTER only.
//   GEGLU  : columns [0,128) gate, [128,256) up; writes 128 outputs per row.
//   plain  : writes 256 outputs per row.
//   SCATTER: plain, but the row goes to sc.ret_y[meta >> 24] + (meta & 0xffffff) * Nout
//            over NVLink; 64 columns per row are staged in shared memory so that 8
//            lanes write each row's 128 bytes as one run.
// half: two warps share each TMEM lane quadrant and split the tile's columns
// (half 0 the first half of the 32-column chunks, half 1 the rest); SCATTER is
// done by half 0 alone (its staging area is per quadrant).
template <bool GEGLU, bool SCATTER>
__device__ __forceinline__ void store_tile(uint32_t taddr, int row, bool row_ok, int n0, int Nout,
                                           const __nv_bfloat16* __restrict__ bias,
                                           __nv_bfloat16* __restrict__ out, const EpScatter& sc,
                                           uint8_t* stg, int lane, int half) {
  constexpr int BN = 256;
  constexpr int kTileN = GEGLU ? BN / 2 : BN;
  constexpr int kChunks = kTileN / 32;
  const int c_begin = SCATTER ? 0 : half * (kChunks / 2);
  const int c_end = SCATTER ? kChunks : c_begin + kChunks / 2;
  if (SCATTER && half != 0) return;
  __nv_bfloat16* orow = out + (int64_t)row * Nout + n0;
  if (SCATTER) {
    // Rows go to their token owners over NVLink. Registers hold one row per
    // thread; stage 64 columns per row in shared memory and let 8 lanes write
    // each row's 128 bytes, so that the peer stores are 128-byte runs.
    const int meta = row_ok ? __ldg(&sc.meta[row]) : -1;
    #pragma unroll 1
    for (int cp = c_begin / 2; cp < c_end / 2; ++cp) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int c = cp * 2 + half;
        uint32_t v[32];
        tc_ld32(taddr + c * 32, v);
        tc_ld_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int n = n0 + c * 32 + q * 8;
          float b[8], o[8];
          if (n < Nout) {
            load8_ldg(bias + n, b);
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) b[i] = 0.f;
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = __uint_as_float(v[q * 8 + i]) + b[i];
          store8(reinterpret_cast<__nv_bfloat16*>(stg + lane * kStgPitch + (half * 4 + q) * 16), o);
        }
      }
      __syncwarp();
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int rr = i * 4 + (lane >> 3), piece = lane & 7;
        const int m = __shfl_sync(0xffffffffu, meta, rr);
        const int n = n0 + cp * 64 + piece * 8;
        if (m >= 0 && n < Nout) {
          const uint4 val = *reinterpret_cast<const uint4*>(stg + rr * kStgPitch + piece * 16);
          *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(sc.ret_y[(m >> 24) & 7]) +
                                    (int64_t)(m & 0xffffff) * Nout + n) = val;
        }
      }
      __syncwarp();
    }
  } else if (GEGLU) {
#pragma unroll 1
    for (int c = c_begin; c < c_end; ++c) {
      uint32_t g[32], u[32];
      tc_ld32(taddr + c * 32, g);
      tc_ld32(taddr + BN / 2 + c * 32, u);
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
    for (int c = c_begin; c < c_end; ++c) {
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
}

}  // namespace tc
}  // namespace moe
