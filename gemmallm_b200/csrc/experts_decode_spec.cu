// Small-N expert feed-forward that does not wait for the routing. With a few dozen
// tokens nearly every expert is hit, so the kernel streams the weights of ALL experts
// and multiplies them with ALL N tokens of the batch (N <= 128): nothing it loads
// depends on the routing, so it starts while the routing kernel before it in the
// stream is still running (programmatic dependent launch) and the routing latency
// disappears behind the weight stream. Only what is STORED depends on the routing,
// and that is known long before the first store that needs it.
// Operand roles: the tokens are the A operand (accumulator lane t = token t; only the
// first NP = 16/32/64/128 rows of the 128-row A tile are loaded, the other lanes
// compute on whatever the shared memory holds and are never read), the weights are
// the B operand with N = 256, so that one MMA consumes 8 KiB of weights at the tensor
// core's full rate (with the weights as the 128-row A operand and few token columns
// the MMA pipe, at about 160 cycles per 4 KiB, could not keep up with HBM).
//   GEGLU tile (e, 128 features): B = 128 gate rows and 128 up rows of
//     gate_and_up.weight, accumulator columns c and 128 + c; the epilogue thread of
//     token t writes h_all[e][t][...] = gelu_tanh(g + bg) * (u + bu) for the tokens
//     routed to expert e (reference model.py:174,180-182).
//   down tile (e, 256 features, K range): A = h_all[e] (lanes of tokens not routed to e
//     hold stale data and are never stored), B = 256 rows of down.weight. Partial sums
//     go to part[ks][row][d], row = the position the counting sort gives the (token,
//     expert) pair: offsets[e] + rank of the token among e's tokens; down tiles of
//     experts without tokens are skipped (model.py:184).
// One persistent CTA per SM. Tiles are claimed from a global counter (GEGLU tiles
// first, then down tiles, expert-major), so a CTA that starts late because the routing
// kernel still holds its SM simply takes fewer tiles; the claiming thread hands each
// tile to the MMA and epilogue warps through a small ring in shared memory. A down
// tile waits (bounded) until all GEGLU tiles of its expert have published their h
// rows; those were claimed earlier by CTAs that are running, so the waits end.
#include <cuda.h>
#include "common.cuh"
#include "tc_ptx.cuh"

namespace moe {

namespace {

using namespace tc;

constexpr int BK = 64;
constexpr int kBox = 128 * BK * 2;   // one 128-row weight box: 16 KiB
constexpr int kEpiThreads = 256;           // 8 epilogue warps: two per TMEM lane quadrant, half the columns each
constexpr int kThreads = 64 + kEpiThreads;
constexpr int kMaxStages = 6;
constexpr int kMaxE = 32;
constexpr int kSmemBudget = 220 * 1024;
constexpr int kRing = 4;

struct Control {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t h_done[2];     // the epilogue threads have stored (and fenced) a GEGLU tile
  uint64_t route_done;    // the epilogue threads have filled mask[] and offsets[]
  uint64_t ring_full[kRing];   // the claiming thread has written ring[slot]
  uint64_t ring_empty[kRing];  // the MMA thread and the epilogue threads have read it
  int ring[kRing];             // claimed tile ids, -1 = no more tiles
  uint32_t tmem_base;
  int abort;
  int offsets[kMaxExperts + 1];
  int tb_start[kMaxExperts + 1];   // SORTED: prefix of NP-row blocks per expert
  uint32_t mask[kMaxE][4];   // bit t of mask[e]: token t is routed to expert e
};

// SORTED variant: which expert a global row block belongs to (binary search in the prefix).
__device__ __forceinline__ int expert_of_block(const Control* ctl, int E, int u) {
  int lo = 0, hi = E;   // invariant: tb_start[lo] <= u < tb_start[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (ctl->tb_start[mid] <= u) lo = mid; else hi = mid;
  }
  return lo;
}


__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// SORTED = false: the kernel described at the top of this file (all tokens against every expert,
//   no wait for the routing). SORTED = true: the same pipeline on the rows the dispatch kernel has
//   sorted by expert, for calls too large for the first form: the unit of work is a block of NP
//   rows (32, 64 or 128) of one expert's segment (A = rows of perm, then of h [M,f]; lanes beyond the segment's end are
//   other experts' rows and are not stored), every role waits for the kernels before this one
//   first, and the partial sums go to part[ks][row][d] in the sorted order.
template <bool SORTED>
__global__ void __launch_bounds__(kThreads, 1)
decode_spec_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_h,
                   const CUtensorMap* __restrict__ tmap_w1, const CUtensorMap* __restrict__ tmap_w2,
                   const int32_t* __restrict__ offsets, const int32_t* __restrict__ idx,
                   const void* const* __restrict__ b1_ptrs, int N, int NP, int k, int E, int d, int f,
                   int ksplit, int64_t part_stride, int stages, int tmem_cols,
                   __nv_bfloat16* __restrict__ h_all, float* __restrict__ part, int* __restrict__ ready,
                   int32_t* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~(uintptr_t)1023);
  const int tok_bytes = NP * 128;
  const int stage_bytes = tok_bytes + 2 * kBox;   // [NP token rows][256 weight rows]
  Control* ctl = reinterpret_cast<Control*>(smem + (size_t)stages * stage_bytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n1 = (f + 127) / 128;   // GEGLU tiles per expert
  const int n2 = (d + 255) / 256;   // down n tiles per expert
  const int kb_all1 = (d + BK - 1) / BK;
  const int kb_all2 = (f + BK - 1) / BK;
  const int kb_per_split = (kb_all2 + ksplit - 1) / ksplit;
  constexpr uint32_t idesc = make_idesc(256);

  int* tile_counter = ready + (MOE_B200_READY_INTS - 1);

  // first tile: the claim is in flight while the barriers and the tensor memory are set up
  int first_tile = 0;
  if (threadIdx.x == 0) first_tile = atomicAdd(tile_counter, 1);
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], 1); }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&ctl->tmem_full[a], 1);
      mbar_init(&ctl->tmem_empty[a], kEpiThreads);
      mbar_init(&ctl->h_done[a], kEpiThreads);
    }
    mbar_init(&ctl->route_done, kEpiThreads);
    for (int i = 0; i < kRing; ++i) { mbar_init(&ctl->ring_full[i], 1); mbar_init(&ctl->ring_empty[i], kEpiThreads + 1); }
    ctl->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  for (int i = threadIdx.x; i < kMaxE * 4; i += kThreads) (&ctl->mask[0][0])[i] = 0u;
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&ctl->tmem_base)),
                 "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctl->tmem_base);
  if constexpr (SORTED) {
    // sorted rows and offsets come from the kernels before this one: wait, then the block table
    pdl_wait();
    for (int e = threadIdx.x; e <= E; e += kThreads) ctl->offsets[e] = __ldcg(&offsets[e]);
    __syncthreads();
    if (warp == 0) {
      int carry = 0;
      for (int e0 = 0; e0 < E; e0 += 32) {
        const int e = e0 + lane;
        const int nb = e < E ? (ctl->offsets[e + 1] - ctl->offsets[e] + NP - 1) / NP : 0;
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
    __syncthreads();
  }
  // SORTED = false: the routing kernel before this one signals its dependents only after it has
  // waited for ITS predecessor, so x is complete here; weights and biases are never written
  // by kernels of this library. Nothing below waits for the routing until it must.
  pdl_launch_dependents();
  const int U = SORTED ? ctl->tb_start[E] : E;     // units of work: row blocks, or experts
  const int T1 = U * n1;                           // GEGLU tiles
  const int total_tiles = T1 + U * n2 * ksplit;

  if (warp == 0) {
    // ---------------- tile claiming + TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int slot = 0;
      uint32_t rphase = 0;
      bool ok = true;
      bool routed = false;
      // The next tile is claimed while the last few stages of the current one are still to
      // be issued: late enough that nobody hoards tiles, early enough to hide the atomic.
      int t_cur = first_tile;
      int t_next = -1;
      int next_ready = 0;
      int cur_ready = 0;   // completion count of t_cur's expert as read one tile earlier
      auto claim_next = [&]() {
        t_next = atomicAdd(tile_counter, 1);
        next_ready = 0;
        if (t_next >= T1 && t_next < total_tiles) {
          // the completion count the next tile will need, read early (no ordering asked here)
          const int u_next = ((t_next - T1) / ksplit) / n2;
          asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(next_ready) : "l"(ready + u_next) : "memory");
        }
      };
      while (ok) {
        const int t = t_cur < total_tiles ? t_cur : -1;
        if (!SORTED && t >= T1) {
          // Down tiles of an expert without tokens are dropped here, by the one thread that
          // decides it; the other roles only ever see tiles that are processed. offsets[] is
          // written by the routing kernel while this kernel runs: wait for that kernel, and
          // read through L2 (the read-only path is for data constant over the kernel's life).
          if (!routed) { pdl_wait(); routed = true; }
          const int e = ((t - T1) / ksplit) / n2;
          if (__ldcg(&offsets[e + 1]) == __ldcg(&offsets[e])) {
            claim_next();
            t_cur = t_next;
            cur_ready = next_ready;
            continue;
          }
        }
        if (!mbar_wait(&ctl->ring_empty[slot], rphase ^ 1u, &ctl->abort, status, 29)) break;
        ctl->ring[slot] = t;
        mbar_arrive(&ctl->ring_full[slot]);
        if (++slot == kRing) { slot = 0; rphase ^= 1u; }
        if (t < 0) break;
        t_next = -1;
        if (t < T1) {
          const int u = t / n1, nt = t - u * n1;
          const int e = SORTED ? expert_of_block(ctl, E, u) : u;
          const int arow = SORTED ? ctl->offsets[e] + (u - ctl->tb_start[e]) * NP : 0;
          const CUtensorMap* tw = tmap_w1 + e;
          const int claim_kb = max(0, kb_all1 - 4);
          for (int kb = 0; kb < kb_all1; ++kb) {
            if (kb == claim_kb) claim_next();
            if (!mbar_wait(&ctl->empty[stage], phase ^ 1u, &ctl->abort, status, 21)) { ok = false; break; }
            uint8_t* sw = smem + (size_t)stage * stage_bytes;
            mbar_expect_tx(&ctl->full[stage], (uint32_t)stage_bytes);
            tma_load_2d(sw, &tmap_x, &ctl->full[stage], kb * BK, arow);
            tma_load_2d(sw + tok_bytes, tw, &ctl->full[stage], kb * BK, nt * 128);
            tma_load_2d(sw + tok_bytes + kBox, tw, &ctl->full[stage], kb * BK, f + nt * 128);
            if (++stage == stages) { stage = 0; phase ^= 1u; }
          }
        } else {
          const int j = t - T1;
          const int ks = j % ksplit;
          const int rest = j / ksplit;
          const int u = rest / n2, nt = rest - u * n2;
          const int e = SORTED ? expert_of_block(ctl, E, u) : u;
          const int arow = SORTED ? ctl->offsets[e] + (u - ctl->tb_start[e]) * NP : e * NP;
          {
            // the h rows of this unit must be complete (bounded wait), and visible to TMA
            if (cur_ready >= n1) {
              asm volatile("fence.acq_rel.gpu;" ::: "memory");
            } else {
              const unsigned long long t0 = global_ns();
              for (uint32_t it = 0; ld_acquire_gpu(&ready[u]) < n1; ++it) {
                if ((it & 63u) == 63u) {
                  if (*reinterpret_cast<volatile int*>(&ctl->abort)) { ok = false; break; }
                  if (global_ns() - t0 > kWaitLimitNs) {
                    *reinterpret_cast<volatile int*>(&ctl->abort) = 1;
                    atomicMax(&status[0], MOE_B200_DEV_TIMEOUT);
                    status[1] = 26;
                    status[2] = (int)blockIdx.x;
                    ok = false;
                    break;
                  }
                }
              }
              if (!ok) break;
            }
            asm volatile("fence.proxy.async;" ::: "memory");
            const CUtensorMap* tw = tmap_w2 + e;
            const int kb0 = ks * kb_per_split;
            const int kb1 = min(kb_all2, kb0 + kb_per_split);
            const int claim_kb = max(kb0, kb1 - 4);
            for (int kb = kb0; kb < kb1; ++kb) {
              if (kb == claim_kb) claim_next();
              if (!mbar_wait(&ctl->empty[stage], phase ^ 1u, &ctl->abort, status, 22)) { ok = false; break; }
              uint8_t* sw = smem + (size_t)stage * stage_bytes;
              mbar_expect_tx(&ctl->full[stage], (uint32_t)stage_bytes);
              tma_load_2d(sw, &tmap_h, &ctl->full[stage], kb * BK, arow);
              tma_load_2d(sw + tok_bytes, tw, &ctl->full[stage], kb * BK, nt * 256);
              tma_load_2d(sw + tok_bytes + kBox, tw, &ctl->full[stage], kb * BK, nt * 256 + 128);
              if (++stage == stages) { stage = 0; phase ^= 1u; }
            }
          }
        }
        if (t_next < 0) claim_next();   // tile skipped or without K blocks
        t_cur = t_next;
        cur_ready = next_ready;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase = 0;
      int slot = 0;
      uint32_t rphase = 0;
      int it = 0;
      bool ok = true;
      while (ok) {
        if (!mbar_wait(&ctl->ring_full[slot], rphase, &ctl->abort, status, 30)) break;
        const int t = *reinterpret_cast<volatile int*>(&ctl->ring[slot]);
        mbar_arrive(&ctl->ring_empty[slot]);
        if (++slot == kRing) { slot = 0; rphase ^= 1u; }
        if (t < 0) break;
        const bool down = t >= T1;
        int kb0 = 0, kb1 = kb_all1;
        if (down) {
          const int ks = (t - T1) % ksplit;
          kb0 = ks * kb_per_split;
          kb1 = min(kb_all2, kb0 + kb_per_split);
        }
        const int a = it & 1;
        if (!mbar_wait(&ctl->tmem_empty[a], acc_phase ^ 1u, &ctl->abort, status, 23)) { ok = false; break; }
        tc_fence_after();
        const uint32_t acc = tmem_base + (uint32_t)(a * 256);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&ctl->full[stage], phase, &ctl->abort, status, 24)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sw = smem_u32(smem + (size_t)stage * stage_bytes);
          // A: 128 token rows from the stage base (only NP of them loaded); B: 256 weight rows
          const uint64_t adesc = make_smem_desc(sw);
          const uint64_t bdesc = make_smem_desc(sw + (uint32_t)tok_bytes);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk)
            tc_mma(acc, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc,
                   (kb > kb0 || kk > 0) ? 1u : 0u);
          tc_commit(&ctl->empty[stage]);
          if (++stage == stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(&ctl->tmem_full[a]);
        if (a == 1) acc_phase ^= 1u;
        ++it;
      }
    }
  } else {
    // ---------------- epilogue: thread = token (accumulator lane), half of the columns ----------------
    const int quad = warp & 3;                 // TMEM lanes 32*quad .. +31 (fixed by the warp's index mod 4)
    const int half = (warp - 2) >> 2;          // which half of the tile's columns this warp handles
    const int r = quad * 32 + lane;            // token = accumulator lane
    const int et = threadIdx.x - 64;           // 0 .. kEpiThreads-1
    bool ok = true;
    uint32_t acc_phase = 0;
    int slot = 0;
    uint32_t rphase = 0;
    int it = 0;
    if constexpr (!SORTED) {
      // routing: wait for the routing kernel, then membership masks and offsets into shared memory
      // (written while this kernel runs, so read through L2, not through the read-only path)
      pdl_wait();
      for (int p = et; p < N * k; p += kEpiThreads) {
        const int e = __ldcg(&idx[p]);
        const int tok = p / k;
        if (e >= 0 && e < E) atomicOr(&ctl->mask[e][tok >> 5], 1u << (tok & 31));
      }
      for (int e = et; e <= E; e += kEpiThreads) ctl->offsets[e] = __ldcg(&offsets[e]);
      mbar_arrive(&ctl->route_done);
      ok = mbar_wait(&ctl->route_done, 0u, &ctl->abort, status, 27);
    }
    while (ok) {
      if (!mbar_wait(&ctl->ring_full[slot], rphase, &ctl->abort, status, 31)) break;
      const int t = *reinterpret_cast<volatile int*>(&ctl->ring[slot]);
      mbar_arrive(&ctl->ring_empty[slot]);
      if (++slot == kRing) { slot = 0; rphase ^= 1u; }
      if (t < 0) break;
      const bool down = t >= T1;
      int u, nt, ks = 0;     // unit of work: expert, or (SORTED) global row block
      if (!down) {
        u = t / n1;
        nt = t - u * n1;
      } else {
        const int j = t - T1;
        ks = j % ksplit;
        const int rest = j / ksplit;
        u = rest / n2;
        nt = rest - u * n2;
      }
      const int e = SORTED ? expert_of_block(ctl, E, u) : u;
      const int a = it & 1;
      // this thread's token (accumulator lane) and whether its result is stored: routed to expert
      // e, or (SORTED) a row of this block, which ends where the expert's segment ends
      int row0 = 0;
      uint32_t mword;        // the warp's lanes 32*quad .. +31
      if constexpr (SORTED) {
        row0 = ctl->offsets[e] + (u - ctl->tb_start[e]) * NP;
        const int left = min(NP, ctl->offsets[e + 1] - row0) - quad * 32;
        mword = left >= 32 ? 0xffffffffu : (left > 0 ? (1u << left) - 1u : 0u);
      } else {
        mword = ctl->mask[e][quad];
      }
      const bool routed_here = (mword >> lane) & 1u;
      // GEGLU biases of this warp's 64 features, fetched before the accumulator is awaited: lane l
      // keeps features l and 32 + l of the half; the loop below hands them round with shuffles
      float bgv[2] = {0.f, 0.f}, buv[2] = {0.f, 0.f};
      if (!down && mword != 0u) {
        const __nv_bfloat16* bias = static_cast<const __nv_bfloat16*>(b1_ptrs[e]);
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          const int feat = nt * 128 + (half * 2 + ch) * 32 + lane;
          if (feat < f) {
            bgv[ch] = __bfloat162float(__ldg(bias + feat));
            buv[ch] = __bfloat162float(__ldg(bias + f + feat));
          }
        }
      }
      if (!mbar_wait(&ctl->tmem_full[a], acc_phase, &ctl->abort, status, 25)) { ok = false; break; }
      tc_fence_after();
      const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(a * 256);
      if (!down) {
        if (mword != 0u) {       // uniform over the warp
          const int n0 = nt * 128;
          __nv_bfloat16* o = h_all + (SORTED ? (int64_t)(row0 + r) : (int64_t)e * NP + r) * f + n0;
          // rolled: half the code, and this code runs from a cold instruction cache the first time
#pragma unroll 1
          for (int ch = 0; ch < 2; ++ch) {
            const int c0 = (half * 2 + ch) * 32;
            const float bgc = ch ? bgv[1] : bgv[0], buc = ch ? buv[1] : buv[0];
            uint32_t g[32], u[32];
            tc_ld32(lane_addr + (uint32_t)c0, g);
            tc_ld32(lane_addr + (uint32_t)(128 + c0), u);
            tc_ld_wait();
#pragma unroll
            for (int c8 = 0; c8 < 32; c8 += 8) {
              float hv[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float gv = __uint_as_float(g[c8 + i]) + __shfl_sync(0xffffffffu, bgc, c8 + i);
                const float uv = __uint_as_float(u[c8 + i]) + __shfl_sync(0xffffffffu, buc, c8 + i);
                hv[i] = gelu_tanh_fast(gv) * uv;
              }
              if (routed_here && n0 + c0 + c8 < f) store8(o + c0 + c8, hv);   // f is a multiple of 8
            }
          }
        }
        // publish: all epilogue threads have stored and fenced, then one adds to the expert's count
        __threadfence();
        mbar_arrive(&ctl->h_done[a]);
        if (et == 0) {
          if (!mbar_wait(&ctl->h_done[a], acc_phase, &ctl->abort, status, 28)) { ok = false; break; }
          __threadfence();
          atomicAdd(&ready[u], 1);
        }
      } else if (mword != 0u) {
        const int n0 = nt * 256;
        int row;
        if constexpr (SORTED) {
          row = row0 + r;
        } else {
          row = ctl->offsets[e] + __popc(mword & ((1u << lane) - 1u));
          for (int w = 0; w < quad; ++w) row += __popc(ctl->mask[e][w]);
        }
        float* o = part + (int64_t)ks * part_stride + (int64_t)row * d + n0;
#pragma unroll 1
        for (int c0 = half * 128; c0 < half * 128 + 128; c0 += 32) {
          uint32_t v[32];
          tc_ld32(lane_addr + (uint32_t)c0, v);
          tc_ld_wait();
          if (routed_here) {
#pragma unroll
            for (int c4 = 0; c4 < 32; c4 += 4) {
              if (n0 + c0 + c4 < d) {      // d is a multiple of 8
                *reinterpret_cast<float4*>(o + c0 + c4) =
                    make_float4(__uint_as_float(v[c4]), __uint_as_float(v[c4 + 1]),
                                __uint_as_float(v[c4 + 2]), __uint_as_float(v[c4 + 3]));
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&ctl->tmem_empty[a]);
      if (a == 1) acc_phase ^= 1u;
      ++it;
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
                 "r"(tmem_cols)
                 : "memory");
  }
  // The last CTA to get here leaves the counters zero for the next call on this workspace:
  // by then every CTA has made its last claim and read its last completion count.
  // A CTA that gave up on a wait counts too: the status word keeps the failure, the counters
  // are clean again for the next call.
  if (threadIdx.x == 0) {
    int* exit_count = ready + (MOE_B200_READY_INTS - 2);
    __threadfence();
    if (atomicAdd(exit_count, 1) == (int)gridDim.x - 1) {
      for (int i = 0; i < U; ++i) ready[i] = 0;
      *tile_counter = 0;
      *exit_count = 0;
    }
  }
}

}  // namespace

// token rows padded to the MMA's N granularity: 16, 32, 64 or 128
int decode_spec_rows(int64_t N) { return N <= 16 ? 16 : N <= 32 ? 32 : N <= 64 ? 64 : 128; }

bool decode_spec_supported(int64_t N, int E, int k) {
  return N >= 1 && N <= 128 && E <= kMaxE && N * k <= kDecodeMaxRows;
}

// `ready`: int32 [MOE_B200_READY_INTS], zeroed by the caller before this launch: one completion
// count per expert, and the tile counter in the last word. h_all: bf16 [E][NP][f].
int launch_experts_tc_decode_spec(const void* x, const int32_t* idx, const int32_t* offsets,
                                  const void* plan, int64_t N, int k, int d, int f, int E, void* h_all,
                                  float* part, int* ready, int32_t* status, cudaStream_t s) {
  if (N == 0) return 0;
  const int NP = decode_spec_rows(N);
  PlanView pv = plan_view(plan, E);
  alignas(64) CUtensorMap tm_x, tm_h;
  int rc = encode_tmap_2d(&tm_x, x, (uint64_t)N, (uint64_t)d, (uint32_t)NP);
  if (rc) return rc;
  rc = encode_tmap_2d(&tm_h, h_all, (uint64_t)E * NP, (uint64_t)f, (uint32_t)NP);
  if (rc) return rc;
  int sms = 0;
  rc = sm_count(&sms);
  if (rc) return rc;
  const int stage_bytes = 2 * kBox + NP * 128;
  int stages = (kSmemBudget - (int)sizeof(Control) - 1024) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  const size_t smem = 1024 + (size_t)stages * stage_bytes + sizeof(Control);
  const int tmem_cols = 512;   // two accumulators of 256 columns
  static PerDeviceOnce once;
  rc = ensure_dynamic_smem(once, decode_spec_kernel<false>, kSmemBudget);
  if (rc) return rc;
  MOE_CUDA_CHECK(launch_pdl(decode_spec_kernel<false>, dim3(sms), dim3(kThreads), smem, s, tm_x, tm_h,
                            static_cast<const CUtensorMap*>(pv.tmap_W1),
                            static_cast<const CUtensorMap*>(pv.tmap_W2), offsets, idx, pv.b1, (int)N, NP,
                            k, E, d, f, decode_splits(f), N * (int64_t)k * d, stages, tmem_cols,
                            static_cast<__nv_bfloat16*>(h_all), part, ready, status));
  return 0;
}

// Rows-sorted form for calls between the decode and the prefill sizes. Rows per block: the
// smallest of 32, 64, 128 that holds one and a half times an expert's share under balanced
// routing (fewer token bytes per stage; a segment that is larger still takes several blocks, and
// streams its expert's weights once per block).
int rows_block(int64_t M, int E) {
  const int64_t share = (3 * ((M + E - 1) / E) + 1) / 2;
  return share <= 32 ? 32 : share <= 64 ? 64 : 128;
}

// K ranges of the down product: about one wave of CTAs' worth of tiles, given at least
// max(ceil(M / block), min(E, M)) row blocks; each range at least 8 blocks of 64. More ranges
// only add partial sums to write and read back (measured at d=1024, f=4096, E=8: 4 ranges are
// best at 512 and 1024 rows, 2 at 2048, 1 or 2 at 4096).
int rows_splits(int64_t M, int d, int f, int E) {
  const int NP = rows_block(M, E);
  int64_t blocks = (M + NP - 1) / NP;
  const int64_t hit = M < E ? M : E;
  if (blocks < hit) blocks = hit;
  const int64_t tiles = blocks * ((d + 255) / 256);
  int64_t want = kNumSMs / tiles;
  const int kb = (f + BK - 1) / BK;
  if (want > kb / 8) want = kb / 8;
  if (want > 8) want = 8;
  return want < 1 ? 1 : (int)want;
}

// Every row block of an expert's segment needs one completion counter.
bool rows_supported(int64_t M, int E) {
  return M > 0 && E >= 1 && E <= kMaxExperts &&
         (M + rows_block(M, E) - 1) / rows_block(M, E) + E <= MOE_B200_READY_INTS - 8;
}

// perm [M,d] sorted by expert, offsets [E+1]; h [M,f] and part [ksplit][M][d] are written.
// `ready` as for launch_experts_tc_decode_spec.
int launch_experts_tc_rows(const void* perm, const int32_t* offsets, const void* plan, int64_t M,
                           int d, int f, int E, int ksplit, void* h, float* part, int* ready,
                           int32_t* status, cudaStream_t s) {
  if (M == 0) return 0;
  const int NP = rows_block(M, E);
  PlanView pv = plan_view(plan, E);
  alignas(64) CUtensorMap tm_x, tm_h;
  int rc = encode_tmap_2d(&tm_x, perm, (uint64_t)M, (uint64_t)d, (uint32_t)NP);
  if (rc) return rc;
  rc = encode_tmap_2d(&tm_h, h, (uint64_t)M, (uint64_t)f, (uint32_t)NP);
  if (rc) return rc;
  int sms = 0;
  rc = sm_count(&sms);
  if (rc) return rc;
  const int stage_bytes = 2 * kBox + NP * 128;
  int stages = (kSmemBudget - (int)sizeof(Control) - 1024) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  const size_t smem = 1024 + (size_t)stages * stage_bytes + sizeof(Control);
  static PerDeviceOnce once;
  rc = ensure_dynamic_smem(once, decode_spec_kernel<true>, kSmemBudget);
  if (rc) return rc;
  MOE_CUDA_CHECK(launch_pdl(decode_spec_kernel<true>, dim3(sms), dim3(kThreads), smem, s, tm_x, tm_h,
                            static_cast<const CUtensorMap*>(pv.tmap_W1),
                            static_cast<const CUtensorMap*>(pv.tmap_W2), offsets,
                            static_cast<const int32_t*>(nullptr), pv.b1, (int)0, NP, 1, E, d, f, ksplit,
                            M * (int64_t)d, stages, 512, static_cast<__nv_bfloat16*>(h), part, ready,
                            status));
  return 0;
}

}  // namespace moe
