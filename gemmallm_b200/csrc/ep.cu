// Expert-parallel exchange kernels: the dispatch and combine of the block as an
// all-to-all written with plain NVLink peer stores (no NCCL on the data path, no
// multicast, no TMA on remote memory).
//
// Tokens are sharded over the G ranks (rank r owns N_local tokens), experts are
// owned by ranks (optionally replicated, see ep_dispatch_kernel); the router runs
// replicated on local tokens.
// Every rank has one "symmetric" buffer of identical layout that its peers can
// write. Per forward (the call's epoch is a device-side counter that ep_begin_kernel
// advances, so the whole call can be captured in a CUDA graph and replayed):
//   0. ep_begin_kernel: epoch += 1, status words and the completion counter cleared.
//   1. ep_dispatch_kernel (cooperative): per-expert counts of the local
//      (token, slot) pairs, published to every rank's cnt_all[r] together with
//      the slot-0 counts and the softmax sums the loss needs; waits for all G
//      rows; derives the row every pair gets in its destination's receive
//      buffer (rows of one expert contiguous, ordered by source rank then
//      token, so the layout is deterministic); pushes the token rows and a
//      return address (source rank, pair id) with 16-byte peer stores; raises
//      flag X on every destination.
//   2. The grouped GEMMs (experts_tc2.cu) wait for flag X from every source at their
//      head and run on the receive buffer. The down pass stores its output rows
//      straight into the token owners' ret_y through peer pointers (scatter
//      epilogue), so the return transfer overlaps the math tile by tile; its last
//      block raises flag Y on every rank.
//   3. The combine kernel waits for flag Y from every owner at its head and reads
//      ret_y in (token, slot) order.
// Every wait on a peer's flag is bounded (2 s) and reports
// MOE_B200_DEV_TIMEOUT through the status word instead of hanging.
// Replaces, for the sharded configuration, reference model.py:226-268.
#include <cooperative_groups.h>
#include <stdio.h>
#include "common.cuh"
#include "ep_sync.cuh"

namespace cg = cooperative_groups;

namespace moe {

namespace {

constexpr int kThreads = 256;
constexpr int kChunk = kDispatchChunk;
constexpr int kEpGroupBlocks = 16;                                   // blocks per group of the two-level prefix
constexpr int kEpGroups = (kNumSMs * 2 + kEpGroupBlocks - 1) / kEpGroupBlocks;
using epsync::ld_acquire_sys;
using epsync::st_release_sys;
using epsync::wait_flag;

// Experts are addressed by "virtual" ids: vmap[e * world + source rank] is the
// virtual expert that rank's pairs for expert e go to, and owner[v] the rank that
// runs it. Without replication v == e. A popular expert can be given several
// virtual ids owned by different ranks (same weights on each): every source rank
// then sends its rows for that expert to one replica, which spreads the expert's
// load and keeps part of its rows off NVLink. E counts real experts (routing
// indices, loss); EV virtual experts (counts, layout).
__global__ void __launch_bounds__(kThreads)
ep_dispatch_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ idx, int64_t N, int row_pieces,
                   int E, int EV, int k, EpPeers peers, int rank, int world,
                   const uint32_t* __restrict__ epoch_ptr,
                   const int32_t* __restrict__ owner, const int32_t* __restrict__ vmap,
                   int32_t* __restrict__ scratch, const float* __restrict__ psum_part,
                   int64_t router_blocks, int32_t* __restrict__ cnt_slot0,
                   float* __restrict__ psum_global, int32_t* __restrict__ offsets_local,
                   float* __restrict__ aux, int64_t n_total, int32_t* __restrict__ status, int split) {
  cg::grid_group grid = cg::this_grid();
  const uint32_t epoch = *reinterpret_cast<const volatile uint32_t*>(epoch_ptr);
  extern __shared__ int s_int[];
  // destination of every (token, slot) pair of the chunk in hand: address of its row at the owner
  unsigned long long* s_dst = reinterpret_cast<unsigned long long*>(s_int);   // [kChunk*k]
  int* s_hist = s_int + 2 * kChunk * k; // [EV] local totals per virtual expert
  int* s_base = s_hist + EV;            // [EV] local rows of earlier chunks
  int* s_dest = s_base + EV;            // [EV] first row of (this rank, virtual expert) at its owner
  int* s_run = s_dest + EV;             // [EV]
  int* s_owner = s_run + EV;            // [EV]
  int* s_vmap = s_owner + EV;           // [E]  virtual expert of real expert e for this source rank
  int* s_slot0 = s_vmap + E;            // [E]  slot-0 histogram (real experts)
  int* s_cnt = s_slot0 + E;             // [world][EV] pair counts of every source rank
  float* s_red = reinterpret_cast<float*>(s_cnt + world * EV);  // [kThreads]
  __shared__ int s_fail;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = gridDim.x;
  const int64_t nchunk = (N + kChunk - 1) / kChunk;
  // scratch: the two accumulators that ep_begin_kernel zeroes come first
  int32_t* grp_cnt = scratch;                                   // [kEpGroups][EV] pair counts per group of 16 blocks
  int32_t* cnt0_acc = grp_cnt + kEpGroups * EV;                 // [E] slot-0 counts of this rank
  float* psum_local = reinterpret_cast<float*>(cnt0_acc + E);   // [E] probability sums of this rank
  int32_t* blk_cnt = cnt0_acc + 2 * E;                          // [G][EV] pair counts per block
  int32_t* chunk_cnt = blk_cnt + (size_t)kNumSMs * 2 * EV;      // [nchunk][EV]
  const int row_ints = EV + 2 * E;                    // published row: pair counts, slot-0 counts, psum bits

  // ---- phase 1: per-chunk histograms --------------------------------------
  // the tables come from the workspace (moe_b200_ep_setup): an entry outside its range would
  // turn into a wild peer store, so it is clamped and reported instead
  if (tid == 0) s_fail = 0;
  for (int v = tid; v < EV; v += kThreads) {
    int o = owner[v];
    if ((unsigned)o >= (unsigned)world) { atomicMax(&status[0], MOE_B200_DEV_BAD_INDEX); o = rank; }
    s_owner[v] = o;
  }
  for (int v = tid; v < EV; v += kThreads) s_base[v] = 0;
  for (int e = tid; e < E; e += kThreads) {
    s_slot0[e] = 0;
    int v = vmap[e * world + rank];
    if ((unsigned)v >= (unsigned)EV) { atomicMax(&status[0], MOE_B200_DEV_BAD_INDEX); v = 0; }
    s_vmap[e] = v;
  }
  __syncthreads();
  // work is dealt in contiguous ranges: chunks for the histograms, (chunk, part of the row)
  // units for the copies, so that a call with fewer chunks than blocks still uses the grid
  const int64_t h_first = nchunk * blockIdx.x / G, h_end = nchunk * (blockIdx.x + 1) / G;
  const int64_t units = nchunk * split;
  const int64_t u_first = units * blockIdx.x / G, u_end = units * (blockIdx.x + 1) / G;
  for (int64_t c = h_first; c < h_end; ++c) {
    for (int v = tid; v < EV; v += kThreads) s_hist[v] = 0;
    __syncthreads();
    const int64_t t0 = c * kChunk;
    const int ntok = (int)((N - t0) < kChunk ? (N - t0) : kChunk);
    for (int p = tid; p < ntok * k; p += kThreads) {
      int e = idx[t0 * k + p];
      if ((unsigned)e >= (unsigned)E) { atomicMax(&status[0], MOE_B200_DEV_BAD_INDEX); continue; }
      atomicAdd(&s_hist[s_vmap[e]], 1);
      if (p % k == 0) atomicAdd(&s_slot0[e], 1);
    }
    __syncthreads();
    for (int v = tid; v < EV; v += kThreads) {
      chunk_cnt[c * EV + v] = s_hist[v];
      s_base[v] += s_hist[v];                       // this block's total so far
    }
    __syncthreads();
  }
  // this block's totals: per block (prefix inside a group of 16 blocks) and, atomically, per
  // group and for the rank's slot-0 counts (integers: the order of the additions is immaterial)
  for (int v = tid; v < EV; v += kThreads) {
    const int n = s_base[v];
    blk_cnt[(size_t)blockIdx.x * EV + v] = n;
    if (n != 0) atomicAdd(&grp_cnt[(blockIdx.x / kEpGroupBlocks) * EV + v], n);
  }
  for (int e = tid; e < E; e += kThreads)
    if (s_slot0[e] != 0) atomicAdd(&cnt0_acc[e], s_slot0[e]);
  // the rank's probability sum of expert e: block e adds the router blocks' partial sums,
  // each thread a strided share in block order, then a tree over the threads (fixed order)
  for (int e = blockIdx.x; e < E; e += G) {
    float acc = 0.f;
    for (int64_t b = tid; b < router_blocks; b += kThreads) acc += psum_part[b * E + e];
    s_red[tid] = acc;
    __syncthreads();
    for (int o = kThreads / 2; o > 0; o >>= 1) {
      if (tid < o) s_red[tid] += s_red[tid + o];
      __syncthreads();
    }
    if (tid == 0) psum_local[e] = s_red[0];
    __syncthreads();
  }
  grid.sync();

  // ---- phase 2: local totals and this block's base; block 0 publishes this rank's row ----
  // totals = sum of the groups; base = the groups in front of this block's group plus the
  // blocks in front of it inside its group (blocks hold contiguous chunk ranges in block order)
  const int64_t c0 = u_first / split;          // chunk of this block's first unit = its first chunk
  {
    const int my_grp = blockIdx.x / kEpGroupBlocks;
    const int ngrp = (G + kEpGroupBlocks - 1) / kEpGroupBlocks;
    for (int v = tid; v < EV; v += kThreads) {
      int tot = 0, before = 0;
      for (int gq = 0; gq < ngrp; ++gq) {
        const int n = __ldcg(&grp_cnt[gq * EV + v]);
        tot += n;
        before += gq < my_grp ? n : 0;
      }
      for (int bb = my_grp * kEpGroupBlocks; bb < (int)blockIdx.x; ++bb)
        before += __ldcg(&blk_cnt[(size_t)bb * EV + v]);
      s_hist[v] = tot;
      s_base[v] = before;
    }
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    int32_t* my_row = peers.cnt_all[rank] + (size_t)rank * row_ints;
    for (int v = tid; v < EV; v += kThreads) my_row[v] = s_hist[v];
    for (int e = tid; e < E; e += kThreads) {
      my_row[EV + e] = __ldcg(&cnt0_acc[e]);
      my_row[EV + E + e] = __float_as_int(__ldcg(&psum_local[e]));
    }
    __syncthreads();
    // copy the row to every peer, then raise the count flag there
    for (int i = tid; i < row_ints * world; i += kThreads) {
      int q = i / row_ints, j = i - q * row_ints;
      if (q != rank) peers.cnt_all[q][(size_t)rank * row_ints + j] = my_row[j];
    }
    __threadfence_system();
    __syncthreads();
    if (tid < world) st_release_sys(peers.flags[tid] + kEpFlagCnt * kEpMaxRanks + rank, epoch);
  }
  // ---- phase 3: wait for every rank's row, derive destination rows ---------
  if (tid < world) {
    if (!wait_flag(peers.flags[rank] + kEpFlagCnt * kEpMaxRanks + tid, epoch, status, 21)) s_fail = 1;
  }
  __syncthreads();
  const bool fail = s_fail != 0;
  const int32_t* all = peers.cnt_all[rank];
  for (int i = tid; i < world * EV; i += kThreads) {
    int g = i / EV, v = i - g * EV;
    s_cnt[i] = fail ? 0 : (int)__ldcv(&all[(size_t)g * row_ints + v]);
  }
  __syncthreads();
  // rows of a virtual expert over all source ranks (s_run is free until the ranking)
  for (int v = tid; v < EV; v += kThreads) {
    int n = 0;
    for (int g = 0; g < world; ++g) n += s_cnt[g * EV + v];
    s_run[v] = n;
  }
  __syncthreads();
  for (int v = tid; v < EV; v += kThreads) {
    const int q = s_owner[v];
    int base = 0;
    for (int v2 = 0; v2 < v; ++v2)
      if (s_owner[v2] == q) base += s_run[v2];
    for (int g = 0; g < rank; ++g) base += s_cnt[g * EV + v];
    s_dest[v] = base;
  }
  if (blockIdx.x == 0 && fail) {
    // a peer never arrived: leave an empty layout so that the kernels after this one do nothing
    for (int i = tid; i <= EV; i += kThreads) offsets_local[i] = 0;
  }
  if (blockIdx.x == 0 && !fail) {
    // rows this rank will receive, per owned virtual expert in increasing id
    if (tid == 0) {
      int acc = 0, li = 0;
      for (int v = 0; v < EV; ++v) {
        if (s_owner[v] != rank) continue;
        offsets_local[li++] = acc;
        acc += s_run[v];
      }
      offsets_local[li] = acc;
    }
    // global slot-0 counts and probability sums, fixed order over ranks; loss
    // E^2 * mean_e(psum[e]/N_total * cnt0[e]/N_total)  (model.py:213-216)
    float part = 0.f;
    for (int e = tid; e < E; e += kThreads) {
      int c0s = 0;
      float ps = 0.f;
      for (int g = 0; g < world; ++g) {
        c0s += (int)__ldcv(&all[(size_t)g * row_ints + EV + e]);
        ps += __int_as_float((int)__ldcv(&all[(size_t)g * row_ints + EV + E + e]));
      }
      cnt_slot0[e] = c0s;
      psum_global[e] = ps;
      part += (ps / (float)n_total) * ((float)c0s / (float)n_total);
    }
    s_red[tid] = part;
    __syncthreads();
    for (int o = kThreads / 2; o > 0; o >>= 1) {
      if (tid < o) s_red[tid] += s_red[tid + o];
      __syncthreads();
    }
    if (tid == 0) aux[0] = s_red[0] / (float)E * (float)(E * E);
  }
  __syncthreads();
  // ---- phase 4: rank the pairs of each chunk, push rows to their owners ----
  // A unit is one part (of `split`) of the 16-byte pieces of a chunk's rows; every block that
  // holds a unit of a chunk ranks the chunk's pairs itself, part 0 writes the rows' metadata.
  {
    constexpr int kInFlight = 8;
    constexpr int kBatch = kThreads * kInFlight;
    int64_t ranked = -1;                          // chunk whose destinations are in s_dst
    int64_t based = c0;                           // s_base holds the rows of chunks before this one
    for (int64_t un = u_first; un < u_end && !fail; ++un) {
      const int64_t c = un / split;
      const int part = (int)(un - c * split);
      const int64_t t0 = c * kChunk;
      const int ntok = (int)((N - t0) < kChunk ? (N - t0) : kChunk);
      const int npair = ntok * k;
      const int pc_lo = (int)((int64_t)row_pieces * part / split);
      const int pc_n = (int)((int64_t)row_pieces * (part + 1) / split) - pc_lo;
      const int items = ntok * pc_n;
      const uint4* src = x + t0 * row_pieces + pc_lo;
      auto load = [&](uint4 (&v)[kInFlight], int i0) {
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
          const int i = i0 + u * kThreads;
          if (i < items) {
            const int tl = i / pc_n, pc = i - tl * pc_n;
            v[u] = __ldg(src + (size_t)tl * row_pieces + pc);
          }
        }
      };
      auto store = [&](const uint4 (&v)[kInFlight], int i0) {
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
          const int i = i0 + u * kThreads;
          if (i < items) {
            const int tl = i / pc_n, pc = i - tl * pc_n;
            for (int j = 0; j < k; ++j) {
              uint4* dst = reinterpret_cast<uint4*>(s_dst[tl * k + j]);
              if (dst != nullptr) dst[pc_lo + pc] = v[u];
            }
          }
        }
      };
      uint4 va[kInFlight], vb[kInFlight];
      load(va, tid);                              // on its way while the ranks are made
      if (c != ranked) {
        __syncthreads();                          // the copies of the chunk before are done with s_dst
        // rows of the chunks between `based` and c precede this chunk's
        for (; based < c; ++based)
          for (int v = tid; v < EV; v += kThreads) s_base[v] += __ldcg(&chunk_cnt[based * EV + v]);
        __syncthreads();
        if (warp == 0) {
          for (int v = lane; v < EV; v += 32) s_run[v] = 0;
          __syncwarp();
          for (int p0 = 0; p0 < npair; p0 += 32) {
            int p = p0 + lane;
            int e = p < npair ? idx[t0 * k + p] : -1;
            bool ok = (unsigned)e < (unsigned)E;
            const int v = ok ? s_vmap[e] : -1 - lane;
            unsigned grp = __match_any_sync(0xffffffffu, v);
            int row = -1, q = 0;
            if (ok) {
              row = s_dest[v] + s_base[v] + s_run[v] + __popc(grp & ((1u << lane) - 1u));
              q = s_owner[v];
            }
            __syncwarp();
            if (ok && (grp >> lane) == 1u) s_run[v] += __popc(grp);
            __syncwarp();
            if (p < npair) {
              s_dst[p] = row >= 0 ? reinterpret_cast<unsigned long long>(
                                        reinterpret_cast<uint4*>(peers.recv_x[q]) + (int64_t)row * row_pieces)
                                  : 0ull;
              if (row >= 0 && part == 0)
                peers.recv_meta[q][row] = (rank << 24) | (int)((t0 * k + p) & 0xffffff);
            }
          }
        }
        __syncthreads();
        ranked = c;
      }
      for (int i0 = tid;;) {
        const int i1 = i0 + kBatch;
        if (i1 < items) load(vb, i1);
        store(va, i0);
        if (i1 >= items) break;
        i0 = i1 + kBatch;
        if (i0 < items) load(va, i0);
        store(vb, i1);
        if (i0 >= items) break;
      }
    }
  }
  __threadfence_system();
  grid.sync();
  if (blockIdx.x == 0 && tid < world && !fail)
    st_release_sys(peers.flags[tid] + kEpFlagX * kEpMaxRanks + rank, epoch);
}

// Head of a call: the epoch advances, the status words and the down pass's completion counter
// start at zero.
__global__ void ep_begin_kernel(uint32_t* epoch, uint32_t* done_counter, int32_t* status,
                                int32_t* zero, int zero_ints) {
  if (threadIdx.x == 0) {
    *epoch = *epoch + 1u;
    *done_counter = 0u;
  }
  if (threadIdx.x < MOE_B200_STATUS_INTS) status[threadIdx.x] = 0;
  // the dispatch kernel's atomic accumulators (group counts, slot-0 counts)
  for (int i = threadIdx.x; i < zero_ints; i += blockDim.x) zero[i] = 0;
}

}  // namespace

int64_t ep_scratch_ints(int64_t N, int EV, int E) {
  return (int64_t)kEpGroups * EV + 2 * (int64_t)E + (int64_t)kNumSMs * 2 * EV + ((N + kChunk - 1) / kChunk) * EV;
}

int launch_ep_dispatch(const void* x, const int32_t* idx, int64_t N, int d, int E, int EV, int k,
                       int dtype, const EpPeers& peers, int rank, int world, const uint32_t* epoch,
                       const int32_t* owner, const int32_t* vmap, int32_t* scratch,
                       const float* psum_part,
                       int32_t* cnt_slot0, float* psum_global, int32_t* offsets_local, float* aux,
                       int64_t n_total, int32_t* status, cudaStream_t s) {
  const int row_pieces = d * (dtype == MOE_B200_BF16 ? 2 : 4) / 16;
  const size_t smem = sizeof(int) * (size_t)(5 * EV + 2 * E + 2 * kChunk * k + world * EV + kThreads);
  const void* fn = (const void*)ep_dispatch_kernel;
  // a cooperative grid must be resident at once: SM count of the current device, occupancy
  // for this call's shared-memory size
  int sms = 0;
  int rc = sm_count(&sms);
  if (rc) return rc;
  int per_sm = 0;
  MOE_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kThreads, smem));
  per_sm = per_sm < 1 ? 1 : (per_sm > 2 ? 2 : per_sm);
  int64_t grid = (int64_t)sms * per_sm;
  if (grid > (int64_t)kNumSMs * 2) grid = (int64_t)kNumSMs * 2;
  int64_t nchunk = (N + kChunk - 1) / kChunk;
  if (nchunk < 1) nchunk = 1;
  // the rows of a chunk are cut into up to four parts of at least 16 pieces: more, smaller units
  // of work even out the blocks' shares, and a call with fewer chunks than blocks still fills the grid
  int split = row_pieces / 16;
  split = split < 1 ? 1 : (split > 4 ? 4 : split);
  if (grid > nchunk * split) grid = nchunk * split;
  int64_t router_blocks = (N + kRouterTokensPerBlock - 1) / kRouterTokensPerBlock;
  const uint4* x4 = static_cast<const uint4*>(x);
  EpPeers pv = peers;
  void* args[] = {(void*)&x4, (void*)&idx, (void*)&N, (void*)&row_pieces, (void*)&E, (void*)&EV,
                  (void*)&k, (void*)&pv, (void*)&rank, (void*)&world, (void*)&epoch, (void*)&owner,
                  (void*)&vmap, (void*)&scratch, (void*)&psum_part, (void*)&router_blocks,
                  (void*)&cnt_slot0,
                  (void*)&psum_global, (void*)&offsets_local, (void*)&aux, (void*)&n_total,
                  (void*)&status, (void*)&split};
  MOE_CUDA_CHECK(cudaLaunchCooperativeKernel(fn, dim3((unsigned)grid), dim3(kThreads), args, smem, s));
  return 0;
}

int launch_ep_begin(uint32_t* epoch, uint32_t* done_counter, int32_t* status, int32_t* scratch, int EV,
                    int E, cudaStream_t s) {
  ep_begin_kernel<<<1, 256, 0, s>>>(epoch, done_counter, status, scratch, kEpGroups * EV + E);
  MOE_CUDA_CHECK(cudaGetLastError());
  return 0;
}

}  // namespace moe
