// Dispatch kernel: histogram of the routing indices, exclusive scan, and the
// permutation of token rows into one expert-contiguous buffer, in a single
// cooperative launch. Replaces the reference's per-slot argsort, the Python
// count loop with its device->host reads, the gather and the split
// (model.py:226-253), and finishes the load-balancing loss (model.py:213-216).
//
// HBM-bound: x [N,d] is read once and written k times with 16-byte accesses.
// Tokens are cut into chunks of 64; every block owns one contiguous range of
// chunks (the first nchunk mod gridDim blocks one chunk more than the rest) in
// both phases. Phase 1 counts experts per chunk and per block into scratch.
// After a grid barrier every block sums the per-block counts (gridDim * E
// numbers: all of them for the expert offsets, those of earlier blocks for its
// base), then for each of its chunks ranks the (token, slot) pairs in token
// order and copies the rows, the loads of one batch of rows in flight while
// the batch before it is stored. Rows of one expert therefore stay in token
// order whatever the grid size.
// With the caller's LayerNorm folded in (norm_stats != nullptr, see norm.cu) a row is
// copied as (x - mean) * rstd * gamma + beta, with (mean, rstd) from the router
// (reference model.py:311-312).
#include <cooperative_groups.h>
#include <stdio.h>
#include "common.cuh"

namespace cg = cooperative_groups;

namespace moe {

namespace {

constexpr int kThreads = 256;
constexpr int kChunk = kDispatchChunk;
constexpr int kScratchHeader = 32;  // ints: [0] = blocks finished

__host__ __device__ inline int64_t num_chunks(int64_t N) { return (N + kChunk - 1) / kChunk; }

// chunks [first, first + count) of block b out of G
__device__ inline void chunk_range(int64_t nchunk, int G, int b, int64_t& first, int64_t& count) {
  const int64_t lo = nchunk / G, extra = nchunk - lo * G;
  count = lo + (b < extra ? 1 : 0);
  first = lo * b + (b < extra ? b : extra);
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
dispatch_kernel(const T* __restrict__ x, const int32_t* __restrict__ idx, int64_t N, int d, int E,
                int k, int32_t* __restrict__ scratch, int32_t* __restrict__ cnt_slot,
                int32_t* __restrict__ offsets, int32_t* __restrict__ row_of, T* __restrict__ perm,
                const float* __restrict__ psum_part, int64_t router_blocks,
                float* __restrict__ psum, float* __restrict__ aux, int32_t* __restrict__ status,
                const float* __restrict__ norm_stats, const T* __restrict__ gamma,
                const T* __restrict__ beta) {
  cg::grid_group grid = cg::this_grid();
  extern __shared__ int s_int[];
  int* s_hist = s_int;             // [E]  chunk histogram, later totals
  int* s_base = s_hist + E;        // [E]  rows of earlier chunks per expert
  int* s_off = s_base + E;         // [E+1]
  int* s_run = s_off + E + 1;      // [E]  running rank inside the chunk
  int* s_slot = s_run + E;         // [k*E]
  int* s_row = s_slot + k * E;     // [kChunk*k]
  float* s_red = reinterpret_cast<float*>(s_row + kChunk * k);  // [kThreads]
  __shared__ int s_last;

  const int tid = threadIdx.x;
  const int G = gridDim.x;
  const int64_t nchunk = num_chunks(N);
  int32_t* done = scratch;
  int32_t* chunk_cnt = scratch + kScratchHeader;     // [nchunk][E]
  int32_t* blk_slot = chunk_cnt + nchunk * E;        // [G][k][E]
  int32_t* blk_cnt = blk_slot + (size_t)kNumSMs * 2 * k * E;   // [G][E]
  int64_t c_first, c_count;
  chunk_range(nchunk, G, blockIdx.x, c_first, c_count);

  // ---- phase 1: histograms -----------------------------------------------
  for (int i = tid; i < k * E; i += kThreads) s_slot[i] = 0;
  for (int e = tid; e < E; e += kThreads) s_base[e] = 0;   // this block's total per expert
  if (blockIdx.x == 0 && tid == 0) *done = 0;
  for (int64_t c = c_first; c < c_first + c_count; ++c) {
    for (int e = tid; e < E; e += kThreads) s_hist[e] = 0;
    __syncthreads();
    const int64_t t0 = c * kChunk;
    const int ntok = (int)((N - t0) < kChunk ? (N - t0) : kChunk);
    for (int p = tid; p < ntok * k; p += kThreads) {
      int e = idx[t0 * k + p];
      if ((unsigned)e >= (unsigned)E) {
        atomicMax(&status[0], MOE_B200_DEV_BAD_INDEX);
        continue;
      }
      atomicAdd(&s_hist[e], 1);
      atomicAdd(&s_slot[(p % k) * E + e], 1);
    }
    __syncthreads();
    for (int e = tid; e < E; e += kThreads) {
      chunk_cnt[c * E + e] = s_hist[e];
      s_base[e] += s_hist[e];
    }
    __syncthreads();
  }
  for (int i = tid; i < k * E; i += kThreads) blk_slot[(size_t)blockIdx.x * k * E + i] = s_slot[i];
  for (int e = tid; e < E; e += kThreads) blk_cnt[(size_t)blockIdx.x * E + e] = s_base[e];

  grid.sync();

  // ---- phase 2: scan ------------------------------------------------------
  for (int e = tid; e < E; e += kThreads) { s_hist[e] = 0; s_base[e] = 0; }
  __syncthreads();
  {
    const int bme = (int)blockIdx.x;
    if (kThreads % E == 0) {
      // every count this thread visits belongs to the same expert: sum in registers,
      // one shared-memory atomic per thread at the end
      const int e = tid % E, step = kThreads / E;
      int tot = 0, before = 0;
#pragma unroll 8
      for (int bb = tid / E; bb < G; bb += step) {
        const int v = __ldcg(&blk_cnt[(size_t)bb * E + e]);
        tot += v;
        before += bb < bme ? v : 0;
      }
      if (tot != 0) atomicAdd(&s_hist[e], tot);
      if (before != 0) atomicAdd(&s_base[e], before);
    } else {
      for (int i = tid; i < G * E; i += kThreads) {
        const int v = __ldcg(&blk_cnt[i]);
        const int bb = i / E, e = i - bb * E;
        if (v != 0) {
          atomicAdd(&s_hist[e], v);
          if (bb < bme) atomicAdd(&s_base[e], v);
        }
      }
    }
  }
  __syncthreads();
  if (tid < 32) {
    // exclusive scan over E <= 256 experts by one warp: 8 consecutive experts per lane
    int loc[kMaxExperts / 32];
    int sum = 0;
#pragma unroll
    for (int i = 0; i < kMaxExperts / 32; ++i) {
      int e = tid * (kMaxExperts / 32) + i;
      loc[i] = sum;
      sum += e < E ? s_hist[e] : 0;
    }
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (tid >= o) incl += v;
    }
    const int excl = incl - sum;
#pragma unroll
    for (int i = 0; i < kMaxExperts / 32; ++i) {
      int e = tid * (kMaxExperts / 32) + i;
      if (e < E) s_off[e] = excl + loc[i];
    }
    if (tid == 31) s_off[E] = incl;
  }
  __syncthreads();
  if (blockIdx.x == 0)
    for (int e = tid; e <= E; e += kThreads) offsets[e] = s_off[e];

  // ---- phase 2: rank and copy ---------------------------------------------
  const int warp = tid >> 5, lane = tid & 31;
  constexpr int kVec = 16 / (int)sizeof(T);
  constexpr int kInFlight = 8;
  constexpr int kBatch = kThreads * kInFlight;
  const int pieces = d / kVec;
  for (int64_t c = c_first; c < c_first + c_count; ++c) {
    const int64_t t0 = c * kChunk;
    const int ntok = (int)((N - t0) < kChunk ? (N - t0) : kChunk);
    const int npair = ntok * k;
    // rows: the chunk's 16-byte pieces are spread over the block, kInFlight loads per
    // thread and batch; each piece is stored once per slot. The first batch is
    // requested before the ranks are known, every later one before the batch in
    // front of it is stored.
    const int items = ntok * pieces;
    const uint4* src = reinterpret_cast<const uint4*>(x + t0 * d);
    auto load = [&](uint4 (&v)[kInFlight], int i0) {
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) {
        const int i = i0 + u * kThreads;
        if (i < items) v[u] = __ldg(src + i);
      }
    };
    auto store = [&](uint4 (&v)[kInFlight], int i0) {
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) {
        const int i = i0 + u * kThreads;
        if (i < items) {
          const int tl = i / pieces, pc = i - tl * pieces;
          if (norm_stats != nullptr) {
            // 16 bytes = 4 fp32 or 8 bf16 elements of row t0 + tl, columns from pc * kVec
            const float mean = __ldg(&norm_stats[2 * (t0 + tl)]);
            const float rstd = __ldg(&norm_stats[2 * (t0 + tl) + 1]);
            T* e = reinterpret_cast<T*>(&v[u]);
#pragma unroll
            for (int q = 0; q < kVec; ++q) {
              const float y = fmaf((to_f32(e[q]) - mean) * rstd, to_f32(__ldg(&gamma[pc * kVec + q])),
                                   to_f32(__ldg(&beta[pc * kVec + q])));
              from_f32(e[q], y);
            }
          }
          for (int j = 0; j < k; ++j) {
            const int row = s_row[tl * k + j];
            if (row >= 0) __stcs(reinterpret_cast<uint4*>(perm + (int64_t)row * d) + pc, v[u]);
          }
        }
      }
    };
    uint4 va[kInFlight], vb[kInFlight];
    load(va, tid);
    if (warp == 0) {
      for (int e = lane; e < E; e += 32) s_run[e] = 0;
      __syncwarp();
      for (int p0 = 0; p0 < npair; p0 += 32) {
        int p = p0 + lane;
        int e = p < npair ? idx[t0 * k + p] : -1;
        bool ok = (unsigned)e < (unsigned)E;
        // lanes with the same expert form a group; rank = earlier lanes of it
        unsigned grp = __match_any_sync(0xffffffffu, ok ? e : -1 - lane);
        int row = -1;
        if (ok) {
          int before = __popc(grp & ((1u << lane) - 1u));
          row = s_off[e] + s_base[e] + s_run[e] + before;
        }
        __syncwarp();
        if (ok && (grp >> lane) == 1u) s_run[e] += __popc(grp);  // highest lane of the group
        __syncwarp();
        if (p < npair) {
          s_row[p] = row;
          row_of[t0 * k + p] = row;
        }
      }
    }
    __syncthreads();
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
    __syncthreads();
    // this chunk's rows precede the next chunk's
    for (int e = tid; e < E; e += kThreads) s_base[e] += chunk_cnt[c * E + e];
    __syncthreads();
  }

  // ---- tail: per-slot counts, probability sums, loss ----------------------
  // per-slot counts: entry i = (slot, expert) is summed over the blocks by one warp
  for (int i = blockIdx.x * (kThreads / 32) + warp; i < k * E; i += G * (kThreads / 32)) {
    int acc = 0;
    for (int b = lane; b < G; b += 32) acc += __ldcg(&blk_slot[(size_t)b * k * E + i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) cnt_slot[i] = acc;
  }
  if (psum_part == nullptr) return;
  for (int e = blockIdx.x; e < E; e += G) {
    float acc = 0.f;
    for (int64_t b = tid; b < router_blocks; b += kThreads) acc += psum_part[b * E + e];
    s_red[tid] = acc;
    __syncthreads();
    for (int o = kThreads / 2; o > 0; o >>= 1) {
      if (tid < o) s_red[tid] += s_red[tid + o];
      __syncthreads();
    }
    if (tid == 0) psum[e] = s_red[0];
    __syncthreads();
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) s_last = (atomicAdd(done, 1) == G - 1);
  __syncthreads();
  if (s_last) {
    __threadfence();
    // E^2 * mean_e( psum[e]/N * cnt0[e]/N ), model.py:213-216 (slot 0 only)
    float acc = 0.f;
    for (int e = tid; e < E; e += kThreads) {
      float prob = __ldcg(&psum[e]) / (float)N;
      float freq = (float)__ldcg(&cnt_slot[e]) / (float)N;
      acc += prob * freq;
    }
    s_red[tid] = acc;
    __syncthreads();
    for (int o = kThreads / 2; o > 0; o >>= 1) {
      if (tid < o) s_red[tid] += s_red[tid + o];
      __syncthreads();
    }
    if (tid == 0) aux[0] = s_red[0] / (float)E * (float)(E * E);
  }
}

}  // namespace

int64_t dispatch_scratch_ints(int64_t N, int E, int k) {
  return kScratchHeader + num_chunks(N) * E + (int64_t)kNumSMs * 2 * k * E + (int64_t)kNumSMs * 2 * E;
}

int launch_dispatch(const void* x, const int32_t* idx, int64_t N, int d, int E, int k, int dtype,
                    int32_t* scratch, int32_t* cnt_slot, int32_t* offsets, int32_t* row_of,
                    void* perm, const float* psum_part, float* psum, float* aux, int32_t* status,
                    cudaStream_t s, const float* norm_stats, const void* gamma, const void* beta) {
  const size_t smem =
      sizeof(int) * (size_t)(4 * E + 1 + k * E + kChunk * k) + sizeof(float) * kThreads;
  const int ti = dtype == MOE_B200_BF16 ? 1 : 0;
  const void* fn = ti ? (const void*)dispatch_kernel<__nv_bfloat16> : (const void*)dispatch_kernel<float>;
  // a cooperative grid must be resident at once: SM count of the current device, and the
  // occupancy for this call's shared-memory size (a host-side computation, no GPU work)
  int sms = 0;
  int rc = sm_count(&sms);
  if (rc) return rc;
  int per_sm = 0;
  MOE_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kThreads, smem));
  per_sm = per_sm < 1 ? 1 : (per_sm > 2 ? 2 : per_sm);
  int64_t grid = (int64_t)sms * per_sm;
  if (grid > (int64_t)kNumSMs * 2) grid = (int64_t)kNumSMs * 2;
  int64_t nchunk = num_chunks(N);
  if (nchunk < 1) nchunk = 1;
  if (grid > nchunk) grid = nchunk;
  int64_t router_blocks = (N + kRouterTokensPerBlock - 1) / kRouterTokensPerBlock;
  void* args[] = {(void*)&x,        (void*)&idx,     (void*)&N,       (void*)&d,
                  (void*)&E,        (void*)&k,       (void*)&scratch, (void*)&cnt_slot,
                  (void*)&offsets,  (void*)&row_of,  (void*)&perm,    (void*)&psum_part,
                  (void*)&router_blocks, (void*)&psum, (void*)&aux,   (void*)&status,
                  (void*)&norm_stats, (void*)&gamma, (void*)&beta};
  MOE_CUDA_CHECK(cudaLaunchCooperativeKernel(fn, dim3((unsigned)grid), dim3(kThreads), args, smem, s));
  return 0;
}

}  // namespace moe

// ---------------------------------------------------------------------------
// Dispatch without caller-provided scratch.
//
// Some callers cannot hand the library a scratch buffer because they are not
// allowed to allocate device memory at the point of the call: code running
// inside a framework's forward hook with a frozen memory pool, a serving loop
// whose allocator is locked while requests are in flight, or a host language
// binding that only receives the tensors of the op's signature. For them the
// per-chunk counters live in this file-scope device array instead. Every GPU
// that loads the library holds kStaticScratchInts * 4 bytes (1 MiB) for the
// lifetime of the process.
//
// The array is shared by every call on that GPU and keeps what the last call
// left in it. Nothing has to be cleared between calls: the kernel zeroes its
// completion counter itself before the grid barrier and overwrites every
// count before reading it. Two calls whose kernels overlap on one GPU (two
// streams, two host threads) race on it; callers must serialise them.
// The first call on a device looks up the array's device address
// (cudaGetSymbolAddress); make that first call outside any stream capture.
namespace moe {
namespace {
constexpr int64_t kStaticScratchInts = 262144;  // 1 MiB
static __device__ __align__(256) int32_t g_static_scratch[kStaticScratchInts];
// g_static_scratch names a host-side shadow here; the device address has to be
// asked for, once per device, with that device current.
int32_t* g_static_scratch_addr[kMaxDevices] = {nullptr};
}  // namespace
}  // namespace moe

extern "C" int moe_b200_dispatch_static(const void* x, const int32_t* idx, int64_t N, int d, int E,
                                        int k, int dtype, int32_t* cnt_slot, int32_t* offsets,
                                        int32_t* row_of, void* perm, const float* psum_part,
                                        float* psum, float* aux, int32_t* status, void* stream) {
  using namespace moe;
  if (dtype != MOE_B200_F32 && dtype != MOE_B200_BF16)
    return set_error(MOE_B200_ERR_DTYPE, "dtype must be MOE_B200_F32 or MOE_B200_BF16");
  if (N < 0 || d < 8 || (d & 7) || E < 1 || E > kMaxExperts || k < 1 || k > kMaxTopK || k > E ||
      N * (int64_t)k >= (int64_t)1 << 31)
    return set_error(MOE_B200_ERR_SHAPE, "N, d, E or k out of range");
  const int64_t need = dispatch_scratch_ints(N, E, k);
  if (need > kStaticScratchInts) {
    char msg[200];
    snprintf(msg, sizeof(msg),
             "moe_b200_dispatch_static: this shape needs %lld scratch words, the built-in array "
             "holds %lld; use moe_b200_dispatch with a caller-provided scratch buffer",
             (long long)need, (long long)kStaticScratchInts);
    return set_error(MOE_B200_ERR_WORKSPACE, msg);
  }
  if (!cnt_slot || !offsets || !status) return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (N > 0 && (!x || !idx || !row_of || !perm)) return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (psum_part && (!psum || !aux))
    return set_error(MOE_B200_ERR_NULL, "psum and aux are required with psum_part");
  if (!aligned16(x) || !aligned16(perm))
    return set_error(MOE_B200_ERR_ALIGN, "x and perm must be 16-byte aligned");
  int dev = 0;
  MOE_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return set_error(MOE_B200_ERR_UNSUPPORTED, "device ordinal too large");
  if (g_static_scratch_addr[dev] == nullptr) {
    int32_t* ptr = nullptr;
    MOE_CUDA_CHECK(cudaGetSymbolAddress((void**)&ptr, g_static_scratch));
    g_static_scratch_addr[dev] = ptr;
  }
  return launch_dispatch(x, idx, N, d, E, k, dtype, g_static_scratch_addr[dev], cnt_slot, offsets,
                         row_of, perm, psum_part, psum, aux, status, (cudaStream_t)stream);
}
