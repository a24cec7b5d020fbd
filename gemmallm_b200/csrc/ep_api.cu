// extern "C" entry points of the expert-parallel configuration (declared in
// include/moe_b200.h): symmetric-buffer and workspace layouts, and the launch
// sequence of one sharded forward.
#include <string.h>
#include "common.cuh"

namespace moe {

namespace {

size_t up1k(size_t v) { return (v + 1023) & ~(size_t)1023; }

int ep_check(int64_t N_local, int d, int f, int E, int k, int dtype, int rank, int world) {
  if (dtype != MOE_B200_BF16)
    return set_error(MOE_B200_ERR_DTYPE, "the expert-parallel path computes in bf16");
  if (world < 1 || world > kEpMaxRanks || rank < 0 || rank >= world)
    return set_error(MOE_B200_ERR_SHAPE, "world must be in [1,8] and rank in [0,world)");
  if (N_local < 0 || d < 8 || (d & 7) || f < 8 || (f & 7) || E < 1 || E > kMaxExperts || k < 1 ||
      k > kMaxTopK || k > E)
    return set_error(MOE_B200_ERR_SHAPE, "N, d, f, E or k out of range");
  if (N_local * (int64_t)k >= (int64_t)1 << 24)
    return set_error(MOE_B200_ERR_SHAPE, "N_local*k must stay below 2^24 (return address field)");
  if (N_local * (int64_t)k * world >= (int64_t)1 << 31)
    return set_error(MOE_B200_ERR_SHAPE, "N*k exceeds int32 rows");
  return 0;
}

void symm_layout(int64_t N_local, int d, int E, int k, int world, size_t* off, size_t* total) {
  const size_t cap = (size_t)N_local * k * world;  // worst case: every pair lands on one rank
  size_t sizes[MOE_B200_EP_SYMM_NUM];
  sizes[MOE_B200_EP_SYMM_FLAGS] = sizeof(uint32_t) * kEpNumFlags * kEpMaxRanks;
  sizes[MOE_B200_EP_SYMM_CNT_ALL] = sizeof(int32_t) * (kMaxExperts + 2 * E) * world;  // any EV <= 256
  sizes[MOE_B200_EP_SYMM_RECV_META] = sizeof(int32_t) * cap;
  sizes[MOE_B200_EP_SYMM_RECV_X] = cap * d * 2;
  sizes[MOE_B200_EP_SYMM_RET_Y] = (size_t)N_local * k * d * 2;
  size_t pos = 0;
  for (int i = 0; i < MOE_B200_EP_SYMM_NUM; ++i) {
    off[i] = pos;
    pos += up1k(sizes[i] ? sizes[i] : 1);
  }
  *total = pos;
}

void ws_layout(int64_t N_local, int d, int f, int E, int k, int world, size_t* off, size_t* total) {
  const size_t M = (size_t)N_local * k;
  const size_t cap = M * world;
  const size_t rb = (size_t)((N_local + kRouterTokensPerBlock - 1) / kRouterTokensPerBlock);
  size_t sizes[MOE_B200_EP_WS_NUM];
  sizes[MOE_B200_EP_WS_STATUS] = 16 * sizeof(int32_t);
  sizes[MOE_B200_EP_WS_LOGITS] = (size_t)N_local * E * sizeof(float);
  sizes[MOE_B200_EP_WS_IDX] = M * sizeof(int32_t);
  sizes[MOE_B200_EP_WS_W] = M * sizeof(float);
  sizes[MOE_B200_EP_WS_PSUM_PART] = rb * E * sizeof(float);
  sizes[MOE_B200_EP_WS_PSUM] = (size_t)E * sizeof(float);
  sizes[MOE_B200_EP_WS_AUX] = sizeof(float);
  sizes[MOE_B200_EP_WS_SCRATCH] = (size_t)ep_scratch_ints(N_local, kMaxExperts, E) * sizeof(int32_t);
  sizes[MOE_B200_EP_WS_CNT_SLOT0] = (size_t)E * sizeof(int32_t);
  sizes[MOE_B200_EP_WS_OFFSETS_LOCAL] = (size_t)(kMaxExperts + 1) * sizeof(int32_t);
  sizes[MOE_B200_EP_WS_OWNER] = (size_t)(kMaxExperts + E * kEpMaxRanks) * sizeof(int32_t);  // owner[EV], vmap[E][world]
  sizes[MOE_B200_EP_WS_H] = cap * f * 2;
  sizes[MOE_B200_EP_WS_Y] = cap * d * 2;
  size_t pos = 0;
  for (int i = 0; i < MOE_B200_EP_WS_NUM; ++i) {
    off[i] = pos;
    pos += up1k(sizes[i] ? sizes[i] : 1);
  }
  *total = pos;
}

}  // namespace
}  // namespace moe

using namespace moe;

extern "C" {

size_t moe_b200_ep_symm_bytes(int64_t N_local, int d, int E, int k, int world) {
  if (ep_check(N_local, d, 8, E, k, MOE_B200_BF16, 0, world)) return 0;
  size_t off[MOE_B200_EP_SYMM_NUM], total;
  symm_layout(N_local, d, E, k, world, off, &total);
  return total;
}

int moe_b200_ep_symm_layout(int64_t N_local, int d, int E, int k, int world, size_t* h_offsets) {
  if (!h_offsets) return set_error(MOE_B200_ERR_NULL, "h_offsets is NULL");
  int rc = ep_check(N_local, d, 8, E, k, MOE_B200_BF16, 0, world);
  if (rc) return rc;
  size_t total;
  symm_layout(N_local, d, E, k, world, h_offsets, &total);
  return 0;
}

size_t moe_b200_ep_workspace_bytes(int64_t N_local, int d, int f, int E, int k, int world) {
  if (ep_check(N_local, d, f, E, k, MOE_B200_BF16, 0, world)) return 0;
  size_t off[MOE_B200_EP_WS_NUM], total;
  ws_layout(N_local, d, f, E, k, world, off, &total);
  return total;
}

int moe_b200_ep_workspace_layout(int64_t N_local, int d, int f, int E, int k, int world,
                                 size_t* h_offsets) {
  if (!h_offsets) return set_error(MOE_B200_ERR_NULL, "h_offsets is NULL");
  int rc = ep_check(N_local, d, f, E, k, MOE_B200_BF16, 0, world);
  if (rc) return rc;
  size_t total;
  ws_layout(N_local, d, f, E, k, world, h_offsets, &total);
  return 0;
}

int moe_b200_ep_forward(const void* x, const void* Wg, const void* bg, const void* plan_local,
                        const void* residual, int64_t N_local, int d, int f, int E, int k,
                        int dtype, int flags, int rank, int world, uint32_t epoch, int EV,
                        const int32_t* h_owner, const int32_t* h_vmap, void* const* h_symm_bases,
                        void* workspace, size_t workspace_bytes, void* out, void* stream) {
  int rc = ep_check(N_local, d, f, E, k, dtype, rank, world);
  if (rc) return rc;
  if (!h_owner || !h_vmap || !h_symm_bases || !workspace) return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (EV < E || EV > kMaxExperts) return set_error(MOE_B200_ERR_SHAPE, "EV must be in [E, 256]");
  if (N_local > 0 && (!x || !Wg || !bg || !out)) return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (epoch == 0) return set_error(MOE_B200_ERR_SHAPE, "epoch must start at 1 and grow by one per call");
  int E_local = 0;
  for (int v = 0; v < EV; ++v) {
    if (h_owner[v] < 0 || h_owner[v] >= world)
      return set_error(MOE_B200_ERR_SHAPE, "expert owner out of range");
    if (h_owner[v] == rank) ++E_local;
  }
  for (int i = 0; i < E * world; ++i)
    if (h_vmap[i] < 0 || h_vmap[i] >= EV)
      return set_error(MOE_B200_ERR_SHAPE, "virtual expert id out of range");
  if (E_local > 0 && !plan_local) return set_error(MOE_B200_ERR_NULL, "plan_local is NULL");
  size_t so[MOE_B200_EP_SYMM_NUM], wo[MOE_B200_EP_WS_NUM], stotal, wtotal;
  symm_layout(N_local, d, E, k, world, so, &stotal);
  ws_layout(N_local, d, f, E, k, world, wo, &wtotal);
  if (workspace_bytes < wtotal) return set_error(MOE_B200_ERR_WORKSPACE, "workspace too small");
  if ((uintptr_t)workspace & 1023) return set_error(MOE_B200_ERR_ALIGN, "workspace must be 1024-byte aligned");
  EpPeers peers;
  memset(&peers, 0, sizeof(peers));
  for (int q = 0; q < world; ++q) {
    char* b = static_cast<char*>(h_symm_bases[q]);
    if (!b || ((uintptr_t)b & 1023)) return set_error(MOE_B200_ERR_ALIGN, "symmetric buffers must be 1024-byte aligned");
    peers.flags[q] = reinterpret_cast<uint32_t*>(b + so[MOE_B200_EP_SYMM_FLAGS]);
    peers.cnt_all[q] = reinterpret_cast<int32_t*>(b + so[MOE_B200_EP_SYMM_CNT_ALL]);
    peers.recv_meta[q] = reinterpret_cast<int32_t*>(b + so[MOE_B200_EP_SYMM_RECV_META]);
    peers.recv_x[q] = b + so[MOE_B200_EP_SYMM_RECV_X];
    peers.ret_y[q] = b + so[MOE_B200_EP_SYMM_RET_Y];
  }
  char* ws = static_cast<char*>(workspace);
  int32_t* status = reinterpret_cast<int32_t*>(ws + wo[MOE_B200_EP_WS_STATUS]);
  float* logits = reinterpret_cast<float*>(ws + wo[MOE_B200_EP_WS_LOGITS]);
  int32_t* idx = reinterpret_cast<int32_t*>(ws + wo[MOE_B200_EP_WS_IDX]);
  float* w = reinterpret_cast<float*>(ws + wo[MOE_B200_EP_WS_W]);
  float* psum_part = reinterpret_cast<float*>(ws + wo[MOE_B200_EP_WS_PSUM_PART]);
  float* psum = reinterpret_cast<float*>(ws + wo[MOE_B200_EP_WS_PSUM]);
  float* aux = reinterpret_cast<float*>(ws + wo[MOE_B200_EP_WS_AUX]);
  int32_t* scratch = reinterpret_cast<int32_t*>(ws + wo[MOE_B200_EP_WS_SCRATCH]);
  int32_t* cnt_slot0 = reinterpret_cast<int32_t*>(ws + wo[MOE_B200_EP_WS_CNT_SLOT0]);
  int32_t* offsets_local = reinterpret_cast<int32_t*>(ws + wo[MOE_B200_EP_WS_OFFSETS_LOCAL]);
  int32_t* owner = reinterpret_cast<int32_t*>(ws + wo[MOE_B200_EP_WS_OWNER]);
  void* h = ws + wo[MOE_B200_EP_WS_H];
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t cap = N_local * (int64_t)k * world;

  MOE_CUDA_CHECK(cudaMemsetAsync(status, 0, 16 * sizeof(int32_t), s));
  // the owner table is uploaded only when it (or the workspace) changes: a copy
  // from pageable memory would otherwise synchronise the stream on every call
  static thread_local const void* cached_ws = nullptr;
  static thread_local int cached_n = 0;
  static thread_local int32_t cached_tab[kMaxExperts + kMaxExperts * kEpMaxRanks];
  int32_t tab[kMaxExperts + kMaxExperts * kEpMaxRanks];
  memset(tab, 0, sizeof(tab));
  memcpy(tab, h_owner, sizeof(int32_t) * EV);
  memcpy(tab + kMaxExperts, h_vmap, sizeof(int32_t) * E * world);
  const int tab_n = kMaxExperts + E * world;
  if (cached_ws != workspace || cached_n != tab_n || memcmp(cached_tab, tab, sizeof(int32_t) * tab_n) != 0) {
    MOE_CUDA_CHECK(cudaMemcpyAsync(owner, tab, sizeof(int32_t) * tab_n, cudaMemcpyHostToDevice, s));
    memcpy(cached_tab, tab, sizeof(int32_t) * tab_n);
    cached_ws = workspace;
    cached_n = tab_n;
  }
  const int32_t* vmap_dev = owner + kMaxExperts;
  if (N_local > 0) {
    rc = launch_router(x, Wg, bg, N_local, d, E, k, dtype, logits, idx, w, psum_part, status, s);
    if (rc) return rc;
  }
  rc = launch_ep_dispatch(x, idx, N_local, d, E, EV, k, dtype, peers, rank, world, epoch, owner,
                          vmap_dev, scratch, psum_part, cnt_slot0, psum, offsets_local, aux,
                          N_local * (int64_t)world, status, s);
  if (rc) return rc;
  rc = launch_ep_wait(peers.flags[rank] + kEpFlagX * kEpMaxRanks, world, epoch, status, 22, s);
  if (rc) return rc;
  EpScatter sc;
  for (int q = 0; q < kEpMaxRanks; ++q) sc.ret_y[q] = peers.ret_y[q];
  sc.meta = peers.recv_meta[rank];
  if (flags & MOE_B200_FLAG_EP_UNFUSED_RETURN) {
    // expert outputs to a local buffer first, then one copy kernel over NVLink
    void* y = ws + wo[MOE_B200_EP_WS_Y];
    if (E_local > 0) {
      rc = (flags & MOE_B200_FLAG_ONE_CTA)
               ? launch_experts_tc(peers.recv_x[rank], offsets_local, plan_local, cap, d, f, E_local,
                                   h, y, status, s)
               : launch_experts_tc2(peers.recv_x[rank], offsets_local, plan_local, cap, d, f, E_local,
                                    h, y, nullptr, status, s);
      if (rc) return rc;
      rc = launch_ep_return(y, offsets_local, E_local, sc, d, s);
      if (rc) return rc;
    }
  } else {
    rc = (flags & MOE_B200_FLAG_ONE_CTA)
             ? launch_experts_tc_ep(peers.recv_x[rank], offsets_local, plan_local, cap, d, f, E_local,
                                    h, sc, status, s)
             : launch_experts_tc2(peers.recv_x[rank], offsets_local, plan_local, cap, d, f, E_local, h,
                                  nullptr, &sc, status, s);
    if (rc) return rc;
  }
  rc = launch_ep_signal(peers, kEpFlagY, rank, world, epoch, s);
  if (rc) return rc;
  rc = launch_ep_wait(peers.flags[rank] + kEpFlagY * kEpMaxRanks, world, epoch, status, 23, s);
  if (rc) return rc;
  return launch_combine(peers.ret_y[rank], nullptr, w, residual, N_local, d, k, dtype, out, s);
}

}  // extern "C"
