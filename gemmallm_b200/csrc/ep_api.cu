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
  sizes[MOE_B200_EP_WS_STATUS] = 32 * sizeof(int32_t);   // 16 status words, then epoch, completion counter
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

int moe_b200_ep_setup(const int32_t* h_owner, const int32_t* h_vmap, int64_t N_local, int d, int f,
                      int E, int k, int world, int EV, void* workspace, size_t workspace_bytes,
                      void* stream) {
  int rc = ep_check(N_local, d, f, E, k, MOE_B200_BF16, 0, world);
  if (rc) return rc;
  if (!h_owner || !h_vmap || !workspace) return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (EV < E || EV > kMaxExperts) return set_error(MOE_B200_ERR_SHAPE, "EV must be in [E, 256]");
  for (int v = 0; v < EV; ++v)
    if (h_owner[v] < 0 || h_owner[v] >= world)
      return set_error(MOE_B200_ERR_SHAPE, "expert owner out of range");
  for (int i = 0; i < E * world; ++i)
    if (h_vmap[i] < 0 || h_vmap[i] >= EV)
      return set_error(MOE_B200_ERR_SHAPE, "virtual expert id out of range");
  size_t wo[MOE_B200_EP_WS_NUM], wtotal;
  ws_layout(N_local, d, f, E, k, world, wo, &wtotal);
  if (workspace_bytes < wtotal) return set_error(MOE_B200_ERR_WORKSPACE, "workspace too small");
  if ((uintptr_t)workspace & 1023) return set_error(MOE_B200_ERR_ALIGN, "workspace must be 1024-byte aligned");
  char* ws = static_cast<char*>(workspace);
  cudaStream_t s = (cudaStream_t)stream;
  int32_t tab[kMaxExperts + kMaxExperts * kEpMaxRanks];
  memset(tab, 0, sizeof(tab));
  memcpy(tab, h_owner, sizeof(int32_t) * EV);
  memcpy(tab + kMaxExperts, h_vmap, sizeof(int32_t) * E * world);
  // status words, the epoch (calls count from 1) and the completion counter
  MOE_CUDA_CHECK(cudaMemsetAsync(ws + wo[MOE_B200_EP_WS_STATUS], 0, 32 * sizeof(int32_t), s));
  MOE_CUDA_CHECK(cudaMemcpyAsync(ws + wo[MOE_B200_EP_WS_OWNER], tab,
                                 sizeof(int32_t) * (kMaxExperts + E * world), cudaMemcpyHostToDevice, s));
  // `tab` lives on this stack frame
  MOE_CUDA_CHECK(cudaStreamSynchronize(s));
  return 0;
}

int moe_b200_ep_forward(const void* x, const void* Wg, const void* bg, const void* plan_local,
                        const void* residual, int64_t N_local, int d, int f, int E, int k,
                        int dtype, int flags, int rank, int world, int EV,
                        int E_local, void* const* h_symm_bases,
                        void* workspace, size_t workspace_bytes, void* out,
                        void* const* h_stage_events, void* stream) {
  int rc = ep_check(N_local, d, f, E, k, dtype, rank, world);
  if (rc) return rc;
  if (!h_symm_bases || !workspace) return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (flags != 0) return set_error(MOE_B200_ERR_UNSUPPORTED, "flags must be 0");
  if (EV < E || EV > kMaxExperts) return set_error(MOE_B200_ERR_SHAPE, "EV must be in [E, 256]");
  if (E_local < 0 || E_local > EV) return set_error(MOE_B200_ERR_SHAPE, "E_local must be in [0, EV]");
  if (N_local > 0 && (!x || !Wg || !bg || !out)) return set_error(MOE_B200_ERR_NULL, "NULL argument");
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
  const int32_t* owner = reinterpret_cast<const int32_t*>(ws + wo[MOE_B200_EP_WS_OWNER]);
  const int32_t* vmap_dev = owner + kMaxExperts;
  void* h = ws + wo[MOE_B200_EP_WS_H];
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t cap = N_local * (int64_t)k * world;

  auto stamp = [&](int which) -> int {
    if (h_stage_events == nullptr) return 0;
    MOE_CUDA_CHECK(cudaEventRecord(static_cast<cudaEvent_t>(h_stage_events[which]), s));
    return 0;
  };
  uint32_t* epoch = reinterpret_cast<uint32_t*>(status + 16);
  uint32_t* done_counter = reinterpret_cast<uint32_t*>(status + 17);
  // the call's epoch lives on the device, so the same launches can be replayed from a CUDA graph
  rc = launch_ep_begin(epoch, done_counter, status, scratch, EV, E, s);
  if (rc) return rc;
  if ((rc = stamp(MOE_B200_EP_EV_START))) return rc;
  if (N_local > 0) {
    rc = launch_router(x, Wg, bg, N_local, d, E, k, dtype, logits, idx, w, psum_part, status, s);
    if (rc) return rc;
  }
  if ((rc = stamp(MOE_B200_EP_EV_ROUTER))) return rc;
  rc = launch_ep_dispatch(x, idx, N_local, d, E, EV, k, dtype, peers, rank, world, epoch, owner,
                          vmap_dev, scratch, psum_part, cnt_slot0, psum, offsets_local, aux,
                          N_local * (int64_t)world, status, s);
  if (rc) return rc;
  if ((rc = stamp(MOE_B200_EP_EV_DISPATCH))) return rc;
  // the GEGLU pass waits for every source's rows at its head; the down pass stores its rows
  // straight into the token owners' ret_y and its last block raises the return flag everywhere;
  // the combine waits for every owner's return flag at its head
  EpScatter sc;
  for (int q = 0; q < kEpMaxRanks; ++q) sc.ret_y[q] = peers.ret_y[q];
  sc.meta = peers.recv_meta[rank];
  EpSync wait_x = {}, signal_y = {}, wait_y = {};
  wait_x.epoch = signal_y.epoch = wait_y.epoch = epoch;
  wait_x.world = signal_y.world = wait_y.world = world;
  wait_x.wait_flags = peers.flags[rank] + kEpFlagX * kEpMaxRanks;
  wait_y.wait_flags = peers.flags[rank] + kEpFlagY * kEpMaxRanks;
  signal_y.done_counter = done_counter;
  for (int q = 0; q < world; ++q) signal_y.signal_flags[q] = peers.flags[q] + kEpFlagY * kEpMaxRanks + rank;
  rc = launch_experts_tc2(peers.recv_x[rank], offsets_local, plan_local, cap, d, f, E_local, h,
                          nullptr, &sc, status, s, nullptr, &wait_x, &signal_y);
  if (rc) return rc;
  if ((rc = stamp(MOE_B200_EP_EV_EXPERTS))) return rc;
  rc = launch_combine(peers.ret_y[rank], nullptr, w, residual, N_local, d, k, dtype, out, s, &wait_y,
                      status);
  if (rc) return rc;
  return stamp(MOE_B200_EP_EV_COMBINE);
}

}  // extern "C"
