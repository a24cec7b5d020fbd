// extern "C" entry points of training mode (declared in include/moe_b200.h): the forward with
// dropout on h and the tensors the backward pass needs (reference model.py:164,183 under
// .train()), and the backward pass itself (what torch.autograd derives for model.py:200-276
// and 173-190 when the reference trains, train.py:140-141).
#include <cuda.h>
#include <string.h>
#include "common.cuh"

namespace moe {
namespace {

size_t up1k(size_t v) { return (v + 1023) & ~(size_t)1023; }

int train_check(int64_t N, int d, int f, int E, int k, int dtype, float p) {
  if (dtype != MOE_B200_BF16)
    return set_error(MOE_B200_ERR_DTYPE, "training mode computes in bf16");
  if (N < 0 || d < 8 || (d & 7) || f < 8 || (f & 7) || E < 1 || E > kMaxExperts || k < 1 ||
      k > kMaxTopK || k > E || N * (int64_t)k >= (int64_t)1 << 31)
    return set_error(MOE_B200_ERR_SHAPE, "N, d, f, E or k out of range");
  if (!(p >= 0.f && p < 1.f)) return set_error(MOE_B200_ERR_SHAPE, "dropout probability must be in [0,1)");
  return 0;
}

int64_t padded_rows(int64_t M, int E) { return ((M + 63) & ~(int64_t)63) + (int64_t)64 * E; }

void tws_layout(int64_t N, int d, int f, int E, int k, size_t* off, size_t* total) {
  const size_t M = (size_t)N * k;
  const size_t Kp = (size_t)padded_rows((int64_t)M, E);
  size_t sizes[MOE_B200_TWS_NUM];
  sizes[MOE_B200_TWS_GU] = M * 2 * f * 2;
  sizes[MOE_B200_TWS_PAIR_OF] = M * sizeof(int32_t);
  sizes[MOE_B200_TWS_KOFF] = (size_t)(E + 1) * sizeof(int32_t);
  sizes[MOE_B200_TWS_DY] = M * d * 2;
  sizes[MOE_B200_TWS_DH] = M * f * 2;
  sizes[MOE_B200_TWS_DXS] = M * d * 2;
  sizes[MOE_B200_TWS_W1T] = (size_t)E * d * 2 * f * 2;
  sizes[MOE_B200_TWS_W2T] = (size_t)E * f * d * 2;
  sizes[MOE_B200_TWS_TMAPS] = (size_t)2 * E * 128;
  sizes[MOE_B200_TWS_XT] = (size_t)d * Kp * 2;
  sizes[MOE_B200_TWS_HT] = (size_t)f * Kp * 2;
  sizes[MOE_B200_TWS_DYT] = (size_t)d * Kp * 2;
  sizes[MOE_B200_TWS_DGUT] = (size_t)2 * f * Kp * 2;
  sizes[MOE_B200_TWS_DL] = (size_t)N * E * sizeof(float);
  sizes[MOE_B200_TWS_DW] = M * sizeof(float);
  sizes[MOE_B200_TWS_ONES] = M * sizeof(float);
  sizes[MOE_B200_TWS_DWG_F32] = ((size_t)E * d + E) * sizeof(float);
  sizes[MOE_B200_TWS_DXR] = (size_t)N * d * 2;
  sizes[MOE_B200_TWS_G_WG] = (size_t)E * d * 2;
  sizes[MOE_B200_TWS_G_BG] = (size_t)E * 2;
  sizes[MOE_B200_TWS_G_W1] = (size_t)E * 2 * f * d * 2;
  sizes[MOE_B200_TWS_G_B1] = (size_t)E * 2 * f * 2;
  sizes[MOE_B200_TWS_G_W2] = (size_t)E * d * f * 2;
  sizes[MOE_B200_TWS_G_B2] = (size_t)E * d * 2;
  size_t pos = 0;
  for (int i = 0; i < MOE_B200_TWS_NUM; ++i) {
    off[i] = pos;
    pos += up1k(sizes[i] ? sizes[i] : 1);
  }
  *total = pos;
}

TrainArgs train_args(char* tws, const size_t* to, float p, uint64_t seed) {
  TrainArgs tr;
  tr.gu = reinterpret_cast<__nv_bfloat16*>(tws + to[MOE_B200_TWS_GU]);
  tr.pair_of = reinterpret_cast<const int32_t*>(tws + to[MOE_B200_TWS_PAIR_OF]);
  const double t = (double)p * 4294967296.0;
  tr.thresh = p <= 0.f ? 0u : (uint32_t)(t >= 4294967295.0 ? 4294967295.0 : t);
  tr.scale = 1.0f / (1.0f - p);
  tr.seed_lo = (uint32_t)seed;
  tr.seed_hi = (uint32_t)(seed >> 32);
  return tr;
}

// Backward of the grouped expert feed-forward (model.py:174-184) on sorted rows: given dy (gradient
// of y, in the training workspace), h (the dropped h of the forward), the saved pre-activations and
// the sorted inputs, writes dxs (gradient of the sorted inputs) and the four parameter gradients.
int experts_backward(const void* perm, const void* h, const int32_t* offsets, const void* plan,
                     int64_t M, int d, int f, int E, const TrainArgs& tr, char* tws, const size_t* to,
                     int32_t* status, cudaStream_t s) {
  const int64_t Kp = padded_rows(M, E);
  const PlanView pv = plan_view(plan, E);
  int32_t* koff = reinterpret_cast<int32_t*>(tws + to[MOE_B200_TWS_KOFF]);
  void* gu = tws + to[MOE_B200_TWS_GU];
  void* dy = tws + to[MOE_B200_TWS_DY];
  void* dh = tws + to[MOE_B200_TWS_DH];
  void* dxs = tws + to[MOE_B200_TWS_DXS];
  const char* tmaps = tws + to[MOE_B200_TWS_TMAPS];
  // experts without rows get no tile in the weight-gradient products
  MOE_CUDA_CHECK(cudaMemsetAsync(tws + to[MOE_B200_TWS_G_W1], 0, (size_t)E * 2 * f * d * 2, s));
  MOE_CUDA_CHECK(cudaMemsetAsync(tws + to[MOE_B200_TWS_G_W2], 0, (size_t)E * d * f * 2, s));
  int rc = launch_pad_offsets(offsets, E, koff, s);
  if (rc) return rc;
  // down Linear (model.py:184): dh = dy W2, dW2 = dy^T h, db2 = column sums of dy
  rc = launch_transpose_weights(pv.W2, E, d, f, tws + to[MOE_B200_TWS_W2T], s);
  if (rc) return rc;
  rc = launch_grouped_rows(dy, M, d, tmaps + (size_t)128 * E, offsets, nullptr, E, f, dh, status, s);
  if (rc) return rc;
  rc = launch_transpose_pad(dy, offsets, koff, E, d, Kp, tws + to[MOE_B200_TWS_DYT], s);
  if (rc) return rc;
  rc = launch_transpose_pad(h, offsets, koff, E, f, Kp, tws + to[MOE_B200_TWS_HT], s);
  if (rc) return rc;
  rc = launch_grouped_cols(tws + to[MOE_B200_TWS_DYT], tws + to[MOE_B200_TWS_HT], Kp, d, f, koff,
                           tws + to[MOE_B200_TWS_G_W2], E, status, s);
  if (rc) return rc;
  rc = launch_colsum(dy, offsets, E, d, tws + to[MOE_B200_TWS_G_B2], s);
  if (rc) return rc;
  // dropout, product and GELU (model.py:180-183): (g, u) -> (dg, du) in place
  rc = launch_geglu_bwd(dh, gu, tr.pair_of, M, f, tr.thresh, tr.scale, tr.seed_lo, tr.seed_hi, s);
  if (rc) return rc;
  // gate_and_up Linear (model.py:174): dx = dgu W1, dW1 = dgu^T x, db1 = column sums of dgu
  rc = launch_transpose_weights(pv.W1, E, 2 * f, d, tws + to[MOE_B200_TWS_W1T], s);
  if (rc) return rc;
  rc = launch_grouped_rows(gu, M, 2 * f, tmaps, offsets, nullptr, E, d, dxs, status, s);
  if (rc) return rc;
  rc = launch_transpose_pad(gu, offsets, koff, E, 2 * f, Kp, tws + to[MOE_B200_TWS_DGUT], s);
  if (rc) return rc;
  rc = launch_transpose_pad(perm, offsets, koff, E, d, Kp, tws + to[MOE_B200_TWS_XT], s);
  if (rc) return rc;
  rc = launch_grouped_cols(tws + to[MOE_B200_TWS_DGUT], tws + to[MOE_B200_TWS_XT], Kp, 2 * f, d, koff,
                           tws + to[MOE_B200_TWS_G_W1], E, status, s);
  if (rc) return rc;
  return launch_colsum(gu, offsets, E, 2 * f, tws + to[MOE_B200_TWS_G_B1], s);
}

}  // namespace
}  // namespace moe

using namespace moe;

extern "C" {

size_t moe_b200_train_workspace_bytes(int64_t N, int d, int f, int E, int k, int dtype) {
  if (train_check(N, d, f, E, k, dtype, 0.f)) return 0;
  size_t off[MOE_B200_TWS_NUM], total;
  tws_layout(N, d, f, E, k, off, &total);
  return total;
}

int moe_b200_train_workspace_layout(int64_t N, int d, int f, int E, int k, int dtype, size_t* h_offsets) {
  if (!h_offsets) return set_error(MOE_B200_ERR_NULL, "h_offsets is NULL");
  int rc = train_check(N, d, f, E, k, dtype, 0.f);
  if (rc) return rc;
  size_t total;
  tws_layout(N, d, f, E, k, h_offsets, &total);
  return 0;
}

int moe_b200_train_setup(int64_t N, int d, int f, int E, int k, int dtype, void* train_ws,
                         size_t train_ws_bytes, void* stream) {
  int rc = train_check(N, d, f, E, k, dtype, 0.f);
  if (rc) return rc;
  if (!train_ws) return set_error(MOE_B200_ERR_NULL, "train_ws is NULL");
  size_t to[MOE_B200_TWS_NUM], total;
  tws_layout(N, d, f, E, k, to, &total);
  if (train_ws_bytes < total) return set_error(MOE_B200_ERR_WORKSPACE, "training workspace too small");
  if ((uintptr_t)train_ws & 1023) return set_error(MOE_B200_ERR_ALIGN, "training workspace must be 1024-byte aligned");
  char* tws = static_cast<char*>(train_ws);
  cudaStream_t s = (cudaStream_t)stream;
  // tensor maps of the transposed weight buffers (their addresses never change)
  const size_t nmaps = (size_t)2 * E;
  unsigned char* maps = static_cast<unsigned char*>(aligned_alloc(128, nmaps * 128));
  if (!maps) return set_error(MOE_B200_ERR_WORKSPACE, "out of host memory");
  for (int e = 0; e < E && rc == 0; ++e) {
    rc = encode_tmap_2d(maps + 128 * (size_t)e, tws + to[MOE_B200_TWS_W1T] + (size_t)e * d * 2 * f * 2,
                        (uint64_t)d, (uint64_t)2 * f, 128);
    if (rc == 0)
      rc = encode_tmap_2d(maps + 128 * (size_t)(E + e), tws + to[MOE_B200_TWS_W2T] + (size_t)e * f * d * 2,
                          (uint64_t)f, (uint64_t)d, 128);
  }
  if (rc == 0) {
    cudaError_t ce = cudaMemcpyAsync(tws + to[MOE_B200_TWS_TMAPS], maps, nmaps * 128, cudaMemcpyHostToDevice, s);
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(s);
    if (ce != cudaSuccess) rc = cuda_error(ce, "upload of the tensor maps");
  }
  free(maps);
  if (rc) return rc;
  return launch_fill_f32(reinterpret_cast<float*>(tws + to[MOE_B200_TWS_ONES]), N * (int64_t)k, 1.0f, s);
}

int moe_b200_forward_train(const void* x, const void* Wg, const void* bg, const void* plan,
                           const void* residual, int64_t N, int d, int f, int E, int k, int dtype,
                           float dropout_p, uint64_t seed, void* workspace, size_t workspace_bytes,
                           void* train_ws, size_t train_ws_bytes, void* out, void* stream) {
  int rc = train_check(N, d, f, E, k, dtype, dropout_p);
  if (rc) return rc;
  if (!workspace || !train_ws) return set_error(MOE_B200_ERR_NULL, "workspace is NULL");
  size_t off[MOE_B200_WS_NUM], to[MOE_B200_TWS_NUM], ttotal;
  rc = moe_b200_workspace_layout(N, d, f, E, k, dtype, off);
  if (rc) return rc;
  if (workspace_bytes < moe_b200_workspace_bytes(N, d, f, E, k, dtype))
    return set_error(MOE_B200_ERR_WORKSPACE, "workspace too small");
  tws_layout(N, d, f, E, k, to, &ttotal);
  if (train_ws_bytes < ttotal) return set_error(MOE_B200_ERR_WORKSPACE, "training workspace too small");
  if (((uintptr_t)workspace & 1023) || ((uintptr_t)train_ws & 1023))
    return set_error(MOE_B200_ERR_ALIGN, "workspaces must be 1024-byte aligned");
  if (N == 0) return 0;
  if (!x || !Wg || !bg || !plan || !out) return set_error(MOE_B200_ERR_NULL, "NULL argument");
  char* ws = static_cast<char*>(workspace);
  char* tws = static_cast<char*>(train_ws);
  int32_t* status = reinterpret_cast<int32_t*>(ws + off[MOE_B200_WS_STATUS]);
  float* logits = reinterpret_cast<float*>(ws + off[MOE_B200_WS_LOGITS]);
  int32_t* idx = reinterpret_cast<int32_t*>(ws + off[MOE_B200_WS_IDX]);
  float* w = reinterpret_cast<float*>(ws + off[MOE_B200_WS_W]);
  float* psum_part = reinterpret_cast<float*>(ws + off[MOE_B200_WS_PSUM_PART]);
  int32_t* row_of = reinterpret_cast<int32_t*>(ws + off[MOE_B200_WS_ROW_OF]);
  int32_t* offsets = reinterpret_cast<int32_t*>(ws + off[MOE_B200_WS_OFFSETS]);
  void* perm = ws + off[MOE_B200_WS_PERM];
  void* h = ws + off[MOE_B200_WS_H];
  void* y = ws + off[MOE_B200_WS_Y];
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t M = N * k;
  MOE_CUDA_CHECK(cudaMemsetAsync(status, 0, (MOE_B200_READY_OFFSET + MOE_B200_READY_INTS) * sizeof(int32_t), s));
  // training always takes the large-N kernels: the backward pass works on their sorted buffers
  rc = moe_b200_router(x, Wg, bg, N, d, E, k, dtype, logits, idx, w, psum_part, status, stream);
  if (rc) return rc;
  rc = moe_b200_dispatch(x, idx, N, d, E, k, dtype, reinterpret_cast<int32_t*>(ws + off[MOE_B200_WS_SCRATCH]),
                         reinterpret_cast<int32_t*>(ws + off[MOE_B200_WS_CNT_SLOT]), offsets, row_of, perm,
                         psum_part, reinterpret_cast<float*>(ws + off[MOE_B200_WS_PSUM]),
                         reinterpret_cast<float*>(ws + off[MOE_B200_WS_AUX]), status, stream);
  if (rc) return rc;
  rc = launch_pair_of(row_of, M, reinterpret_cast<int32_t*>(tws + to[MOE_B200_TWS_PAIR_OF]), s);
  if (rc) return rc;
  const TrainArgs tr = train_args(tws, to, dropout_p, seed);
  rc = launch_experts_tc2(perm, offsets, plan, M, d, f, E, h, y, nullptr, status, s, &tr);
  if (rc) return rc;
  return moe_b200_combine(y, row_of, w, residual, N, d, k, dtype, out, stream);
}

int moe_b200_backward(const void* x, const void* Wg, const void* plan, const void* grad_out,
                      float grad_aux, int64_t N, int d, int f, int E, int k, int dtype,
                      float dropout_p, uint64_t seed, void* workspace, size_t workspace_bytes,
                      void* train_ws, size_t train_ws_bytes, void* grad_x, void* stream) {
  int rc = train_check(N, d, f, E, k, dtype, dropout_p);
  if (rc) return rc;
  if (!workspace || !train_ws) return set_error(MOE_B200_ERR_NULL, "workspace is NULL");
  size_t off[MOE_B200_WS_NUM], to[MOE_B200_TWS_NUM], ttotal;
  rc = moe_b200_workspace_layout(N, d, f, E, k, dtype, off);
  if (rc) return rc;
  if (workspace_bytes < moe_b200_workspace_bytes(N, d, f, E, k, dtype))
    return set_error(MOE_B200_ERR_WORKSPACE, "workspace too small");
  tws_layout(N, d, f, E, k, to, &ttotal);
  if (train_ws_bytes < ttotal) return set_error(MOE_B200_ERR_WORKSPACE, "training workspace too small");
  if (N == 0) return 0;
  if (!x || !Wg || !plan || !grad_out || !grad_x) return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (!aligned16(grad_out) || !aligned16(grad_x) || !aligned16(x))
    return set_error(MOE_B200_ERR_ALIGN, "buffers must be 16-byte aligned");
  char* ws = static_cast<char*>(workspace);
  char* tws = static_cast<char*>(train_ws);
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t M = N * k;
  const int64_t Kp = padded_rows(M, E);
  int32_t* status = reinterpret_cast<int32_t*>(ws + off[MOE_B200_WS_STATUS]);
  const float* logits = reinterpret_cast<const float*>(ws + off[MOE_B200_WS_LOGITS]);
  const int32_t* idx = reinterpret_cast<const int32_t*>(ws + off[MOE_B200_WS_IDX]);
  const float* w = reinterpret_cast<const float*>(ws + off[MOE_B200_WS_W]);
  const int32_t* cnt_slot = reinterpret_cast<const int32_t*>(ws + off[MOE_B200_WS_CNT_SLOT]);
  const int32_t* offsets = reinterpret_cast<const int32_t*>(ws + off[MOE_B200_WS_OFFSETS]);
  const int32_t* row_of = reinterpret_cast<const int32_t*>(ws + off[MOE_B200_WS_ROW_OF]);
  const void* perm = ws + off[MOE_B200_WS_PERM];
  const void* h = ws + off[MOE_B200_WS_H];
  const void* y = ws + off[MOE_B200_WS_Y];
  const int32_t* pair_of = reinterpret_cast<const int32_t*>(tws + to[MOE_B200_TWS_PAIR_OF]);
  int32_t* koff = reinterpret_cast<int32_t*>(tws + to[MOE_B200_TWS_KOFF]);
  void* gu = tws + to[MOE_B200_TWS_GU];
  void* dy = tws + to[MOE_B200_TWS_DY];
  void* dh = tws + to[MOE_B200_TWS_DH];
  void* dxs = tws + to[MOE_B200_TWS_DXS];
  void* w1t = tws + to[MOE_B200_TWS_W1T];
  void* w2t = tws + to[MOE_B200_TWS_W2T];
  const char* tmaps = tws + to[MOE_B200_TWS_TMAPS];
  float* dl = reinterpret_cast<float*>(tws + to[MOE_B200_TWS_DL]);
  float* dw = reinterpret_cast<float*>(tws + to[MOE_B200_TWS_DW]);
  const float* ones = reinterpret_cast<const float*>(tws + to[MOE_B200_TWS_ONES]);
  float* dwg32 = reinterpret_cast<float*>(tws + to[MOE_B200_TWS_DWG_F32]);
  void* dxr = tws + to[MOE_B200_TWS_DXR];
  const PlanView pv = plan_view(plan, E);
  const TrainArgs tr = train_args(tws, to, dropout_p, seed);

  // combine (model.py:271) and router (model.py:206-223)
  rc = launch_combine_bwd(grad_out, y, pair_of, w, M, d, k, dy, dw, s);
  if (rc) return rc;
  rc = launch_router_bwd(logits, idx, w, dw, cnt_slot, grad_aux, x, Wg, N, d, E, k, dl, dwg32,
                         dwg32 + (size_t)E * d, tws + to[MOE_B200_TWS_G_WG], tws + to[MOE_B200_TWS_G_BG],
                         dxr, s);
  if (rc) return rc;
  // the experts (model.py:174-184)
  rc = experts_backward(perm, h, offsets, plan, M, d, f, E, tr, tws, to, status, s);
  if (rc) return rc;
  // gather (model.py:248-253) and the router's share: dx[t] = sum_j dxs[row_of[t,j]] + dxr[t]
  return launch_combine(dxs, row_of, ones, dxr, N, d, k, dtype, grad_x, s);
}

// ---- the expert feed-forward alone (the reference's dense FeedForward, model.py:154-190, is one
// group; any grouping by offsets works) ----

int moe_b200_experts_train(const void* x_sorted, const int32_t* offsets, const void* plan, int64_t M,
                           int d, int f, int E, float dropout_p, uint64_t seed, void* train_ws,
                           size_t train_ws_bytes, void* h, void* y, int32_t* status, void* stream) {
  int rc = train_check(M, d, f, E, 1, MOE_B200_BF16, dropout_p);
  if (rc) return rc;
  if (M == 0) return 0;
  if (!x_sorted || !offsets || !plan || !train_ws || !h || !y || !status)
    return set_error(MOE_B200_ERR_NULL, "NULL argument");
  size_t to[MOE_B200_TWS_NUM], ttotal;
  tws_layout(M, d, f, E, 1, to, &ttotal);
  if (train_ws_bytes < ttotal) return set_error(MOE_B200_ERR_WORKSPACE, "training workspace too small");
  if ((uintptr_t)train_ws & 1023) return set_error(MOE_B200_ERR_ALIGN, "training workspace must be 1024-byte aligned");
  char* tws = static_cast<char*>(train_ws);
  cudaStream_t s = (cudaStream_t)stream;
  // row r is pair r: the dropout mask of element (r, c) depends on the row's position only
  rc = launch_iota(reinterpret_cast<int32_t*>(tws + to[MOE_B200_TWS_PAIR_OF]), M, s);
  if (rc) return rc;
  const TrainArgs tr = train_args(tws, to, dropout_p, seed);
  return launch_experts_tc2(x_sorted, offsets, plan, M, d, f, E, h, y, nullptr, status, s, &tr);
}

int moe_b200_experts_backward(const void* x_sorted, const void* h, const int32_t* offsets,
                              const void* plan, const void* grad_y, int64_t M, int d, int f, int E,
                              float dropout_p, uint64_t seed, void* train_ws, size_t train_ws_bytes,
                              void* grad_x, int32_t* status, void* stream) {
  int rc = train_check(M, d, f, E, 1, MOE_B200_BF16, dropout_p);
  if (rc) return rc;
  if (M == 0) return 0;
  if (!x_sorted || !h || !offsets || !plan || !grad_y || !train_ws || !grad_x || !status)
    return set_error(MOE_B200_ERR_NULL, "NULL argument");
  size_t to[MOE_B200_TWS_NUM], ttotal;
  tws_layout(M, d, f, E, 1, to, &ttotal);
  if (train_ws_bytes < ttotal) return set_error(MOE_B200_ERR_WORKSPACE, "training workspace too small");
  char* tws = static_cast<char*>(train_ws);
  cudaStream_t s = (cudaStream_t)stream;
  const TrainArgs tr = train_args(tws, to, dropout_p, seed);
  MOE_CUDA_CHECK(cudaMemcpyAsync(tws + to[MOE_B200_TWS_DY], grad_y, (size_t)M * d * 2, cudaMemcpyDeviceToDevice, s));
  rc = experts_backward(x_sorted, h, offsets, plan, M, d, f, E, tr, tws, to, status, s);
  if (rc) return rc;
  MOE_CUDA_CHECK(cudaMemcpyAsync(grad_x, tws + to[MOE_B200_TWS_DXS], (size_t)M * d * 2, cudaMemcpyDeviceToDevice, s));
  return 0;
}

}  // extern "C"
