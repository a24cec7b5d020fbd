// extern "C" surface of libmoe_b200 (declared in include/moe_b200.h): argument
// checks on the host, workspace layout, plan construction, and the launch
// sequence of the whole block (reference MOE.forward, model.py:200-276).
#include <cuda.h>
#include <stdio.h>
#include <string.h>
#include "common.cuh"

namespace moe {

static thread_local char g_err[256] = "ok";

int set_error(int code, const char* msg) {
  snprintf(g_err, sizeof(g_err), "%s", msg);
  return code;
}
int cuda_error(cudaError_t e, const char* where) {
  snprintf(g_err, sizeof(g_err), "CUDA error %d (%s) at %s", (int)e, cudaGetErrorString(e), where);
  return 1000 + (int)e;
}

int64_t dispatch_scratch_ints(int64_t N, int E, int k);

static int check_shape(int64_t N, int d, int f, int E, int k, int dtype) {
  if (dtype != MOE_B200_F32 && dtype != MOE_B200_BF16)
    return set_error(MOE_B200_ERR_DTYPE, "dtype must be MOE_B200_F32 or MOE_B200_BF16");
  if (N < 0 || N > (int64_t)1 << 28) return set_error(MOE_B200_ERR_SHAPE, "N out of range");
  if (d < 8 || (d & 7)) return set_error(MOE_B200_ERR_SHAPE, "d must be a positive multiple of 8");
  if (f < 8 || (f & 7)) return set_error(MOE_B200_ERR_SHAPE, "f must be a positive multiple of 8");
  if (E < 1 || E > kMaxExperts) return set_error(MOE_B200_ERR_SHAPE, "E must be in [1,256]");
  if (k < 1 || k > kMaxTopK || k > E) return set_error(MOE_B200_ERR_SHAPE, "k must be in [1,min(8,E)]");
  if (N * (int64_t)k >= (int64_t)1 << 31) return set_error(MOE_B200_ERR_SHAPE, "N*k exceeds int32 rows");
  return 0;
}

static size_t align_up(size_t v) { return (v + 1023) & ~(size_t)1023; }

static void layout(int64_t N, int d, int f, int E, int k, int dtype, size_t* off, size_t* total) {
  const size_t es = dtype == MOE_B200_BF16 ? 2 : 4;
  const size_t M = (size_t)N * k;
  const size_t rb = (size_t)((N + kRouterTokensPerBlock - 1) / kRouterTokensPerBlock);
  size_t sizes[MOE_B200_WS_NUM];
  sizes[MOE_B200_WS_STATUS] = (MOE_B200_READY_OFFSET + MOE_B200_READY_INTS) * sizeof(int32_t);
  sizes[MOE_B200_WS_LOGITS] = (size_t)N * E * sizeof(float);
  sizes[MOE_B200_WS_IDX] = M * sizeof(int32_t);
  sizes[MOE_B200_WS_W] = M * sizeof(float);
  sizes[MOE_B200_WS_PSUM_PART] = rb * E * sizeof(float);
  sizes[MOE_B200_WS_PSUM] = (size_t)E * sizeof(float);
  sizes[MOE_B200_WS_AUX] = sizeof(float);
  sizes[MOE_B200_WS_SCRATCH] = (size_t)dispatch_scratch_ints(N, E, k) * sizeof(int32_t);
  if (front_split_supported(N, E, k, dtype) &&
      (size_t)front_small_exchange_ints(N, E, k) * sizeof(int32_t) > sizes[MOE_B200_WS_SCRATCH])
    sizes[MOE_B200_WS_SCRATCH] = (size_t)front_small_exchange_ints(N, E, k) * sizeof(int32_t);
  sizes[MOE_B200_WS_CNT_SLOT] = (size_t)k * E * sizeof(int32_t);
  sizes[MOE_B200_WS_OFFSETS] = (size_t)(E + 1) * sizeof(int32_t);
  sizes[MOE_B200_WS_ROW_OF] = M * sizeof(int32_t);
  sizes[MOE_B200_WS_PERM] = M * d * es;
  sizes[MOE_B200_WS_H] = M * f * es;
  if (dtype == MOE_B200_BF16 && decode_spec_supported(N, E, k)) {
    // the routing-independent small-N kernel keeps one slab of h per expert
    const size_t slabs = (size_t)E * decode_spec_rows(N) * f * es;
    if (slabs > sizes[MOE_B200_WS_H]) sizes[MOE_B200_WS_H] = slabs;
  }
  sizes[MOE_B200_WS_Y] = M * d * es;
  sizes[MOE_B200_WS_PART] =
      (dtype == MOE_B200_BF16 && M <= kDecodeMaxRows) ? (size_t)decode_splits(f) * M * d * sizeof(float) : 0;
  if (dtype == MOE_B200_BF16 && (int64_t)M > kDecodeMaxRows && (int64_t)M <= kRowsPathMaxRows)
    sizes[MOE_B200_WS_PART] = (size_t)rows_splits((int64_t)M, d, f, E) * M * d * sizeof(float);
  sizes[MOE_B200_WS_NORM_W] = (size_t)E * d * es;
  sizes[MOE_B200_WS_NORM_C] = (size_t)2 * E * sizeof(float);
  sizes[MOE_B200_WS_STATS] = (size_t)N * 2 * sizeof(float);
  sizes[MOE_B200_WS_XN] = (int64_t)M <= kRowsPathMaxRows ? (size_t)N * d * es : 0;
  size_t pos = 0;
  for (int i = 0; i < MOE_B200_WS_NUM; ++i) {
    off[i] = pos;
    pos += align_up(sizes[i] ? sizes[i] : 1);
  }
  *total = pos;
}

}  // namespace moe

using namespace moe;

extern "C" {

int moe_b200_version(void) { return MOE_B200_ABI_VERSION; }

const char* moe_b200_last_error_string(void) { return g_err; }

size_t moe_b200_workspace_bytes(int64_t N, int d, int f, int E, int k, int dtype) {
  if (check_shape(N, d, f, E, k, dtype)) return 0;
  size_t off[MOE_B200_WS_NUM], total;
  layout(N, d, f, E, k, dtype, off, &total);
  return total;
}

int moe_b200_workspace_layout(int64_t N, int d, int f, int E, int k, int dtype, size_t* h_offsets) {
  if (h_offsets == nullptr) return set_error(MOE_B200_ERR_NULL, "h_offsets is NULL");
  int rc = check_shape(N, d, f, E, k, dtype);
  if (rc) return rc;
  size_t total;
  layout(N, d, f, E, k, dtype, h_offsets, &total);
  return 0;
}

size_t moe_b200_plan_bytes(int E) {
  if (E < 1 || E > kMaxExperts) return 0;
  return plan_ptr_bytes(E) + (size_t)kPlanMapsPerExpert * E * 128;
}

int moe_b200_plan_build(const void* const* h_W1, const void* const* h_b1, const void* const* h_W2,
                        const void* const* h_b2, int E, int d, int f, int dtype, void* plan,
                        size_t plan_bytes, void* stream) {
  if (!h_W1 || !h_b1 || !h_W2 || !h_b2 || !plan) return set_error(MOE_B200_ERR_NULL, "NULL argument");
  int rc = check_shape(0, d, f, E, 1, dtype);
  if (rc) return rc;
  if (plan_bytes < moe_b200_plan_bytes(E)) return set_error(MOE_B200_ERR_WORKSPACE, "plan buffer too small");
  if (!aligned16(plan) || ((uintptr_t)plan & 127)) return set_error(MOE_B200_ERR_ALIGN, "plan must be 128-byte aligned");
  for (int e = 0; e < E; ++e) {
    if (!h_W1[e] || !h_b1[e] || !h_W2[e] || !h_b2[e]) return set_error(MOE_B200_ERR_NULL, "NULL expert parameter");
    if (!aligned16(h_W1[e]) || !aligned16(h_W2[e]) || !aligned16(h_b1[e]) || !aligned16(h_b2[e]))
      return set_error(MOE_B200_ERR_ALIGN, "expert parameters must be 16-byte aligned");
  }
  const size_t bytes = moe_b200_plan_bytes(E);
  // staged on the host stack/heap; cudaMemcpyAsync from pageable memory copies
  // the source before it returns
  static thread_local unsigned char* stage = nullptr;
  static thread_local size_t stage_cap = 0;
  if (stage_cap < bytes) {
    free(stage);
    stage = static_cast<unsigned char*>(aligned_alloc(128, (bytes + 127) & ~(size_t)127));
    stage_cap = bytes;
  }
  memset(stage, 0, bytes);
  const void** ptrs = reinterpret_cast<const void**>(stage);
  for (int e = 0; e < E; ++e) {
    ptrs[e] = h_W1[e];
    ptrs[E + e] = h_b1[e];
    ptrs[2 * E + e] = h_W2[e];
    ptrs[3 * E + e] = h_b2[e];
  }
  if (dtype == MOE_B200_BF16) {
    rc = build_weight_tensor_maps(h_W1, h_W2, E, d, f, stage + plan_ptr_bytes(E));
    if (rc) return rc;
  }
  MOE_CUDA_CHECK(cudaMemcpyAsync(plan, stage, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
  // the staging buffer is reused by the next call on this thread
  MOE_CUDA_CHECK(cudaStreamSynchronize((cudaStream_t)stream));
  return 0;
}

int64_t moe_b200_router_blocks(int64_t N) {
  return (N + kRouterTokensPerBlock - 1) / kRouterTokensPerBlock;
}

size_t moe_b200_dispatch_scratch_bytes(int64_t N, int E, int k) {
  if (N < 0 || E < 1 || E > kMaxExperts || k < 1 || k > kMaxTopK) return 0;
  return (size_t)dispatch_scratch_ints(N, E, k) * sizeof(int32_t);
}

int moe_b200_router(const void* x, const void* Wg, const void* bg, int64_t N, int d, int E, int k,
                    int dtype, float* out_logits, int32_t* out_idx, float* out_w, float* psum_part,
                    int32_t* status, void* stream) {
  int rc = check_shape(N, d, 8, E, k, dtype);
  if (rc) return rc;
  if (N == 0) return 0;
  if (!x || !Wg || !bg || !out_idx || !out_w || !psum_part) return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (!aligned16(x) || !aligned16(Wg)) return set_error(MOE_B200_ERR_ALIGN, "x and Wg must be 16-byte aligned");
  return launch_router(x, Wg, bg, N, d, E, k, dtype, out_logits, out_idx, out_w, psum_part, status,
                       (cudaStream_t)stream);
}

int moe_b200_dispatch(const void* x, const int32_t* idx, int64_t N, int d, int E, int k, int dtype,
                      int32_t* scratch, int32_t* cnt_slot, int32_t* offsets, int32_t* row_of,
                      void* perm, const float* psum_part, float* psum, float* aux, int32_t* status,
                      void* stream) {
  int rc = check_shape(N, d, 8, E, k, dtype);
  if (rc) return rc;
  if (!scratch || !cnt_slot || !offsets || !status) return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (N > 0 && (!x || !idx || !row_of || !perm)) return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (psum_part && (!psum || !aux)) return set_error(MOE_B200_ERR_NULL, "psum and aux are required with psum_part");
  if (!aligned16(x) || !aligned16(perm)) return set_error(MOE_B200_ERR_ALIGN, "x and perm must be 16-byte aligned");
  return launch_dispatch(x, idx, N, d, E, k, dtype, scratch, cnt_slot, offsets, row_of, perm,
                         psum_part, psum, aux, status, (cudaStream_t)stream);
}

int moe_b200_norm_fold(const void* Wg, const void* bg, const void* norm_weight, const void* norm_bias,
                       int E, int d, int dtype, void* out_Wn, float* out_c, void* stream) {
  int rc = check_shape(0, d, 8, E, 1, dtype);
  if (rc) return rc;
  if (!Wg || !bg || !norm_weight || !norm_bias || !out_Wn || !out_c)
    return set_error(MOE_B200_ERR_NULL, "NULL argument");
  return launch_norm_fold(Wg, bg, norm_weight, norm_bias, E, d, dtype, out_Wn, out_c, (cudaStream_t)stream);
}

int moe_b200_router_norm(const void* x, const void* Wn, const float* c, float eps, int64_t N, int d,
                         int E, int k, int dtype, float* out_logits, int32_t* out_idx, float* out_w,
                         float* psum_part, float* out_stats, int32_t* status, void* stream) {
  int rc = check_shape(N, d, 8, E, k, dtype);
  if (rc) return rc;
  if (N == 0) return 0;
  if (!x || !Wn || !c || !out_idx || !out_w || !psum_part || !out_stats)
    return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (!(eps >= 0.f)) return set_error(MOE_B200_ERR_SHAPE, "eps must be non-negative");
  if (!aligned16(x) || !aligned16(Wn)) return set_error(MOE_B200_ERR_ALIGN, "x and Wn must be 16-byte aligned");
  return launch_router(x, Wn, nullptr, N, d, E, k, dtype, out_logits, out_idx, out_w, psum_part, status,
                       (cudaStream_t)stream, c, eps, out_stats);
}

int moe_b200_dispatch_norm(const void* x, const int32_t* idx, const float* stats,
                           const void* norm_weight, const void* norm_bias, int64_t N, int d, int E,
                           int k, int dtype, int32_t* scratch, int32_t* cnt_slot, int32_t* offsets,
                           int32_t* row_of, void* perm, const float* psum_part, float* psum,
                           float* aux, int32_t* status, void* stream) {
  int rc = check_shape(N, d, 8, E, k, dtype);
  if (rc) return rc;
  if (!scratch || !cnt_slot || !offsets || !status) return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (N > 0 && (!x || !idx || !row_of || !perm || !stats || !norm_weight || !norm_bias))
    return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (psum_part && (!psum || !aux)) return set_error(MOE_B200_ERR_NULL, "psum and aux are required with psum_part");
  if (!aligned16(x) || !aligned16(perm)) return set_error(MOE_B200_ERR_ALIGN, "x and perm must be 16-byte aligned");
  return launch_dispatch(x, idx, N, d, E, k, dtype, scratch, cnt_slot, offsets, row_of, perm,
                         psum_part, psum, aux, status, (cudaStream_t)stream, stats, norm_weight,
                         norm_bias);
}

int moe_b200_layernorm(const void* x, const void* norm_weight, const void* norm_bias, float eps,
                       int64_t N, int d, int dtype, void* out, void* stream) {
  int rc = check_shape(N, d, 8, 1, 1, dtype);
  if (rc) return rc;
  if (N == 0) return 0;
  if (!x || !norm_weight || !norm_bias || !out) return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (!aligned16(x) || !aligned16(out) || !aligned16(norm_weight) || !aligned16(norm_bias))
    return set_error(MOE_B200_ERR_ALIGN, "buffers must be 16-byte aligned");
  return launch_layernorm_rows(x, norm_weight, norm_bias, eps, N, d, dtype, out, nullptr,
                               (cudaStream_t)stream);
}

int moe_b200_experts(const void* perm, const int32_t* offsets, const void* plan, int64_t M, int d,
                     int f, int E, int dtype, int flags, void* h, void* y, int32_t* status,
                     void* stream) {
  int rc = check_shape(0, d, f, E, 1, dtype);
  if (rc) return rc;
  if (M < 0 || M >= (int64_t)1 << 31) return set_error(MOE_B200_ERR_SHAPE, "M out of range");
  if (M == 0) return 0;
  if (!perm || !offsets || !plan || !h || !y || !status) return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (!aligned16(perm) || !aligned16(h) || !aligned16(y)) return set_error(MOE_B200_ERR_ALIGN, "buffers must be 16-byte aligned");
  if (flags != 0) return set_error(MOE_B200_ERR_UNSUPPORTED, "flags must be 0");
  if (dtype == MOE_B200_BF16)
    return launch_experts_tc2(perm, offsets, plan, M, d, f, E, h, y, nullptr, status,
                              (cudaStream_t)stream);
  return launch_experts_simt(perm, offsets, plan, M, d, f, E, dtype, h, y, (cudaStream_t)stream);
}

int moe_b200_rows_splits(int64_t M, int d, int f, int E) { return M > 0 && f >= 8 && d >= 8 && E >= 1 ? rows_splits(M, d, f, E) : 0; }

int moe_b200_experts_rows(const void* perm, const int32_t* offsets, const void* plan, int64_t M,
                          int d, int f, int E, int ksplit, void* h, float* part, int32_t* ready,
                          int32_t* status, void* stream) {
  int rc = check_shape(0, d, f, E, 1, MOE_B200_BF16);
  if (rc) return rc;
  if (M < 0 || M >= (int64_t)1 << 31) return set_error(MOE_B200_ERR_SHAPE, "M out of range");
  if (M == 0) return 0;
  if (!rows_supported(M, E)) return set_error(MOE_B200_ERR_UNSUPPORTED, "too many 128-row blocks for the completion counters");
  if (ksplit < 1 || ksplit > 8 || ksplit > (f + 63) / 64) return set_error(MOE_B200_ERR_SHAPE, "ksplit must be in [1,8] and at most the number of 64-wide K blocks");
  if (!perm || !offsets || !plan || !h || !part || !ready || !status) return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (!aligned16(perm) || !aligned16(h) || !aligned16(part)) return set_error(MOE_B200_ERR_ALIGN, "buffers must be 16-byte aligned");
  MOE_CUDA_CHECK(cudaMemsetAsync(ready, 0, MOE_B200_READY_INTS * sizeof(int32_t), (cudaStream_t)stream));
  return launch_experts_tc_rows(perm, offsets, plan, M, d, f, E, ksplit, h, part, ready, status,
                                (cudaStream_t)stream);
}

int moe_b200_front_small(const void* x, const void* Wg, const void* bg, int64_t N, int d, int E,
                         int k, int dtype, float* out_logits, int32_t* out_idx, float* out_w,
                         int32_t* cnt_slot, int32_t* offsets, int32_t* row_of, void* perm,
                         float* psum, float* aux, void* stream) {
  int rc = check_shape(N, d, 8, E, k, dtype);
  if (rc) return rc;
  if (!front_small_supported(N, E, k, dtype))
    return set_error(MOE_B200_ERR_UNSUPPORTED,
                     "moe_b200_front_small needs bf16, 1 <= N <= 512, N*k <= 1024, E <= 32");
  if (!x || !Wg || !bg || !out_idx || !out_w || !cnt_slot || !offsets || !row_of || !perm || !psum || !aux)
    return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (!aligned16(x) || !aligned16(Wg) || !aligned16(perm))
    return set_error(MOE_B200_ERR_ALIGN, "x, Wg and perm must be 16-byte aligned");
  return launch_front_small(x, Wg, bg, N, d, E, k, out_logits, out_idx, out_w, cnt_slot, offsets,
                            row_of, perm, psum, aux, (cudaStream_t)stream);
}

int64_t moe_b200_front_exchange_ints(int64_t N, int E, int k) {
  return (N >= 1 && E >= 1 && k >= 1) ? front_small_exchange_ints(N, E, k) : 0;
}

int moe_b200_front_small_split(const void* x, const void* Wg, const void* bg, int64_t N, int d, int E,
                               int k, int dtype, float* out_logits, int32_t* out_idx, float* out_w,
                               int32_t* cnt_slot, int32_t* offsets, int32_t* row_of, void* perm,
                               float* psum, float* aux, int32_t* exchange, int32_t* counter,
                               int32_t* status, void* stream) {
  int rc = check_shape(N, d, 8, E, k, dtype);
  if (rc) return rc;
  if (!front_split_supported(N, E, k, dtype))
    return set_error(MOE_B200_ERR_UNSUPPORTED,
                     "moe_b200_front_small_split needs bf16, 1 <= N <= 2048, E <= 32");
  if (!x || !Wg || !bg || !out_idx || !out_w || !cnt_slot || !offsets || !row_of || !perm || !psum ||
      !aux || !exchange || !counter || !status)
    return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (!aligned16(x) || !aligned16(Wg) || !aligned16(perm))
    return set_error(MOE_B200_ERR_ALIGN, "x, Wg and perm must be 16-byte aligned");
  MOE_CUDA_CHECK(cudaMemsetAsync(counter, 0, sizeof(int32_t), (cudaStream_t)stream));
  return launch_front_small(x, Wg, bg, N, d, E, k, out_logits, out_idx, out_w, cnt_slot, offsets,
                            row_of, perm, psum, aux, (cudaStream_t)stream, exchange, counter, status);
}

int moe_b200_decode_tiny(const void* x, const void* Wg, const void* bg, const void* plan,
                         const void* residual, int64_t N, int d, int f, int E, int k,
                         float* out_logits, int32_t* out_idx, float* out_w, int32_t* cnt_slot,
                         int32_t* offsets, int32_t* row_of, void* perm, float* psum, float* aux,
                         void* h, void* out, int32_t* status, void* stream) {
  int rc = check_shape(N, d, f, E, k, MOE_B200_BF16);
  if (rc) return rc;
  if (!decode_tiny_supported(N, d, f, E, k, MOE_B200_BF16))
    return set_error(MOE_B200_ERR_UNSUPPORTED,
                     "moe_b200_decode_tiny needs 1 <= N <= 8, E <= 32, d and f multiples of 8");
  if (!x || !Wg || !bg || !plan || !out_idx || !out_w || !cnt_slot || !offsets || !row_of || !perm ||
      !psum || !aux || !h || !out || !status)
    return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (!aligned16(x) || !aligned16(Wg) || !aligned16(perm) || !aligned16(h) || !aligned16(out) ||
      (residual && !aligned16(residual)))
    return set_error(MOE_B200_ERR_ALIGN, "x, Wg, perm, h, out and residual must be 16-byte aligned");
  return launch_decode_tiny(x, Wg, bg, N, d, f, E, k, plan, residual, out_logits, out_idx, out_w,
                            cnt_slot, offsets, row_of, perm, psum, aux, h, out, status,
                            (cudaStream_t)stream);
}

int moe_b200_decode_splits(int f) { return f >= 8 ? decode_splits(f) : 0; }

int64_t moe_b200_decode_max_rows(void) { return kDecodeMaxRows; }

int moe_b200_experts_decode_fused(const void* perm, const int32_t* offsets, const void* plan,
                                  int64_t M, int d, int f, int E, void* h, float* part,
                                  int32_t* ready, int32_t* status, void* stream) {
  int rc = check_shape(0, d, f, E, 1, MOE_B200_BF16);
  if (rc) return rc;
  if (M < 0 || M > kDecodeMaxRows) return set_error(MOE_B200_ERR_SHAPE, "M exceeds the small-N path's row limit");
  if (M == 0) return 0;
  if (!perm || !offsets || !plan || !h || !part || !ready || !status) return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (!aligned16(perm) || !aligned16(h) || !aligned16(part)) return set_error(MOE_B200_ERR_ALIGN, "buffers must be 16-byte aligned");
  MOE_CUDA_CHECK(cudaMemsetAsync(ready, 0, MOE_B200_READY_INTS * sizeof(int32_t), (cudaStream_t)stream));
  return launch_experts_tc_decode_fused(perm, offsets, plan, M, d, f, E, h, part, ready, status,
                                        (cudaStream_t)stream);
}

int moe_b200_experts_gemv(const void* perm, const int32_t* offsets, const void* plan, int64_t M, int d,
                          int f, int E, void* h, float* part, void* stream) {
  int rc = check_shape(0, d, f, E, 1, MOE_B200_BF16);
  if (rc) return rc;
  if (M < 0 || M > kDecodeMaxRows) return set_error(MOE_B200_ERR_SHAPE, "M exceeds the small-N path's row limit");
  if (M == 0) return 0;
  if (!perm || !offsets || !plan || !h || !part) return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (!aligned16(perm) || !aligned16(h) || !aligned16(part)) return set_error(MOE_B200_ERR_ALIGN, "buffers must be 16-byte aligned");
  return launch_experts_gemv(perm, offsets, plan, M, d, f, E, decode_splits(f), h, part, (cudaStream_t)stream);
}

int moe_b200_decode_spec_rows(int64_t N) { return decode_spec_rows(N); }

int moe_b200_experts_decode_spec(const void* x, const int32_t* idx, const int32_t* offsets,
                                 const void* plan, int64_t N, int k, int d, int f, int E,
                                 void* h_all, float* part, int32_t* ready, int32_t* status,
                                 void* stream) {
  int rc = check_shape(N, d, f, E, k, MOE_B200_BF16);
  if (rc) return rc;
  if (!decode_spec_supported(N, E, k)) return set_error(MOE_B200_ERR_UNSUPPORTED, "needs N <= 128, E <= 32, N*k within the small-N row limit");
  if (!x || !idx || !offsets || !plan || !h_all || !part || !ready || !status) return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (!aligned16(x) || !aligned16(h_all) || !aligned16(part)) return set_error(MOE_B200_ERR_ALIGN, "buffers must be 16-byte aligned");
  MOE_CUDA_CHECK(cudaMemsetAsync(ready, 0, MOE_B200_READY_INTS * sizeof(int32_t), (cudaStream_t)stream));
  return launch_experts_tc_decode_spec(x, idx, offsets, plan, N, k, d, f, E, h_all, part, ready, status,
                                       (cudaStream_t)stream);
}

int moe_b200_combine_decode(const float* part, int ksplit, int64_t M, const int32_t* row_of,
                            const int32_t* idx, const float* w, const void* plan, int E,
                            const void* residual, int64_t N, int d, int k, void* out, void* stream) {
  int rc = check_shape(N, d, 8, E, k, MOE_B200_BF16);
  if (rc) return rc;
  if (N == 0) return 0;
  if (!part || !row_of || !idx || !w || !plan || !out) return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (ksplit < 1 || ksplit > 8 || M < 0) return set_error(MOE_B200_ERR_SHAPE, "ksplit or M out of range");
  if (!aligned16(part) || !aligned16(out) || !aligned16(residual)) return set_error(MOE_B200_ERR_ALIGN, "buffers must be 16-byte aligned");
  return launch_combine_decode(part, ksplit, M, row_of, idx, w, plan, E, residual, N, d, k, out, (cudaStream_t)stream);
}

int moe_b200_combine(const void* y, const int32_t* row_of, const float* w, const void* residual,
                     int64_t N, int d, int k, int dtype, void* out, void* stream) {
  int rc = check_shape(N, d, 8, k, k, dtype);
  if (rc) return rc;
  if (N == 0) return 0;
  if (!y || !row_of || !w || !out) return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (!aligned16(y) || !aligned16(out) || !aligned16(residual))
    return set_error(MOE_B200_ERR_ALIGN, "buffers must be 16-byte aligned");
  return launch_combine(y, row_of, w, residual, N, d, k, dtype, out, (cudaStream_t)stream);
}

int moe_b200_forward(const void* x, const void* Wg, const void* bg, const void* plan,
                     const void* residual, const void* norm_weight, const void* norm_bias,
                     float norm_eps, int64_t N, int d, int f, int E, int k, int dtype, int flags,
                     void* workspace, size_t workspace_bytes, void* out, void* stream) {
  int rc = check_shape(N, d, f, E, k, dtype);
  if (rc) return rc;
  if (!workspace) return set_error(MOE_B200_ERR_NULL, "workspace is NULL");
  size_t off[MOE_B200_WS_NUM], total;
  layout(N, d, f, E, k, dtype, off, &total);
  if (workspace_bytes < total) return set_error(MOE_B200_ERR_WORKSPACE, "workspace too small");
  if (((uintptr_t)workspace & 1023)) return set_error(MOE_B200_ERR_ALIGN, "workspace must be 1024-byte aligned");
  if (N > 0 && (!x || !Wg || !bg || !plan || !out)) return set_error(MOE_B200_ERR_NULL, "NULL argument");
  const bool norm = norm_weight != nullptr;
  if (norm && (!norm_bias || !aligned16(norm_weight) || !aligned16(norm_bias) || !(norm_eps >= 0.f)))
    return set_error(MOE_B200_ERR_NULL, "norm_bias (16-byte aligned) and a non-negative eps are required with norm_weight");
  char* ws = static_cast<char*>(workspace);
  int32_t* status = reinterpret_cast<int32_t*>(ws + off[MOE_B200_WS_STATUS]);
  float* logits = reinterpret_cast<float*>(ws + off[MOE_B200_WS_LOGITS]);
  int32_t* idx = reinterpret_cast<int32_t*>(ws + off[MOE_B200_WS_IDX]);
  float* w = reinterpret_cast<float*>(ws + off[MOE_B200_WS_W]);
  float* psum_part = reinterpret_cast<float*>(ws + off[MOE_B200_WS_PSUM_PART]);
  float* psum = reinterpret_cast<float*>(ws + off[MOE_B200_WS_PSUM]);
  float* aux = reinterpret_cast<float*>(ws + off[MOE_B200_WS_AUX]);
  int32_t* scratch = reinterpret_cast<int32_t*>(ws + off[MOE_B200_WS_SCRATCH]);
  int32_t* cnt_slot = reinterpret_cast<int32_t*>(ws + off[MOE_B200_WS_CNT_SLOT]);
  int32_t* offsets = reinterpret_cast<int32_t*>(ws + off[MOE_B200_WS_OFFSETS]);
  int32_t* row_of = reinterpret_cast<int32_t*>(ws + off[MOE_B200_WS_ROW_OF]);
  void* perm = ws + off[MOE_B200_WS_PERM];
  void* h = ws + off[MOE_B200_WS_H];
  void* y = ws + off[MOE_B200_WS_Y];
  float* part = reinterpret_cast<float*>(ws + off[MOE_B200_WS_PART]);
  cudaStream_t s = (cudaStream_t)stream;
  if (flags & ~MOE_B200_FLAG_WS_CLEAN) return set_error(MOE_B200_ERR_UNSUPPORTED, "unknown flag");
  // a size switch, not a backend switch: up to 256 rows the weight-streaming kernels
  const bool small_n = dtype == MOE_B200_BF16 && N * k <= kDecodeMaxRows;

  // as many rows as experts: most experts are hit, stream all of them without waiting for the
  // routing (measured at d=1024, f=4096, E=8, k=2: 43-45 us from 4 to 64 tokens, against 23 / 34 /
  // 40 / 50 / 66 us for the one-launch kernel below at 1 / 2 / 3 / 4 / 6 tokens, whose time grows
  // with every expert that is hit)
  const bool spec = small_n && front_small_supported(N, E, k, dtype) && decode_spec_supported(N, E, k) &&
                    N * k >= (int64_t)E;
  // a handful of tokens, a row or two per expert: routing, both products and the weighted sum
  // in one cooperative launch
  const bool tiny = small_n && !spec && decode_tiny_supported(N, d, f, E, k, dtype);
  // between the decode and the prefill sizes: the streaming kernel on the sorted rows
  const bool rows_path = dtype == MOE_B200_BF16 && !small_n && N * k <= kRowsPathMaxRows &&
                         rows_supported(N * k, E);
  const bool counters = small_n || rows_path;
  // status words, and the completion counters behind them where a kernel uses them, in one memset
  if (!(counters && (flags & MOE_B200_FLAG_WS_CLEAN)))
    MOE_CUDA_CHECK(cudaMemsetAsync(
        status, 0, (counters ? MOE_B200_READY_OFFSET + MOE_B200_READY_INTS : MOE_B200_STATUS_INTS) * sizeof(int32_t), s));
  const bool front = (small_n || rows_path) &&
                     (front_small_supported(N, E, k, dtype) || front_split_supported(N, E, k, dtype));
  float* stats = reinterpret_cast<float*>(ws + off[MOE_B200_WS_STATS]);
  if (norm && N > 0 && (front || small_n || rows_path)) {
    // up to 4096 rows the kernels read x through TMA: normalise the few rows once
    void* xn = ws + off[MOE_B200_WS_XN];
    rc = launch_layernorm_rows(x, norm_weight, norm_bias, norm_eps, N, d, dtype, xn, nullptr, s);
    if (rc) return rc;
    x = xn;
  }
  const bool fold = norm && N > 0 && x != ws + off[MOE_B200_WS_XN];
  if (tiny)
    return launch_decode_tiny(x, Wg, bg, N, d, f, E, k, plan, residual, logits, idx, w, cnt_slot,
                              offsets, row_of, perm, psum, aux, h, out, status, s);
  if (front) {
    // router and dispatch of up to a few hundred tokens in one launch
    // (beyond 128 tokens its blocks share the work and meet at a counter behind the status words)
    rc = launch_front_small(x, Wg, bg, N, d, E, k, logits, idx, w, cnt_slot, offsets, row_of, perm,
                            psum, aux, s, scratch,
                            status + MOE_B200_READY_OFFSET + MOE_B200_READY_INTS - 4, status);
    if (rc) return rc;
  } else {
    if (fold) {
      void* wn = ws + off[MOE_B200_WS_NORM_W];
      float* nc = reinterpret_cast<float*>(ws + off[MOE_B200_WS_NORM_C]);
      rc = launch_norm_fold(Wg, bg, norm_weight, norm_bias, E, d, dtype, wn, nc, s);
      if (rc) return rc;
      rc = moe_b200_router_norm(x, wn, nc, norm_eps, N, d, E, k, dtype, logits, idx, w, psum_part,
                                stats, status, stream);
      if (rc) return rc;
      rc = moe_b200_dispatch_norm(x, idx, stats, norm_weight, norm_bias, N, d, E, k, dtype, scratch,
                                  cnt_slot, offsets, row_of, perm, psum_part, psum, aux, status, stream);
      if (rc) return rc;
    } else {
      rc = moe_b200_router(x, Wg, bg, N, d, E, k, dtype, logits, idx, w, psum_part, status, stream);
      if (rc) return rc;
      rc = moe_b200_dispatch(x, idx, N, d, E, k, dtype, scratch, cnt_slot, offsets, row_of, perm,
                             N > 0 ? psum_part : nullptr, psum, aux, status, stream);
      if (rc) return rc;
    }
  }
  if (small_n) {
    // few tokens per expert: weight streaming with narrow tiles and split-K
    if (spec)
      rc = launch_experts_tc_decode_spec(x, idx, offsets, plan, N, k, d, f, E, h, part,
                                         status + MOE_B200_READY_OFFSET, status, s);
    else   // a row or two per expert: matrix-vector streaming of the experts that were hit
      rc = launch_experts_gemv(perm, offsets, plan, N * k, d, f, E, decode_splits(f), h, part, s);
    if (rc) return rc;
    return moe_b200_combine_decode(part, decode_splits(f), N * k, row_of, idx, w, plan, E, residual,
                                   N, d, k, out, stream);
  }
  if (rows_path) {
    const int ks = rows_splits(N * k, d, f, E);
    rc = launch_experts_tc_rows(perm, offsets, plan, N * k, d, f, E, ks, h, part,
                                status + MOE_B200_READY_OFFSET, status, s);
    if (rc) return rc;
    return moe_b200_combine_decode(part, ks, N * k, row_of, idx, w, plan, E, residual, N, d, k, out,
                                   stream);
  }
  rc = moe_b200_experts(perm, offsets, plan, N * k, d, f, E, dtype, 0, h, y, status, stream);
  if (rc) return rc;
  return moe_b200_combine(y, row_of, w, residual, N, d, k, dtype, out, stream);
}

int moe_b200_read_status(const int32_t* status, int32_t* h_status, void* stream) {
  if (!status || !h_status) return set_error(MOE_B200_ERR_NULL, "NULL argument");
  MOE_CUDA_CHECK(cudaMemcpyAsync(h_status, status, 16 * sizeof(int32_t), cudaMemcpyDeviceToHost,
                                 (cudaStream_t)stream));
  MOE_CUDA_CHECK(cudaStreamSynchronize((cudaStream_t)stream));
  return h_status[0];
}

}  // extern "C"
