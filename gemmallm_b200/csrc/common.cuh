// Shared helpers of libmoe_b200: error plumbing, vector load/store of bf16/fp32
// rows as fp32, and the internal launch prototypes each .cu file exports.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stddef.h>
#include "../../include/moe_b200.h"

namespace moe {

constexpr int kMaxExperts = 256;
constexpr int kMaxTopK = 8;
constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs

// Tokens per router block and per dispatch chunk. Both kernels partition the
// token range the same way, in token order.
constexpr int kRouterTokensPerBlock = 64;
constexpr int kDispatchChunk = 64;

// The small-N (weight-streaming) expert path is taken up to this many sorted rows (N*k).
constexpr int64_t kDecodeMaxRows = 256;
constexpr int64_t kRowsPathMaxRows = 4096;   // above: the prefill kernels (256-row tiles)

int set_error(int code, const char* msg);
int cuda_error(cudaError_t e, const char* where);

#define MOE_CUDA_CHECK(expr)                                  \
  do {                                                        \
    cudaError_t e__ = (expr);                                 \
    if (e__ != cudaSuccess) return moe::cuda_error(e__, #expr); \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Function attributes, occupancy results and SM counts belong to a device, and one
// process may drive several: every cache of them is indexed by the device that is
// current at the call.
constexpr int kMaxDevices = 64;
inline int device_slot(int* slot) {
  int dev = 0;
  MOE_CUDA_CHECK(cudaGetDevice(&dev));
  *slot = (dev >= 0 && dev < kMaxDevices) ? dev : -1;
  return 0;
}
struct PerDeviceOnce {
  bool done[kMaxDevices] = {};
};
// Raise a kernel's dynamic shared-memory limit once per device.
template <typename Fn>
inline int ensure_dynamic_smem(PerDeviceOnce& once, Fn fn, size_t bytes) {
  int slot = -1;
  int rc = device_slot(&slot);
  if (rc) return rc;
  if (slot < 0 || !once.done[slot]) {
    MOE_CUDA_CHECK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    if (slot >= 0) once.done[slot] = true;
  }
  return 0;
}

// ---- device helpers -------------------------------------------------------

template <typename T> struct Vec8;  // 8 consecutive elements of a row, as fp32

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Load 8 consecutive elements starting at p (16-byte aligned for bf16,
// 32-byte aligned pairs of float4 for fp32) into fp32 registers.
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  uint4 r = *reinterpret_cast<const uint4*>(p);
  v[0] = bf16_lo(r.x); v[1] = bf16_hi(r.x);
  v[2] = bf16_lo(r.y); v[3] = bf16_hi(r.y);
  v[4] = bf16_lo(r.z); v[5] = bf16_hi(r.z);
  v[6] = bf16_lo(r.w); v[7] = bf16_hi(r.w);
}
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  float4 a = *reinterpret_cast<const float4*>(p);
  float4 b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8_ldg(const __nv_bfloat16* p, float (&v)[8]) {
  uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
  v[0] = bf16_lo(r.x); v[1] = bf16_hi(r.x);
  v[2] = bf16_lo(r.y); v[3] = bf16_hi(r.y);
  v[4] = bf16_lo(r.z); v[5] = bf16_hi(r.z);
  v[6] = bf16_lo(r.w); v[7] = bf16_hi(r.w);
}
__device__ __forceinline__ void load8_ldg(const float* p, float (&v)[8]) {
  float4 a = __ldg(reinterpret_cast<const float4*>(p));
  float4 b = __ldg(reinterpret_cast<const float4*>(p + 4));
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 r;
  r.x = pack_bf16x2(v[0], v[1]);
  r.y = pack_bf16x2(v[2], v[3]);
  r.z = pack_bf16x2(v[4], v[5]);
  r.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = r;
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void from_f32(float& o, float v) { o = v; }
__device__ __forceinline__ void from_f32(__nv_bfloat16& o, float v) { o = __float2bfloat16_rn(v); }

// GELU, tanh form, exactly the expression of F.gelu(approximate="tanh")
// (used at model.py:181): 0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))).
__device__ __forceinline__ float gelu_tanh_precise(float g) {
  const float kBeta = 0.7978845608028654f;  // sqrt(2/pi)
  float inner = kBeta * (g + 0.044715f * g * g * g);
  return 0.5f * g * (1.0f + tanhf(inner));
}
__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float gelu_tanh_fast(float g) {
  const float kBeta = 0.7978845608028654f;
  float g2 = g * g;
  float inner = g * fmaf(0.044715f * kBeta, g2, kBeta);
  float hg = 0.5f * g;
  return fmaf(hg, tanh_approx(inner), hg);
}

// Programmatic dependent launch: a kernel launched with launch_pdl may start while
// the kernel before it in the stream is still draining; everything it does before
// pdl_wait() must not touch that kernel's outputs. pdl_wait() returns when the
// earlier kernel has completed and its writes are visible; without the launch
// attribute it returns at once. pdl_launch_dependents() lets the next kernel's
// blocks be scheduled as soon as resources free up.
// Rule for loads: what a kernel that may still be running when this one starts has
// written is read with ordinary or __ldcg loads AFTER pdl_wait(), never with __ldg /
// ld.global.nc: those promise data that is constant over the kernel's lifetime, and
// the compiler is free to move them above the wait (it did: two roles of one kernel
// then disagreed about the routing). A kernel that signals its dependents only after
// its own wait extends the guarantee to everything before it in the chain; one that
// signals first (decode_spec_kernel, combine_decode_kernel) does not.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Plan buffer layout (device memory owned by the caller).
//   [0, 4*E*8)            : W1[E], b1[E], W2[E], b2[E] device pointers
//   then, 128-byte aligned: tensor maps (128 bytes each) W1[E], W2[E] with
//   128-row boxes, then W1[E], W2[E] with 64-row boxes for the small-N path
struct PlanView {
  const void* const* W1;
  const void* const* b1;
  const void* const* W2;
  const void* const* b2;
  const void* tmap_W1;  // CUtensorMap[E]
  const void* tmap_W2;  // CUtensorMap[E]
  const void* tmap_W1_dec;
  const void* tmap_W2_dec;
};
constexpr int kPlanMapsPerExpert = 4;
__host__ __device__ inline size_t plan_ptr_bytes(int E) {
  return ((size_t)4 * E * sizeof(void*) + 127) & ~(size_t)127;
}
__host__ __device__ inline PlanView plan_view(const void* plan, int E) {
  const char* p = static_cast<const char*>(plan);
  PlanView v;
  v.W1 = reinterpret_cast<const void* const*>(p);
  v.b1 = v.W1 + E;
  v.W2 = v.b1 + E;
  v.b2 = v.W2 + E;
  v.tmap_W1 = p + plan_ptr_bytes(E);
  v.tmap_W2 = p + plan_ptr_bytes(E) + (size_t)128 * E;
  v.tmap_W1_dec = p + plan_ptr_bytes(E) + (size_t)128 * 2 * E;
  v.tmap_W2_dec = p + plan_ptr_bytes(E) + (size_t)128 * 3 * E;
  return v;
}

// ---- expert-parallel exchange ------------------------------------------------
constexpr int kEpMaxRanks = 8;
enum { kEpFlagCnt = 0, kEpFlagX = 1, kEpFlagY = 2, kEpNumFlags = 3 };

// Pointers into every rank's symmetric buffer (index = rank), valid on this GPU.
struct EpPeers {
  uint32_t* flags[kEpMaxRanks];     // [kEpNumFlags][kEpMaxRanks] epoch words, one per (kind, source)
  int32_t* cnt_all[kEpMaxRanks];    // [world][EV+2E] per source: pair counts, slot-0 counts, psum bits
  int32_t* recv_meta[kEpMaxRanks];  // [cap] return address of a received row: source << 24 | pair id
  void* recv_x[kEpMaxRanks];        // [cap][d] received token rows, grouped by owned expert
  void* ret_y[kEpMaxRanks];         // [N_local*k][d] expert outputs returned to the token owner
};
// Expert-parallel hand-shakes folded into the neighbouring kernels. Epochs only grow; a flag
// word holds the epoch of the last call that raised it. `epoch` points to the call's epoch in
// the workspace (written by ep_begin_kernel at the head of the call).
//   wait_flags != nullptr: before touching its inputs the kernel waits (bounded) until
//     wait_flags[0 .. world) have reached *epoch;
//   done_counter != nullptr: the last block of the grid to finish raises signal_flags[q] + rank
//     on every rank q (after a system-scope fence: its own and, through the counter, every
//     other block's peer stores are visible first).
struct EpSync {
  const uint32_t* epoch;
  const uint32_t* wait_flags;
  uint32_t* done_counter;
  uint32_t* signal_flags[kEpMaxRanks];   // per destination rank: word this rank raises there
  int world;
};

// Destination of the down pass's rows in the expert-parallel configuration.
struct EpScatter {
  void* ret_y[kEpMaxRanks];
  const int32_t* meta;
};

// Training-mode extras of the GEGLU pass (reference model.py:164,183: nn.Dropout on h, and
// what the backward pass needs): the pre-activations gate/up with their biases go to
// gu [M, 2f] (columns [0,f) gate, [f,2f) up), and h is multiplied by the dropout mask of its
// (token, slot) pair: element (pair, c) is kept iff its Philox word (philox.cuh) is >= thresh,
// and scaled by `scale` = 1 / (1 - p).
struct TrainArgs {
  __nv_bfloat16* gu;
  const int32_t* pair_of;   // [M] token * k + slot of every sorted row
  uint32_t thresh;          // p * 2^32; 0 keeps everything
  float scale;
  uint32_t seed_lo, seed_hi;
};

// ---- launchers implemented in the other translation units -----------------
int launch_router(const void* x, const void* Wg, const void* bg, int64_t N, int d, int E, int k,
                  int dtype, float* out_logits, int32_t* out_idx, float* out_w, float* psum_part,
                  int32_t* status, cudaStream_t s, const float* norm_c = nullptr, float eps = 0.f,
                  float* stats = nullptr);
int launch_dispatch(const void* x, const int32_t* idx, int64_t N, int d, int E, int k, int dtype,
                    int32_t* chunk_cnt, int32_t* cnt_slot, int32_t* offsets, int32_t* row_of,
                    void* perm, const float* psum_part, float* psum, float* aux, int32_t* status,
                    cudaStream_t s, const float* norm_stats = nullptr, const void* gamma = nullptr,
                    const void* beta = nullptr);
int launch_norm_fold(const void* Wg, const void* bg, const void* gamma, const void* beta, int E,
                     int d, int dtype, void* Wn, float* c, cudaStream_t s);
int launch_layernorm_rows(const void* x, const void* gamma, const void* beta, float eps, int64_t N,
                          int d, int dtype, void* out, float* stats, cudaStream_t s);
int launch_experts_simt(const void* perm, const int32_t* offsets, const void* plan, int64_t M,
                        int d, int f, int E, int dtype, void* h, void* y, cudaStream_t s);
int launch_combine(const void* y, const int32_t* row_of, const float* w, const void* residual,
                   int64_t N, int d, int k, int dtype, void* out, cudaStream_t s,
                   const EpSync* ep_wait = nullptr, int32_t* status = nullptr);
int build_weight_tensor_maps(const void* const* h_W1, const void* const* h_W2, int E, int d, int f,
                             void* h_tmaps /* kPlanMapsPerExpert*E*128 bytes */);
int launch_experts_tc2(const void* perm, const int32_t* offsets, const void* plan, int64_t M, int d,
                       int f, int E, void* h, void* y, const EpScatter* sc, int32_t* status,
                       cudaStream_t s, const TrainArgs* train = nullptr, const EpSync* ep_wait = nullptr,
                       const EpSync* ep_signal = nullptr);
// One grouped product out[rows of e] = A[rows of e] . B_e^T (+ bias_e), B_e given by the e-th
// tensor map of tmaps_b ([Nout, K] row-major, 128-row boxes); bias may be nullptr.
int launch_grouped_rows(const void* A, int64_t M, int K, const void* tmaps_b, const int32_t* offsets,
                        const void* const* bias, int E, int Nout, void* out, int32_t* status,
                        cudaStream_t s);
// Grouped over the contraction index: out_e [Ra, Rb] = At[:, K_e] . Bt[:, K_e]^T for the column
// ranges K_e = [koff[e], koff[e+1]) (multiples of 64) of At [Ra, Kpad] and Bt [Rb, Kpad];
// out [E][Ra][Rb]. Experts with an empty range are skipped (their slice is left untouched).
int launch_grouped_cols(const void* At, const void* Bt, int64_t Kpad, int Ra, int Rb,
                        const int32_t* koff, void* out, int E, int32_t* status, cudaStream_t s);
int64_t ep_scratch_ints(int64_t N, int EV, int E);
int launch_ep_begin(uint32_t* epoch, uint32_t* done_counter, int32_t* status, int32_t* scratch, int EV,
                    int E, cudaStream_t s);
int launch_ep_dispatch(const void* x, const int32_t* idx, int64_t N, int d, int E, int EV, int k,
                       int dtype, const EpPeers& peers, int rank, int world, const uint32_t* epoch,
                       const int32_t* owner, const int32_t* vmap, int32_t* scratch,
                       const float* psum_part,
                       int32_t* cnt_slot0, float* psum_global, int32_t* offsets_local, float* aux,
                       int64_t n_total, int32_t* status, cudaStream_t s);
bool front_small_supported(int64_t N, int E, int k, int dtype);
int64_t front_small_exchange_ints(int64_t N, int E, int k);
bool front_split_supported(int64_t N, int E, int k, int dtype);
int launch_front_small(const void* x, const void* Wg, const void* bg, int64_t N, int d, int E, int k,
                       float* out_logits, int32_t* out_idx, float* out_w, int32_t* cnt_slot,
                       int32_t* offsets, int32_t* row_of, void* perm, float* psum, float* aux,
                       cudaStream_t s, int* xch = nullptr, int* counter = nullptr,
                       int32_t* status = nullptr);
int encode_tmap_2d(void* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);
int sm_count(int* sms);
int decode_splits(int f);
int decode_spec_rows(int64_t N);
bool decode_spec_supported(int64_t N, int E, int k);
int launch_experts_tc_decode_spec(const void* x, const int32_t* idx, const int32_t* offsets,
                                  const void* plan, int64_t N, int k, int d, int f, int E, void* h_all,
                                  float* part, int* ready, int32_t* status, cudaStream_t s);
int rows_splits(int64_t M, int d, int f, int E);
bool rows_supported(int64_t M, int E);
int launch_experts_tc_rows(const void* perm, const int32_t* offsets, const void* plan, int64_t M,
                           int d, int f, int E, int ksplit, void* h, float* part, int* ready,
                           int32_t* status, cudaStream_t s);
int launch_experts_tc_decode_fused(const void* perm, const int32_t* offsets, const void* plan,
                                   int64_t M, int d, int f, int E, void* h, float* part, int* ready,
                                   int32_t* status, cudaStream_t s, int spec = -1);
int launch_combine_decode(const float* part, int ksplit, int64_t M, const int32_t* row_of,
                          const int32_t* idx, const float* w, const void* plan, int E,
                          const void* residual, int64_t N, int d, int k, void* out, cudaStream_t s);

// Router for 17 to 64 experts on the tcgen05 path (router_tc.cu); same results as launch_router.
bool router_tc_supported(int64_t N, int d, int E, int k);
int launch_router_tc(const void* x, const void* Wg, const void* bg, int64_t N, int d, int E, int k,
                     float* out_logits, int32_t* out_idx, float* out_w, float* psum_part,
                     int32_t* status, cudaStream_t s);
// The whole block for one to eight tokens in one cooperative launch (experts_tiny.cu):
// routing results as launch_front_small, h [N*k, f] scratch, out [N, d].
bool decode_tiny_supported(int64_t N, int d, int f, int E, int k, int dtype);
int launch_decode_tiny(const void* x, const void* Wg, const void* bg, int64_t N, int d, int f, int E,
                       int k, const void* plan, const void* residual, float* logits, int32_t* idx,
                       float* w, int32_t* cnt_slot, int32_t* offsets, int32_t* row_of, void* perm,
                       float* psum, float* aux, void* h, void* out, int32_t* status, cudaStream_t s);
int launch_experts_gemv(const void* perm, const int32_t* offsets, const void* plan, int64_t M, int d,
                        int f, int E, int ksplit, void* h, float* part, cudaStream_t s);

// ---- backward.cu ----
int launch_pair_of(const int32_t* row_of, int64_t M, int32_t* pair_of, cudaStream_t s);
int launch_pad_offsets(const int32_t* offsets, int E, int32_t* koff, cudaStream_t s);
int launch_combine_bwd(const void* dout, const void* y, const int32_t* pair_of, const float* w,
                       int64_t M, int d, int k, void* dy, float* dw, cudaStream_t s);
int launch_router_bwd(const float* logits, const int32_t* idx, const float* w, const float* dw,
                      const int32_t* cnt0, float grad_aux, const void* x, const void* Wg, int64_t N,
                      int d, int E, int k, float* dl, float* dWg_f32, float* dbg_f32, void* dWg,
                      void* dbg, void* dxr, cudaStream_t s);
int launch_fill_f32(float* p, int64_t n, float v, cudaStream_t s);
int launch_iota(int32_t* p, int64_t n, cudaStream_t s);
int launch_geglu_bwd(const void* dh, void* gu, const int32_t* pair_of, int64_t M, int f,
                     uint32_t thresh, float scale, uint32_t seed_lo, uint32_t seed_hi, cudaStream_t s);
int launch_transpose_weights(const void* const* src_ptrs, int E, int R, int C, void* dst, cudaStream_t s);
int launch_transpose_pad(const void* src, const int32_t* offsets, const int32_t* koff, int E, int C,
                         int64_t Kpad, void* dst, cudaStream_t s);
int launch_colsum(const void* src, const int32_t* offsets, int E, int C, void* db, cudaStream_t s);

}  // namespace moe
