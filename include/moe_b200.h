/*
 * moe_b200.h — C ABI of libmoe_b200.so: the Mixture-of-Experts feed-forward
 * block of GemmaLLM (reference model.py:192-276, expert model.py:154-190)
 * as hand-written CUDA kernels for NVIDIA B200 (sm_100a).
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless its name starts with h_.
 *   - Every call is asynchronous on the given stream (a cudaStream_t passed as
 *     void*; NULL = the legacy default stream) unless stated otherwise.
 *   - Return value: 0 = ok; negative = argument error found on the host before
 *     any launch (nothing ran); positive = CUDA runtime error code + 1000.
 *     Errors detected on the device (a wait that ran out, a bad index) are
 *     written to the workspace status word; read it with moe_b200_read_status.
 *   - The library owns no device memory and never allocates: the caller
 *     passes inputs, outputs, a workspace and a "plan" buffer.
 *   - Matrices are row-major and contiguous. Tokens are rows: x is [N, d].
 *   - dtype: MOE_B200_F32 or MOE_B200_BF16 applies to x, the parameters and
 *     the output alike. The router always computes in fp32.
 *
 * Symbols: N tokens, d = hidden size, f = per-branch expert width
 * (gate_and_up.weight is [2f, d]: rows [0,f) gate, rows [f,2f) up,
 * model.py:180), E experts, k = experts per token (the reference fixes k = 2,
 * model.py:210).
 */
#ifndef MOE_B200_H
#define MOE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MOE_B200_ABI_VERSION 2

enum { MOE_B200_F32 = 0, MOE_B200_BF16 = 1 };

/* host-side argument errors */
enum {
  MOE_B200_OK = 0,
  MOE_B200_ERR_NULL = -1,      /* a required pointer is NULL */
  MOE_B200_ERR_SHAPE = -2,     /* N, d, f, E or k out of the supported range */
  MOE_B200_ERR_ALIGN = -3,     /* a pointer or row pitch is not 16-byte aligned */
  MOE_B200_ERR_DTYPE = -4,     /* unknown dtype */
  MOE_B200_ERR_WORKSPACE = -5, /* workspace or plan buffer too small */
  MOE_B200_ERR_DRIVER = -6,    /* tensor-map encoding entry point unavailable */
  MOE_B200_ERR_UNSUPPORTED = -7
};

/* device-side status codes (workspace status word 0) */
enum {
  MOE_B200_DEV_OK = 0,
  MOE_B200_DEV_TIMEOUT = 1,   /* a bounded wait inside a kernel ran out */
  MOE_B200_DEV_BAD_INDEX = 2  /* an expert index outside [0,E) was seen */
};

/* flags for moe_b200_forward */
enum {
  MOE_B200_FLAG_DEFAULT = 0,
  /* The caller guarantees that the status region of `workspace`
   * (MOE_B200_WS_STATUS, status words and counters) is all zero on entry: it was
   * zeroed once, and every call on this workspace since then has ended with
   * device status 0 (such calls leave the region zero). Saves the memset in
   * front of the first kernel of calls of up to 4096 rows, which then overlaps
   * the tail of the kernel before it. After a non-zero device status the region
   * has to be zeroed again by the caller. */
  MOE_B200_FLAG_WS_CLEAN = 1
};

/* Layout of the status region: word 0 = device status code, words 1..15 detail;
 * from word MOE_B200_READY_OFFSET on, MOE_B200_READY_INTS completion counters of
 * moe_b200_experts_decode_fused. */
#define MOE_B200_STATUS_INTS 16
#define MOE_B200_READY_OFFSET 64
#define MOE_B200_READY_INTS 320

/* Indices into the array filled by moe_b200_workspace_layout. */
enum {
  MOE_B200_WS_STATUS = 0, /* int32[16] status, then the counters (see MOE_B200_READY_OFFSET) */
  MOE_B200_WS_LOGITS,     /* float [N,E]   router logits (model.py:206) */
  MOE_B200_WS_IDX,        /* int32 [N,k]   chosen experts, slot 0 = best (model.py:210) */
  MOE_B200_WS_W,          /* float [N,k]   renormalised scores (model.py:219-223) */
  MOE_B200_WS_PSUM_PART,  /* float [router blocks, E] partial sums of softmax */
  MOE_B200_WS_PSUM,       /* float [E]     sum over tokens of softmax (model.py:215) */
  MOE_B200_WS_AUX,        /* float [1]     load-balancing loss (model.py:216) */
  MOE_B200_WS_SCRATCH,    /* int32 [moe_b200_dispatch_scratch_bytes/4] dispatch scratch */
  MOE_B200_WS_CNT_SLOT,   /* int32 [k,E]   per-slot expert counts (model.py:237-245) */
  MOE_B200_WS_OFFSETS,    /* int32 [E+1]   start row of each expert in the sorted buffers */
  MOE_B200_WS_ROW_OF,     /* int32 [N,k]   sorted-buffer row of (token, slot) */
  MOE_B200_WS_PERM,       /* T [N*k, d]    tokens sorted by expert (model.py:248-253) */
  MOE_B200_WS_H,          /* T [N*k, f]    gelu_tanh(gate)*up (model.py:180-182) */
  MOE_B200_WS_Y,          /* T [N*k, d]    expert outputs, sorted order (model.py:184) */
  MOE_B200_WS_PART,       /* float [splits, N*k, d] split-K partial sums of the small-N path
                           * (present when N*k <= moe_b200_decode_max_rows(), bf16) */
  MOE_B200_WS_NORM_W,     /* T [E,d]       gate.weight * norm weight (moe_b200_norm_fold) */
  MOE_B200_WS_NORM_C,     /* float [2E]    constants of the folded router */
  MOE_B200_WS_STATS,      /* float [N,2]   mean and 1/std of every row of x */
  MOE_B200_WS_XN,         /* T [N,d]       normalised rows, calls of up to 4096 rows only */
  MOE_B200_WS_NUM
};

/* ABI version of the loaded library (no reference counterpart: the reference
 * is a Python class, model.py:192). Synchronous. */
int moe_b200_version(void);

/* Text for the last non-zero return value on this thread. Synchronous. */
const char* moe_b200_last_error_string(void);

/* Bytes of workspace moe_b200_forward needs; 0 on bad arguments. Replaces the
 * temporaries the reference allocates per call (model.py:226-268).
 * Synchronous, touches no GPU. */
size_t moe_b200_workspace_bytes(int64_t N, int d, int f, int E, int k, int dtype);

/* Byte offset of each workspace region (h_offsets[MOE_B200_WS_NUM]). */
int moe_b200_workspace_layout(int64_t N, int d, int f, int E, int k, int dtype,
                              size_t* h_offsets);

/* Bytes of the plan buffer for E experts. */
size_t moe_b200_plan_bytes(int E);

/* Record the E experts' parameter pointers (and, for bf16, their TMA tensor
 * maps) in the caller's plan buffer. Stands for the reference's
 * nn.ModuleList of FeedForward (model.py:197): h_W1[e] = gate_and_up.weight
 * [2f,d], h_b1[e] = gate_and_up.bias [2f], h_W2[e] = down.weight [d,f],
 * h_b2[e] = down.bias [d] (model.py:162-163). Call again whenever a
 * parameter's storage moves. The host arrays may be freed on return. */
int moe_b200_plan_build(const void* const* h_W1, const void* const* h_b1,
                        const void* const* h_W2, const void* const* h_b2,
                        int E, int d, int f, int dtype,
                        void* plan, size_t plan_bytes, void* stream);

/* An expert Linear with its LoRA branch folded in (fine_tuning=True,
 * model.py:175-179 and 185-189): out_W = W + scale * B A, out_b = b + scale *
 * (B a_bias + b_lora), so that x out_W^T + out_b = x W^T + b + scale * (B (A x +
 * a_bias) + b_lora). W [out,in], A [rank,in] (lora_*_a.weight), a_bias [rank],
 * B [out,rank] (lora_*_b.weight), b_lora [out]; fp32 arithmetic, one rounding.
 * The merged tensors go into a plan like any other parameters. */
int moe_b200_lora_merge(const void* W, const void* b, const void* A, const void* a_bias,
                        const void* B, const void* b_lora, float scale,
                        int out_features, int in_features, int rank, int dtype,
                        void* out_W, void* out_b, void* stream);

/* Part 1 — router: logits = x Wg^T + bg (model.py:206), fp32 softmax
 * (model.py:207), top-k (model.py:210), renormalise (model.py:219-223), and
 * the sums the load-balancing loss needs (model.py:213-216).
 *   out_logits  float [N,E]  or NULL
 *   out_idx     int32 [N,k]  slot 0 = highest probability
 *   out_w       float [N,k]
 *   psum_part   float [moe_b200_router_blocks(N), E] scratch
 */
int moe_b200_router(const void* x, const void* Wg, const void* bg,
                    int64_t N, int d, int E, int k, int dtype,
                    float* out_logits, int32_t* out_idx, float* out_w,
                    float* psum_part, int32_t* status, void* stream);

int64_t moe_b200_router_blocks(int64_t N);

/* Part 2 — dispatch: histogram of idx, exclusive scan, and permutation of the
 * token rows into one expert-contiguous buffer; replaces the per-slot argsort,
 * count loop, gather and split of model.py:226-253. Rows of one expert keep
 * token order (stable).
 *   scratch    moe_b200_dispatch_scratch_bytes(N,E,k) bytes: per-chunk and
 *              per-block expert counts, per-block per-slot counts; contents
 *              need no initialisation and are overwritten by every call
 *   cnt_slot   int32 [k,E]   (top_expert_counts, second_expert_counts, ...)
 *   offsets    int32 [E+1]
 *   row_of     int32 [N,k]
 *   perm       T [N*k, d]
 *   psum_part/psum/aux: when psum_part is non-NULL the router's partial sums
 *   are reduced in a fixed order into psum[E] and the load-balancing loss
 *   aux[0] (model.py:213-216); otherwise these three may be NULL.
 */
int moe_b200_dispatch(const void* x, const int32_t* idx,
                      int64_t N, int d, int E, int k, int dtype,
                      int32_t* scratch, int32_t* cnt_slot, int32_t* offsets,
                      int32_t* row_of, void* perm,
                      const float* psum_part, float* psum, float* aux,
                      int32_t* status, void* stream);

size_t moe_b200_dispatch_scratch_bytes(int64_t N, int E, int k);

/* moe_b200_dispatch for callers that cannot give it a scratch buffer because
 * they may not allocate device memory where they call from (a forward hook
 * under a frozen memory pool, a serving loop whose allocator is locked while
 * requests are in flight, a language binding that only sees the op's own
 * tensors). No counterpart in the reference. Same arguments and results as
 * moe_b200_dispatch without `scratch`: the counters live in a 1 MiB array
 * built into the library (held by every GPU that loads it until the process
 * exits). After the first call on a device it takes no device memory and calls
 * no allocating routine; that first call loads the library's kernels on the
 * device and looks the array's address up (so make it once at start-up).
 *   - Limit: moe_b200_dispatch_scratch_bytes(N,E,k) <= 1 MiB (e.g. N=65536,
 *     E=64, k=4 fits); larger shapes return MOE_B200_ERR_WORKSPACE.
 *   - The first call on each device looks up the array's device address; make
 *     that call before any stream capture starts.
 *   - All calls on one GPU share the array; it needs no clearing between
 *     calls, but calls whose kernels overlap on the GPU race on it. */
int moe_b200_dispatch_static(const void* x, const int32_t* idx,
                             int64_t N, int d, int E, int k, int dtype,
                             int32_t* cnt_slot, int32_t* offsets,
                             int32_t* row_of, void* perm,
                             const float* psum_part, float* psum, float* aux,
                             int32_t* status, void* stream);

/* Part 3 — experts: for every expert e and its rows [offsets[e], offsets[e+1])
 * of perm: h = gelu_tanh(x W1g^T + b1g) * (x W1u^T + b1u), y = h W2^T + b2
 * (FeedForward.forward, model.py:173-190 with fine_tuning=False, dropout in
 * eval mode). M = N*k rows. bf16 runs on tcgen05 tensor cores with fp32
 * accumulation; fp32 runs on CUDA cores. h [M,f] and y [M,d] are outputs.
 * flags: reserved, pass 0. */
int moe_b200_experts(const void* perm, const int32_t* offsets, const void* plan,
                     int64_t M, int d, int f, int E, int dtype, int flags,
                     void* h, void* y, int32_t* status, void* stream);

/* Part 3 for calls between the decode and the prefill sizes (bf16): the weight-streaming
 * pipeline of moe_b200_experts_decode_spec on the rows sorted by expert. With a few hundred
 * rows per expert the prefill kernels' 256-row tiles are mostly padding, their token operand
 * is as many bytes as the weights and the down product has fewer tiles than there are SMs;
 * here the unit is a block of 32, 64 or 128 rows of one expert's segment, the weights are the wide MMA
 * operand and the down product's K is cut into `ksplit` ranges. h [M,f] is written as by
 * moe_b200_experts; the down product arrives as part[s][M][d] WITHOUT down.bias, for
 * moe_b200_combine_decode (model.py:174-184 per expert, another summation order over K).
 * ready: int32[MOE_B200_READY_INTS], zeroed by this call; moe_b200_rows_splits gives the
 * ksplit moe_b200_forward uses. Needs (row blocks) + E <= MOE_B200_READY_INTS - 8.
 * Residency rule and time-out behaviour as for moe_b200_experts_decode_fused. */
int moe_b200_experts_rows(const void* perm, const int32_t* offsets, const void* plan,
                          int64_t M, int d, int f, int E, int ksplit, void* h, float* part,
                          int32_t* ready, int32_t* status, void* stream);
int moe_b200_rows_splits(int64_t M, int d, int f, int E);

/* Parts 1+2 for a handful of tokens in ONE single-block launch: same results as
 * moe_b200_router followed by moe_b200_dispatch (model.py:206-253), for bf16,
 * 1 <= N <= 512, N*k <= 1024, E <= 32; other shapes return
 * MOE_B200_ERR_UNSUPPORTED. psum [E] and aux [1] are final (no partial sums). */
int moe_b200_front_small(const void* x, const void* Wg, const void* bg,
                         int64_t N, int d, int E, int k, int dtype,
                         float* out_logits, int32_t* out_idx, float* out_w,
                         int32_t* cnt_slot, int32_t* offsets, int32_t* row_of, void* perm,
                         float* psum, float* aux, void* stream);

/* The same results from blocks that share the work: beyond 128 tokens every block of
 * moe_b200_front_small would repeat the whole routing; here block b routes tokens 16b..16b+15,
 * the blocks exchange their counts through `exchange` (int32, at least
 * moe_b200_front_exchange_ints(N,E,k) words) and meet at `counter` (one int32, zeroed by this
 * call; bounded wait, MOE_B200_DEV_TIMEOUT in `status` if a block never arrives). bf16,
 * 1 <= N <= 2048, E <= 32. Up to 128 tokens it runs exactly moe_b200_front_small. The logits differ from that function's in the
 * order their partial sums are added; everything derived from them is derived the same way. */
int moe_b200_front_small_split(const void* x, const void* Wg, const void* bg,
                               int64_t N, int d, int E, int k, int dtype,
                               float* out_logits, int32_t* out_idx, float* out_w,
                               int32_t* cnt_slot, int32_t* offsets, int32_t* row_of, void* perm,
                               float* psum, float* aux, int32_t* exchange, int32_t* counter,
                               int32_t* status, void* stream);
int64_t moe_b200_front_exchange_ints(int64_t N, int E, int k);

/* Part 3, small-N ("decode") variant, bf16 only, M <= moe_b200_decode_max_rows():
 * the same products as moe_b200_experts, arranged for weight streaming when
 * only a few rows reach each expert (the reference runs the same
 * FeedForward.forward whatever the row count, model.py:256-257), in ONE launch:
 * the down tiles of a 32-row block start as soon as that block's GEGLU tiles
 * have finished, while other blocks' weights are still streaming. h [M,f] is
 * written as usual; the down product is split over K into
 * moe_b200_decode_splits(f) fp32 buffers part[s][M][d] WITHOUT down.bias;
 * moe_b200_combine_decode sums them.
 * `ready`: int32[MOE_B200_READY_INTS] completion counters, zeroed by this call.
 * The kernel's blocks wait on one another, so all of them must be resident: one
 * block per SM of an otherwise idle GPU. If other work holds SMs for seconds,
 * the bounded waits end with MOE_B200_DEV_TIMEOUT in status and the outputs are
 * unspecified; the context stays usable. */
int moe_b200_experts_decode_fused(const void* perm, const int32_t* offsets, const void* plan,
                                  int64_t M, int d, int f, int E, void* h, float* part,
                                  int32_t* ready, int32_t* status, void* stream);
int moe_b200_decode_splits(int f);
int64_t moe_b200_decode_max_rows(void);

/* Part 3 for a row or two per expert (decode with a few tokens), bf16, M <=
 * moe_b200_decode_max_rows(): h [M,f] and part[s][M][d] as moe_b200_experts_decode_fused,
 * from two weight-streaming launches (GEGLU, then the down product split over K into
 * moe_b200_decode_splits(f) ranges) in which the weights are the 16-row operand of
 * mma.sync and thousands of warps stream at once even when only two experts are hit
 * (model.py:174-184; the reference skips experts without rows, model.py:256, so does this).
 * Its blocks do not wait on one another: no residency requirement. */
int moe_b200_experts_gemv(const void* perm, const int32_t* offsets, const void* plan,
                          int64_t M, int d, int f, int E, void* h, float* part, void* stream);

/* The whole block for one to eight tokens in ONE cooperative launch (model.py:206-276 and
 * the caller's model.py:319): routing as moe_b200_front_small (same results: logits may be
 * NULL, idx, w, cnt_slot, offsets, row_of, perm, psum, aux), then the hit experts' GEGLU
 * product into h [N*k,f] (scratch), a grid barrier, the down product from weight rows that
 * were requested into shared memory before the GEGLU product, and
 * out[t] = sum_j w[t,j] * bf16(y[t,j]) (+ residual[t]) in slot order, as
 * moe_b200_combine_decode. bf16, 1 <= N <= 8, E <= 32, d and f multiples of 8.
 * moe_b200_forward takes this path when, in addition, N*k < E (few experts hit). One block
 * per SM; the launch itself guarantees that they are resident together. status: the 16
 * status words (a time-out of the weight rows' arrival is reported there and the rows are
 * then read from global memory). */
int moe_b200_decode_tiny(const void* x, const void* Wg, const void* bg, const void* plan,
                         const void* residual, int64_t N, int d, int f, int E, int k,
                         float* out_logits, int32_t* out_idx, float* out_w, int32_t* cnt_slot,
                         int32_t* offsets, int32_t* row_of, void* perm, float* psum, float* aux,
                         void* h, void* out, int32_t* status, void* stream);

/* Part 3 for small N without waiting for the routing: the same partial sums
 * part[s][M][d] as moe_b200_experts_decode_fused (row order of moe_b200_dispatch), but
 * computed from the UNSORTED tokens x [N,d]: every expert's weights are streamed and
 * multiplied with all N tokens, and only the (token, expert) pairs of idx [N,k] are
 * stored. Nothing the kernel loads depends on idx/offsets, so under programmatic
 * dependent launch it overlaps the routing kernel before it in the stream
 * (model.py:174-184 per expert; the reference skips experts without tokens,
 * model.py:256, this kernel reads their GEGLU weights anyway: worth it when most
 * experts are hit; moe_b200_forward uses it from N*k >= E on). bf16, N <= 128, E <= 32, N*k <=
 * moe_b200_decode_max_rows(). h_all: bf16 [E][moe_b200_decode_spec_rows(N)][f]
 * scratch; ready: int32[MOE_B200_READY_INTS], zeroed by this call. Residency rule
 * and timeout behaviour as for moe_b200_experts_decode_fused. */
int moe_b200_experts_decode_spec(const void* x, const int32_t* idx, const int32_t* offsets,
                                 const void* plan, int64_t N, int k, int d, int f, int E,
                                 void* h_all, float* part, int32_t* ready, int32_t* status,
                                 void* stream);
int moe_b200_decode_spec_rows(int64_t N);

/* Parts 4+5 after the small-N expert kernels: y = sum_s part[s] + down.bias of
 * the row's expert (idx), rounded to bf16, then the weighted sum and residual
 * of moe_b200_combine (model.py:184, 264-271, 319). */
int moe_b200_combine_decode(const float* part, int ksplit, int64_t M,
                            const int32_t* row_of, const int32_t* idx, const float* w,
                            const void* plan, int E, const void* residual,
                            int64_t N, int d, int k, void* out, void* stream);

/* Parts 4+5 — combine: out[t] = sum_j w[t,j] * y[row_of[t,j]] in slot order
 * in fp32 (model.py:264-271), plus residual[t] when residual is non-NULL (the
 * caller's `tensor += skip_connection`, model.py:319), rounded once to T. */
int moe_b200_combine(const void* y, const int32_t* row_of, const float* w,
                     const void* residual, int64_t N, int d, int k, int dtype,
                     void* out, void* stream);

/* ---- The caller's LayerNorm folded into the block -----------------------------
 * In the reference the block's input is LayerNorm(x) (norm2, model.py:298,311-312).
 * With norm_weight/norm_bias [d] given, x is the tensor BEFORE that norm: the
 * router forms the row statistics in its own pass over x and computes the logits
 * of the normalised row from folded weights, the dispatch normalises the rows
 * while it copies them, and the normalised tensor is never written to memory.
 * (eps inside the square root, biased variance: torch.nn.LayerNorm.) */

/* Wn [E,d] = Wg * norm_weight (rounded to T), c [2E]: c[e] = sum_j Wn[e][j],
 * c[E+e] = sum_j norm_bias[j] * Wg[e][j] + bg[e]; then
 * LayerNorm(x) . Wg[e] + bg[e] = rstd * (x . Wn[e] - mean * c[e]) + c[E+e]. */
int moe_b200_norm_fold(const void* Wg, const void* bg, const void* norm_weight,
                       const void* norm_bias, int E, int d, int dtype,
                       void* out_Wn, float* out_c, void* stream);

/* moe_b200_router on LayerNorm(x) (model.py:311-312, 206-223): Wn and c from
 * moe_b200_norm_fold; out_stats float [N,2] receives (mean, 1/std) of every row. */
int moe_b200_router_norm(const void* x, const void* Wn, const float* c, float eps,
                         int64_t N, int d, int E, int k, int dtype,
                         float* out_logits, int32_t* out_idx, float* out_w,
                         float* psum_part, float* out_stats, int32_t* status, void* stream);

/* moe_b200_dispatch that writes LayerNorm(x) rows into perm: stats from
 * moe_b200_router_norm, norm_weight/norm_bias [d]. */
int moe_b200_dispatch_norm(const void* x, const int32_t* idx, const float* stats,
                           const void* norm_weight, const void* norm_bias,
                           int64_t N, int d, int E, int k, int dtype,
                           int32_t* scratch, int32_t* cnt_slot, int32_t* offsets,
                           int32_t* row_of, void* perm,
                           const float* psum_part, float* psum, float* aux,
                           int32_t* status, void* stream);

/* out [N,d] = LayerNorm(x) row by row (model.py:298,312); what moe_b200_forward
 * runs in front of calls of up to 4096 rows, whose kernels read x through TMA. */
int moe_b200_layernorm(const void* x, const void* norm_weight, const void* norm_bias, float eps,
                       int64_t N, int d, int dtype, void* out, void* stream);

/* The whole block: MOE.forward (model.py:200-276) for x [N,d] -> out [N,d],
 * with the optional fused residual. Wg [E,d], bg [E] are gate.weight/bias
 * (model.py:195). norm_weight/norm_bias: NULL, or the LayerNorm in front of the
 * block (see above; x is then the un-normalised tensor, which is usually also
 * the residual). After it the workspace holds logits, idx, w, counts,
 * offsets, psum and the loss (see moe_b200_workspace_layout). The size of the
 * call selects the kernels (bf16): one to eight tokens with fewer than E rows
 * moe_b200_decode_tiny; up to moe_b200_decode_max_rows() rows the single-launch
 * front and a weight-streaming expert kernel; up to 4096 rows the front and the
 * streaming kernel on sorted rows; beyond that router, dispatch, the two grouped
 * GEMM passes and combine. */
int moe_b200_forward(const void* x, const void* Wg, const void* bg,
                     const void* plan, const void* residual,
                     const void* norm_weight, const void* norm_bias, float norm_eps,
                     int64_t N, int d, int f, int E, int k, int dtype, int flags,
                     void* workspace, size_t workspace_bytes,
                     void* out, void* stream);

/* ---- Attention core of the decoder layer ---------------------------------------
 * What the reference's Attention.forward does between its Linears (model.py:104-142),
 * for the decoder the block sits in: qkv [B,S,(q_heads + 2 kv_heads) * 64] bf16 is the
 * output of the fused QKV Linear (queries, then keys, then values, model.py:104); every
 * group of q_heads / kv_heads query heads shares one KV head (model.py:112-115); queries
 * and keys are rotated with pos_emb float [>= S, 128] (row m = [cos | signed sin] of
 * position m, model.py:14-36, 50-57); scores = q k^T * scaler + mask, softmax, times V
 * (model.py:127-132); the result of head h at token s is multiplied by
 * sigmoid(gate[b,s,h]) (gate bf16 [B,S,q_heads], the head-gate Linear's output,
 * model.py:139-142). mask: NULL or float [S,S], added to every sequence's scores.
 * out bf16 [B,S,q_heads * 64]. head_dim 64, S <= 128; else MOE_B200_ERR_UNSUPPORTED. */
int moe_b200_attention(const void* qkv, const void* gate, const float* pos_emb, const float* mask,
                       int64_t B, int S, int q_heads, int kv_heads, int head_dim, float scaler,
                       void* out, void* stream);

/* ---- Training mode ---------------------------------------------------------------
 * The reference trains through this block (loss.backward(), train.py:140-141): under
 * .train() FeedForward.forward applies nn.Dropout to h (model.py:164,183), and
 * torch.autograd differentiates model.py:200-276 and 173-190. These entry points are
 * that forward and its backward pass for bf16. Both work on the block's ordinary
 * workspace (which the forward fills and the backward reads: call the backward before
 * the next forward on the same workspace) plus a training workspace for the saved
 * pre-activations, the transposed operands and the parameter gradients. */
enum {
  MOE_B200_TWS_GU = 0,   /* bf16 [N*k, 2f] gate/up pre-activations; (dg, du) after the backward */
  MOE_B200_TWS_PAIR_OF,  /* int32 [N*k]    token * k + slot of every sorted row */
  MOE_B200_TWS_KOFF,     /* int32 [E+1]    expert starts, each padded to a multiple of 64 */
  MOE_B200_TWS_DY, MOE_B200_TWS_DH, MOE_B200_TWS_DXS,   /* gradients of y, h, sorted x */
  MOE_B200_TWS_W1T, MOE_B200_TWS_W2T,                   /* transposed weights [E][d][2f], [E][f][d] */
  MOE_B200_TWS_TMAPS,    /* tensor maps of W1T[e], W2T[e] (moe_b200_train_setup) */
  MOE_B200_TWS_XT, MOE_B200_TWS_HT, MOE_B200_TWS_DYT, MOE_B200_TWS_DGUT, /* [cols][padded rows] */
  MOE_B200_TWS_DL,       /* float [N,E]   gradient of the router logits */
  MOE_B200_TWS_DW,       /* float [N,k]   gradient of the renormalised scores */
  MOE_B200_TWS_ONES,     /* float [N,k]   ones (moe_b200_train_setup) */
  MOE_B200_TWS_DWG_F32,  /* float [E*d + E] accumulators of the gate gradients */
  MOE_B200_TWS_DXR,      /* bf16 [N,d]    the router's share of grad_x */
  /* results of moe_b200_backward, bf16: */
  MOE_B200_TWS_G_WG,     /* [E,d]      gradient of gate.weight */
  MOE_B200_TWS_G_BG,     /* [E]        gate.bias */
  MOE_B200_TWS_G_W1,     /* [E,2f,d]   experts.e.gate_and_up.weight */
  MOE_B200_TWS_G_B1,     /* [E,2f]     experts.e.gate_and_up.bias */
  MOE_B200_TWS_G_W2,     /* [E,d,f]    experts.e.down.weight */
  MOE_B200_TWS_G_B2,     /* [E,d]      experts.e.down.bias */
  MOE_B200_TWS_NUM
};
size_t moe_b200_train_workspace_bytes(int64_t N, int d, int f, int E, int k, int dtype);
int moe_b200_train_workspace_layout(int64_t N, int d, int f, int E, int k, int dtype,
                                    size_t* h_offsets);
/* Once per training workspace (synchronous): tensor maps of its transposed-weight
 * buffers, constants. */
int moe_b200_train_setup(int64_t N, int d, int f, int E, int k, int dtype, void* train_ws,
                         size_t train_ws_bytes, void* stream);

/* MOE.forward in training mode (model.py:200-276 with model.py:183 active): as
 * moe_b200_forward on the large-N kernels at every N, with dropout on h. The mask is
 * counter-based: element (token * k + slot, column c) of h is dropped iff word c % 4 of
 * Philox4x32-10(counter = (c / 4, token * k + slot, 0, 0), key = seed) is below
 * dropout_p * 2^32; kept elements are scaled by 1 / (1 - dropout_p). The same
 * dropout_p and seed must be given to moe_b200_backward. */
int moe_b200_forward_train(const void* x, const void* Wg, const void* bg, const void* plan,
                           const void* residual, int64_t N, int d, int f, int E, int k, int dtype,
                           float dropout_p, uint64_t seed, void* workspace, size_t workspace_bytes,
                           void* train_ws, size_t train_ws_bytes, void* out, void* stream);

/* Backward of moe_b200_forward_train: grad_out [N,d] = gradient of the block's output,
 * grad_aux = gradient of the load-balancing loss (a host scalar). Writes grad_x [N,d]
 * (gradient of x; a fused residual's gradient is grad_out itself) and the parameter
 * gradients into the MOE_B200_TWS_G_* regions. The expert counts inside the loss carry
 * no gradient (torch.bincount, model.py:213). */
int moe_b200_backward(const void* x, const void* Wg, const void* plan, const void* grad_out,
                      float grad_aux, int64_t N, int d, int f, int E, int k, int dtype,
                      float dropout_p, uint64_t seed, void* workspace, size_t workspace_bytes,
                      void* train_ws, size_t train_ws_bytes, void* grad_x, void* stream);

/* The expert feed-forward alone in training mode: FeedForward.forward under .train()
 * (model.py:173-190 with model.py:183 active) for the rows of every group of `offsets`; the
 * reference's dense FeedForward (use_moe=False, model.py:302,316) is one group. The training
 * workspace is laid out by moe_b200_train_workspace_layout(M, d, f, E, 1, dtype) and prepared
 * by moe_b200_train_setup with the same arguments. Row r's dropout mask is that of pair r. */
int moe_b200_experts_train(const void* x_sorted, const int32_t* offsets, const void* plan,
                           int64_t M, int d, int f, int E, float dropout_p, uint64_t seed,
                           void* train_ws, size_t train_ws_bytes, void* h, void* y,
                           int32_t* status, void* stream);
/* Its backward: grad_y [M,d] -> grad_x [M,d], parameter gradients in the MOE_B200_TWS_G_W1 /
 * G_B1 / G_W2 / G_B2 regions; x_sorted and h are the forward's input and (dropped) h. */
int moe_b200_experts_backward(const void* x_sorted, const void* h, const int32_t* offsets,
                              const void* plan, const void* grad_y, int64_t M, int d, int f, int E,
                              float dropout_p, uint64_t seed, void* train_ws, size_t train_ws_bytes,
                              void* grad_x, int32_t* status, void* stream);

/* ---- Expert-parallel configuration ------------------------------------------
 * Tokens are sharded over `world` ranks (one process per GPU, rank r owns
 * N_local tokens) and experts are owned by rank h_expert_owner[e]; the
 * reference has no multi-GPU path, these entry points extend MOE.forward
 * (model.py:200-276) to that sharding. Dispatch and combine are all-to-all
 * exchanges written as peer stores inside the kernels; the caller provides, on
 * every rank, one "symmetric" buffer of moe_b200_ep_symm_bytes bytes that all
 * ranks can address (h_symm_bases[q] = rank q's buffer as mapped in THIS
 * process), zero-filled once before the first call. bf16 only. */
enum {
  MOE_B200_EP_SYMM_FLAGS = 0, /* uint32 [3][8] epoch words */
  MOE_B200_EP_SYMM_CNT_ALL,   /* int32 [world][256+2E] counts published by every rank */
  MOE_B200_EP_SYMM_RECV_META, /* int32 [cap] return address of each received row */
  MOE_B200_EP_SYMM_RECV_X,    /* bf16 [cap][d] received rows, cap = N_local*k*world */
  MOE_B200_EP_SYMM_RET_Y,     /* bf16 [N_local*k][d] expert outputs in (token, slot) order */
  MOE_B200_EP_SYMM_NUM
};
enum {
  MOE_B200_EP_WS_STATUS = 0, /* int32 [16] status words, then the call counter */
  MOE_B200_EP_WS_LOGITS, MOE_B200_EP_WS_IDX, MOE_B200_EP_WS_W,
  MOE_B200_EP_WS_PSUM_PART, MOE_B200_EP_WS_PSUM, /* float [E], summed over all ranks */
  MOE_B200_EP_WS_AUX,          /* loss over all N_local*world tokens (model.py:213-216) */
  MOE_B200_EP_WS_SCRATCH, MOE_B200_EP_WS_CNT_SLOT0, /* int32 [E], all ranks */
  MOE_B200_EP_WS_OFFSETS_LOCAL, /* int32 [E_local+1] rows received per owned (virtual) expert */
  MOE_B200_EP_WS_OWNER,        /* int32 owner[256], vmap[E][world]: written by moe_b200_ep_setup */
  MOE_B200_EP_WS_H,            /* bf16 [cap][f] */
  MOE_B200_EP_WS_NUM
};
size_t moe_b200_ep_symm_bytes(int64_t N_local, int d, int E, int k, int world);
int moe_b200_ep_symm_layout(int64_t N_local, int d, int E, int k, int world, size_t* h_offsets);
size_t moe_b200_ep_workspace_bytes(int64_t N_local, int d, int f, int E, int k, int world);
int moe_b200_ep_workspace_layout(int64_t N_local, int d, int f, int E, int k, int world,
                                 size_t* h_offsets);

/* Expert placement, uploaded once into the workspace (synchronous; call it again
 * when the placement changes or the workspace is a new allocation). Experts are
 * addressed by virtual ids v in [0, EV): h_owner[v] is the rank that runs v,
 * h_vmap[e * world + r] the virtual expert that rank r's rows for expert e go to.
 * Without replication EV = E and h_vmap[e * world + r] = e. Giving a popular
 * expert several virtual ids on different ranks (with the same weights in each
 * rank's plan) splits its rows between them. Also zeroes the status words and
 * the call counter: call it on all ranks together, with the symmetric buffers
 * zero-filled. */
int moe_b200_ep_setup(const int32_t* h_owner, const int32_t* h_vmap, int64_t N_local, int d, int f,
                      int E, int k, int world, int EV, void* workspace, size_t workspace_bytes,
                      void* stream);

/* One sharded forward on this rank: router on the local tokens, count exchange,
 * dispatch push to the expert owners, grouped GEMMs on the received rows with
 * the down pass writing straight to the token owners, combine (+ residual).
 * The workspace must have been prepared by moe_b200_ep_setup with the same
 * shape. plan_local covers the E_local virtual experts this rank owns, in
 * increasing virtual id. flags: reserved, pass 0.
 * h_stage_events: NULL, or MOE_B200_EP_EV_NUM cudaEvent_t handles that the call
 * records on `stream` at the stage boundaries (for per-stage timing; the waits
 * on peers are part of the stages they end).
 * All ranks must make the same sequence of calls on workspaces and symmetric
 * buffers that were set up together: the hand-shakes are numbered by a call
 * counter that lives in the workspace (so the launches of one call can be
 * captured in a CUDA graph and replayed). A peer that never arrives makes the
 * bounded waits run out: status word = MOE_B200_DEV_TIMEOUT. */
int moe_b200_ep_forward(const void* x, const void* Wg, const void* bg, const void* plan_local,
                        const void* residual, int64_t N_local, int d, int f, int E, int k,
                        int dtype, int flags, int rank, int world, int EV,
                        int E_local, void* const* h_symm_bases,
                        void* workspace, size_t workspace_bytes, void* out,
                        void* const* h_stage_events, void* stream);
enum {
  MOE_B200_EP_EV_START = 0, /* before the router */
  MOE_B200_EP_EV_ROUTER,    /* router done */
  MOE_B200_EP_EV_DISPATCH,  /* counts exchanged, own rows pushed to their owners */
  MOE_B200_EP_EV_EXPERTS,   /* every source's rows waited for, both grouped GEMMs done, outputs
                             * stored to the token owners */
  MOE_B200_EP_EV_COMBINE,   /* every owner's outputs waited for, combine done */
  MOE_B200_EP_EV_NUM
};

/* Copy the 16 status words to the host after synchronising the stream.
 * Returns h_status[0]. Synchronous. */
int moe_b200_read_status(const int32_t* status, int32_t* h_status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOE_B200_H */
