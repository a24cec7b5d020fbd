// Router and dispatch of a small call in ONE launch: the kernel around front_small_body
// (front_small.cuh), its launcher and the size limits.
#include "front_small.cuh"

namespace moe {

namespace {

constexpr int kThreads = kFrontThreads;
constexpr int kMaxTok = kFrontMaxTok;
constexpr int kMaxE = kFrontMaxE;
constexpr int kMaxPairs = kFrontMaxPairs;

template <int NT, bool SPLIT>
__global__ void __launch_bounds__(kThreads, 1)
front_small_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ Wg,
                   const __nv_bfloat16* __restrict__ bg, int Ntotal, int d, int E, int k,
                   float* __restrict__ out_logits, int32_t* __restrict__ out_idx,
                   float* __restrict__ out_w, int32_t* __restrict__ cnt_slot,
                   int32_t* __restrict__ offsets, int32_t* __restrict__ row_of,
                   __nv_bfloat16* __restrict__ perm, float* __restrict__ psum,
                   float* __restrict__ aux, int* __restrict__ xch, int* __restrict__ counter,
                   int32_t* __restrict__ status) {
  extern __shared__ float smem[];
  pdl_wait();                 // x may come from the kernel before this one
  pdl_launch_dependents();
  front_small_body<NT, SPLIT>(smem, (int)blockIdx.x, (int)gridDim.x, x, Wg, bg, Ntotal, d, E, k,
                              out_logits, out_idx, out_w, cnt_slot, offsets, row_of, perm, psum, aux,
                              xch, counter, status);
}

template <int NT>
int launch(const void* x, const void* Wg, const void* bg, int N, int d, int E, int k,
           float* out_logits, int32_t* out_idx, float* out_w, int32_t* cnt_slot, int32_t* offsets,
           int32_t* row_of, void* perm, float* psum, float* aux, int* xch, int* counter,
           int32_t* status, cudaStream_t s) {
  // beyond 128 tokens repeating the routing in every block costs more than one exchange
  const bool split = xch != nullptr && counter != nullptr && status != nullptr && N > 128;
  const int ntok = split ? 16 : N;
  const size_t smem = front_small_smem_bytes(NT, ntok, E, k);
  static PerDeviceOnce once_whole, once_split;
  int rc = ensure_dynamic_smem(once_whole, front_small_kernel<NT, false>, 160 * 1024);
  if (rc) return rc;
  rc = ensure_dynamic_smem(once_split, front_small_kernel<NT, true>, 160 * 1024);
  if (rc) return rc;
  // one block per 16 tokens
  const int blocks = N <= 16 ? 1 : (N + 15) / 16;
  auto fn = split ? front_small_kernel<NT, true> : front_small_kernel<NT, false>;
  MOE_CUDA_CHECK(launch_pdl(fn, dim3(blocks), dim3(kThreads), smem, s,
                            static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(Wg),
                            static_cast<const __nv_bfloat16*>(bg), N, d, E, k, out_logits, out_idx,
                            out_w, cnt_slot, offsets, row_of, static_cast<__nv_bfloat16*>(perm), psum,
                            aux, xch, counter, status));
  return 0;
}

}  // namespace

bool front_small_supported(int64_t N, int E, int k, int dtype) {
  return dtype == MOE_B200_BF16 && N >= 1 && N <= kMaxTok && N * k <= kMaxPairs && E <= kMaxE;
}

// With the exchange buffer and the counter (blocks share the work): as many tokens as give a grid
// whose blocks are all resident at once with room to spare.
bool front_split_supported(int64_t N, int E, int k, int dtype) {
  return dtype == MOE_B200_BF16 && N >= 1 && N <= 16 * 128 && E <= kMaxE && k <= kMaxTopK;
}

// xch: int32 scratch of at least front_small_exchange_ints(N, E, k) words and counter: one int32
// that is zero on entry (both only used beyond 128 tokens; without them every block repeats the
// whole routing at every size).
int64_t front_small_exchange_ints(int64_t N, int E, int k) {
  const int64_t nb = (N + 15) / 16;
  return nb * k * E + nb * E;
}

int launch_front_small(const void* x, const void* Wg, const void* bg, int64_t N, int d, int E, int k,
                       float* out_logits, int32_t* out_idx, float* out_w, int32_t* cnt_slot,
                       int32_t* offsets, int32_t* row_of, void* perm, float* psum, float* aux,
                       cudaStream_t s, int* xch, int* counter, int32_t* status) {
  if (E <= 8) return launch<1>(x, Wg, bg, (int)N, d, E, k, out_logits, out_idx, out_w, cnt_slot, offsets, row_of, perm, psum, aux, xch, counter, status, s);
  if (E <= 16) return launch<2>(x, Wg, bg, (int)N, d, E, k, out_logits, out_idx, out_w, cnt_slot, offsets, row_of, perm, psum, aux, xch, counter, status, s);
  return launch<4>(x, Wg, bg, (int)N, d, E, k, out_logits, out_idx, out_w, cnt_slot, offsets, row_of, perm, psum, aux, xch, counter, status, s);
}

}  // namespace moe
