// Core of the reference's Attention.forward (model.py:96-152) between its two Linears, for
// head_dim 64 and contexts up to 128 tokens, in one kernel:
//   split of the fused QKV projection (model.py:104), KV heads shared by groups of query heads
//   (the repeat_interleave of model.py:112-115 becomes "all heads of a group read the same K/V
//   in shared memory"), RoPE on queries and keys from the model's own table (model.py:123-124,
//   table rows [cos | signed sin] of model.py:14-36), scores = q k^T / sqrt(head_dim) + mask
//   (model.py:127-130), softmax (:131), times V (:132), times the sigmoid head gate (:139-142).
// The [B, H, S, S] score tensor of the reference is never written: a block owns one
// (sequence, KV head), keeps that head's rotated K and transposed V in shared memory, and each
// warp runs whole query heads through mma.sync m16n8k16 with the probabilities staying in
// registers between the two products. HBM traffic = QKV in, output out.
#include "common.cuh"

namespace moe {

namespace {

constexpr int HD = 64;            // head_dim
constexpr int kMaxS = 128;        // context limit of this kernel
constexpr int kWarpsAtt = 8;

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// out[i] = x[i] * pe[i] + x[i ^ 1] * pe[HD + i]: the reference's cat(x, swap_pairs(x)) * pos_emb,
// halves added (model.py:50-57); eight consecutive elements at a time.
__device__ __forceinline__ void rope8(const float (&x)[8], const float* __restrict__ pe, int c,
                                      float (&o)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = x[i] * pe[c + i] + x[i ^ 1] * pe[HD + c + i];
}

// Shared memory: K [S][72] bf16 (rotated), Vt [64][S+8] bf16, per warp Q [16][72] bf16,
// pos_emb [S][128] f32, mask [S][S] f32 (optional).
template <int S_TILES>   // ceil(S / 16), 1..8
__global__ void __launch_bounds__(kWarpsAtt * 32)
attention_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ gate,
                 const float* __restrict__ pos_emb, const float* __restrict__ mask, int S, int H,
                 int KV, float scaler, __nv_bfloat16* __restrict__ out) {
  constexpr int SP = S_TILES * 16;        // padded context
  constexpr int KP = HD + 8;              // K / Q row pitch (bf16): conflict-free fragment loads
  constexpr int VP = SP + 8;              // Vt row pitch
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smem_raw);           // [SP][KP]
  __nv_bfloat16* sVt = sK + SP * KP;                                        // [HD][VP]
  __nv_bfloat16* sQ = sVt + HD * VP;                                        // [warps][16][KP]
  float* sPE = reinterpret_cast<float*>(sQ + kWarpsAtt * 16 * KP);          // [SP][2*HD]
  float* sM = sPE + SP * 2 * HD;                                            // [SP][SP] when mask

  const int b = blockIdx.x / KV, kvh = blockIdx.x - b * KV;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int row_elems = (H + 2 * KV) * HD;                   // one token's fused QKV row
  const __nv_bfloat16* base = qkv + (size_t)b * S * row_elems;
  const int heads_per_kv = H / KV;

  // ---- stage the table, the mask, rotated K and transposed V ----
  for (int i = threadIdx.x; i < SP * 2 * HD; i += blockDim.x) {
    const int s = i / (2 * HD);
    sPE[i] = s < S ? pos_emb[i] : 0.f;
  }
  if (mask != nullptr)
    for (int i = threadIdx.x; i < SP * SP; i += blockDim.x) {
      const int r = i / SP, c = i - r * SP;
      sM[i] = (r < S && c < S) ? mask[r * S + c] : (c < S ? 0.f : -INFINITY);
    }
  __syncthreads();
  for (int i = threadIdx.x; i < SP * (HD / 8); i += blockDim.x) {
    const int s = i / (HD / 8), c = (i - s * (HD / 8)) * 8;
    float kx[8], vx[8], ko[8];
    if (s < S) {
      load8(base + (size_t)s * row_elems + (H + kvh) * HD + c, kx);
      load8(base + (size_t)s * row_elems + (H + KV + kvh) * HD + c, vx);
      rope8(kx, sPE + s * 2 * HD, c, ko);
    } else {
#pragma unroll
      for (int q = 0; q < 8; ++q) ko[q] = vx[q] = 0.f;
    }
    store8(sK + s * KP + c, ko);
#pragma unroll
    for (int q = 0; q < 8; ++q) sVt[(c + q) * VP + s] = __float2bfloat16_rn(vx[q]);
  }
  __syncthreads();

  __nv_bfloat16* myQ = sQ + warp * 16 * KP;
  // A warp's work: (query head, 16-row tile) items. The rows of the next item and its gate
  // values are requested before the products of the current one, so that a warp always has
  // loads in flight.
  const int my_heads = warp < heads_per_kv ? (heads_per_kv - warp + kWarpsAtt - 1) / kWarpsAtt : 0;
  const int items = my_heads * S_TILES;
  const uint4 zero4 = make_uint4(0, 0, 0, 0);
  auto fetch = [&](int item, uint4 (&raw)[4], float& ga, float& gb) {
    const int h = kvh * heads_per_kv + warp + (item / S_TILES) * kWarpsAtt, mt = item % S_TILES;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int i = lane + 32 * q;
      const int s = mt * 16 + (i >> 3), c = (i & 7) * 8;
      raw[q] = s < S ? __ldg(reinterpret_cast<const uint4*>(base + (size_t)s * row_elems + h * HD + c)) : zero4;
    }
    const int r0 = mt * 16 + g;
    ga = r0 < S ? __bfloat162float(gate[((size_t)b * S + r0) * H + h]) : 0.f;
    gb = r0 + 8 < S ? __bfloat162float(gate[((size_t)b * S + r0 + 8) * H + h]) : 0.f;
  };
  uint4 raw[4];
  float gate_a = 0.f, gate_b = 0.f;
  if (items > 0) fetch(0, raw, gate_a, gate_b);
  for (int item = 0; item < items; ++item) {
    {
      const int h = kvh * heads_per_kv + warp + (item / S_TILES) * kWarpsAtt, mt = item % S_TILES;
      // ---- 16 query rows of this head, rotated, into the warp's staging area ----
      __syncwarp();
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int i = lane + 32 * q;
        const int sl = i >> 3, c = (i & 7) * 8;
        const int s = mt * 16 + sl;
        const uint32_t w[4] = {raw[q].x, raw[q].y, raw[q].z, raw[q].w};
        float qx[8], qo[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) { qx[2 * e] = bf16_lo(w[e]); qx[2 * e + 1] = bf16_hi(w[e]); }
        if (s < S) {
          rope8(qx, sPE + s * 2 * HD, c, qo);
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) qo[e] = 0.f;
        }
        store8(myQ + sl * KP + c, qo);
      }
      const float cur_ga = gate_a, cur_gb = gate_b;
      if (item + 1 < items) fetch(item + 1, raw, gate_a, gate_b);
      __syncwarp();
      // ---- scores of 16 query rows against all keys ----
      float sc[2 * S_TILES][4];
#pragma unroll
      for (int n = 0; n < 2 * S_TILES; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) sc[n][i] = 0.f;
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk) {
        const __nv_bfloat16* qa = myQ + g * KP + kk * 16 + 2 * t;
        const uint32_t a0 = *reinterpret_cast<const uint32_t*>(qa);
        const uint32_t a1 = *reinterpret_cast<const uint32_t*>(qa + 8 * KP);
        const uint32_t a2 = *reinterpret_cast<const uint32_t*>(qa + 8);
        const uint32_t a3 = *reinterpret_cast<const uint32_t*>(qa + 8 * KP + 8);
#pragma unroll
        for (int n = 0; n < 2 * S_TILES; ++n) {
          const __nv_bfloat16* kb = sK + (n * 8 + g) * KP + kk * 16 + 2 * t;
          mma16816(sc[n], a0, a1, a2, a3, *reinterpret_cast<const uint32_t*>(kb),
                   *reinterpret_cast<const uint32_t*>(kb + 8));
        }
      }
      // ---- scale, mask, softmax over the keys (rows g and g + 8 of the tile) ----
      const int r0 = mt * 16 + g, r1 = r0 + 8;
      float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
      for (int n = 0; n < 2 * S_TILES; ++n) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int col = n * 8 + 2 * t + (i & 1);
          const int row = (i < 2) ? r0 : r1;
          float v = sc[n][i] * scaler;
          if (mask != nullptr) v += sM[row * SP + col];
          else if (col >= S) v = -INFINITY;
          sc[n][i] = v;
        }
        m0 = fmaxf(m0, fmaxf(sc[n][0], sc[n][1]));
        m1 = fmaxf(m1, fmaxf(sc[n][2], sc[n][3]));
      }
#pragma unroll
      for (int o = 1; o <= 2; o <<= 1) {
        m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, o));
        m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, o));
      }
      float l0 = 0.f, l1 = 0.f;
#pragma unroll
      for (int n = 0; n < 2 * S_TILES; ++n) {
        sc[n][0] = __expf(sc[n][0] - m0); sc[n][1] = __expf(sc[n][1] - m0);
        sc[n][2] = __expf(sc[n][2] - m1); sc[n][3] = __expf(sc[n][3] - m1);
        l0 += sc[n][0] + sc[n][1];
        l1 += sc[n][2] + sc[n][3];
      }
#pragma unroll
      for (int o = 1; o <= 2; o <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, o);
        l1 += __shfl_xor_sync(0xffffffffu, l1, o);
      }
      const float inv0 = 1.f / l0, inv1 = 1.f / l1;
      // ---- probabilities (bf16, straight from the accumulator registers) times V ----
      float o_acc[HD / 8][4];
#pragma unroll
      for (int n = 0; n < HD / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) o_acc[n][i] = 0.f;
#pragma unroll
      for (int kk = 0; kk < S_TILES; ++kk) {
        const uint32_t a0 = pack_bf16x2(sc[2 * kk][0] * inv0, sc[2 * kk][1] * inv0);
        const uint32_t a1 = pack_bf16x2(sc[2 * kk][2] * inv1, sc[2 * kk][3] * inv1);
        const uint32_t a2 = pack_bf16x2(sc[2 * kk + 1][0] * inv0, sc[2 * kk + 1][1] * inv0);
        const uint32_t a3 = pack_bf16x2(sc[2 * kk + 1][2] * inv1, sc[2 * kk + 1][3] * inv1);
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) {
          const __nv_bfloat16* vb = sVt + (n * 8 + g) * VP + kk * 16 + 2 * t;
          mma16816(o_acc[n], a0, a1, a2, a3, *reinterpret_cast<const uint32_t*>(vb),
                   *reinterpret_cast<const uint32_t*>(vb + 8));
        }
      }
      // ---- sigmoid head gate (model.py:139-142); the tile leaves through the warp's staging
      // area (free since the score products) as 128-byte runs per row ----
      const float g0 = 1.f / (1.f + __expf(-cur_ga)), g1 = 1.f / (1.f + __expf(-cur_gb));
      __syncwarp();
#pragma unroll
      for (int n = 0; n < HD / 8; ++n) {
        *reinterpret_cast<uint32_t*>(myQ + g * KP + n * 8 + 2 * t) = pack_bf16x2(o_acc[n][0] * g0, o_acc[n][1] * g0);
        *reinterpret_cast<uint32_t*>(myQ + (g + 8) * KP + n * 8 + 2 * t) = pack_bf16x2(o_acc[n][2] * g1, o_acc[n][3] * g1);
      }
      __syncwarp();
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int i = lane + 32 * q;
        const int sl = i >> 3, c = (i & 7) * 8;
        const int srow = mt * 16 + sl;
        if (srow < S)
          *reinterpret_cast<uint4*>(out + ((size_t)b * S + srow) * H * HD + h * HD + c) =
              *reinterpret_cast<const uint4*>(myQ + sl * KP + c);
      }
    }
  }
}

template <int ST>
int launch_att(const void* qkv, const void* gate, const float* pos_emb, const float* mask, int B, int S,
               int H, int KV, float scaler, void* out, cudaStream_t s) {
  constexpr int SP = ST * 16;
  const size_t smem = (size_t)(SP * (HD + 8) + HD * (SP + 8) + kWarpsAtt * 16 * (HD + 8)) * 2 +
                      (size_t)SP * 2 * HD * 4 + (mask != nullptr ? (size_t)SP * SP * 4 : 0);
  static PerDeviceOnce once;
  int rc = ensure_dynamic_smem(once, attention_kernel<ST>, 227 * 1024);
  if (rc) return rc;
  if (smem > 227 * 1024) return set_error(MOE_B200_ERR_UNSUPPORTED, "context too long for the shared-memory layout");
  attention_kernel<ST><<<(unsigned)(B * KV), kWarpsAtt * 32, smem, s>>>(
      static_cast<const __nv_bfloat16*>(qkv), static_cast<const __nv_bfloat16*>(gate), pos_emb, mask, S,
      H, KV, scaler, static_cast<__nv_bfloat16*>(out));
  MOE_CUDA_CHECK(cudaGetLastError());
  return 0;
}

}  // namespace
}  // namespace moe

using namespace moe;

extern "C" int moe_b200_attention(const void* qkv, const void* gate, const float* pos_emb,
                                  const float* mask, int64_t B, int S, int q_heads, int kv_heads,
                                  int head_dim, float scaler, void* out, void* stream) {
  if (head_dim != HD) return set_error(MOE_B200_ERR_UNSUPPORTED, "head_dim must be 64");
  if (S < 1 || S > kMaxS) return set_error(MOE_B200_ERR_UNSUPPORTED, "context must be in [1,128]");
  if (B < 0 || B > (1 << 24) || q_heads < 1 || kv_heads < 1 || q_heads % kv_heads != 0)
    return set_error(MOE_B200_ERR_SHAPE, "B or head counts out of range");
  if (B == 0) return 0;
  if (!qkv || !gate || !pos_emb || !out) return set_error(MOE_B200_ERR_NULL, "NULL argument");
  if (!aligned16(qkv) || !aligned16(out)) return set_error(MOE_B200_ERR_ALIGN, "buffers must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  switch ((S + 15) / 16) {
    case 1: return launch_att<1>(qkv, gate, pos_emb, mask, (int)B, S, q_heads, kv_heads, scaler, out, s);
    case 2: return launch_att<2>(qkv, gate, pos_emb, mask, (int)B, S, q_heads, kv_heads, scaler, out, s);
    case 3: return launch_att<3>(qkv, gate, pos_emb, mask, (int)B, S, q_heads, kv_heads, scaler, out, s);
    case 4: return launch_att<4>(qkv, gate, pos_emb, mask, (int)B, S, q_heads, kv_heads, scaler, out, s);
    case 5: return launch_att<5>(qkv, gate, pos_emb, mask, (int)B, S, q_heads, kv_heads, scaler, out, s);
    case 6: return launch_att<6>(qkv, gate, pos_emb, mask, (int)B, S, q_heads, kv_heads, scaler, out, s);
    case 7: return launch_att<7>(qkv, gate, pos_emb, mask, (int)B, S, q_heads, kv_heads, scaler, out, s);
    default: return launch_att<8>(qkv, gate, pos_emb, mask, (int)B, S, q_heads, kv_heads, scaler, out, s);
  }
}
