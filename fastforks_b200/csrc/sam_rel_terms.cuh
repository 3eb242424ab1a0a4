// The two products behind SAM's decomposed relative-position bias, for every query of a square grid:
//   rel_h[b, head, (y, x), k] = q[b, (y, x), head, :] . rel_pos_h[y - k + side - 1, :]
//   rel_w[b, head, (y, x), k] = q[b, (y, x), head, :] . rel_pos_w[x - k + side - 1, :]      (k = 0 .. side - 1)
// q is the UNSCALED query of head dim 64, read in place from the packed qkv tensor; the tables are the module's
// parameters themselves ([2 * side - 1, 64]): the [side, side, 64] gather the upstream code builds first
// (get_rel_pos) never exists. HBM-bound work on the FMA pipe: q is read once, the results are written once.
//
// One CTA takes the queries that share one coordinate (which = 0: a grid row y, for rel_h; which = 1: a grid column
// x, for rel_w), because they share the `side` table rows: those are staged in shared memory as fp32, one thread
// then owns a query row (64 values in registers) and walks the table rows with broadcast 16-byte loads.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace b200 {

struct RelTermsParams {
  const void* q;
  int64_t q_sb, q_sn, q_sh;  // element strides of q: batch, token, head
  const void* rel_pos_h;     // [2 * side - 1, 64]
  const void* rel_pos_w;
  void* rel_h;               // [batch, heads, side * side, side], contiguous
  void* rel_w;
  int batch, heads, side;
};

constexpr int kRelThreads = 256;
constexpr int kRelMaxSide = 64;  // shared memory: side rows of 64 floats

template <typename T>
__device__ __forceinline__ float2 rel_unpack2(uint32_t v);
template <>
__device__ __forceinline__ float2 rel_unpack2<__half>(uint32_t v) {
  return __half22float2(*reinterpret_cast<const __half2*>(&v));
}
template <>
__device__ __forceinline__ float2 rel_unpack2<__nv_bfloat16>(uint32_t v) {
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
template <typename T>
__device__ __forceinline__ uint32_t rel_pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t rel_pack2<__half>(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t rel_pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <typename T>
__global__ void __launch_bounds__(kRelThreads) sam_rel_terms_kernel(const RelTermsParams p) {
  __shared__ __align__(16) float table[kRelMaxSide][64];  // table[k] = rel_pos[c - k + side - 1]
  const int side = p.side, n_tokens = side * side;
  const int which = blockIdx.y;               // 0: rel_h (fixed y), 1: rel_w (fixed x)
  const int b = blockIdx.x / side, c = blockIdx.x - b * side;
  const T* rel_pos = static_cast<const T*>(which == 0 ? p.rel_pos_h : p.rel_pos_w);
  for (int i = threadIdx.x; i < side * 32; i += kRelThreads) {
    const int k = i >> 5, pair = i & 31;
    const float2 v = rel_unpack2<T>(reinterpret_cast<const uint32_t*>(rel_pos + static_cast<int64_t>(c - k + side - 1) * 64)[pair]);
    table[k][2 * pair] = v.x;
    table[k][2 * pair + 1] = v.y;
  }
  __syncthreads();
  T* out = static_cast<T*>(which == 0 ? p.rel_h : p.rel_w);
  const int rows = side * p.heads;  // the queries of this CTA: `side` tokens x heads
  // blockIdx.z splits the rows: every thread has at most one, so that a 64 x 64 grid (768 rows per coordinate) makes
  // three CTAs per coordinate instead of one CTA that walks three rows per thread on an otherwise idle GPU.
  for (int r = blockIdx.z * kRelThreads + threadIdx.x; r < rows; r += gridDim.z * kRelThreads) {
    const int j = r / p.heads, head = r - j * p.heads;
    const int n = which == 0 ? c * side + j : j * side + c;
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const T*>(p.q) + b * p.q_sb + n * p.q_sn + head * p.q_sh);
    float q[64];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const uint4 v = __ldg(src + u);
      const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = rel_unpack2<T>(w4[e]);
        q[u * 8 + e * 2] = f.x;
        q[u * 8 + e * 2 + 1] = f.y;
      }
    }
    T* dst = out + ((static_cast<int64_t>(b) * p.heads + head) * n_tokens + n) * side;
    // side is even (checked by the host). Four table rows at a time where they exist: four independent chains of
    // fused multiply-adds hide the latency of the shared-memory loads behind them; a leftover pair goes alone.
    int k = 0;
    for (; k + 4 <= side; k += 4) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ch = 0; ch < 64; ch += 4) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float4 t = *reinterpret_cast<const float4*>(&table[k + u][ch]);
          acc[u] = fmaf(q[ch], t.x, acc[u]);
          acc[u] = fmaf(q[ch + 1], t.y, acc[u]);
          acc[u] = fmaf(q[ch + 2], t.z, acc[u]);
          acc[u] = fmaf(q[ch + 3], t.w, acc[u]);
        }
      }
      *reinterpret_cast<uint32_t*>(dst + k) = rel_pack2<T>(acc[0], acc[1]);
      *reinterpret_cast<uint32_t*>(dst + k + 2) = rel_pack2<T>(acc[2], acc[3]);
    }
    for (; k < side; k += 2) {
      float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
      for (int ch = 0; ch < 64; ch += 4) {
        const float4 t0 = *reinterpret_cast<const float4*>(&table[k][ch]);
        const float4 t1 = *reinterpret_cast<const float4*>(&table[k + 1][ch]);
        acc0 = fmaf(q[ch], t0.x, acc0); acc0 = fmaf(q[ch + 1], t0.y, acc0);
        acc0 = fmaf(q[ch + 2], t0.z, acc0); acc0 = fmaf(q[ch + 3], t0.w, acc0);
        acc1 = fmaf(q[ch], t1.x, acc1); acc1 = fmaf(q[ch + 1], t1.y, acc1);
        acc1 = fmaf(q[ch + 2], t1.z, acc1); acc1 = fmaf(q[ch + 3], t1.w, acc1);
      }
      *reinterpret_cast<uint32_t*>(dst + k) = rel_pack2<T>(acc0, acc1);
    }
  }
}

}  // namespace b200
