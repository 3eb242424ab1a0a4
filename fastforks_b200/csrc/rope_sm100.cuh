// DINOv3's rotary position embedding, in place on the q and k views of a packed qkv tensor, head dim 64:
//   out[j]      = (x[j] cos[j] - x[j + 32] sin[j]) * m
//   out[j + 32] = (x[j + 32] cos[j] + x[j] sin[j]) * m          j = 0 .. 31   (= x cos + rotate_half(x) sin)
// with m = q_scale for q and 1 for k, in fp32, rounded once. The first `prefix` tokens of a sequence (class token
// and registers) are not rotated: their q is only scaled, their k is left alone. The table `cs` holds, per patch
// token, 32 cosines then 32 sines in fp32 (dims j and j + 32 share an angle).
//
// HBM-bound, one read and one write of q and k: a thread takes eight dims j and their partners j + 32 (two 16-byte
// loads, two 16-byte stores); the threads of a CTA cover one token's (q | k, head, dim group) units so that a warp's
// accesses are contiguous in the packed layout, and the token's table row is read by every head from L1.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace b200 {

struct RopeParams {
  void* q;
  void* k;
  int64_t q_sb, q_sn, q_sh;  // element strides: batch, token, head
  int64_t k_sb, k_sn, k_sh;
  const float* cs;           // [tokens - prefix, 2, 32]
  int batch, heads, tokens, prefix;
  float q_scale;
};

constexpr int kRopeThreads = 128;

template <typename T>
__device__ __forceinline__ float2 rope_unpack2(uint32_t v);
template <>
__device__ __forceinline__ float2 rope_unpack2<__half>(uint32_t v) {
  return __half22float2(*reinterpret_cast<const __half2*>(&v));
}
template <>
__device__ __forceinline__ float2 rope_unpack2<__nv_bfloat16>(uint32_t v) {
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
template <typename T>
__device__ __forceinline__ uint32_t rope_pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t rope_pack2<__half>(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t rope_pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <typename T>
__global__ void __launch_bounds__(kRopeThreads) rope_qk_kernel(const RopeParams p) {
  const int units = 8 * p.heads;  // per token: (q | k) x heads x four groups of eight dims
  const long long rows = static_cast<long long>(p.batch) * p.tokens;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const int b = static_cast<int>(row / p.tokens), n = static_cast<int>(row - static_cast<long long>(b) * p.tokens);
    const int np = n - p.prefix;
    for (int u = threadIdx.x; u < units; u += kRopeThreads) {
      const int is_k = u >= 4 * p.heads ? 1 : 0;
      const int v = u - is_k * 4 * p.heads;
      const int h = v >> 2, g = v & 3;
      if (np < 0 && is_k) continue;  // prefix tokens: k is left alone
      T* x = is_k ? static_cast<T*>(p.k) + b * p.k_sb + n * p.k_sn + h * p.k_sh
                  : static_cast<T*>(p.q) + b * p.q_sb + n * p.q_sn + h * p.q_sh;
      uint4* lo_ptr = reinterpret_cast<uint4*>(x + 8 * g);
      uint4* hi_ptr = reinterpret_cast<uint4*>(x + 32 + 8 * g);
      const uint4 lo = *lo_ptr, hi = *hi_ptr;
      const uint32_t lw[4] = {lo.x, lo.y, lo.z, lo.w}, hw[4] = {hi.x, hi.y, hi.z, hi.w};
      const float m = is_k ? 1.f : p.q_scale;
      uint32_t lo_out[4], hi_out[4];
      if (np < 0) {  // prefix tokens: q is scaled only
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 x1 = rope_unpack2<T>(lw[i]), x2 = rope_unpack2<T>(hw[i]);
          lo_out[i] = rope_pack2<T>(x1.x * m, x1.y * m);
          hi_out[i] = rope_pack2<T>(x2.x * m, x2.y * m);
        }
      } else {
        const float4* cos4 = reinterpret_cast<const float4*>(p.cs + static_cast<long long>(np) * 64 + 8 * g);
        const float4* sin4 = reinterpret_cast<const float4*>(p.cs + static_cast<long long>(np) * 64 + 32 + 8 * g);
        const float4 c0 = __ldg(cos4), c1 = __ldg(cos4 + 1), s0 = __ldg(sin4), s1 = __ldg(sin4 + 1);
        const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 x1 = rope_unpack2<T>(lw[i]), x2 = rope_unpack2<T>(hw[i]);
          // the product is rounded before the subtraction / addition takes it in (no contraction into an FMA with a
          // differently rounded partner): x1 c - x2 s is computed as fma(x1, c, -(x2 s)) on both halves alike
          const float a0 = __fmaf_rn(x1.x, c[2 * i], -__fmul_rn(x2.x, s[2 * i]));
          const float a1 = __fmaf_rn(x1.y, c[2 * i + 1], -__fmul_rn(x2.y, s[2 * i + 1]));
          const float b0 = __fmaf_rn(x2.x, c[2 * i], __fmul_rn(x1.x, s[2 * i]));
          const float b1 = __fmaf_rn(x2.y, c[2 * i + 1], __fmul_rn(x1.y, s[2 * i + 1]));
          lo_out[i] = rope_pack2<T>(a0 * m, a1 * m);
          hi_out[i] = rope_pack2<T>(b0 * m, b1 * m);
        }
      }
      *lo_ptr = make_uint4(lo_out[0], lo_out[1], lo_out[2], lo_out[3]);
      *hi_ptr = make_uint4(hi_out[0], hi_out[1], hi_out[2], hi_out[3]);
    }
  }
}

}  // namespace b200
