// GEMM with a fused epilogue for the layers around attention, on sm_100a:
//
//   y[p, n] = act((sum_k x[p, k] w[n, k] + bias[n]) * scale[n] + res[p, n])         (bias, scale, res optional)
//
// x [M, K] (row stride lda) and w [N, K] (row-major) are fp16 or bf16, accumulation is fp32 in tensor memory, bias
// and res have the type of x, scale is fp32, y has the type of x and may alias res (a thread reads the residual of
// the columns it is about to write, nobody else touches them). act: 0 none, 1 relu, 5 gelu (erf), 6 gelu (tanh form).
//
// Persistent CTAs, one per SM, walk output tiles of BM rows x BN columns (128 x 128, 128 x 256 or 256 x 256, chosen
// by the host: the product needs 2 * 64 * (BM + BN) bytes from L2 for every 2 * 64 * BM * BN flops, and without
// multicast the L2 bandwidth, not the tensor pipe, bounds the narrow tiles):
//   * a loader thread stages x and w tiles of 64 k-values through a ring of shared-memory stages with TMA
//     (128-byte swizzle, rows and k-values past the end read as zero, no multicast);
//   * an MMA thread issues tcgen05.mma (M = 128, N = BN, K = 16, both operands K-major) into accumulators in
//     tensor memory: two alternating ones for BM = 128, so that the next tile's products run during the epilogue;
//     for BM = 256 the two accumulators are the upper and the lower 128 rows of one tile (two MMAs per k-step that
//     share the w tile);
//   * eight epilogue warps read a finished accumulator 32 columns at a time, turn the chunk through shared memory
//     (a thread owns a row in tensor memory, but a warp should write whole rows), apply the epilogue and write y
//     with 16-byte stores that fill their sectors.
// Every barrier wait is bounded (sm100_ptx.cuh); a wait that runs out sets the CTA's abort flag and the role bit
// in the status word, and all warps fall through to the common exit.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "sm100_ptx.cuh"

namespace b200 {

constexpr int kGemmBK = 64;
constexpr int kGemmThreads = 320;  // warp 0 loader, warp 1 MMA, warps 2..9 epilogue
constexpr int kGemmEpiWarp0 = 2;
enum : uint32_t { kStatusGemmLoader = 64, kStatusGemmMma = 128, kStatusGemmEpilogue = 256 };
enum : int { kActNone = 0, kActRelu = 1, kActGelu = 5, kActGeluTanh = 6 };

struct GemmParams {
  int m, n, k;
  int tiles_m, tiles_n;
  const void* bias;    // [n] or null
  const float* scale;  // [n] or null
  const void* res;     // [m, lres] or null
  int64_t lres;
  void* y;
  int64_t ldy;
  int act;
  uint32_t* status;
};

template <int BM, int BN>
struct GemmSmem {
  static constexpr int kStages = BM == 256 ? 3 : BN == 256 ? 4 : 5;
  static constexpr int kBytesA = BM * kGemmBK * 2, kBytesB = BN * kGemmBK * 2;
  alignas(1024) uint8_t a[kStages][kBytesA];
  alignas(1024) uint8_t b[kStages][kBytesB];
  alignas(16) float turn[8][32][32];  // per epilogue warp: 32 rows x 32 columns of fp32 on their way from row owners to row writers
  uint64_t full[kStages], empty[kStages];
  uint64_t acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  uint32_t abort;
};

__device__ __forceinline__ float gemm_act(float v, int act) {
  switch (act) {
    case kActRelu:
      return fmaxf(v, 0.f);
    case kActGelu:
      return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
    case kActGeluTanh: {
      float t;
      const float u = 0.7978845608028654f * v * (1.f + 0.044715f * v * v);
      asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
      return 0.5f * v * (1.f + t);
    }
    default:
      return v;
  }
}

template <typename T>
__device__ __forceinline__ float2 gemm_unpack2(uint32_t v) {
  if constexpr (std::is_same<T, __half>::value) return __half22float2(*reinterpret_cast<const __half2*>(&v));
  else return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
template <typename T>
__device__ __forceinline__ uint32_t gemm_pack2(float lo, float hi) {
  if constexpr (std::is_same<T, __half>::value) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

template <typename T, int BM, int BN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_epilogue_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w, const GemmParams p) {
  static_assert((BM == 128 && (BN == 128 || BN == 256)) || (BM == 256 && BN == 256), "tile shapes that are built");
  using Smem = GemmSmem<BM, BN>;
  constexpr int kStages = Smem::kStages;
  constexpr bool kTall = BM == 256;  // both accumulators belong to one tile
  extern __shared__ uint8_t smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&sm.full[i], 1);
      mbar_init(&sm.empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.acc_full[i], 1);
      mbar_init(&sm.acc_empty[i], kTall ? 4 : 8);  // one arrival per epilogue warp that reads the accumulator
    }
    sm.abort = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc(&sm.tmem_base, 512);  // two accumulators of up to 256 fp32 columns
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_w);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  grid_dependency_wait();  // programmatic stream serialisation: see the attention kernel
  const uint32_t tmem = sm.tmem_base;
  volatile uint32_t* abort_flag = &sm.abort;
  const int tiles = p.tiles_m * p.tiles_n;
  const int k_blocks = (p.k + kGemmBK - 1) / kGemmBK;

  if (warp == 0) {
    // ======================= loader ==================================================================
    if (lane == 0) {
      bool ok = true;
      int g = 0;  // stage uses so far
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        // m runs fastest: CTAs that work at the same time share a w tile (it meets them in L2)
        const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
        for (int kb = 0; kb < k_blocks; ++kb, ++g) {
          const int st = g % kStages;
          ok = mbar_wait_relaxed(&sm.empty[st], ((g / kStages) & 1) ^ 1, abort_flag);
          if (!ok) break;
          mbar_arrive_expect_tx(&sm.full[st], Smem::kBytesA + Smem::kBytesB);
          // a box holds 128 rows: one per 128 rows of either operand
#pragma unroll
          for (int h = 0; h < BM / 128; ++h)
            tma_load_2d(sm.a[st] + h * 128 * kGemmBK * 2, &tm_x, &sm.full[st], kb * kGemmBK, tm * BM + h * 128);
#pragma unroll
          for (int h = 0; h < BN / 128; ++h)
            tma_load_2d(sm.b[st] + h * 128 * kGemmBK * 2, &tm_w, &sm.full[st], kb * kGemmBK, tn * BN + h * 128);
        }
      }
      if (!ok && atomicExch(const_cast<uint32_t*>(abort_flag), 1u) == 0) atomicOr(p.status, kStatusGemmLoader);
      if (*abort_flag != 0) {  // let every copy that was issued land before the CTA goes
        uint32_t no_abort = 0;
        for (int j = (g > kStages ? g - kStages : 0); j < g; ++j) mbar_wait_relaxed(&sm.full[j % kStages], (j / kStages) & 1, &no_abort);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ======================= MMA issuer ==============================================================
    if (lane == 0) {
      constexpr uint32_t fmt = std::is_same<T, __half>::value ? UMMA_F16 : UMMA_BF16;
      constexpr uint32_t idesc = umma_idesc_f16(fmt, 128, BN, 0, 0);
      const uint64_t a_desc0 = umma_smem_desc_sw128(smem_u32(sm.a[0]), 1024, 16);
      const uint64_t b_desc0 = umma_smem_desc_sw128(smem_u32(sm.b[0]), 1024, 16);
      bool ok = true;
      int g = 0, it = 0;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++it) {
        // The epilogue must have read the accumulator(s) this tile writes: for 128-row tiles the one used two tiles
        // ago, for 256-row tiles both halves of the tile before.
        if constexpr (kTall) {
          if (it >= 1) ok = mbar_wait(&sm.acc_empty[0], (it - 1) & 1, abort_flag) && mbar_wait(&sm.acc_empty[1], (it - 1) & 1, abort_flag);
        } else {
          if (it >= 2) ok = mbar_wait(&sm.acc_empty[it & 1], ((it >> 1) - 1) & 1, abort_flag);
        }
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t acc = tmem + (kTall ? 0 : (it & 1) * 256);
        for (int kb = 0; kb < k_blocks; ++kb, ++g) {
          const int st = g % kStages;
          ok = mbar_wait(&sm.full[st], (g / kStages) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
          const uint64_t a = a_desc0 + static_cast<uint64_t>(st) * (Smem::kBytesA >> 4);
          const uint64_t b = b_desc0 + static_cast<uint64_t>(st) * (Smem::kBytesB >> 4);
#pragma unroll
          for (int h = 0; h < BM / 128; ++h)
#pragma unroll
            for (int kk = 0; kk < kGemmBK / 16; ++kk)
              umma_ss(acc + h * 256, a + h * ((128 * kGemmBK * 2) >> 4) + 2 * kk, b + 2 * kk, idesc, (kb | kk) != 0 ? 1u : 0u);
          umma_commit(&sm.empty[st]);
        }
        if (ok) {
          if constexpr (kTall) {
            umma_commit(&sm.acc_full[0]);
            umma_commit(&sm.acc_full[1]);
          } else {
            umma_commit(&sm.acc_full[it & 1]);
          }
        }
      }
      if (!ok && atomicExch(const_cast<uint32_t*>(abort_flag), 1u) == 0) atomicOr(p.status, kStatusGemmMma);
    }
    __syncwarp();
  } else {
    // ======================= epilogue warps ==========================================================
    const int e = warp - kGemmEpiWarp0;          // 0..7
    const int quarter = warp & 3;                // the tensor-memory lanes this warp may read: 32 * (warp % 4) ..
    const int part = e >> 2;                     // 128-row tiles: which half of the columns; 256-row tiles: which half of the rows
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    constexpr int kCols = kTall ? BN : BN / 2;   // columns per warp
    float(*turn)[32] = sm.turn[e];
    bool ok = true;
    int it = 0;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++it) {
      const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
      const int buf = kTall ? part : (it & 1);
      const uint32_t parity = kTall ? (it & 1) : ((it >> 1) & 1);
      if (!__all_sync(0xffffffffu, mbar_wait(&sm.acc_full[buf], parity, abort_flag))) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int row0 = tm * BM + (kTall ? part * 128 : 0) + quarter * 32;  // first of this warp's 32 rows
      const int col0 = tn * BN + (kTall ? 0 : part * kCols);
      const uint32_t acc = tmem + lane_addr + buf * 256 + (kTall ? 0 : part * kCols);
#pragma unroll 1
      for (int c = 0; c < kCols; c += 32) {
        if (col0 + c >= p.n) break;  // warp-uniform: the whole chunk lies past the last column
        // The residual of the eight columns this lane will write, asked for before anything else of the chunk:
        // the loads fly while the accumulator is read and turned.
        const int cg = lane & 3;                  // which eight columns of the chunk
        const int col = col0 + c + cg * 8;
        uint4 rv[4];
        if (p.res != nullptr && col < p.n) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int row = row0 + (lane >> 2) + 8 * i;
            rv[i] = row < p.m ? *reinterpret_cast<const uint4*>(static_cast<const T*>(p.res) + static_cast<int64_t>(row) * p.lres + col)
                              : make_uint4(0, 0, 0, 0);
          }
        }
        float v[32];
        tmem_ld_x32(acc + c, reinterpret_cast<uint32_t*>(v));
        // Row owner -> row writer: thread `lane` holds row `lane`; afterwards lane l holds, for i = 0..3, the eight
        // columns (l % 4) * 8.. of row l / 4 + 8 i, so that a store instruction of the warp writes eight rows of
        // 64 contiguous bytes. 16-byte chunks are placed at chunk ^ (row % 8): conflict-free both ways.
#pragma unroll
        for (int q = 0; q < 8; ++q)
          *reinterpret_cast<float4*>(&turn[lane][((q ^ (lane & 7)) << 2)]) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        __syncwarp();
        if (col < p.n) {                          // n is a multiple of 8: eight columns are inside or outside together
          float bias8[8], scale8[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            bias8[q] = 0.f;
            scale8[q] = 1.f;
          }
          if (p.bias != nullptr) {
            const uint4 bv = __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(p.bias) + col));
            const uint32_t w4[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 f = gemm_unpack2<T>(w4[q]);
              bias8[2 * q] = f.x;
              bias8[2 * q + 1] = f.y;
            }
          }
          if (p.scale != nullptr) {
            const float4 s0 = __ldg(reinterpret_cast<const float4*>(p.scale + col));
            const float4 s1 = __ldg(reinterpret_cast<const float4*>(p.scale + col + 4));
            scale8[0] = s0.x; scale8[1] = s0.y; scale8[2] = s0.z; scale8[3] = s0.w;
            scale8[4] = s1.x; scale8[5] = s1.y; scale8[6] = s1.z; scale8[7] = s1.w;
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int r = (lane >> 2) + 8 * i;
            const int row = row0 + r;
            if (row >= p.m) break;
            const float4 lo = *reinterpret_cast<const float4*>(&turn[r][(((2 * cg) ^ (r & 7)) << 2)]);
            const float4 hi = *reinterpret_cast<const float4*>(&turn[r][(((2 * cg + 1) ^ (r & 7)) << 2)]);
            float x[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
            for (int q = 0; q < 8; ++q) x[q] = (x[q] + bias8[q]) * scale8[q];
            if (p.res != nullptr) {
              const uint32_t w4[4] = {rv[i].x, rv[i].y, rv[i].z, rv[i].w};
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float2 f = gemm_unpack2<T>(w4[q]);
                x[2 * q] += f.x;
                x[2 * q + 1] += f.y;
              }
            }
            if (p.act != kActNone) {
#pragma unroll
              for (int q = 0; q < 8; ++q) x[q] = gemm_act(x[q], p.act);
            }
            uint4 out;
            out.x = gemm_pack2<T>(x[0], x[1]);
            out.y = gemm_pack2<T>(x[2], x[3]);
            out.z = gemm_pack2<T>(x[4], x[5]);
            out.w = gemm_pack2<T>(x[6], x[7]);
            *reinterpret_cast<uint4*>(static_cast<T*>(p.y) + static_cast<int64_t>(row) * p.ldy + col) = out;
          }
        }
        __syncwarp();  // the chunk has been read back before the next one overwrites it
      }
      // every column of this warp is in registers or written: the accumulator may be overwritten
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.acc_empty[buf]);
    }
    if (!ok && lane == 0) {
      if (atomicExch(const_cast<uint32_t*>(abort_flag), 1u) == 0) atomicOr(p.status, kStatusGemmEpilogue);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace b200
