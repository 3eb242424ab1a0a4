// Non-causal multi-head attention forward for head dim 64 on sm_100a:
//   O = softmax(scale * Q K^T + bias) V,   fp16 / bf16 operands, fp32 accumulation.
//
// One CTA owns one or two 128-row query tiles of one (batch, head) and walks the keys in tiles of 128:
//   * a loader warp stages Q once and K / V tiles through a ring of shared-memory stages with TMA
//     (128-byte swizzle, rows past the end of the sequence read as zero);
//   * an MMA warp issues S = Q K^T (tcgen05.mma, M=128 N=128 K=64) into tensor memory and
//     O += P V (M=128 N=64 K=128) with P read straight from tensor memory, where it overlays S;
//   * two softmax warpgroups, one per query tile, own one row of S per thread: they read the row
//     from tensor memory, keep the running maximum and sum, and write P back as 16-bit values.
//     While one warpgroup runs its exponentials the tensor pipe works for the other tile.
// The running maximum is only raised when it grows by more than 2^8, so rescaling O (a tensor-memory
// round trip) is rare; the final division by the row sum happens once in the epilogue.
//
// Every barrier wait is bounded (see sm100_ptx.cuh). A wait that runs out raises the CTA's abort
// flag, records the role in the global status word, and all warps fall through to the common exit,
// which waits for TMA copies still in flight and frees tensor memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "sm100_ptx.cuh"

namespace b200 {

constexpr int kTileRows = 128;                       // query rows per tile == keys per tile
constexpr int kHeadDim = 64;                         // the only head dim of this path
constexpr int kTileBytes = kTileRows * kHeadDim * 2; // one Q / K / V tile in shared memory
constexpr int kSoftmaxThreads = 256;                 // two warpgroups
constexpr int kLoaderWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kThreads = 384;                        // 2 softmax warpgroups + 1 warpgroup of helpers (2 idle warps)
constexpr int kSoftmaxRegs = 224, kHelperRegs = 48;   // per-thread register budgets after the hand-over
constexpr int kLaunchRegs = 168;                      // what a 384-thread CTA gets per thread at launch
// setmaxnreg.inc blocks until the CTA's pool holds the registers: the budgets must fit what the launch allocated,
// or the second warpgroup waits for ever.
static_assert(2 * 128 * kSoftmaxRegs + 128 * kHelperRegs <= kLaunchRegs * kThreads, "register hand-over does not balance");
constexpr uint32_t kTmemCols = 512;                  // S0 S1 (128 each) + O0 O1 (64 each) = 384 -> next power of two
constexpr uint32_t kTmemS = 0, kTmemO = 256;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;            // log2 units: P stays below 2^8 between rescales

enum : uint32_t { kStatusLoader = 1, kStatusMma = 2, kStatusSoftmax = 4 };
enum : int { kBiasNone = 0, kBiasDense = 1, kBiasDecomposed = 2 };

struct BiasView {
  const void* ptr;
  int64_t sb, sh, sn;  // element strides: batch, head, query row
  int dtype;           // 0 fp16, 1 bf16, 2 fp32
};

struct AttnParams {
  int batch, heads, q_tokens, kv_tokens;
  int items_per_head;  // CTAs per (batch, head): ceil(q_tiles / 2)
  int kv_tiles;
  float scale_log2;    // scale * log2(e)
  void* o;
  int64_t o_sb, o_sn, o_sh;
  BiasView bias;       // dense bias, or rel_h of the decomposed form
  BiasView bias2;      // rel_w of the decomposed form
  int rel_kw;
  uint32_t* status;    // device word that collects role bits of expired waits
};

template <int STAGES, bool P_IN_SMEM>
struct alignas(1024) AttnSmem {
  uint8_t q[2][kTileBytes];
  uint8_t k[STAGES][kTileBytes];
  uint8_t v[STAGES][kTileBytes];
  uint8_t p[P_IN_SMEM ? 2 : 1][P_IN_SMEM ? 2 * kTileBytes : 1024];  // P as two 64-key column blocks
  uint64_t q_full[2];
  uint64_t k_full[STAGES], k_empty[STAGES];
  uint64_t v_full[STAGES], v_empty[STAGES];
  uint64_t s_full[2], p_full[2], o_full[2];
  uint32_t tmem_base;
  uint32_t abort;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float load_bias_elem(const void* base, int dtype, int64_t idx) {
  if (dtype == 2) return __ldg(reinterpret_cast<const float*>(base) + idx);
  if (dtype == 0) return __half2float(__ldg(reinterpret_cast<const __half*>(base) + idx));
  return __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16*>(base) + idx));
}

template <typename T, int BIAS, int STAGES, bool P_IN_SMEM>
__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  using Smem = AttnSmem<STAGES, P_IN_SMEM>;
  extern __shared__ uint8_t smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int item = blockIdx.x % p.items_per_head;
  const int bh = blockIdx.x / p.items_per_head;
  const int b = bh / p.heads;
  const int h = bh % p.heads;
  const int q_row0 = item * 2 * kTileRows;
  const int n_tiles = (p.q_tokens - q_row0 > kTileRows) ? 2 : 1;  // query tiles of this CTA
  const int kv_tiles = p.kv_tiles;

  // ---- set-up: barriers, tensor memory -------------------------------------------------------
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.q_full[i], 1);
      mbar_init(&sm.s_full[i], 1);
      mbar_init(&sm.p_full[i], kTileRows);
      mbar_init(&sm.o_full[i], 1);
    }
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&sm.k_full[i], 1);
      mbar_init(&sm.k_empty[i], 1);
      mbar_init(&sm.v_full[i], 1);
      mbar_init(&sm.v_empty[i], 1);
    }
    sm.abort = 0;
    mbar_init_fence();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(&sm.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  if (warp == kLoaderWarp && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm.tmem_base;
  volatile uint32_t* abort_flag = &sm.abort;

  if (warp >= kLoaderWarp) {
    reg_dealloc<kHelperRegs>();
  if (warp == kLoaderWarp) {
    // ======================= loader =========================================================
    if (lane == 0) {
      bool ok = true;
      for (int t = 0; t < n_tiles; ++t) {
        mbar_arrive_expect_tx(&sm.q_full[t], kTileBytes);
        tma_load_4d(sm.q[t], &tm_q, &sm.q_full[t], 0, q_row0 + t * kTileRows, h, b);
      }
      int issued_k = 0, issued_v = 0;
      for (int j = 0; j < kv_tiles && ok; ++j) {
        const int st = j % STAGES;
        const uint32_t ph = (j / STAGES) & 1;
        ok = mbar_wait(&sm.k_empty[st], ph ^ 1, abort_flag);
        if (!ok) break;
        mbar_arrive_expect_tx(&sm.k_full[st], kTileBytes);
        tma_load_4d(sm.k[st], &tm_k, &sm.k_full[st], 0, j * kTileRows, h, b);
        issued_k = j + 1;
        ok = mbar_wait(&sm.v_empty[st], ph ^ 1, abort_flag);
        if (!ok) break;
        mbar_arrive_expect_tx(&sm.v_full[st], kTileBytes);
        tma_load_4d(sm.v[st], &tm_v, &sm.v_full[st], 0, j * kTileRows, h, b);
        issued_v = j + 1;
      }
      if (!ok) {
        if (atomicExch(const_cast<uint32_t*>(abort_flag), 1u) == 0) atomicOr(p.status, kStatusLoader);
      }
      if (*abort_flag != 0) {
        // Nobody may be consuming any more: wait (bounded, ignoring the abort flag) for every copy
        // that was issued, so that none writes into shared memory after the CTA has gone.
        uint32_t no_abort = 0;
        for (int t = 0; t < n_tiles; ++t) mbar_wait(&sm.q_full[t], 0, &no_abort);
        for (int j = (issued_k > STAGES ? issued_k - STAGES : 0); j < issued_k; ++j)
          mbar_wait(&sm.k_full[j % STAGES], (j / STAGES) & 1, &no_abort);
        for (int j = (issued_v > STAGES ? issued_v - STAGES : 0); j < issued_v; ++j)
          mbar_wait(&sm.v_full[j % STAGES], (j / STAGES) & 1, &no_abort);
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // ======================= MMA issuer ======================================================
    if (lane == 0) {
      constexpr uint32_t fmt = std::is_same<T, __half>::value ? UMMA_F16 : UMMA_BF16;
      constexpr uint32_t idesc_qk = umma_idesc_f16(fmt, kTileRows, kTileRows, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_f16(fmt, kTileRows, kHeadDim, 0, 1);
      bool ok = true;

      auto issue_qk = [&](int t, int st) {
        const uint64_t a = umma_smem_desc_sw128(smem_u32(sm.q[t]), 1024, 16);
        const uint64_t bd = umma_smem_desc_sw128(smem_u32(sm.k[st]), 1024, 16);
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk)  // 32 bytes of K per step inside the swizzle atom
          umma_ss(tmem + kTmemS + t * kTileRows, a + 2 * kk, bd + 2 * kk, idesc_qk, kk > 0);
      };
      auto issue_pv = [&](int t, int st, bool first) {
        const uint64_t bd = umma_smem_desc_sw128(smem_u32(sm.v[st]), 1024, 0);
#pragma unroll
        for (int kk = 0; kk < kTileRows / 16; ++kk) {  // 16 keys = two 8-row groups of V per step
          const uint32_t acc = (!first || kk > 0) ? 1u : 0u;
          if constexpr (P_IN_SMEM) {
            const uint64_t a =
                umma_smem_desc_sw128(smem_u32(sm.p[t]) + (kk / 4) * kTileBytes, 1024, 16) + 2 * (kk % 4);
            umma_ss(tmem + kTmemO + t * kHeadDim, a, bd + kk * (2048 >> 4), idesc_pv, acc);
          } else {
            umma_ts(tmem + kTmemO + t * kHeadDim, tmem + kTmemS + t * kTileRows + kk * 8, bd + kk * (2048 >> 4),
                    idesc_pv, acc);
          }
        }
      };

      // S_t(0) for both tiles
      ok = mbar_wait(&sm.k_full[0], 0, abort_flag);
      for (int t = 0; t < n_tiles && ok; ++t) {
        ok = mbar_wait(&sm.q_full[t], 0, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        issue_qk(t, 0);
        umma_commit(&sm.s_full[t]);
      }
      if (ok) umma_commit(&sm.k_empty[0]);

      for (int j = 0; j < kv_tiles && ok; ++j) {
        const int st = j % STAGES;
        const uint32_t ph = (j / STAGES) & 1;
        const bool more = j + 1 < kv_tiles;
        const int st1 = (j + 1) % STAGES;
        const uint32_t ph1 = ((j + 1) / STAGES) & 1;
        if (more) {
          ok = mbar_wait(&sm.k_full[st1], ph1, abort_flag);
          if (!ok) break;
        }
        ok = mbar_wait(&sm.v_full[st], ph, abort_flag);
        if (!ok) break;
        for (int t = 0; t < n_tiles; ++t) {
          ok = mbar_wait(&sm.p_full[t], j & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
          issue_pv(t, st, j == 0);
          if (more) {
            issue_qk(t, st1);
            umma_commit(&sm.s_full[t]);
          } else {
            umma_commit(&sm.o_full[t]);
          }
        }
        if (!ok) break;
        umma_commit(&sm.v_empty[st]);
        if (more) umma_commit(&sm.k_empty[st1]);
      }
      if (!ok) {
        if (atomicExch(const_cast<uint32_t*>(abort_flag), 1u) == 0) atomicOr(p.status, kStatusMma);
      }
    }
    __syncwarp();
  }
  } else {
    // ======================= softmax warpgroups ==============================================
    reg_alloc<kSoftmaxRegs>();
    const int t = warp >> 2;                     // query tile of this warpgroup
    const int row_in_tile = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    if (t < n_tiles) {
      const int q_row = q_row0 + t * kTileRows + row_in_tile;
      const bool row_valid = q_row < p.q_tokens;
      const uint32_t s_addr = tmem + lane_addr + kTmemS + t * kTileRows;
      const uint32_t o_addr = tmem + lane_addr + kTmemO + t * kHeadDim;
      const float c = p.scale_log2;
      float m_ref = -INFINITY;
      float l_sum = 0.f;
      bool ok = true;

      int64_t bias_row = 0, bias2_row = 0;
      if constexpr (BIAS != kBiasNone) {
        const int qr = row_valid ? q_row : 0;
        bias_row = b * p.bias.sb + h * p.bias.sh + qr * p.bias.sn;
        if constexpr (BIAS == kBiasDecomposed) bias2_row = b * p.bias2.sb + h * p.bias2.sh + qr * p.bias2.sn;
      }

      for (int j = 0; j < kv_tiles; ++j) {
        ok = __all_sync(0xffffffffu, mbar_wait(&sm.s_full[t], j & 1, abort_flag));
        if (!ok) break;
        tc_fence_after_sync();

        float s[kTileRows];
        {
          uint32_t* su = reinterpret_cast<uint32_t*>(s);
          tmem_ld_x64(s_addr, su);
          tmem_ld_x64(s_addr + 64, su + 64);
        }
        const int kv0 = j * kTileRows;
        const int kv_valid = min(kTileRows, p.kv_tokens - kv0);

        if constexpr (BIAS == kBiasDense) {
#pragma unroll
          for (int i = 0; i < kTileRows; ++i) {
            const float bv = (i < kv_valid) ? load_bias_elem(p.bias.ptr, p.bias.dtype, bias_row + kv0 + i) : 0.f;
            s[i] = fmaf(s[i], c, bv * kLog2e);
          }
        } else if constexpr (BIAS == kBiasDecomposed) {
          int ih = kv0 / p.rel_kw;
          int iw = kv0 - ih * p.rel_kw;
          float bh_val = (kv0 < p.kv_tokens) ? load_bias_elem(p.bias.ptr, p.bias.dtype, bias_row + ih) : 0.f;
#pragma unroll
          for (int i = 0; i < kTileRows; ++i) {
            float bv = 0.f;
            if (i < kv_valid) bv = bh_val + load_bias_elem(p.bias2.ptr, p.bias2.dtype, bias2_row + iw);
            s[i] = fmaf(s[i], c, bv * kLog2e);
            if (++iw == p.rel_kw) {
              iw = 0;
              ++ih;
              if (i + 1 < kv_valid) bh_val = load_bias_elem(p.bias.ptr, p.bias.dtype, bias_row + ih);
            }
          }
        }
        if (kv_valid < kTileRows) {
#pragma unroll
          for (int i = 0; i < kTileRows; ++i)
            if (i >= kv_valid) s[i] = -INFINITY;
        }

        float mx0 = s[0], mx1 = s[1], mx2 = s[2], mx3 = s[3];
#pragma unroll
        for (int i = 4; i < kTileRows; i += 4) {
          mx0 = fmaxf(mx0, s[i]);
          mx1 = fmaxf(mx1, s[i + 1]);
          mx2 = fmaxf(mx2, s[i + 2]);
          mx3 = fmaxf(mx3, s[i + 3]);
        }
        float m_tile = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        if constexpr (BIAS == kBiasNone) m_tile *= c;

        // Raise the reference maximum only when it pays (or on the first tile).
        const bool raise = m_tile > m_ref + kRescaleThreshold;  // -inf + 8 = -inf: true for any finite first tile
        float alpha = 1.f;
        if (raise) {
          alpha = fast_exp2(m_ref - m_tile);  // m_ref = -inf -> 0
          m_ref = m_tile;
        }
        if (j > 0 && __any_sync(0xffffffffu, raise)) {
          float o[kHeadDim];
          uint32_t* ou = reinterpret_cast<uint32_t*>(o);
          tmem_ld_x64(o_addr, ou);
#pragma unroll
          for (int i = 0; i < kHeadDim; ++i) o[i] *= alpha;
          tmem_st_x32(o_addr, ou);
          tmem_st_x32(o_addr + 32, ou + 32);
        }
        l_sum *= alpha;
        const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;

        float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
        uint32_t pk[kTileRows / 2];
#pragma unroll
        for (int i = 0; i < kTileRows; i += 4) {
          float p0, p1, p2, p3;
          if constexpr (BIAS == kBiasNone) {
            p0 = fast_exp2(fmaf(s[i], c, -m_use));
            p1 = fast_exp2(fmaf(s[i + 1], c, -m_use));
            p2 = fast_exp2(fmaf(s[i + 2], c, -m_use));
            p3 = fast_exp2(fmaf(s[i + 3], c, -m_use));
          } else {
            p0 = fast_exp2(s[i] - m_use);
            p1 = fast_exp2(s[i + 1] - m_use);
            p2 = fast_exp2(s[i + 2] - m_use);
            p3 = fast_exp2(s[i + 3] - m_use);
          }
          l0 += p0;
          l1 += p1;
          l2 += p2;
          l3 += p3;
          pk[i / 2] = pack2<T>(p0, p1);
          pk[i / 2 + 1] = pack2<T>(p2, p3);
        }
        l_sum += (l0 + l1) + (l2 + l3);

        if constexpr (P_IN_SMEM) {
          // Row r of the K-major, 128-byte-swizzled P tile: 16-byte chunk c of a 64-key block sits at
          // r * 128 + ((c ^ (r & 7)) * 16).
          uint8_t* prow = sm.p[t] + row_in_tile * 128;
#pragma unroll
          for (int ch = 0; ch < 16; ++ch) {
            uint4 val = make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
            uint8_t* dst = prow + (ch / 8) * kTileBytes + (((ch & 7) ^ (row_in_tile & 7)) << 4);
            *reinterpret_cast<uint4*>(dst) = val;
          }
          fence_proxy_async_smem();
        } else {
          tmem_st_x32(s_addr, pk);
          tmem_st_x32(s_addr + 32, pk + 32);
        }
        tmem_st_wait();
        tc_fence_before_sync();
        mbar_arrive(&sm.p_full[t]);
      }

      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&sm.o_full[t], 0, abort_flag));
      if (ok) {
        tc_fence_after_sync();
        float o[kHeadDim];
        tmem_ld_x64(o_addr, reinterpret_cast<uint32_t*>(o));
        if (row_valid) {
          const float inv = 1.f / l_sum;
          T* dst = reinterpret_cast<T*>(p.o) + b * p.o_sb + static_cast<int64_t>(q_row) * p.o_sn + h * p.o_sh;
#pragma unroll
          for (int ch = 0; ch < kHeadDim / 8; ++ch) {
            uint4 val;
            val.x = pack2<T>(o[ch * 8 + 0] * inv, o[ch * 8 + 1] * inv);
            val.y = pack2<T>(o[ch * 8 + 2] * inv, o[ch * 8 + 3] * inv);
            val.z = pack2<T>(o[ch * 8 + 4] * inv, o[ch * 8 + 5] * inv);
            val.w = pack2<T>(o[ch * 8 + 6] * inv, o[ch * 8 + 7] * inv);
            *reinterpret_cast<uint4*>(dst + ch * 8) = val;
          }
        }
      } else if (lane == 0) {
        if (atomicExch(const_cast<uint32_t*>(abort_flag), 1u) == 0) atomicOr(p.status, kStatusSoftmax);
      }
    }
  }

  // ---- common exit ----------------------------------------------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace b200
