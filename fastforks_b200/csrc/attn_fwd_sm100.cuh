// Non-causal multi-head attention forward for head dim 64 on sm_100a:
//   O = softmax(scale * Q K^T + bias) V,   fp16 / bf16 operands, fp32 accumulation.
//
// Persistent CTAs (one per SM) take work items - one or two 128-row query tiles of one (batch, head) - and walk
// the keys of each in tiles of 128:
//   * a loader warp stages Q once and K / V tiles through rings of shared-memory stages with TMA
//     (128-byte swizzle, rows past the end of the sequence read as zero); K runs two tiles ahead of V;
//   * one thread per query tile issues S = Q K^T (tcgen05.mma, M=128 N=128 K=64) into tensor memory and
//     O += P V (M=128 N=64 K=128) with P read straight from tensor memory. S_t(j+1) is issued as soon
//     as the softmax threads have pulled S_t(j) into registers, so the tensor pipe never sits on the
//     softmax critical path;
//   * two softmax warpgroups, one per query tile, own one row of S per thread: they read the row
//     from tensor memory, keep the running maximum and sum, and write P back as 16-bit values.
//     The exponential section is passed between the two warpgroups like a token ("ping-pong"), so
//     one warpgroup saturates the MUFU unit while the other loads, reduces and stores.
// The running maximum is only raised when it grows by more than 2^8, so rescaling O (a tensor-memory
// round trip) is rare; the final division by the row sum happens once in the epilogue.
//
// Every barrier wait is bounded (see sm100_ptx.cuh). A wait that runs out raises the CTA's abort
// flag, records the role in the global status word, and all warps fall through to the common exit,
// which waits for TMA copies still in flight and frees tensor memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstddef>
#include <type_traits>

#include "sm100_ptx.cuh"

namespace b200 {

constexpr int kTileRows = 128;                        // query rows per tile == keys per tile
constexpr int kHeadDim = 64;                          // the only head dim of this path
constexpr int kTileBytes = kTileRows * kHeadDim * 2;  // one Q / K / V tile in shared memory
constexpr int kLoaderWarp = 8;
constexpr int kMmaWarp = 9;                           // warps 9 and 10 issue the MMAs of query tile 0 and 1
constexpr int kStoreWarp = 11;                        // issues the TMA stores of the output tiles
constexpr int kThreads = 384;                         // 2 softmax warpgroups + 1 warpgroup of helpers
constexpr int kSoftmaxRegs = 224, kHelperRegs = 56;   // per-thread register budgets after the hand-over
constexpr int kLaunchRegs = 168;                      // what a 384-thread CTA gets per thread at launch
// setmaxnreg.inc blocks until the CTA's pool holds the registers: the budgets must fit what the launch
// allocated, or the second warpgroup waits for ever.
static_assert(2 * 128 * kSoftmaxRegs + 128 * kHelperRegs <= kLaunchRegs * kThreads,
              "register hand-over does not balance");
constexpr int kStages = 3;       // K / V ring stages (the dense-tile bias form gives one of each to its bias tiles)
constexpr int kStagesDense = 2;
constexpr int kKLead = 2;                             // K tiles are consumed two iterations ahead of V tiles
constexpr uint32_t kTmemCols = 512;                   // S0 S1 (128 each), O0 O1 (64 each), P0 P1 (64 each)
constexpr uint32_t kTmemS = 0, kTmemO = 256, kTmemP = 384;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;             // log2 units: P stays below 2^8 between rescales

enum : uint32_t { kStatusLoader = 1, kStatusMma = 2, kStatusSoftmax = 4, kStatusStore = 16 };  // 8: the wait self-test

// Key-split mode: the key-tile steps of all items form one line (two-tile items first, head by head, then the
// one-tile items) and every CTA takes one contiguous run of it, cut so that the runs cost the same. A step of a
// two-tile item costs kPairCost units, a step of a one-tile item kSingleCost (a lone softmax warpgroup takes 0.78 of
// the time two interleaved ones take for both tiles).
constexpr int kPairCost = 64, kSingleCost = 50;
// An item that is cut has one part per CTA of a run of consecutive CTAs. A part's result is, per query tile, its
// unnormalised output as [16 column groups][128 rows] of float4 (consecutive threads, consecutive addresses), the
// rows' reference maxima and their row sums. How the parts meet:
//   * the part with the item's first keys ("owner") is its CTA's LAST item, every later part its CTA's FIRST item,
//     so as a rule the later parts are complete long before the owner is;
//   * a later part writes its result to the workspace (plain stores by the softmax threads, who go on at once) and
//     the CTA's store warp, once they are all written, fences and counts the part on the item's counter;
//   * the owner first looks at the counter: when every later part is counted, it folds them into the result it
//     still holds in registers and writes the output (the usual case: one look, no store). Otherwise it leaves its
//     result like the others and is counted like them;
//   * whoever counts last while parts are in the workspace - a store warp - folds them all and writes the output
//     rows itself (slow, rare, and the only route when the test flag takes the owner's short cut away).
// Nobody ever waits for another CTA, so no two CTAs need to be resident together (grids of several streams may
// share the GPU in any way) and no wait can run out.
constexpr int kPartialFloats = kTileRows * kHeadDim + 2 * kTileRows;
// How long an owner keeps looking at its item's counter before it gives its result to the workspace like a later
// part. A later part is its CTA's first item, so it is counted early in that CTA's life: the look only ever takes
// time when all CTAs have very short runs, or when the later part's CTA has not been scheduled yet.
constexpr uint64_t kOwnerPatienceNs = 30000;
// kItemPartial: a later part, always its CTA's first item. kItemOwner: the part with the item's first keys, always
// its CTA's last item; the item's counter is the one of this CTA.
enum : int { kItemWhole = 0, kItemPartial = 1, kItemOwner = 2 };

// Bias forms. kBiasDecomposed14 is the decomposed form specialised for a 14 x 14 key grid (SAM's windows): both
// tables of a row sit in registers and every column's pair of indices is a compile-time constant.
// kBiasDecomposed64 is the decomposed form specialised for rel_kw == 64, rel_kh a multiple of 8, with 16-bit, 16-byte aligned
// rel_w rows (SAM's global layers): a key tile then spans exactly two rel_h entries and the whole rel_w row twice.
// kBiasDenseTiles is the dense form for 16-bit biases whose rows are 16-byte aligned: the loader warp brings the
// 128 x 128 bias tile of every (query tile, key tile) into shared memory with TMA, like K and V, instead of every
// softmax thread walking its own row in global memory.
enum : int { kBiasNone = 0, kBiasDense = 1, kBiasDecomposed = 2, kBiasDecomposed64 = 3, kBiasDecomposed14 = 4, kBiasDenseTiles = 5 };
constexpr int kRelStageWords = 33;  // per-row staging of rel_h | rel_w in shared memory: up to 32 values, odd stride

struct BiasView {
  const void* ptr;
  int64_t sb, sh, sn;  // element strides: batch, head, query row
  int dtype;           // 0 fp16, 1 bf16, 2 fp32
};

struct AttnParams {
  int batch, heads, q_tokens, kv_tokens;
  int q_tiles;         // 128-row query tiles per (batch, head)
  // How the host split the work (plan_split in b200_attn.cu): every head has `pairs_per_head` two-tile items, which
  // cover its first 2 * pairs_per_head tiles, and `singles_per_head` one-tile items for the rest. The first
  // `split_na` CTAs of the grid take `split_ka` two-tile items each and the others `split_kb`; the first `split_na`
  // CTAs take `split_a` one-tile items each (one more for the first `split_ea` of them), the others `split_b`
  // (one more for the first `split_eb`).
  int pairs_per_head, singles_per_head;
  int split_na, split_ka, split_kb, split_a, split_ea, split_b, split_eb;
  // Dealt mode: the last `conv_pairs` two-tile items (those a last, partial round of the grid would hold) are worked on
  // as 2 * conv_pairs one-tile items instead, numbered in front of the other one-tile items; `kept_pairs` stay whole.
  int conv_pairs, kept_pairs;
  int kv_tiles;
  float scale_log2;    // scale * log2(e)
  void* o;
  int64_t o_sb, o_sn, o_sh;
  BiasView bias;       // dense bias, or rel_h of the decomposed form
  BiasView bias2;      // rel_w of the decomposed form
  int rel_kh, rel_kw;
  uint64_t magic_pairs, magic_singles, magic_heads, magic_rel_kw;  // fast_div constants of pairs_per_head, singles_per_head, heads (the batch size if batch_fastest), rel_kw
  int batch_fastest;   // items are numbered with the batch index running fastest (else the head index): see decode_item
  int rel_staged;      // decomposed form: rel_kh + rel_kw <= 32, rows are staged in shared memory per item
  int bias_vec;        // dense form: rows are 16-byte aligned, full tiles are read with vector loads
  uint32_t* status;    // device word that collects role bits of expired waits
  // Key-split mode (chunked != 0; see kPairCost). pairs_per_head = q_tiles / 2 and singles_per_head = q_tiles % 2 then.
  int chunked;
  int pair_items, single_items;  // two-tile and one-tile items of the whole problem
  long long cost_total;          // kv_tiles * (pair_items * kPairCost + single_items * kSingleCost)
  float* ws_partial;             // [grid][first item / last item][query tile][kPartialFloats]
  uint32_t* ws_counts;           // [grid][query tile]: counted parts of the item that CTA owns; 0 between launches
  long long cost_base;           // cost_total / grid and cost_total % grid: CTA c begins at cost
  int cost_rem;                  //   c * cost_base + min(c, cost_rem)
  uint64_t magic_kv_tiles;       // fast_div constant of kv_tiles
  int test_flags;                // 1: the owner never takes its short cut (every merge runs in a store warp)
};

// One CTA's share of the work (see cta_work).
struct CtaWork {
  int pairs, singles, pair_start, pair_stride, single_start, single_stride;
  // Key ranges. Every item runs over all kv_tiles key tiles, except, in key-split mode, the first item of a CTA
  // (it may begin at key tile ja0: its earlier keys belong to the CTA before) and the last one (it may end at
  // jb_last: the rest belongs to the next `last_parts` CTAs, whose partial results this CTA merges into its own).
  int first_item, ja0, jb_last, last_parts;
  int first_back, first_fwd;  // CTAs before / after this one that hold other parts of its first item (ja0 > 0)
  int steps_all, steps_pairs;  // key-tile steps of all items and of the two-tile items
};

template <int STAGES, bool BIAS_TILES>
struct alignas(1024) AttnSmemT {
  static constexpr int kRing = STAGES;
  uint8_t q[2][2][kTileBytes];  // [query-tile slot][item parity]: the next item's Q is loaded while this one computes
  uint8_t k[STAGES][kTileBytes];
  uint8_t v[STAGES][kTileBytes];
  uint8_t o_stage[2][kTileBytes];  // an item's output tile per query-tile slot, in the TMA tile layout (128-byte swizzle)
  uint64_t q_full[2][2];   // Q_t of an item has landed                      (TMA)
  uint64_t q_empty[2][2];  // that item's last Q_t K^T has finished          (MMA commit)
  uint64_t k_full[STAGES], k_empty[STAGES];
  uint64_t v_full[STAGES], v_empty[STAGES];
  uint64_t bias_full[2];   // dense-tile bias form: the bias tile of query tile t's current step has landed (TMA)
  uint64_t bias_free[2];   // ... and has been read by the softmax warps                                  (4 softmax warps)
  uint64_t s_full[2];   // S_t(j) is in tensor memory                     (MMA commit)
  uint64_t s_free[2];   // S_t(j) has been read into registers             (4 softmax warps)
  uint64_t p_full[2];   // P_t(j) is in tensor memory, O_t rescaled        (4 softmax warps)
  uint64_t pv_done[2];  // O_t += P_t(j) V(j) has finished                 (MMA commit)
  uint64_t o_free[2];   // the item's O_t has been read by its epilogue     (4 softmax warps)
  uint64_t turn[2];     // the other warpgroup has released t from inside its exponentials: t may start (4 warps; barrier form of the token)
  uint64_t o_staged[2];      // the item's output tile t is in o_stage[t]           (4 softmax warps)
  uint64_t o_stage_free[2];  // the TMA store of that tile has read o_stage[t]       (store thread)
  uint64_t drain[2];         // abort path only: the MMAs query tile t's thread had in flight have finished (MMA commit)
  uint64_t merge_go[2];      // the owner's first thread has looked at the item's counter and set `merge_ready` (1)
  uint32_t merge_ready[2];   // every later part of the owner's item is counted: the owner folds them in itself
  uint32_t o_store[2][2];    // [t][item parity] what the hand-over o_staged[t] of a cut item means: 1 a staged tile, 2 a part in the workspace
  uint32_t turn_count[2][4];  // flag form of the token: releases so far by warp w of warpgroup t (see kFlagTurn)
  uint32_t tmem_base;
  uint32_t abort;
  CtaWork work;  // written once at set-up; kept here rather than in registers of every role
  // decomposed forms: each softmax thread's own rel_h | rel_w row, times log2(e); dense-tile form: per query tile the
  // two 64-column halves of the current 128 x 128 bias tile (16-bit, 128-byte swizzle)
  // (a TMA destination with the 128-byte swizzle starts on a 1024-byte boundary)
  union alignas(BIAS_TILES ? 1024 : 16) {
    float rel_stage[2][kTileRows][kRelStageWords];
    uint8_t bias_tile[BIAS_TILES ? 2 : 1][2][BIAS_TILES ? kTileBytes : 16];
  };
};
using AttnSmem = AttnSmemT<kStages, false>;
using AttnSmemDense = AttnSmemT<kStagesDense, true>;
// The set-up walks the barriers as one array and picks the arrival count by position.
static_assert(offsetof(AttnSmem, merge_go) + sizeof(uint64_t[2]) == offsetof(AttnSmem, merge_ready) &&
                  offsetof(AttnSmem, o_free) + 2 * sizeof(uint64_t[2]) == offsetof(AttnSmem, o_staged) &&
                  offsetof(AttnSmem, q_full) < offsetof(AttnSmem, merge_go),
              "barrier order in AttnSmemT: q_full ... o_free, turn, o_staged ... merge_go, nothing else in between");
static_assert(offsetof(AttnSmemDense, bias_tile) % 1024 == 0, "bias tiles: 1024-byte aligned for the 128-byte swizzle");

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// (a.x * b.x + c.x, a.y * b.y + c.y) in one instruction of the FMA pipe.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n\t"
      ".reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\t"
      "mov.b64 rb, {%4, %5};\n\t"
      "mov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t"
      "}\n"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}

__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t"
      ".reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\t"
      "mov.b64 rb, {%4, %5};\n\t"
      "add.rn.f32x2 rd, ra, rb;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t"
      "}\n"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}

// One arrival for the whole warp, after all its lanes have reached this point.
__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}

// The same, pinned in the instruction stream: `dep` is routed through the instruction, so every later
// computation that reads `dep` is scheduled after the arrival instead of being hoisted above it.
__device__ __forceinline__ void warp_arrive_pinned(uint64_t* bar, int lane, float& dep) {
  __syncwarp();
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.eq.s32 p, %2, 0;\n\t"
      "@p mbarrier.arrive.shared::cta.b64 _, [%1];\n\t"
      "}\n"
      : "+f"(dep)
      : "r"(smem_u32(bar)), "r"(lane)
      : "memory");
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

// Two packed 16-bit values (fp16 when `is_half`, else bf16) as floats.
__device__ __forceinline__ float2 unpack2(uint32_t v, bool is_half) {
  if (is_half) return __half22float2(*reinterpret_cast<const __half2*>(&v));
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}

__device__ __forceinline__ float load_bias_elem(const void* base, int dtype, int64_t idx) {
  if (dtype == 2) return __ldg(reinterpret_cast<const float*>(base) + idx);
  if (dtype == 0) return __half2float(__ldg(reinterpret_cast<const __half*>(base) + idx));
  return __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16*>(base) + idx));
}

// The same with the table's type known at compile time, and the dispatch that makes it so. A run of loads must sit
// in ONE arm of the type decision: with the decision inside every load (load_bias_elem in a loop) each load sits
// behind its own branches, the compiler does not move the loads across them, and their latencies add up instead of
// overlapping (measured on SAM's 14 x 14 windows: 28 loads per row and item, 7 us per item).
template <int DT>
__device__ __forceinline__ float load_bias_elem_t(const void* base, int64_t idx) {
  if constexpr (DT == 2) return __ldg(reinterpret_cast<const float*>(base) + idx);
  else if constexpr (DT == 0) return __half2float(__ldg(reinterpret_cast<const __half*>(base) + idx));
  else return __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16*>(base) + idx));
}

template <typename F>
__device__ __forceinline__ void for_bias_dtype(int dtype, F&& f) {
  if (dtype == 2) f(std::integral_constant<int, 2>{});
  else if (dtype == 0) f(std::integral_constant<int, 0>{});
  else f(std::integral_constant<int, 1>{});
}

// n / d for the divisors the host knows at launch: magic = ceil(2^64 / d) (0 stands for d == 1), exact for every
// n * d < 2^64. An integer division in device code takes its reciprocal from the MUFU unit, which the softmax warps
// keep saturated; the multiply does not.
__host__ __device__ __forceinline__ int fast_div(int n, uint64_t magic) {
#ifdef __CUDA_ARCH__
  return magic == 0 ? n : static_cast<int>(__umul64hi(static_cast<uint64_t>(static_cast<uint32_t>(n)), magic));
#else  // the host runs the same plan for b200_attn_plan
  return magic == 0 ? n : static_cast<int>((static_cast<unsigned __int128>(static_cast<uint32_t>(n)) * magic) >> 64);
#endif
}

// s[i] = s[i] * c + rel_h[(KV0 + i) / 14] + rel_w[(KV0 + i) % 14] for the keys of a 14 x 14 grid that fall into this
// tile; `stage` (shared memory) holds the row's 14 rel_h and 14 rel_w values, already times log2(e). All indices are
// constants: rel_w sits in registers for the section, each rel_h value is read once.
template <int KV0>
__device__ __forceinline__ void add_rel14(float* s, const float* stage, float c) {
  float rw[14];
#pragma unroll
  for (int m = 0; m < 14; ++m) rw[m] = stage[14 + m];
  const float2 cc = make_float2(c, c);
#pragma unroll
  for (int i = 0; i < kTileRows; i += 2) {
    constexpr int kKeys = 14 * 14;  // even, so a pair of columns is inside or outside together
    const int col = KV0 + i;
    if (col < kKeys) {
      const float2 b2 = fadd2(make_float2(stage[col / 14], stage[(col + 1) / 14]), make_float2(rw[col % 14], rw[(col + 1) % 14]));
      const float2 r = ffma2(make_float2(s[i], s[i + 1]), cc, b2);
      s[i] = r.x;
      s[i + 1] = r.y;
    }
  }
}

static_assert(sizeof(AttnSmem) + 1024 <= 227 * 1024 && sizeof(AttnSmemDense) + 1024 <= 227 * 1024, "shared memory of one CTA");

// One unit of work: one or two 128-row query tiles of one (batch, head) over the key tiles [ja, jb).
struct WorkItem {
  int b, h, q_row0, n_tiles;
  int ja, jb;  // key tiles of this CTA's part
  int kind;    // kItemWhole, kItemPartial (leaves its result in the workspace) or kItemOwner (merges the later parts)
};

// Key-split mode: the step of the line at which CTA `cta` begins (cta == grid: the end of the line).
__host__ __device__ __forceinline__ long long chunk_bound(const AttnParams& p, int cta, int grid) {
  (void)grid;
  const long long cost = cta * p.cost_base + (cta < p.cost_rem ? cta : p.cost_rem);  // no division by the grid size
  const long long pair_steps = static_cast<long long>(p.pair_items) * p.kv_tiles;
  const long long pair_cost = pair_steps * kPairCost;
  return cost <= pair_cost ? cost / kPairCost : pair_steps + (cost - pair_cost) / kSingleCost;
}

// The items of one CTA: `pairs` two-tile items, then `singles` one-tile items. Every CTA's list runs from two-tile
// to one-tile items: the second warpgroup and its MMA thread finish their last item and leave, they never have to
// skip one in the middle (a role that skips barrier phases cannot wait on them by parity any more).
//
// Dealt mode: two-tile items are numbered head by head, one-tile items likewise, and both kinds are dealt round
// robin, so that the CTAs work on neighbouring items of the same heads at the same time (their K / V tiles meet in
// L2 and the DRAM pages in use stay few; consecutive runs per CTA were measured 10 % slower on the short-sequence
// shapes). One-tile items cost about 0.8 of a two-tile item, so the host mixes the two kinds per head until the
// CTAs' loads are level, and the one-tile items go to the less loaded CTAs first.
//
// Key-split mode (long sequences, where whole items are too coarse to level 148 CTAs): see kPairCost. The only
// divisions are by constants and by kv_tiles (a multiply): a 64-bit division here cost a microsecond of set-up.
__host__ __device__ __forceinline__ CtaWork cta_work(const AttnParams& p, int cta, int grid) {
  CtaWork cw;
  if (p.chunked) {
    const long long sb = chunk_bound(p, cta, grid), se = chunk_bound(p, cta + 1, grid);
    const int first = fast_div(static_cast<int>(sb), p.magic_kv_tiles), last = fast_div(static_cast<int>(se - 1), p.magic_kv_tiles);
    const int items = se > sb ? last - first + 1 : 0;
    cw.first_item = first;
    cw.ja0 = static_cast<int>(sb - static_cast<long long>(first) * p.kv_tiles);
    cw.jb_last = static_cast<int>(se - static_cast<long long>(last) * p.kv_tiles);
    const int pairs_left = p.pair_items - first;
    cw.pairs = pairs_left < 0 ? 0 : pairs_left < items ? pairs_left : items;
    cw.singles = items - cw.pairs;
    const long long pair_steps = static_cast<long long>(p.pair_items) * p.kv_tiles;
    cw.steps_all = static_cast<int>(se - sb);
    const long long pair_end = se < pair_steps ? se : pair_steps;
    cw.steps_pairs = pair_end > sb ? static_cast<int>(pair_end - sb) : 0;
    cw.last_parts = 0;
    // Only a part that holds the item's first keys owns it (a run inside one item is a middle part: it owns nothing).
    if (items > 0 && cw.jb_last < p.kv_tiles && (items > 1 || cw.ja0 == 0)) {
      const long long item_end = static_cast<long long>(last + 1) * p.kv_tiles;
      while (cta + 1 + cw.last_parts < grid && chunk_bound(p, cta + 1 + cw.last_parts, grid) < item_end) ++cw.last_parts;
    }
    cw.first_back = cw.first_fwd = 0;
    if (items > 0 && cw.ja0 > 0) {
      const long long item_begin = static_cast<long long>(first) * p.kv_tiles, item_end = item_begin + p.kv_tiles;
      while (chunk_bound(p, cta - cw.first_back, grid) > item_begin) ++cw.first_back;  // bound(0) = 0 ends it
      while (cta + 1 + cw.first_fwd < grid && chunk_bound(p, cta + 1 + cw.first_fwd, grid) < item_end) ++cw.first_fwd;
    }
    cw.pair_start = cw.pair_stride = cw.single_start = cw.single_stride = 0;
    return cw;
  }
  cw.pair_start = cta;
  cw.pair_stride = grid;
  const int nb = grid - p.split_na;  // CTAs of the second kind; their one-tile items are numbered first
  if (cta < p.split_na) {
    cw.pairs = p.split_ka;
    cw.singles = p.split_a + (cta < p.split_ea ? 1 : 0);
    cw.single_start = nb * p.split_b + p.split_eb + cta;
    cw.single_stride = p.split_na;
  } else {
    const int c = cta - p.split_na;
    cw.pairs = p.split_kb;
    cw.singles = p.split_b + (c < p.split_eb ? 1 : 0);
    cw.single_start = c;
    cw.single_stride = nb;
  }
  cw.first_item = 0;
  cw.ja0 = 0;
  cw.jb_last = p.kv_tiles;
  cw.last_parts = cw.first_back = cw.first_fwd = 0;
  cw.steps_all = (cw.pairs + cw.singles) * p.kv_tiles;
  cw.steps_pairs = cw.pairs * p.kv_tiles;
  return cw;
}

// The it-th item of a CTA's list. SPLIT: the kernel form for key-split mode (the other form never meets a part
// of an item: every item is whole and its key range a constant, and the code for parts is not even compiled).
template <bool SPLIT>
__host__ __device__ __forceinline__ WorkItem decode_item(const AttnParams& p, const CtaWork& cw, int it) {
  WorkItem w;
  int bh;
  const bool pair = it < cw.pairs;
  if (pair) {
    const int id = SPLIT ? cw.first_item + it : cw.pair_start + it * cw.pair_stride;
    bh = fast_div(id, p.magic_pairs);
    w.q_row0 = (id - bh * p.pairs_per_head) * 2 * kTileRows;
    w.n_tiles = 2;
  } else {
    int id = SPLIT ? cw.first_item + it - p.pair_items : cw.single_start + (it - cw.pairs) * cw.single_stride;
    if (!SPLIT && id < 2 * p.conv_pairs) {  // one half of a two-tile item that is worked on as two one-tile items
      const int pair = p.kept_pairs + (id >> 1);
      bh = fast_div(pair, p.magic_pairs);
      w.q_row0 = (2 * (pair - bh * p.pairs_per_head) + (id & 1)) * kTileRows;
    } else {
      if (!SPLIT) id -= 2 * p.conv_pairs;
      bh = fast_div(id, p.magic_singles);
      w.q_row0 = (2 * p.pairs_per_head + (id - bh * p.singles_per_head)) * kTileRows;
    }
    w.n_tiles = 1;
  }
  // `bh` numbers the (batch, head) pairs head-fastest as a rule: neighbouring CTAs then work on one image's heads.
  // With a dense bias that all images share it is batch-fastest (magic_heads then belongs to the batch size): the
  // CTAs that need one head's bias tiles run together and the tiles meet in L2 instead of coming from DRAM per image.
  const int hi = fast_div(bh, p.magic_heads);
  const int lo = bh - hi * (p.batch_fastest ? p.batch : p.heads);
  w.b = p.batch_fastest ? lo : hi;
  w.h = p.batch_fastest ? hi : lo;
  if (SPLIT) {
    w.ja = it == 0 ? cw.ja0 : 0;
    w.jb = it == cw.pairs + cw.singles - 1 ? cw.jb_last : p.kv_tiles;
    w.kind = w.ja > 0 ? kItemPartial : w.jb < p.kv_tiles ? kItemOwner : kItemWhole;
  } else {
    w.ja = 0;
    w.jb = p.kv_tiles;
    w.kind = kItemWhole;
  }
  return w;
}

// Workspace slot of part `part` of a cut item whose first part belongs to CTA `first_cta`: that CTA's last-item
// slot for part 0, the first-item slot of CTA first_cta + part otherwise.
__device__ __forceinline__ float* partial_slot(float* ws_partial, int first_cta, int part, int t) {
  return ws_partial + ((static_cast<size_t>(first_cta + part) * 2 + (part == 0 ? 1 : 0)) * 2 + t) * kPartialFloats;
}

// One warp folds all `n_parts` parts of query tile t of item w, which are all in the workspace, and writes the
// tile's output rows. The slow route of the key-split mode: it only runs when the owner of a cut item could not
// fold the later parts in itself, so it is written for few registers, not for speed.
// `out_tile`: the output element of the tile's first row and first column; `rows`: rows of the tile inside the
// sequence; `row_stride`: elements between rows.
template <typename T>
__device__ __forceinline__ void merge_parts_to_output(float* ws_partial, T* out_tile, int64_t row_stride, int rows, int t,
                                                    int first_cta, int n_parts, int lane) {
  __threadfence();  // acquire side of the count that made this warp the last one
  for (int rg = 0; rg < kTileRows / 32; ++rg) {
    const int row = rg * 32 + lane;
    float m_all = -INFINITY;
    for (int part = 0; part < n_parts; ++part)
      m_all = fmaxf(m_all, __ldcg(partial_slot(ws_partial, first_cta, part, t) + kTileRows * kHeadDim + row));
    // Part 0 scaled, then every later part added with one fused multiply-add each, in part order: the order and the
    // operations of the owner's short cut in the kernel, so that both routes give the same bits.
    float l_all = 0.f;
    for (int part = 0; part < n_parts; ++part) {
      const float* slot = partial_slot(ws_partial, first_cta, part, t);
      const float m_p = __ldcg(slot + kTileRows * kHeadDim + row);
      const float f = m_p == m_all ? 1.f : fast_exp2(m_p - m_all);
      const float l_p = __ldcg(slot + kTileRows * kHeadDim + kTileRows + row);
      l_all = part == 0 ? l_p * f : fmaf(l_p, f, l_all);
    }
    const float inv = 1.f / l_all;
    for (int c4 = 0; c4 < kHeadDim / 4; ++c4) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int part = 0; part < n_parts; ++part) {
        const float* slot = partial_slot(ws_partial, first_cta, part, t);
        const float m_p = __ldcg(slot + kTileRows * kHeadDim + row);
        const float f = m_p == m_all ? 1.f : fast_exp2(m_p - m_all);
        const float4 x = __ldcg(reinterpret_cast<const float4*>(slot) + c4 * kTileRows + row);
        if (part == 0) {
          acc = make_float4(x.x * f, x.y * f, x.z * f, x.w * f);
        } else {
          acc.x = fmaf(x.x, f, acc.x);
          acc.y = fmaf(x.y, f, acc.y);
          acc.z = fmaf(x.z, f, acc.z);
          acc.w = fmaf(x.w, f, acc.w);
        }
      }
      if (row < rows) {
        uint2 val;
        val.x = pack2<T>(acc.x * inv, acc.y * inv);
        val.y = pack2<T>(acc.z * inv, acc.w * inv);
        *reinterpret_cast<uint2*>(out_tile + row * row_stride + 4 * c4) = val;
      }
    }
  }
}

// Persistent kernel: every CTA works through its own list of items (cta_work). All barrier phases and ring
// positions are running counters, so the loader prefetches the next item's Q / K / V while the current one is
// still being computed and tensor memory and barriers are set up once per CTA.
template <typename T, int BIAS, bool SHORT, bool SPLIT>
__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                const __grid_constant__ CUtensorMap tm_bias, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  using Smem = std::conditional_t<BIAS == kBiasDenseTiles, AttnSmemDense, AttnSmem>;
  constexpr int kStagesK = Smem::kRing, kStagesV = Smem::kRing;
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int kv_tiles = p.kv_tiles;
  // Keys of the last tile, rounded up to the MMA granule: its S needs no more columns, its P V no more steps.
  const int kv_last = p.kv_tokens - (kv_tiles - 1) * kTileRows;
  const int kv_last16 = (kv_last + 15) & ~15;

  // ---- set-up: barriers, tensor memory -------------------------------------------------------
  // The barriers lie one after another in Smem (q_full first, merge_go last): the lanes of warp 0 share them out,
  // one thread doing all fifty in turn was a visible part of a short launch. Arrival counts: 1 for a TMA
  // transaction or an MMA commit, 4 for the warps of a softmax warpgroup (128 arrivals on one word take hundreds
  // of clocks), 2 for the K / V rings' empty barriers (one commit per query tile; an item with one tile commits twice).
  if (warp == 0) {
    uint64_t* const first = &sm.q_full[0][0];
    const int n_bars = static_cast<int>(&sm.merge_go[1] - first) + 1;
    for (int i = lane; i < n_bars; i += 32) {
      uint64_t* bar = first + i;
      const bool four = (bar >= &sm.bias_free[0] && bar <= &sm.bias_free[1]) || (bar >= &sm.s_free[0] && bar <= &sm.s_free[1]) ||
                        (bar >= &sm.p_full[0] && bar <= &sm.p_full[1]) || (bar >= &sm.o_free[0] && bar <= &sm.o_staged[1]);
      const bool two = (bar >= &sm.k_empty[0] && bar <= &sm.k_empty[kStagesK - 1]) ||
                       (bar >= &sm.v_empty[0] && bar <= &sm.v_empty[kStagesV - 1]);
      mbar_init(bar, four ? 4 : two ? 2 : 1);
    }
    if (lane == 0) sm.abort = 0;
    if (lane < 8) (&sm.turn_count[0][0])[lane] = 0;
    mbar_init_fence();
  } else if (threadIdx.x == 32) {
    sm.work = cta_work(p, static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x));
  }
  if (warp == kMmaWarp) {
    tmem_alloc(&sm.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  if (warp == kLoaderWarp && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_o);
    if constexpr (BIAS == kBiasDenseTiles) tma_prefetch_desc(&tm_bias);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  // The launch allows this grid to start while the kernel before it in the stream is still draining (programmatic
  // stream serialisation): the set-up above touches no global memory and overlaps that kernel's tail; everything
  // below reads or writes global memory and waits here until the earlier kernel has completed and its writes are
  // visible. Without an earlier kernel, or without the launch attribute, the wait returns at once.
  grid_dependency_wait();
  const uint32_t tmem = sm.tmem_base;
  volatile uint32_t* abort_flag = &sm.abort;
  const CtaWork& cw = sm.work;
  const int my_items = cw.pairs + cw.singles;

  if (warp >= kLoaderWarp) {
    reg_dealloc<kHelperRegs>();
    if (warp == kLoaderWarp) {
      // ======================= loader =======================================================
      if (lane == 0) {
        bool ok = true;
        int gk = 0, gv = 0;        // K / V tiles issued so far (ring position and phase)
        int q_count[2] = {0, 0};   // Q tiles issued so far per query-tile slot
        for (int it = 0; it < my_items && ok; ++it) {
          const WorkItem w = decode_item<SPLIT>(p, cw, it);
          const int slot = it & 1;
          for (int t = 0; t < w.n_tiles && ok; ++t) {
            ok = mbar_wait_relaxed(&sm.q_empty[t][slot], ((it >> 1) & 1) ^ 1, abort_flag);
            if (!ok) break;
            mbar_arrive_expect_tx(&sm.q_full[t][slot], kTileBytes);
            tma_load_4d(sm.q[t][slot], &tm_q, &sm.q_full[t][slot], 0, w.q_row0 + t * kTileRows, w.h, w.b);
            q_count[t] = it + 1;
          }
          const int steps = w.jb - w.ja;  // the key tiles of this CTA's part of the item
          for (int i = 0; i < steps + kKLead && ok; ++i) {
            if (i < steps) {
              const int st = gk % kStagesK;
              ok = mbar_wait_relaxed(&sm.k_empty[st], ((gk / kStagesK) & 1) ^ 1, abort_flag);
              if (!ok) break;
              mbar_arrive_expect_tx(&sm.k_full[st], kTileBytes);
              tma_load_4d(sm.k[st], &tm_k, &sm.k_full[st], 0, (w.ja + i) * kTileRows, w.h, w.b);
              ++gk;
            }
            const int iv = i - kKLead;
            if (iv >= 0) {
              const int st = gv % kStagesV;
              ok = mbar_wait_relaxed(&sm.v_empty[st], ((gv / kStagesV) & 1) ^ 1, abort_flag);
              if (!ok) break;
              mbar_arrive_expect_tx(&sm.v_full[st], kTileBytes);
              tma_load_4d(sm.v[st], &tm_v, &sm.v_full[st], 0, (w.ja + iv) * kTileRows, w.h, w.b);
              ++gv;
            }
          }
        }
        if (!ok) {
          if (atomicExch(const_cast<uint32_t*>(abort_flag), 1u) == 0) atomicOr(p.status, kStatusLoader);
        }
        if (*abort_flag != 0) {
          // Nobody may be consuming any more: wait (bounded, ignoring the abort flag) for every copy
          // that was issued, so that none writes into shared memory after the CTA has gone.
          uint32_t no_abort = 0;
          for (int t = 0; t < 2; ++t)
            for (int i = (q_count[t] > 2 ? q_count[t] - 2 : 0); i < q_count[t]; ++i)
              mbar_wait_relaxed(&sm.q_full[t][i & 1], (i >> 1) & 1, &no_abort);
          for (int j = (gk > kStagesK ? gk - kStagesK : 0); j < gk; ++j)
            mbar_wait_relaxed(&sm.k_full[j % kStagesK], (j / kStagesK) & 1, &no_abort);
          for (int j = (gv > kStagesV ? gv - kStagesV : 0); j < gv; ++j)
            mbar_wait_relaxed(&sm.v_full[j % kStagesV], (j / kStagesV) & 1, &no_abort);
        }
      }
      if constexpr (BIAS == kBiasDenseTiles) {
        // A second lane of the loader warp brings the bias tiles: one 128 x 128 tile (two 64-column boxes) per query
        // tile and step, single-buffered per query tile. It runs at the softmax warps' pace (a tile's buffer is free
        // once they have read the previous one, early in a step), which must not hold up the K / V loads that run
        // tiles ahead: hence a lane of its own. Columns and rows past the end of the bias read as zero.
        if (lane == 1) {
          bool ok = true;
          int gb[2] = {0, 0};  // bias tiles issued so far per query-tile slot
          for (int it = 0; it < my_items && ok; ++it) {
            const WorkItem w = decode_item<SPLIT>(p, cw, it);
            for (int j = w.ja; j < w.jb && ok; ++j) {
              for (int t = 0; t < w.n_tiles && ok; ++t) {
                ok = mbar_wait_relaxed(&sm.bias_free[t], (gb[t] & 1) ^ 1, abort_flag);
                if (!ok) break;
                mbar_arrive_expect_tx(&sm.bias_full[t], 2 * kTileBytes);
                const int bz = p.bias.sh != 0 ? w.h : 0, bw = p.bias.sb != 0 ? w.b : 0;  // a stride of 0 broadcasts
                tma_load_4d(sm.bias_tile[t][0], &tm_bias, &sm.bias_full[t], j * kTileRows, w.q_row0 + t * kTileRows, bz, bw);
                tma_load_4d(sm.bias_tile[t][1], &tm_bias, &sm.bias_full[t], j * kTileRows + 64, w.q_row0 + t * kTileRows, bz, bw);
                ++gb[t];
              }
            }
          }
          if (!ok) {
            if (atomicExch(const_cast<uint32_t*>(abort_flag), 1u) == 0) atomicOr(p.status, kStatusLoader);
          }
          if (*abort_flag != 0) {  // let the copies in flight land (at most one tile per slot)
            uint32_t no_abort = 0;
            for (int t = 0; t < 2; ++t)
              if (gb[t] > 0) mbar_wait_relaxed(&sm.bias_full[t], (gb[t] - 1) & 1, &no_abort);
          }
        }
      }
      __syncwarp();
    } else if (warp == kMmaWarp || warp == kMmaWarp + 1) {
      // ======================= MMA issuers: one thread per query tile ==========================
      const int t = warp - kMmaWarp;
      if (lane == 0) {
        constexpr uint32_t fmt = std::is_same<T, __half>::value ? UMMA_F16 : UMMA_BF16;
        constexpr uint32_t idesc_qk = umma_idesc_f16(fmt, kTileRows, kTileRows, 0, 0);
        constexpr uint32_t idesc_pv = umma_idesc_f16(fmt, kTileRows, kHeadDim, 0, 1);
        const uint32_t idesc_qk_last = umma_idesc_f16(fmt, kTileRows, kv_last16, 0, 0);
        bool ok = true;

        // Everything the issue loops need is computed once or counted along: one thread feeds the tensor pipe, and
        // every instruction between two tcgen05.mma shows up as an idle pipe when the MMAs are this small.
        const uint64_t q_desc0 = umma_smem_desc_sw128(smem_u32(sm.q[t][0]), 1024, 16);
        const uint64_t k_desc0 = umma_smem_desc_sw128(smem_u32(sm.k[0]), 1024, 16);
        const uint64_t v_desc0 = umma_smem_desc_sw128(smem_u32(sm.v[0]), 1024, 0);
        constexpr uint64_t kStageStep = kTileBytes >> 4;  // descriptor distance between two tiles in shared memory
        const uint32_t s_tm = tmem + kTmemS + t * kTileRows;
        const uint32_t o_tm = tmem + kTmemO + t * kHeadDim;
        const uint32_t p_tm = tmem + kTmemP + t * kHeadDim;
        uint64_t* const s_full = &sm.s_full[t];
        uint64_t* const s_free = &sm.s_free[t];
        uint64_t* const p_full = &sm.p_full[t];
        uint64_t* const pv_done = &sm.pv_done[t];

        // This slot's items are a prefix of the CTA's list (two-tile items come first), so its key-tile steps form
        // one stream gs = 0, 1, ...: step gs is key tile j of item it and uses ring tile gs (stage st, in its
        // ph-th use). S is issued two steps ahead of its use, across item boundaries too, so that a new item starts
        // at once. The positions are counted along: a division by kv_tiles here would queue its reciprocal behind the
        // softmax warps' exponentials on the MUFU unit, which cost the long-sequence runs 15 %.
        const int my_doubles = cw.pairs;
        const int total_steps = t == 0 ? cw.steps_all : cw.steps_pairs;
        // `j` is the key tile and `jend` where this CTA's part of the item ends (the part starts at key tile 0
        // except, in key-split mode, for the CTA's first item).
        struct Pos {
          int gs, it, j, jend, st;
          uint32_t ph;
        };
        const int ja0 = SPLIT ? cw.ja0 : 0, jb_last = cw.jb_last;
        // Without key split every part is a whole item: `jend` is never read and costs no register.
        auto is_first = [&](const Pos& x) { return SPLIT ? x.j == (x.it == 0 ? ja0 : 0) : x.j == 0; };
        auto is_last = [&](const Pos& x) { return SPLIT ? x.j == x.jend - 1 : x.j == kv_tiles - 1; };
        auto advance = [&](Pos& x) {
          ++x.gs;
          if (SPLIT ? ++x.j == x.jend : ++x.j == kv_tiles) {
            x.j = 0;
            ++x.it;
            x.jend = x.it == my_items - 1 ? jb_last : kv_tiles;
          }
          if (++x.st == kStagesK) {
            x.st = 0;
            x.ph ^= 1;
          }
        };
        const Pos start = {0, 0, ja0, my_items == 1 ? jb_last : kv_tiles, 0, 0u};
        static_assert(kStagesK == kStagesV, "one ring position serves both rings");

        // S_t(gs) = Q_t K^T. The last key tile of an item only computes the columns that hold keys.
        auto issue_qk = [&](const Pos& x) -> bool {
          const int slot = x.it & 1;
          // The K tile landed long ago as a rule: its test is issued first and runs behind the wait that does wait.
          const bool k_early = mbar_test_wait(&sm.k_full[x.st], x.ph);
          if (is_first(x) && !mbar_wait(&sm.q_full[t][slot], (x.it >> 1) & 1, abort_flag)) return false;
          if (x.gs > 0 && !mbar_wait(s_free, (x.gs - 1) & 1, abort_flag)) return false;  // S_t has been read
          if (!k_early && !mbar_wait(&sm.k_full[x.st], x.ph, abort_flag)) return false;
          tc_fence_after_sync();
          const uint64_t a = q_desc0 + static_cast<uint64_t>(slot) * kStageStep;
          const uint64_t bd = k_desc0 + static_cast<uint64_t>(x.st) * kStageStep;
          const uint32_t idesc = (x.j == kv_tiles - 1) ? idesc_qk_last : idesc_qk;
#pragma unroll
          for (int kk = 0; kk < kHeadDim / 16; ++kk)  // 32 bytes of K per step inside the swizzle atom
            umma_ss(s_tm, a + 2 * kk, bd + 2 * kk, idesc, kk > 0 ? 1u : 0u);
          umma_commit(s_full);
          umma_commit(&sm.k_empty[x.st]);
          if (x.it >= my_doubles) umma_commit(&sm.k_empty[x.st]);  // one-tile item: stand in for the absent second tile
          if (is_last(x)) umma_commit(&sm.q_empty[t][slot]);  // the item's last reader of Q_t
          return true;
        };
        // O_t (+)= P_t(gs) V, 16 keys (two 8-row groups of the V tile) per MMA.
        auto issue_pv = [&](const Pos& x) -> bool {
          const bool v_early = mbar_test_wait(&sm.v_full[x.st], x.ph);
          if (!mbar_wait(p_full, x.gs & 1, abort_flag)) return false;
          if (!v_early && !mbar_wait(&sm.v_full[x.st], x.ph, abort_flag)) return false;
          // The first P V of an item overwrites O_t: the previous item's epilogue must have read it.
          if (is_first(x) && x.it > 0 && !mbar_wait(&sm.o_free[t], (x.it - 1) & 1, abort_flag)) return false;
          tc_fence_after_sync();
          const uint64_t bd = v_desc0 + static_cast<uint64_t>(x.st) * kStageStep;
          if (x.j != kv_tiles - 1) {
            umma_ts(o_tm, p_tm, bd, idesc_pv, is_first(x) ? 0u : 1u);
#pragma unroll
            for (int kk = 1; kk < kTileRows / 16; ++kk)
              umma_ts(o_tm, p_tm + kk * 8, bd + kk * (2048 >> 4), idesc_pv, 1u);
          } else {
            const int steps = kv_last16 / 16;  // at least one
            umma_ts(o_tm, p_tm, bd, idesc_pv, is_first(x) ? 0u : 1u);
#pragma unroll
            for (int kk = 1; kk < kTileRows / 16; ++kk)
              if (kk < steps) umma_ts(o_tm, p_tm + kk * 8, bd + kk * (2048 >> 4), idesc_pv, 1u);
          }
          umma_commit(pv_done);
          umma_commit(&sm.v_empty[x.st]);
          if (x.it >= my_doubles) umma_commit(&sm.v_empty[x.st]);
          return true;
        };

        Pos xq = start;  // the Q K^T stream runs two steps ahead of the P V stream
        for (int i = 0; i < 2 && xq.gs < total_steps && ok; ++i) {
          ok = issue_qk(xq);
          advance(xq);
        }
        for (Pos xp = start; xp.gs < total_steps && ok; advance(xp)) {
          ok = issue_pv(xp);
          if (ok && xq.gs < total_steps) {
            ok = issue_qk(xq);
            advance(xq);
          }
        }
        if (!ok) {
          if (atomicExch(const_cast<uint32_t*>(abort_flag), 1u) == 0) atomicOr(p.status, kStatusMma);
        }
        if (*abort_flag != 0) {
          // Some role gave up: products this thread issued may still be running, and their commits must not
          // arrive on barriers of a CTA that is gone (nor tensor memory be freed under them). One last commit on
          // a barrier of its own, waited for with the usual limit and without looking at the abort flag.
          uint32_t no_abort = 0;
          umma_commit(&sm.drain[t]);
          mbar_wait(&sm.drain[t], 0, &no_abort);
        }
      }
      __syncwarp();
    } else if (warp == kStoreWarp) {
      // ======================= output stores ====================================================
      // Lane 0 sends each finished output tile from its staging buffer to global memory with a TMA store (rows
      // past the end of the sequence are clipped by the tensor map) and hands the buffer back once it has been read.
      // For a part of an item that is cut along the keys the hand-over may instead mean "the part is in the
      // workspace": lane 0 then fences and counts it, and if that made the item complete the whole warp folds
      // the parts and writes the output rows (see kPartialFloats).
      if constexpr (!SPLIT) {
        if (lane == 0) {
          bool ok = true;
          for (int it = 0; it < my_items && ok; ++it) {
            const WorkItem w = decode_item<SPLIT>(p, cw, it);
            for (int t = 0; t < w.n_tiles && ok; ++t) {
              // Slot 1's items are a prefix of the CTA's list, so this is the it-th use of either slot's buffer.
              ok = mbar_wait(&sm.o_staged[t], it & 1, abort_flag);
              if (!ok) break;
              tma_store_4d(&tm_o, sm.o_stage[t], 0, w.q_row0 + t * kTileRows, w.h, w.b);
              tma_store_commit();
            }
            // The buffers are not needed again before the next item's epilogue: one wait for both stores.
            tma_store_wait_read<0>();
            for (int t = 0; t < w.n_tiles && ok; ++t) mbar_arrive(&sm.o_stage_free[t]);
          }
          // Every store has read its buffer by now (the wait above); the writes themselves complete with the kernel.
          if (!ok) {
            if (atomicExch(const_cast<uint32_t*>(abort_flag), 1u) == 0) atomicOr(p.status, kStatusStore);
          }
        }
        __syncwarp();
      } else {
        bool ok = true;
        for (int it = 0; it < my_items && ok; ++it) {
          const WorkItem w = decode_item<SPLIT>(p, cw, it);
          for (int t = 0; t < w.n_tiles && ok; ++t) {
            uint32_t what = 1;
            if (lane == 0) {
              ok = mbar_wait(&sm.o_staged[t], it & 1, abort_flag);
              if (ok && w.kind != kItemWhole) what = *reinterpret_cast<volatile uint32_t*>(&sm.o_store[t][it & 1]);
              if (ok && what == 1) {
                tma_store_4d(&tm_o, sm.o_stage[t], 0, w.q_row0 + t * kTileRows, w.h, w.b);
                tma_store_commit();
              }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            what = __shfl_sync(0xffffffffu, what, 0);
            if (!ok || w.kind == kItemWhole) continue;
            const bool owner = w.kind == kItemOwner;
            const int first_cta = owner ? static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x) - cw.first_back;
            const int n_parts = owner ? 1 + cw.last_parts : cw.first_back + 1 + cw.first_fwd;
            uint32_t* counter = p.ws_counts + first_cta * 2 + t;
            if (what == 1) {  // the owner folded the later parts in itself: only the counter is left to clear
              if (lane == 0) *counter = 0u;
              continue;
            }
            uint32_t last = 0;
            if (lane == 0) {
              __threadfence();  // the softmax threads' stores, ordered before the hand-over, before the count
              last = atomicAdd(counter, 1u) == static_cast<uint32_t>(n_parts - 1) ? 1u : 0u;
              if (last) {
                __threadfence();
                *counter = 0u;  // nobody else touches it any more: ready for the next launch
              }
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            if (last) {
              const int row0 = w.q_row0 + t * kTileRows;
              T* out_tile = static_cast<T*>(p.o) + w.b * p.o_sb + static_cast<int64_t>(row0) * p.o_sn + w.h * p.o_sh;
              merge_parts_to_output<T>(p.ws_partial, out_tile, p.o_sn, p.q_tokens - row0, t, first_cta, n_parts, lane);
            }
          }
          if (lane == 0) {
            tma_store_wait_read<0>();
            for (int t = 0; t < w.n_tiles && ok; ++t) mbar_arrive(&sm.o_stage_free[t]);
          }
          __syncwarp();
        }
        if (!ok && lane == 0) {
          if (atomicExch(const_cast<uint32_t*>(abort_flag), 1u) == 0) atomicOr(p.status, kStatusStore);
        }
        __syncwarp();
      }
    }
  } else {
    // ======================= softmax warpgroups ================================================
    reg_alloc<kSoftmaxRegs>();
    const int t = warp >> 2;  // query-tile slot of this warpgroup
    const int row_in_tile = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t s_addr = tmem + lane_addr + kTmemS + t * kTileRows;
    const uint32_t o_addr = tmem + lane_addr + kTmemO + t * kHeadDim;
    const uint32_t p_addr = tmem + lane_addr + kTmemP + t * kHeadDim;
    const float c = p.scale_log2;
    int g = 0;        // key-tile steps of this slot so far (phases of s_full, s_free, p_full, pv_done)
    int gp = 0;       // steps so far in items where both warpgroups work (phases of the turn barriers)
    bool ok = true;
    bool bad = false;  // this lane gave up a wait since the last vote
    bool s_early = false, pv_early = false, stage_early = false;  // early barrier tests (see the step loop)
    // Epilogue of the previous item, still to be done: its last P V phase, reference maximum, row sum, kind.
    bool pend = false;
    uint32_t pend_phase = 0;
    float pend_l = 0.f;
    float pend_m_of_split = 0.f;  // key-split form only: the pending item's reference maximum
    int pend_it = 0;
    // O_t / l -> staging buffer -> (store thread) global for the pending item; frees O_t for the next item's first P V.
    // Each thread writes its 128-byte row as eight 16-byte chunks at the positions of the 128-byte swizzle.
    // `pv_tested`, `stage_tested`: results of early tests of the two barriers (false = not tested or still pending).
    // A part of an item that is cut along the keys (key-split mode) either folds the other parts into its O_t and
    // row sum and goes on as usual, or leaves O_t, the reference maxima and the row sums in the workspace.
    // `at_end`: the call after the CTA's last item, the only one that can meet an owner (the calls inside the step
    // loop finish an item that has a successor): the owner's code is compiled into that one call only.
    auto finish_item = [&](bool pv_tested, bool stage_tested, auto at_end) -> bool {
      [[maybe_unused]] constexpr bool kAtEnd = decltype(at_end)::value;
      if (!__all_sync(0xffffffffu, pv_tested || mbar_wait(&sm.pv_done[t], pend_phase, abort_flag))) return false;
      tc_fence_after_sync();
      float o[kHeadDim];
      tmem_ld_x64(o_addr, reinterpret_cast<uint32_t*>(o));
      tc_fence_before_sync();
      warp_arrive(&sm.o_free[t], lane);
      float l_all = pend_l;
      if constexpr (SPLIT) {
        // Which kind of item the pending one is follows from its place in the list (first: a later part if it
        // begins past key tile 0; last: the owner if it ends early) - nothing is carried along in registers.
        const bool later_part = pend_it == 0 && cw.ja0 > 0;
        const bool owner = kAtEnd && !later_part && pend_it == my_items - 1 && cw.jb_last < kv_tiles;
        if (later_part || owner) {  // CTA-uniform: a part of an item that is cut along the keys (see kPartialFloats)
          const int first_cta = owner ? static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x) - cw.first_back;
          const int n_parts = owner ? 1 + cw.last_parts : cw.first_back + 1 + cw.first_fwd;
          const float m_own = pend_m_of_split;
          bool fold = false;
          if constexpr (kAtEnd) if (owner && (p.test_flags & 1) == 0) {
            // The tile's first thread looks at the item's counter - for a while, when the later parts are not all
            // counted yet (CTAs with short runs finish together) - and passes the result on through shared memory.
            if (row_in_tile == 0) {
              const uint32_t* counter = p.ws_counts + first_cta * 2 + t;
              bool ready = ld_acquire_gpu(counter) == static_cast<uint32_t>(n_parts - 1);
              if (!ready) {
                const uint64_t t0 = global_timer_ns();
                while (!ready && global_timer_ns() - t0 < kOwnerPatienceNs) {
                  __nanosleep(200);
                  ready = ld_acquire_gpu(counter) == static_cast<uint32_t>(n_parts - 1);
                }
              }
              sm.merge_ready[t] = ready ? 1u : 0u;
              mbar_arrive(&sm.merge_go[t]);
            }
            if (!__all_sync(0xffffffffu, mbar_wait(&sm.merge_go[t], 0, abort_flag))) return false;  // used once per CTA
            fold = *reinterpret_cast<volatile uint32_t*>(&sm.merge_ready[t]) != 0;
          }
          if (kAtEnd && fold) {
            // The same arithmetic, in the same order, as merge_parts_to_output: whichever route an item takes, its
            // output has the same bits.
            __threadfence();  // the later parts' results, counted before the look, before these loads
            float m_all = m_own;
            for (int part = 1; part < n_parts; ++part)
              m_all = fmaxf(m_all, __ldcg(partial_slot(p.ws_partial, first_cta, part, t) + kTileRows * kHeadDim + row_in_tile));
            const float f_own = m_own == m_all ? 1.f : fast_exp2(m_own - m_all);
            l_all = pend_l * f_own;
#pragma unroll
            for (int i = 0; i < kHeadDim; ++i) o[i] *= f_own;
            for (int part = 1; part < n_parts; ++part) {
              const float* slot = partial_slot(p.ws_partial, first_cta, part, t);
              const float m_p = __ldcg(slot + kTileRows * kHeadDim + row_in_tile);
              const float f = m_p == m_all ? 1.f : fast_exp2(m_p - m_all);
              l_all = fmaf(__ldcg(slot + kTileRows * kHeadDim + kTileRows + row_in_tile), f, l_all);
              const float4* src4 = reinterpret_cast<const float4*>(slot) + row_in_tile;
#pragma unroll
              for (int c4 = 0; c4 < kHeadDim / 4; ++c4) {
                const float4 x = __ldcg(src4 + c4 * kTileRows);
                o[4 * c4 + 0] = fmaf(x.x, f, o[4 * c4 + 0]);
                o[4 * c4 + 1] = fmaf(x.y, f, o[4 * c4 + 1]);
                o[4 * c4 + 2] = fmaf(x.z, f, o[4 * c4 + 2]);
                o[4 * c4 + 3] = fmaf(x.w, f, o[4 * c4 + 3]);
              }
            }
            if (row_in_tile == 0) sm.o_store[t][pend_it & 1] = 1u;
          } else {
            float* slot = partial_slot(p.ws_partial, first_cta, static_cast<int>(blockIdx.x) - first_cta, t);
            float4* dst = reinterpret_cast<float4*>(slot) + row_in_tile;
#pragma unroll
            for (int c4 = 0; c4 < kHeadDim / 4; ++c4)
              __stcg(dst + c4 * kTileRows, make_float4(o[4 * c4], o[4 * c4 + 1], o[4 * c4 + 2], o[4 * c4 + 3]));
            __stcg(slot + kTileRows * kHeadDim + row_in_tile, m_own);
            __stcg(slot + kTileRows * kHeadDim + kTileRows + row_in_tile, pend_l);
            if (row_in_tile == 0) sm.o_store[t][pend_it & 1] = 2u;
            // The hand-over now means "the part is in the workspace": the store warp fences and counts it. Like a
            // staged tile it must not come before the store warp is done with the item before (it may be folding
            // parts for a long time): waits by parity tell only neighbouring phases of a barrier apart.
            if (pend_it > 0 &&
                !__all_sync(0xffffffffu, stage_tested || mbar_wait(&sm.o_stage_free[t], (pend_it - 1) & 1, abort_flag)))
              return false;
            warp_arrive(&sm.o_staged[t], lane);
            pend = false;
            return true;
          }
        }
      }
      const float inv = 1.f / l_all;
      // The buffer's previous tile (the item before the pending one) must have been read by its store.
      if (pend_it > 0 &&
          !__all_sync(0xffffffffu, stage_tested || mbar_wait(&sm.o_stage_free[t], (pend_it - 1) & 1, abort_flag)))
        return false;
      const uint32_t row = smem_u32(sm.o_stage[t]) + row_in_tile * (kHeadDim * 2);
#pragma unroll
      const float2 inv2 = make_float2(inv, inv), zero2 = make_float2(0.f, 0.f);
#pragma unroll
      for (int ch = 0; ch < kHeadDim / 8; ++ch) {
        uint4 val;
        // packed multiplies (x * inv + 0 rounds like x * inv)
        const float2 a = ffma2(make_float2(o[ch * 8 + 0], o[ch * 8 + 1]), inv2, zero2);
        const float2 b = ffma2(make_float2(o[ch * 8 + 2], o[ch * 8 + 3]), inv2, zero2);
        const float2 c2 = ffma2(make_float2(o[ch * 8 + 4], o[ch * 8 + 5]), inv2, zero2);
        const float2 d = ffma2(make_float2(o[ch * 8 + 6], o[ch * 8 + 7]), inv2, zero2);
        val.x = pack2<T>(a.x, a.y);
        val.y = pack2<T>(b.x, b.y);
        val.z = pack2<T>(c2.x, c2.y);
        val.w = pack2<T>(d.x, d.y);
        st_shared_v4(row + ((ch ^ (row_in_tile & 7)) << 4), val);
      }
      fence_proxy_async_smem();  // the TMA store reads what these generic-proxy stores wrote
      warp_arrive(&sm.o_staged[t], lane);
      pend = false;
      return true;
    };

    for (int it = 0; it < my_items && ok; ++it) {
      const WorkItem w = decode_item<SPLIT>(p, cw, it);
      if (t >= w.n_tiles) break;  // only one-tile items follow
      const int b = w.b, h = w.h;
      const int q_row = w.q_row0 + t * kTileRows + row_in_tile;
      const bool row_valid = q_row < p.q_tokens;
      const bool pingpong = w.n_tiles == 2;
      const int ja = w.ja, jb = w.jb;  // this CTA's key tiles of the item
      float m_ref = -INFINITY;
      float l_sum = 0.f;

      int64_t bias_row = 0, bias2_row = 0;
      // kBiasDecomposed64: rel_h of this row as raw 16-byte groups of eight values, each good for four key tiles
      // (a tile spans two rows of the key grid); the next group is fetched four tiles ahead and never converted
      // before it is used. One load per four tiles: every global load in the step costs, two per tile were 20 us of 144.
      uint4 rh_cur = make_uint4(0, 0, 0, 0), rh_nxt = make_uint4(0, 0, 0, 0);
      if constexpr (BIAS != kBiasNone) {
        const int qr = row_valid ? q_row : 0;
        bias_row = b * p.bias.sb + h * p.bias.sh + qr * p.bias.sn;
        if constexpr (BIAS == kBiasDecomposed || BIAS == kBiasDecomposed64 || BIAS == kBiasDecomposed14)
          bias2_row = b * p.bias2.sb + h * p.bias2.sh + qr * p.bias2.sn;
        if constexpr (BIAS == kBiasDecomposed14) {
          // This thread's rows, read back by this thread only: no synchronisation needed.
          float* stage = sm.rel_stage[t][row_in_tile];
          for_bias_dtype(p.bias.dtype, [&](auto dt) {  // rel_h and rel_w are of one type
            constexpr int kDt = decltype(dt)::value;
            float tmp[28];
#pragma unroll
            for (int i = 0; i < 14; ++i) {  // all loads in flight together
              tmp[i] = load_bias_elem_t<kDt>(p.bias.ptr, bias_row + i);
              tmp[14 + i] = load_bias_elem_t<kDt>(p.bias2.ptr, bias2_row + i);
            }
#pragma unroll
            for (int i = 0; i < 28; ++i) stage[i] = tmp[i] * kLog2e;
          });
        }
        if constexpr (BIAS == kBiasDecomposed64) {
          // The row's 64 rel_w values (32 words of 16-bit pairs) are the same for every key tile: they are staged
          // once per item in this thread's own row of the staging area (read back by this thread only, so no
          // synchronisation), and the first pair of rel_h values is fetched; later pairs are fetched a step ahead.
          const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.bias2.ptr) + bias2_row);
          uint32_t* stage = reinterpret_cast<uint32_t*>(sm.rel_stage[t][row_in_tile]);
          uint4 v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) v[u] = __ldg(src + u);
          // rel_h comes in groups of eight values, each good for four key tiles: the part's first group now, the
          // one after it too (the loop fetches a group four tiles ahead, at every fourth tile).
          const uint4* rh_src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.bias.ptr) + bias_row);
          rh_cur = __ldg(rh_src + (ja >> 2));
          if (2 * ((ja & ~3) + 4) < p.rel_kh) rh_nxt = __ldg(rh_src + (ja >> 2) + 1);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            stage[u * 4 + 0] = v[u].x;
            stage[u * 4 + 1] = v[u].y;
            stage[u * 4 + 2] = v[u].z;
            stage[u * 4 + 3] = v[u].w;
          }
        }
        if constexpr (BIAS == kBiasDecomposed) {
          if (p.rel_staged) {  // this thread's rows, read back by this thread only: no synchronisation needed
            float* stage = sm.rel_stage[t][row_in_tile];
            for_bias_dtype(p.bias.dtype, [&](auto dt) {  // rel_h and rel_w are of one type
              constexpr int kDt = decltype(dt)::value;
              float tmp[kRelStageWords - 1];
#pragma unroll
              for (int i = 0; i < kRelStageWords - 1; ++i) {  // all loads in flight together
                const bool in_h = i < p.rel_kh;
                const bool in_w = !in_h && i < p.rel_kh + p.rel_kw;
                tmp[i] = in_h   ? load_bias_elem_t<kDt>(p.bias.ptr, bias_row + i)
                         : in_w ? load_bias_elem_t<kDt>(p.bias2.ptr, bias2_row + (i - p.rel_kh))
                                : 0.f;
              }
#pragma unroll
              for (int i = 0; i < kRelStageWords - 1; ++i) stage[i] = tmp[i] * kLog2e;
            });
          }
        }
      }

      for (int j = ja; j < jb; ++j) {
        const int rj = j - ja;  // step within this CTA's part of the item
        const int step = g + rj;
        // One vote per step on whether any lane's wait ran out during the previous one.
        if (__any_sync(0xffffffffu, bad)) {
          ok = false;
          break;
        }
        bad |= !mbar_wait_warp_after(s_early, &sm.s_full[t], step & 1, abort_flag);
        tc_fence_after_sync();
        // dense-tile bias: the tile's barrier is tested here, its result is needed after the S load
        [[maybe_unused]] bool bias_early = false;
        if constexpr (BIAS == kBiasDenseTiles) bias_early = mbar_test_wait(&sm.bias_full[t], step & 1);

        float s[kTileRows];
        {
          uint32_t* su = reinterpret_cast<uint32_t*>(s);
          // One 128-column load (a quarter of the tcgen05 instructions of four 32-column ones: -2 %).
          tmem_ld_x128(s_addr, su);
        }
        // S_t is in registers: the tensor pipe may overwrite it with the tile after next.
        tc_fence_before_sync();
        warp_arrive(&sm.s_free[t], lane);
        // Tests of the barriers this step will wait on, issued here so that their latency (100-150 clocks each with
        // tensor memory allocated) runs behind the arithmetic; a test that finds its phase pending is repeated as a
        // real wait where the result is needed.
        const bool need_turn = pingpong && (t == 1 || gp + rj > 0);
        const uint32_t turn_parity = (t == 0) ? ((gp + rj - 1) & 1) : ((gp + rj) & 1);
        // The token between the warpgroups has two forms. Barrier form: all four warps of the other warpgroup arrive
        // on `turn`. Flag form (kFlagTurn): warp w only waits for warp w of the other warpgroup - the one it shares
        // its SM sub-partition and MUFU unit with - through a counter in shared memory, which is cheaper to poll than
        // a barrier and does not tie a warp to the slowest of four. Measured per kernel form: the flag form is
        // 2-6 % faster in the short and the key-split kernels and 4-7 % slower in the plain long one.
        constexpr bool kFlagTurn = SHORT || SPLIT;
        const uint32_t turn_need = (t == 0) ? static_cast<uint32_t>(gp + rj) : static_cast<uint32_t>(gp + rj + 1);
        const bool turn_early = (need_turn && !kFlagTurn) ? mbar_test_wait(&sm.turn[t], turn_parity) : true;

        const int kv0 = j * kTileRows;
        const int kv_valid = min(kTileRows, p.kv_tokens - kv0);
        float rh0 = 0.f, rh1 = 0.f;  // kBiasDecomposed64: rel_h of the tile's two 64-column halves, natural units

        if constexpr (BIAS == kBiasDenseTiles) {
          // The tile is in shared memory (loader warp, TMA): this thread's row is sixteen 16-byte chunks, eight per
          // 64-column half, at the positions of the 128-byte swizzle. Logits stay in natural units, s * scale + bias,
          // one packed FMA per pair of columns; log2(e) rides on the FMA in front of the exponential.
          bad |= !mbar_wait_warp_after(bias_early, &sm.bias_full[t], step & 1, abort_flag);
          const bool is_half = p.bias.dtype == 0;
          const float scale_nat = c * 0.6931471805599453f;  // scale_log2 / log2(e)
          auto add_tile = [&](auto half_tag) {
            constexpr bool kHalf = decltype(half_tag)::value;
            const float2 cc = make_float2(scale_nat, scale_nat);
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
              const uint32_t row = smem_u32(sm.bias_tile[t][hf]) + row_in_tile * 128;
#pragma unroll
              for (int ch = 0; ch < 8; ++ch) {
                const uint4 v = ld_shared_v4(row + ((ch ^ (row_in_tile & 7)) << 4));
                const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const int i = hf * 64 + ch * 8 + e * 2;
                  const float2 r = ffma2(make_float2(s[i], s[i + 1]), cc, unpack2(w4[e], kHalf));
                  s[i] = r.x;
                  s[i + 1] = r.y;
                }
              }
            }
          };
          if (is_half) add_tile(std::true_type{});
          else add_tile(std::false_type{});
          warp_arrive(&sm.bias_free[t], lane);  // the loader may bring the next step's tile
        } else if constexpr (BIAS == kBiasDense) {
          if (p.bias_vec && kv_valid == kTileRows && p.bias.dtype != 2) {
            // 16-bit bias, aligned rows, full tile: 32 columns (four 16-byte loads) at a time
            const bool is_half = p.bias.dtype == 0;
            const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.bias.ptr) + bias_row + kv0);
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
              uint4 v[4];
#pragma unroll
              for (int u = 0; u < 4; ++u) v[u] = __ldg(src + ch * 4 + u);
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const uint32_t w4[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 bv = unpack2(w4[e], is_half);
                  const int i = ch * 32 + u * 8 + e * 2;
                  s[i] = fmaf(s[i], c, bv.x * kLog2e);
                  s[i + 1] = fmaf(s[i + 1], c, bv.y * kLog2e);
                }
              }
            }
          } else {
            for_bias_dtype(p.bias.dtype, [&](auto dt) {
              constexpr int kDt = decltype(dt)::value;
#pragma unroll
              for (int i = 0; i < kTileRows; ++i) {
                const float bv = (i < kv_valid) ? load_bias_elem_t<kDt>(p.bias.ptr, bias_row + kv0 + i) : 0.f;
                s[i] = fmaf(s[i], c, bv * kLog2e);
              }
            });
          }
        } else if constexpr (BIAS == kBiasDecomposed64) {
          // Keys kv0 .. kv0+127 are (row 2j, all 64 columns) then (row 2j+1, all 64 columns) of the key grid.
          const bool is_half = p.bias2.dtype == 0;
          // This form keeps the logits in natural units, s * scale + rel_w, one packed FMA per pair of columns: the
          // factor log2(e) rides on the FMA in front of the exponential, and rel_h, constant over each 64-column
          // half, is added to that half's maximum and to that FMA's addend instead of to every column.
          const int jj = j & 3;
          if (jj == 0 && j > ja) {
            rh_cur = rh_nxt;
            if (2 * (j + 4) < p.rel_kh)  // rel_kh is a multiple of 8 in this form: the group is inside the row
              rh_nxt = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.bias.ptr) + bias_row) + (j >> 2) + 1);
          }
          const uint32_t rh_word = jj == 0 ? rh_cur.x : jj == 1 ? rh_cur.y : jj == 2 ? rh_cur.z : rh_cur.w;
          const float2 rh01 = unpack2(rh_word, is_half);
          rh0 = rh01.x;
          rh1 = rh01.y;
          const uint32_t* stage = reinterpret_cast<const uint32_t*>(sm.rel_stage[t][row_in_tile]);
          // The table's type is decided once per step, not once per word.
          auto add_rel64 = [&](auto half_tag) {
            constexpr bool kHalf = decltype(half_tag)::value;
            const float scale_nat = c * 0.6931471805599453f;  // scale_log2 / log2(e)
            const float2 cc = make_float2(scale_nat, scale_nat);
#pragma unroll
            for (int e = 0; e < 32; ++e) {  // one word = rel_w of columns 2e, 2e+1, used by keys 2e.. and 64+2e..
              const float2 rw = unpack2(stage[e], kHalf);
              const int i = 2 * e;
              const float2 lo = ffma2(make_float2(s[i], s[i + 1]), cc, rw);
              const float2 hi = ffma2(make_float2(s[i + 64], s[i + 65]), cc, rw);
              s[i] = lo.x;
              s[i + 1] = lo.y;
              s[i + 64] = hi.x;
              s[i + 65] = hi.y;
            }
          };
          if (is_half) add_rel64(std::true_type{});
          else add_rel64(std::false_type{});
        } else if constexpr (BIAS == kBiasDecomposed14) {
          if (j == 0) add_rel14<0>(s, sm.rel_stage[t][row_in_tile], c);
          else add_rel14<kTileRows>(s, sm.rel_stage[t][row_in_tile], c);
        } else if constexpr (BIAS == kBiasDecomposed) {
          int ih = fast_div(kv0, p.magic_rel_kw);
          int iw = kv0 - ih * p.rel_kw;
          if (p.rel_staged) {
            const float* rh = sm.rel_stage[t][row_in_tile];
            const float* rw = rh + p.rel_kh;
            float bh_val = rh[ih];
#pragma unroll
            for (int i = 0; i < kTileRows; ++i) {
              if (i < kv_valid) s[i] = fmaf(s[i], c, bh_val + rw[iw]);
              if (++iw == p.rel_kw) {
                iw = 0;
                ++ih;
                if (i + 1 < kv_valid) bh_val = rh[ih];
              }
            }
          } else {
            for_bias_dtype(p.bias.dtype, [&](auto dt) {  // rel_h and rel_w are of one type
              constexpr int kDt = decltype(dt)::value;
              float bh_val = load_bias_elem_t<kDt>(p.bias.ptr, bias_row + ih);
#pragma unroll
              for (int i = 0; i < kTileRows; ++i) {
                float bv = 0.f;
                if (i < kv_valid) bv = bh_val + load_bias_elem_t<kDt>(p.bias2.ptr, bias2_row + iw);
                s[i] = fmaf(s[i], c, bv * kLog2e);
                if (++iw == p.rel_kw) {
                  iw = 0;
                  ++ih;
                  if (i + 1 < kv_valid) bh_val = load_bias_elem_t<kDt>(p.bias.ptr, bias_row + ih);
                }
              }
            });
          }
        }
        if (kv_valid < kTileRows) {
          // Short schedule: the ragged tile it is chosen for ends between columns 64 and 96 (197 keys: 69 in the
          // second tile): only those 32 columns need a compare, the last 32 hold no key at all.
          if (SHORT && kv_valid >= 64 && kv_valid <= 96) {
#pragma unroll
            for (int i = 64; i < 96; ++i)
              if (i >= kv_valid) s[i] = -INFINITY;
#pragma unroll
            for (int i = 96; i < kTileRows; ++i) s[i] = -INFINITY;
          } else {
#pragma unroll
            for (int i = 0; i < kTileRows; ++i)
              if (i >= kv_valid) s[i] = -INFINITY;
          }
        }

        float m_tile;
        if constexpr (BIAS == kBiasDecomposed64) {
          // One maximum per 64-column half (two chains each), rel_h added to each, then to base-2 units.
          float a0 = max3(s[0], s[1], s[2]), a1 = max3(s[3], s[4], s[5]);
          float b0 = max3(s[64], s[65], s[66]), b1 = max3(s[67], s[68], s[69]);
#pragma unroll
          for (int i = 6; i + 3 < 64; i += 4) {
            a0 = max3(a0, s[i], s[i + 1]);
            a1 = max3(a1, s[i + 2], s[i + 3]);
            b0 = max3(b0, s[64 + i], s[65 + i]);
            b1 = max3(b1, s[66 + i], s[67 + i]);
          }
          a0 = max3(a0, s[62], s[63]);  // 6 + 4 * 14 = 62: two columns left per half
          b0 = max3(b0, s[126], s[127]);
          m_tile = fmaxf(fmaxf(a0, a1) + rh0, fmaxf(b0, b1) + rh1) * kLog2e;
        } else {
          float mx0 = max3(s[0], s[1], s[2]), mx1 = max3(s[3], s[4], s[5]);
          float mx2 = max3(s[6], s[7], s[8]), mx3 = max3(s[9], s[10], s[11]);
#pragma unroll
          for (int i = 12; i + 7 < kTileRows; i += 8) {
            mx0 = max3(mx0, s[i], s[i + 1]);
            mx1 = max3(mx1, s[i + 2], s[i + 3]);
            mx2 = max3(mx2, s[i + 4], s[i + 5]);
            mx3 = max3(mx3, s[i + 6], s[i + 7]);
          }
          mx0 = max3(mx0, s[124], s[125]);  // 12 + 8 * 14 = 124: four columns left
          mx1 = max3(mx1, s[126], s[127]);
          m_tile = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
          if constexpr (BIAS == kBiasNone) m_tile *= c;
          if constexpr (BIAS == kBiasDenseTiles) m_tile *= kLog2e;  // natural units -> base-2 units
        }

        // Raise the reference maximum only when it pays (or on the first tile).
        const bool raise = m_tile > m_ref + kRescaleThreshold;  // -inf + 8 = -inf: true for any finite first tile
        float alpha = 1.f;
        if (raise) {
          alpha = fast_exp2(m_ref - m_tile);  // m_ref = -inf -> 0
          m_ref = m_tile;
        }
        l_sum *= alpha;
        const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;

        // ---- exponentials ---------------------------------------------------------------------------
        // Both warpgroups feed the MUFU unit, but they must not run in lockstep (their loads and reductions
        // would leave the unit idle together, and equal loops sharing a unit drift into lockstep). So each
        // may only start a section once the other has released it from inside its previous one: warpgroup 0
        // starts step q+1 after warpgroup 1's release in step q, warpgroup 1 starts step q after warpgroup 0's
        // release in step q. The release comes after 96 of the 128 columns (measured against 32, 64, 80, 112 and
        // 128 in the long schedule: 64 was 3 % slower on eleven key tiles, 128 - exclusive sections - 7 %; in the
        // short one 64 against 96: 1 % slower).
        if (need_turn) {
          if constexpr (kFlagTurn) {
            const volatile uint32_t* released = &sm.turn_count[t ^ 1][warp & 3];
            uint32_t polls = 0;
            while (*released < turn_need) {  // bounded: a few seconds of polling at most
              if ((++polls & 0xfff) == 0 && (*abort_flag != 0 || polls > (1u << 26))) {
                bad = true;
                break;
              }
            }
          } else {
            bad |= !mbar_wait_warp_after(turn_early, &sm.turn[t], turn_parity, abort_flag);
          }
        }
        float2 l2a = make_float2(0.f, 0.f), l2b = make_float2(0.f, 0.f);
        const float2 c2 = (BIAS == kBiasNone)           ? make_float2(c, c)
                          : (BIAS == kBiasDecomposed64 || BIAS == kBiasDenseTiles) ? make_float2(kLog2e, kLog2e)
                                                        : make_float2(1.f, 1.f);
        float nm = -m_use;
        uint32_t pk[kTileRows / 2];
        // Release point of the section: let the other warpgroup start (the rest of the section reads `nm` through
        // the arrival, which pins it in the instruction stream) and issue the tests of the barriers needed next.
        auto release_point = [&]() {
          if (pingpong) {
            if constexpr (kFlagTurn) {
              // pinned like the barrier form: `nm` is routed through the store
              asm volatile(
                  "{\n\t"
                  ".reg .pred p;\n\t"
                  "setp.eq.s32 p, %3, 0;\n\t"
                  "@p st.volatile.shared.u32 [%1], %2;\n\t"
                  "}\n"
                  : "+f"(nm)
                  : "r"(smem_u32(&sm.turn_count[t][warp & 3])), "r"(static_cast<uint32_t>(gp + rj + 1)), "r"(lane)
                  : "memory");
            } else {
              warp_arrive_pinned(&sm.turn[t ^ 1], lane, nm);
            }
          }
          // On an item's first tile the P V in question is the last one of the pending item (same barrier, and
          // (step - 1) & 1 is that item's last phase), waited for by its epilogue together with the staging buffer.
          pv_early = (rj > 0 || pend) ? mbar_test_wait(&sm.pv_done[t], (step - 1) & 1) : true;
          stage_early = (rj == 0 && pend && pend_it > 0) ? mbar_test_wait(&sm.o_stage_free[t], (pend_it - 1) & 1) : false;
          s_early = mbar_test_wait(&sm.s_full[t], (step + 1) & 1);  // the next step's S (unused after the last step)
        };
        // Exponentials of 32 * CHUNKS columns from column 32 * FIRST on.
        auto exp_columns = [&](auto first, auto chunks) {
          constexpr int kFirst = decltype(first)::value * 32, kCount = decltype(chunks)::value * 32;
          float nm_half = nm;
          if constexpr (BIAS == kBiasDecomposed64) nm_half = fmaf(kFirst < 64 ? rh0 : rh1, kLog2e, nm);  // a section is one half
          const float2 nm2 = make_float2(nm_half, nm_half);
#pragma unroll
          for (int i = kFirst; i < kFirst + kCount; i += 4) {
            const float2 xa = ffma2(make_float2(s[i], s[i + 1]), c2, nm2);
            const float2 xb = ffma2(make_float2(s[i + 2], s[i + 3]), c2, nm2);
            const float2 pa = make_float2(fast_exp2(xa.x), fast_exp2(xa.y));
            const float2 pb = make_float2(fast_exp2(xb.x), fast_exp2(xb.y));
            l2a = fadd2(l2a, pa);
            l2b = fadd2(l2b, pb);
            pk[i / 2] = pack2<T>(pa.x, pa.y);
            pk[i / 2 + 1] = pack2<T>(pb.x, pb.y);
          }
        };
        using std::integral_constant;
        exp_columns(integral_constant<int, 0>{}, integral_constant<int, 2>{});
        if constexpr (SHORT) {
          // Short-sequence schedule. The last 32 columns of a ragged last key tile that hold no key at all (197 keys:
          // 69 in the second tile) need no exponentials: their logits are -inf and their P is never read (P V stops
          // at the last key's k-step). One CTA-uniform branch: -6 % on [256,12,197,64]. With eleven key tiles
          // the branch is taken once in eleven steps and its effect on the step's schedule costs more than it
          // saves (+4 % on [32,24,1370,64] bf16), hence a schedule of its own.
          exp_columns(integral_constant<int, 2>{}, integral_constant<int, 1>{});
          release_point();
          if (kv_valid > 96) {
            exp_columns(integral_constant<int, 3>{}, integral_constant<int, 1>{});
          } else {
#pragma unroll
            for (int i = 48; i < 64; ++i) pk[i] = 0u;
          }
        } else {
          exp_columns(integral_constant<int, 2>{}, integral_constant<int, 1>{});
          release_point();
          exp_columns(integral_constant<int, 3>{}, integral_constant<int, 1>{});
        }
        l_sum += (l2a.x + l2a.y) + (l2b.x + l2b.y);

        // P_t and O_t may only change once P_t(j-1) V has finished: it was issued when this warpgroup
        // delivered P_t(j-1), a whole exponential section ago. On the first tile of an item the P V in
        // question is the last one of the previous item, and this is where that item's output is written:
        // its epilogue hides behind this item's first exponentials instead of stalling the pipeline.
        if (rj == 0) {
          if (pend) {
            ok = finish_item(pv_early, stage_early, std::false_type{});
            if (!ok) break;
          }
        } else {
          bad |= !mbar_wait_warp_after(pv_early, &sm.pv_done[t], (step - 1) & 1, abort_flag);
          tc_fence_after_sync();
          if (__any_sync(0xffffffffu, raise)) {
            float o[kHeadDim];
            uint32_t* ou = reinterpret_cast<uint32_t*>(o);
            tmem_ld_x64(o_addr, ou);
#pragma unroll
            for (int i = 0; i < kHeadDim; ++i) o[i] *= alpha;
            tmem_st_x32(o_addr, ou);
            tmem_st_x32(o_addr + 32, ou + 32);
          }
        }
        tmem_st_x64(p_addr, pk);
        tmem_st_wait();
        tc_fence_before_sync();
        warp_arrive(&sm.p_full[t], lane);
      }
      if (!ok) break;
      if (__any_sync(0xffffffffu, bad)) {
        ok = false;
        break;
      }

      // The item's output is written later (see above); remember what its epilogue needs.
      pend = true;
      pend_phase = (g + (jb - ja) - 1) & 1;
      pend_l = l_sum;
      if constexpr (SPLIT) pend_m_of_split = m_ref;
      pend_it = it;
      g += jb - ja;
      if (w.n_tiles == 2) gp += jb - ja;
    }
    if (ok && pend) ok = finish_item(false, false, std::true_type{});
    if (!ok && lane == 0) {
      if (atomicExch(const_cast<uint32_t*>(abort_flag), 1u) == 0) atomicOr(p.status, kStatusSoftmax);
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
