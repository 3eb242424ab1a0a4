// C ABI of libb200attn.so: argument checks, TMA descriptor construction and kernel launches.
// Declarations and the reference interfaces they replace are in include/b200_attn.h.
#include "../../include/b200_attn.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <type_traits>

#include "attn_fwd_sm100.cuh"
#include "gemm_sm100.cuh"
#include "rope_sm100.cuh"
#include "sam_rel_terms.cuh"

namespace {

using namespace b200;

// Role bits of waits that gave up; one word per device that loaded the library.
__device__ uint32_t g_status_word;

// A wait that can never be satisfied, with a caller-chosen limit: exercises the path every kernel wait takes when
// it gives up (error bit in the status word, normal return) without faulting, trapping or hanging anything.
__global__ void wait_limit_selftest_kernel(uint64_t limit_ns, uint32_t* status) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);  // nobody ever arrives
    mbar_init_fence();
  }
  __syncthreads();
  const uint64_t t0 = global_timer_ns();
  bool done = false;
  while (!done && global_timer_ns() - t0 <= limit_ns) done = mbar_try_wait(&bar, 0);
  if (!done && threadIdx.x == 0) atomicOr(status, 8u);
}

// ceil(2^64 / d) for the kernel's fast_div; 0 stands for d <= 1.
uint64_t div_magic(int d) { return d <= 1 ? 0 : ~uint64_t(0) / static_cast<uint64_t>(d) + 1; }

thread_local char tl_error[512] = "";


int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tl_error, sizeof(tl_error), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  return fail(B200_ATTN_CUDA_ERROR_BASE + static_cast<int>(e), "%s: %s", what, cudaGetErrorString(e));
}

// cuTensorMapEncodeTiled, fetched through the runtime so that the library needs no link-time libcuda.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      sym = nullptr;
    return reinterpret_cast<EncodeTiledFn>(sym);
  }();
  return fn;
}

// A [batch, tokens, heads, 64] view with arbitrary (16-byte multiple) strides as a 4-D tensor map whose
// box is one 128-row x 64-column tile of one head, written to shared memory with the 128-byte swizzle.
int make_tile_map(CUtensorMap* map, const void* base, uint32_t dtype, int batch, int heads, int tokens,
                  const int64_t stride[3], const char* name) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return fail(B200_ATTN_CUDA_ERROR_BASE, "cuTensorMapEncodeTiled is not available from this driver");
  // A dimension of extent 1 is only ever addressed at coordinate 0: any legal stride will do.
  const int64_t sb = batch > 1 ? stride[0] : kHeadDim;
  const int64_t sn = tokens > 1 ? stride[1] : kHeadDim;
  const int64_t sh = heads > 1 ? stride[2] : kHeadDim;
  cuuint64_t dims[4] = {kHeadDim, static_cast<cuuint64_t>(tokens), static_cast<cuuint64_t>(heads),
                        static_cast<cuuint64_t>(batch)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(sn) * 2, static_cast<cuuint64_t>(sh) * 2,
                           static_cast<cuuint64_t>(sb) * 2};
  cuuint32_t box[4] = {kHeadDim, kTileRows, 1, 1};
  cuuint32_t elem[4] = {1, 1, 1, 1};
  CUresult r = enc(map, dtype == B200_ATTN_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                   const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(B200_ATTN_UNSUPPORTED, "tensor map for %s rejected by the driver (CUresult %d)", name, static_cast<int>(r));
  return B200_ATTN_OK;
}

// Tensor maps made before, per thread: a model calls the operator with the same views (and, through torch's
// caching allocator, the same addresses) in every block and every forward, and for launch-bound shapes (one image of
// 197 tokens) four calls of the driver's encoder cost more host time than the rest of the launch. A map depends on
// nothing but the key, so a hit is exact; the oldest entry of a slot's set goes on a miss.
struct TileMapKey {
  const void* base;
  int64_t stride[3];
  int batch, heads, tokens;
  uint32_t dtype;
  bool operator==(const TileMapKey& o) const {
    return base == o.base && stride[0] == o.stride[0] && stride[1] == o.stride[1] && stride[2] == o.stride[2] && batch == o.batch &&
           heads == o.heads && tokens == o.tokens && dtype == o.dtype;
  }
};
constexpr int kTileMapSets = 256, kTileMapWays = 2;  // 512 maps, 95 KB per thread: a 24-block encoder uses about a hundred
struct TileMapCache {
  TileMapKey key[kTileMapSets][kTileMapWays];
  CUtensorMap map[kTileMapSets][kTileMapWays];
  bool used[kTileMapSets][kTileMapWays];
  uint8_t next[kTileMapSets];
};
thread_local TileMapCache tl_tile_maps{};

int cached_tile_map(CUtensorMap* map, const void* base, uint32_t dtype, int batch, int heads, int tokens, const int64_t stride[3],
                    const char* name) {
  const TileMapKey key{base, {stride[0], stride[1], stride[2]}, batch, heads, tokens, dtype};
  const size_t h = (reinterpret_cast<uintptr_t>(base) >> 7) * 0x9E3779B97F4A7C15ull >> 56;  // 8 bits
  TileMapCache& c = tl_tile_maps;
  for (int w = 0; w < kTileMapWays; ++w)
    if (c.used[h][w] && c.key[h][w] == key) {
      *map = c.map[h][w];
      return B200_ATTN_OK;
    }
  if (const int rc = make_tile_map(map, base, dtype, batch, heads, tokens, stride, name)) return rc;
  const int w = c.next[h];
  c.next[h] = static_cast<uint8_t>((w + 1) % kTileMapWays);
  c.key[h][w] = key;
  c.map[h][w] = *map;
  c.used[h][w] = true;
  return B200_ATTN_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int check_view(const char* name, const void* ptr, const int64_t s[3], int batch, int heads, int tokens) {
  if (ptr == nullptr) return fail(B200_ATTN_BAD_CONFIG, "%s is NULL", name);
  if (!aligned16(ptr)) return fail(B200_ATTN_UNSUPPORTED, "%s is not 16-byte aligned", name);
  const int ext[3] = {batch, tokens, heads};
  const char* dim[3] = {"batch", "token", "head"};
  for (int i = 0; i < 3; ++i) {
    if (ext[i] <= 1) continue;
    if (s[i] <= 0 || s[i] % 8 != 0)
      return fail(B200_ATTN_UNSUPPORTED, "%s %s stride %lld must be a positive multiple of 8 elements", name, dim[i],
                  static_cast<long long>(s[i]));
    if (s[i] >= (int64_t(1) << 38))
      return fail(B200_ATTN_UNSUPPORTED, "%s %s stride %lld is too large for a tensor map", name, dim[i],
                  static_cast<long long>(s[i]));
  }
  return B200_ATTN_OK;
}

// A dense bias that the kernel can fetch tile by tile through TMA like K and V: 16-bit, 16-byte aligned base, every
// stride that is used (the stride of a dimension of extent 1 never is) a non-negative multiple of 8 elements that a
// tensor map can hold, rows at a positive stride.
bool dense_bias_in_tiles(const B200AttnArgs* a) {
  if (a->bias == nullptr || a->bias_dtype == B200_ATTN_F32 || !aligned16(a->bias)) return false;
  const int64_t tb = a->batch > 1 ? a->bias_stride[0] : 0, th = a->heads > 1 ? a->bias_stride[1] : 0;
  const int64_t tn = a->q_tokens > 1 ? a->bias_stride[2] : 8;
  const int64_t limit = int64_t(1) << 38;
  return tn > 0 && tn % 8 == 0 && tb >= 0 && tb % 8 == 0 && th >= 0 && th % 8 == 0 && tn < limit && tb < limit && th < limit;
}
// ... and that every image shares: the items are then numbered batch-fastest (decode_item).
bool bias_shared_by_the_batch(const B200AttnArgs* a) {
  return dense_bias_in_tiles(a) && a->batch > 1 && a->bias_stride[0] == 0;
}

int bias_elem_size(uint32_t dtype) { return dtype == B200_ATTN_F32 ? 4 : 2; }

// The argument checks shared by b200_attn_fwd and b200_attn_query. Sets *bias_mode and *schedule.
int validate(const B200AttnArgs* a, int* bias_mode, int* schedule) {
  if (a == nullptr) return fail(B200_ATTN_BAD_CONFIG, "args is NULL");
  if (a->struct_size != sizeof(B200AttnArgs))
    return fail(B200_ATTN_BAD_CONFIG, "struct_size %u does not match this library's B200AttnArgs (%zu bytes)",
                a->struct_size, sizeof(B200AttnArgs));
  if (a->dtype != B200_ATTN_F16 && a->dtype != B200_ATTN_BF16)
    return fail(B200_ATTN_BAD_CONFIG, "dtype %u: q, k, v, o must be fp16 (0) or bf16 (1)", a->dtype);
  if (a->head_dim != kHeadDim)
    return fail(B200_ATTN_UNSUPPORTED, "head_dim %d: only head dim 64 is built", a->head_dim);
  if (a->batch < 1 || a->heads < 1 || a->q_tokens < 1 || a->kv_tokens < 1)
    return fail(B200_ATTN_UNSUPPORTED, "empty problem: batch %d heads %d q_tokens %d kv_tokens %d", a->batch, a->heads,
                a->q_tokens, a->kv_tokens);
  if (!(a->scale > 0.f) || !std::isfinite(a->scale))
    return fail(B200_ATTN_UNSUPPORTED, "scale %g must be finite and positive", static_cast<double>(a->scale));
  int rc;
  if ((rc = check_view("q", a->q, a->q_stride, a->batch, a->heads, a->q_tokens))) return rc;
  if ((rc = check_view("k", a->k, a->k_stride, a->batch, a->heads, a->kv_tokens))) return rc;
  if ((rc = check_view("v", a->v, a->v_stride, a->batch, a->heads, a->kv_tokens))) return rc;
  if ((rc = check_view("o", a->o, a->o_stride, a->batch, a->heads, a->q_tokens))) return rc;
  const int64_t items = (static_cast<int64_t>(a->q_tokens) + 2 * kTileRows - 1) / (2 * kTileRows);
  if (items * a->batch * a->heads > 0x7fffffffLL)
    return fail(B200_ATTN_UNSUPPORTED, "problem too large for one launch (%lld CTAs)",
                static_cast<long long>(items * a->batch * a->heads));

  *bias_mode = kBiasNone;
  const bool has_rel = a->rel_h != nullptr || a->rel_w != nullptr;
  if (a->bias != nullptr && has_rel)
    return fail(B200_ATTN_BAD_CONFIG, "bias and rel_h / rel_w are mutually exclusive");
  if (a->bias != nullptr) {
    if (a->bias_dtype > B200_ATTN_F32) return fail(B200_ATTN_BAD_CONFIG, "bias_dtype %u unknown", a->bias_dtype);
    if (reinterpret_cast<uintptr_t>(a->bias) % bias_elem_size(a->bias_dtype) != 0)
      return fail(B200_ATTN_UNSUPPORTED, "bias pointer is not aligned to its element size");
    for (int i = 0; i < 3; ++i)
      if (a->bias_stride[i] < 0) return fail(B200_ATTN_UNSUPPORTED, "bias strides must be non-negative");
    *bias_mode = kBiasDense;
  } else if (has_rel) {
    if (a->rel_h == nullptr || a->rel_w == nullptr)
      return fail(B200_ATTN_BAD_CONFIG, "rel_h and rel_w must be given together");
    if (a->rel_dtype > B200_ATTN_F32) return fail(B200_ATTN_BAD_CONFIG, "rel_dtype %u unknown", a->rel_dtype);
    if (a->rel_kh < 1 || a->rel_kw < 1 || static_cast<int64_t>(a->rel_kh) * a->rel_kw != a->kv_tokens)
      return fail(B200_ATTN_UNSUPPORTED, "rel_kh * rel_kw (%d * %d) must equal kv_tokens %d", a->rel_kh, a->rel_kw,
                  a->kv_tokens);
    const int es = bias_elem_size(a->rel_dtype);
    if (reinterpret_cast<uintptr_t>(a->rel_h) % es != 0 || reinterpret_cast<uintptr_t>(a->rel_w) % es != 0)
      return fail(B200_ATTN_UNSUPPORTED, "rel_h / rel_w pointers are not aligned to their element size");
    for (int i = 0; i < 3; ++i)
      if (a->rel_h_stride[i] < 0 || a->rel_w_stride[i] < 0)
        return fail(B200_ATTN_UNSUPPORTED, "rel_h / rel_w strides must be non-negative");
    *bias_mode = kBiasDecomposed;
  }

  if (a->workspace != nullptr && (reinterpret_cast<uintptr_t>(a->workspace) & 255) != 0)
    return fail(B200_ATTN_UNSUPPORTED, "workspace is not 256-byte aligned");
  if (a->workspace_bytes < 0 || (a->workspace == nullptr && a->workspace_bytes != 0))
    return fail(B200_ATTN_BAD_CONFIG, "workspace_bytes %lld without a workspace", static_cast<long long>(a->workspace_bytes));
  if (a->schedule < B200_ATTN_SCHED_AUTO || a->schedule > B200_ATTN_SCHED_SHORT)
    return fail(B200_ATTN_BAD_CONFIG, "schedule %d unknown", a->schedule);
  if (a->test_flags != 0 && a->test_flags != 1) return fail(B200_ATTN_BAD_CONFIG, "test_flags %d unknown", a->test_flags);
  // Short schedule: at most two key tiles and a last one whose final 32 columns hold no key (its exponentials are skipped).
  const int kv_tiles = (a->kv_tokens + kTileRows - 1) / kTileRows;
  const int kv_last = a->kv_tokens - (kv_tiles - 1) * kTileRows;
  const bool short_pays = kv_tiles <= 2 && kv_last <= kTileRows - 32;
  *schedule = a->schedule != B200_ATTN_SCHED_AUTO ? a->schedule : short_pays ? B200_ATTN_SCHED_SHORT : B200_ATTN_SCHED_LONG;
  tl_error[0] = '\0';
  return B200_ATTN_OK;
}

// What a launch needs to know about the current device, looked up once per device: the SM count, the address of the
// status word and which kernels already have their shared-memory opt-in (the opt-in is per device and per kernel).
// The runtime calls behind these cost more than the rest of the host path of a launch-bound call.
constexpr int kMaxDevices = 64;
constexpr int kKernelForms = 36;  // 2 dtypes x 6 bias forms x (short, long, long with key split)
struct DeviceState {
  std::atomic<bool> ready{false};
  int sms = 0;
  uint32_t* status = nullptr;
  std::atomic<bool> opted_in[kKernelForms];
  std::atomic<bool> gemm_opted_in[6];  // 2 dtypes x 3 tile shapes
};
DeviceState g_devices[kMaxDevices];
std::mutex g_devices_mutex;

int device_state(DeviceState** out) {
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (device < 0 || device >= kMaxDevices)
    return fail(B200_ATTN_UNSUPPORTED, "device ordinal %d: at most %d devices are supported", device, kMaxDevices);
  DeviceState& d = g_devices[device];
  if (!d.ready.load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> lock(g_devices_mutex);
    if (!d.ready.load(std::memory_order_relaxed)) {
      e = cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, device);
      if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute(multiprocessor count)");
      e = cudaGetSymbolAddress(reinterpret_cast<void**>(&d.status), g_status_word);
      if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(status word)");
      for (auto& f : d.opted_in) f.store(false, std::memory_order_relaxed);
      for (auto& f : d.gemm_opted_in) f.store(false, std::memory_order_relaxed);
      d.ready.store(true, std::memory_order_release);
    }
  }
  *out = &d;
  return B200_ATTN_OK;
}

// Cost of a one-tile item in units of a two-tile item of the same head. Measured in CUDA graphs: a key-tile step of a
// lone softmax warpgroup takes 0.79 of a step of two interleaved ones, and either kind of item pays about three
// quarters of a step for its epilogue and hand-over: 0.85 for items of two key tiles, 0.80 for eleven.
double dealt_single_cost(int kv_tiles) { return (0.79 * kv_tiles + 0.75) / (kv_tiles + 0.75); }

// Split the query tiles of every (batch, head) into two-tile and one-tile items and deal them to the CTAs so that
// the most loaded CTA finishes as early as possible. Candidates: every count of two-tile items per head from
// q_tiles / 2 down; for each, the two-tile items go to the CTAs in consecutive runs of k or k + 1 and the one-tile
// items fill up the less loaded CTAs first. Fills the split fields of `prm` and returns the grid size.
unsigned plan_split(AttnParams& prm, long long heads_total, int sms, double* span_out) {
  const int tiles = prm.q_tiles;
  const double kDealtSingleCost = dealt_single_cost(prm.kv_tiles);
  double best_span = 0;
  int best_pairs = -1;
  struct Plan {
    int grid, na, ka, kb, a, ea, b, eb, conv;
  } best{}, cur{};
  const int first = tiles / 2, last = tiles / 2 - 8;
  for (int pairs = first; pairs >= 0 && pairs >= last; --pairs) {
    const long long P = pairs * heads_total, S = (tiles - 2LL * pairs) * heads_total;
    const long long grid = P + S < sms ? P + S : sms;
    cur.grid = static_cast<int>(grid);
    cur.na = static_cast<int>(P % grid);
    cur.kb = static_cast<int>(P / grid);
    cur.ka = cur.kb + 1;
    if (cur.na == 0) cur.ka = cur.kb;  // no CTA of the first kind
    // Level the loads with the one-tile items: group A (na CTAs, ka two-tile items), group B (the rest, kb).
    const long long nb = grid - cur.na;
    long long a = 0, b = 0, ea = 0, eb = 0, left = S;
    while (left > 0) {
      const double level_a = cur.na > 0 ? cur.ka + kDealtSingleCost * a : 1e300;
      const double level_b = nb > 0 ? cur.kb + kDealtSingleCost * b : 1e300;
      if (level_b <= level_a) {
        if (left >= nb) { ++b; left -= nb; } else { eb = left; left = 0; }
      } else {
        if (left >= cur.na) { ++a; left -= cur.na; } else { ea = left; left = 0; }
      }
    }
    cur.a = static_cast<int>(a); cur.ea = static_cast<int>(ea); cur.b = static_cast<int>(b); cur.eb = static_cast<int>(eb);
    double span = 0;
    if (cur.na > 0) span = std::fmax(span, cur.ka + kDealtSingleCost * (a + (ea > 0 ? 1 : 0)));
    if (nb > 0) span = std::fmax(span, cur.kb + kDealtSingleCost * (b + (eb > 0 ? 1 : 0)));
    cur.conv = 0;
    if (best_pairs < 0 || span < best_span - 1e-9) {
      best_span = span;
      best_pairs = pairs;
      best = cur;
    }
    // The same count of two-tile items per head, but the na items of the last, partial round taken apart into 2 na
    // one-tile items: every CTA then has kb two-tile items and the one-tile items level the rest. It pays when that
    // round is thin (300 items on 148 CTAs: 4 of them would run a third item while 144 wait) and the lists are short
    // (measured: -6 % at two items per CTA, -3 % at four, nothing at eight: taken from 3 % of predicted gain on).
    if (cur.na > 0 && cur.kb > 0) {
      const long long singles = S + 2LL * cur.na;
      Plan alt = cur;
      alt.conv = cur.na;
      alt.na = 0;
      alt.ka = cur.kb;
      alt.a = alt.ea = 0;
      alt.b = static_cast<int>(singles / grid);
      alt.eb = static_cast<int>(singles % grid);
      const double alt_span = cur.kb + kDealtSingleCost * (alt.b + (alt.eb > 0 ? 1 : 0));
      if (alt_span < 0.97 * span && alt_span < best_span - 1e-9) {
        best_span = alt_span;
        best_pairs = pairs;
        best = alt;
      }
    }
  }
  prm.pairs_per_head = best_pairs;
  prm.singles_per_head = tiles - 2 * best_pairs;
  prm.split_na = best.na; prm.split_ka = best.ka; prm.split_kb = best.kb;
  prm.split_a = best.a; prm.split_ea = best.ea; prm.split_b = best.b; prm.split_eb = best.eb;
  prm.conv_pairs = best.conv;
  prm.kept_pairs = static_cast<int>(best_pairs * heads_total) - best.conv;
  prm.magic_pairs = div_magic(prm.pairs_per_head);
  prm.magic_singles = div_magic(prm.singles_per_head);
  *span_out = best_span;
  return static_cast<unsigned>(best.grid);
}

// Bytes of workspace per CTA of a key-split launch (partial results), and where the items' counters begin.
constexpr size_t kPartialBytes = 4 * static_cast<size_t>(kPartialFloats) * sizeof(float);  // first / last item x two query tiles
size_t workspace_flags_offset(int sms) { return static_cast<size_t>(sms) * kPartialBytes; }
size_t workspace_bytes_for(int sms) { return (workspace_flags_offset(sms) + static_cast<size_t>(sms) * 2 * sizeof(uint32_t) + 255) & ~size_t(255); }

// Key-split plan (the kernel's cta_work has the other half): all key-tile steps in one line, cut into one run per
// CTA by cost. Worth it only where whole items level badly: `dealt_span` is the longest list of the dealt plan in
// two-tile items. Both plans are compared in key-tile steps of a two-tile item, with what was measured on B200
// ([4,16,1370,64]: 63 -> 61 us, [1,12,4096,64]: 108 -> 88 us, [2,16,1370,64]: 41 -> 36 us; [8,6,1370,64], whose
// dealt plan is within 7 % of level, 45 -> 50 us): a step of the key-split kernel takes 6 % longer, a run costs
// about two steps for its merges on top of half a step for every item it starts, and runs of fewer than eight
// steps are all set-up and merge (the grid shrinks rather than cut finer).
// Returns the grid size, or 0 when the dealt plan stays.
constexpr int kMinRunSteps = 8;
constexpr double kSplitStepFactor = 1.06, kSplitMergeSteps = 2.0;
unsigned plan_chunks(AttnParams& prm, const B200AttnArgs* a, long long heads_total, int sms, double dealt_span) {
  if (a->workspace == nullptr || prm.kv_tiles < 3) return 0;
  if (static_cast<size_t>(a->workspace_bytes) < workspace_bytes_for(sms)) return 0;
  const long long pairs = (prm.q_tiles / 2) * heads_total, singles = (prm.q_tiles % 2) * heads_total;
  if ((pairs + singles) * prm.kv_tiles > 0x3fffffffLL) return 0;  // steps are counted in 32 bits
  const long long cost = prm.kv_tiles * (pairs * kPairCost + singles * b200::kSingleCost);
  const long long grid = std::min<long long>(sms, std::max<long long>(1, cost / (kMinRunSteps * kPairCost)));
  const double items_dealt = std::ceil(dealt_span);
  const double dealt = dealt_span * prm.kv_tiles + 0.5 * items_dealt;
  const double run = static_cast<double>(cost) / kPairCost / static_cast<double>(grid);
  const double chunked = kSplitStepFactor * run + 0.5 * (run / prm.kv_tiles + 1.0) + kSplitMergeSteps;
  if (chunked > 0.97 * dealt) return 0;
  prm.chunked = 1;
  prm.pairs_per_head = prm.q_tiles / 2;
  prm.singles_per_head = prm.q_tiles % 2;
  prm.magic_pairs = div_magic(prm.pairs_per_head);
  prm.magic_singles = div_magic(prm.singles_per_head);
  prm.pair_items = static_cast<int>(pairs);
  prm.single_items = static_cast<int>(singles);
  prm.cost_total = cost;
  prm.cost_base = cost / grid;
  prm.cost_rem = static_cast<int>(cost % grid);
  prm.magic_kv_tiles = div_magic(prm.kv_tiles);
  prm.test_flags = a->test_flags;
  prm.ws_partial = static_cast<float*>(a->workspace);
  prm.ws_counts = reinterpret_cast<uint32_t*>(static_cast<char*>(a->workspace) + workspace_flags_offset(sms));
  return static_cast<unsigned>(grid);
}

// Scratch memory of b200_attn_fwd_static: a workspace for devices of up to kStaticMaxSms SMs (a B200 has 148) that
// lives in the module itself, 21.6 MB on every GPU that loads the library, until the process ends.
constexpr int kStaticMaxSms = 160;
constexpr size_t kStaticWorkspaceBytes =
    (static_cast<size_t>(kStaticMaxSms) * kPartialBytes + static_cast<size_t>(kStaticMaxSms) * 2 * sizeof(uint32_t) + 255) & ~size_t(255);
static __device__ __align__(256) unsigned char g_static_workspace[kStaticWorkspaceBytes];
struct StaticScratch {
  std::atomic<bool> ready{false};
  void* ptr = nullptr;  // device address of g_static_workspace on this device
};
StaticScratch g_static_scratch[kMaxDevices];

// The work plan of a call on a device with `sms` SMs: fills the plan fields of `prm`, returns the grid size.
unsigned plan_work(AttnParams& prm, const B200AttnArgs* a, int sms) {
  const long long heads_total = static_cast<long long>(a->batch) * a->heads;
  double dealt_span = 0;
  unsigned grid = plan_split(prm, heads_total, sms, &dealt_span);
  if (const unsigned chunk_grid = plan_chunks(prm, a, heads_total, sms, dealt_span)) grid = chunk_grid;
  return grid;
}

template <typename T, int BIAS, bool SHORT, bool SPLIT>
int launch(const AttnParams& planned, unsigned grid, DeviceState& dev, const CUtensorMap& mq, const CUtensorMap& mk,
           const CUtensorMap& mv, const CUtensorMap& mo, const CUtensorMap& mb, cudaStream_t stream) {
  auto kernel = attn_fwd_kernel<T, BIAS, SHORT, SPLIT>;
  constexpr int smem = static_cast<int>(BIAS == kBiasDenseTiles ? sizeof(AttnSmemDense) : sizeof(AttnSmem)) + 1024;
  constexpr int form = (BIAS * 2 + (std::is_same<T, __half>::value ? 0 : 1)) * 3 + (SHORT ? 1 : SPLIT ? 2 : 0);
  static_assert(form < kKernelForms, "kernel form index");
  if (!dev.opted_in[form].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(shared memory)");
    dev.opted_in[form].store(true, std::memory_order_release);
  }
  // Persistent CTAs: one per SM (shared memory and tensor memory allow no more), fewer when there is less work.
  // Programmatic stream serialisation: the CTAs of this grid may be scheduled while the previous kernel of the stream
  // drains; the kernel waits for that kernel's completion itself (grid_dependency_wait) before it touches global
  // memory, so its set-up (barriers, tensor memory, descriptor prefetch) and the launch latency hide behind the
  // predecessor's tail.
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(grid);
  config.blockDim = dim3(kThreads);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&config, kernel, mq, mk, mv, mo, mb, planned);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "attention kernel launch");
  return B200_ATTN_OK;
}

// The short schedule exists for every bias form but the 64-wide one (its key counts are multiples of 64, where the
// long schedule loses nothing worth a second set of kernels); the key-split form only for the long schedule (a
// sequence of at most two key tiles is never split).
template <typename T, int BIAS>
int launch_sched(bool short_sched, const AttnParams& planned, unsigned grid, DeviceState& dev, const CUtensorMap& mq,
                 const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo, const CUtensorMap& mb, cudaStream_t stream) {
  if (planned.chunked) return launch<T, BIAS, false, true>(planned, grid, dev, mq, mk, mv, mo, mb, stream);
  if constexpr (BIAS != kBiasDecomposed64) {
    if (short_sched) return launch<T, BIAS, true, false>(planned, grid, dev, mq, mk, mv, mo, mb, stream);
  }
  return launch<T, BIAS, false, false>(planned, grid, dev, mq, mk, mv, mo, mb, stream);
}

// The dense bias [B | 1, H | 1, Nq, Nk] (a stride of 0 broadcasts that dimension) as a 4-D tensor map whose box is
// 128 rows x 64 columns with the 128-byte swizzle; a broadcast dimension gets extent 1 and the kernel addresses it at 0.
int make_bias_map(CUtensorMap* map, const B200AttnArgs* a) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return fail(B200_ATTN_CUDA_ERROR_BASE, "cuTensorMapEncodeTiled is not available from this driver");
  const int64_t sb = a->batch > 1 ? a->bias_stride[0] : 0, sh = a->heads > 1 ? a->bias_stride[1] : 0, sn = a->bias_stride[2];
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(a->kv_tokens), static_cast<cuuint64_t>(a->q_tokens),
                        static_cast<cuuint64_t>(sh != 0 ? a->heads : 1), static_cast<cuuint64_t>(sb != 0 ? a->batch : 1)};
  // a dimension of extent 1 is only ever addressed at 0: any legal stride will do
  const int64_t row = a->q_tokens > 1 ? sn : a->kv_tokens + (8 - a->kv_tokens % 8) % 8;
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(row) * 2, static_cast<cuuint64_t>(dims[2] > 1 ? sh : row) * 2,
                           static_cast<cuuint64_t>(dims[3] > 1 ? sb : row) * 2};
  cuuint32_t box[4] = {64, kTileRows, 1, 1};
  cuuint32_t elem[4] = {1, 1, 1, 1};
  const CUresult r = enc(map, a->bias_dtype == B200_ATTN_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                         const_cast<void*>(a->bias), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(B200_ATTN_UNSUPPORTED, "tensor map for the bias rejected by the driver (CUresult %d)", static_cast<int>(r));
  return B200_ATTN_OK;
}

// The bias maps a thread made last, like the tile maps of q, k, v and o: a model passes the same few bias tensors
// call after call (one per block or per window shift).
struct BiasMapKey {
  const void* base;
  int64_t stride[3];
  int batch, heads, q_tokens, kv_tokens;
  uint32_t dtype;
  bool operator==(const BiasMapKey& o) const {
    return base == o.base && stride[0] == o.stride[0] && stride[1] == o.stride[1] && stride[2] == o.stride[2] &&
           batch == o.batch && heads == o.heads && q_tokens == o.q_tokens && kv_tokens == o.kv_tokens && dtype == o.dtype;
  }
};
constexpr int kBiasMapSlots = 16;
struct BiasMapCache {
  BiasMapKey key[kBiasMapSlots];
  CUtensorMap map[kBiasMapSlots];
  bool used[kBiasMapSlots];
};
thread_local BiasMapCache tl_bias_maps{};

int cached_bias_map(CUtensorMap* map, const B200AttnArgs* a) {
  const BiasMapKey key{a->bias, {a->bias_stride[0], a->bias_stride[1], a->bias_stride[2]}, a->batch, a->heads,
                       a->q_tokens, a->kv_tokens, a->bias_dtype};
  const size_t slot = (reinterpret_cast<uintptr_t>(a->bias) >> 8) * 0x9E3779B97F4A7C15ull >> 60;  // 4 bits
  BiasMapCache& c = tl_bias_maps;
  if (c.used[slot] && c.key[slot] == key) {
    *map = c.map[slot];
    return B200_ATTN_OK;
  }
  if (const int rc = make_bias_map(map, a)) return rc;
  c.key[slot] = key;
  c.map[slot] = *map;
  c.used[slot] = true;
  return B200_ATTN_OK;
}

}  // namespace

extern "C" {

int b200_attn_query(const B200AttnArgs* args, int32_t* schedule) {
  int bias_mode = 0, sched = 0;
  const int rc = validate(args, &bias_mode, &sched);
  if (rc == B200_ATTN_OK && schedule != nullptr) *schedule = sched;
  return rc;
}

int b200_attn_fwd(const B200AttnArgs* a, void* stream_ptr) {
  int bias_mode = 0, sched = 0;
  int rc = validate(a, &bias_mode, &sched);
  if (rc != B200_ATTN_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);

  CUtensorMap mq, mk, mv, mo;
  if ((rc = cached_tile_map(&mq, a->q, a->dtype, a->batch, a->heads, a->q_tokens, a->q_stride, "q"))) return rc;
  if ((rc = cached_tile_map(&mk, a->k, a->dtype, a->batch, a->heads, a->kv_tokens, a->k_stride, "k"))) return rc;
  if ((rc = cached_tile_map(&mv, a->v, a->dtype, a->batch, a->heads, a->kv_tokens, a->v_stride, "v"))) return rc;
  if ((rc = cached_tile_map(&mo, a->o, a->dtype, a->batch, a->heads, a->q_tokens, a->o_stride, "o"))) return rc;

  AttnParams prm;
  std::memset(&prm, 0, sizeof(prm));
  prm.batch = a->batch;
  prm.heads = a->heads;
  prm.q_tokens = a->q_tokens;
  prm.kv_tokens = a->kv_tokens;
  prm.q_tiles = (a->q_tokens + kTileRows - 1) / kTileRows;
  prm.kv_tiles = (a->kv_tokens + kTileRows - 1) / kTileRows;
  prm.scale_log2 = a->scale * kLog2e;
  prm.magic_heads = div_magic(a->heads);
  prm.o = a->o;
  prm.o_sb = a->o_stride[0];
  prm.o_sn = a->o_stride[1];
  prm.o_sh = a->o_stride[2];
  if (bias_mode == kBiasDense) {
    prm.bias = BiasView{a->bias, a->bias_stride[0], a->bias_stride[1], a->bias_stride[2],
                        static_cast<int>(a->bias_dtype)};
    // Vector loads need every row segment that starts at a multiple of 128 columns to be 16-byte aligned.
    prm.bias_vec = aligned16(a->bias) && a->bias_stride[0] % 8 == 0 && a->bias_stride[1] % 8 == 0 &&
                   a->bias_stride[2] % 8 == 0;
    if (dense_bias_in_tiles(a)) bias_mode = kBiasDenseTiles;
  } else if (bias_mode == kBiasDecomposed) {
    prm.bias = BiasView{a->rel_h, a->rel_h_stride[0], a->rel_h_stride[1], a->rel_h_stride[2],
                        static_cast<int>(a->rel_dtype)};
    prm.bias2 = BiasView{a->rel_w, a->rel_w_stride[0], a->rel_w_stride[1], a->rel_w_stride[2],
                         static_cast<int>(a->rel_dtype)};
    prm.rel_kh = a->rel_kh;
    prm.rel_kw = a->rel_kw;
    prm.magic_rel_kw = div_magic(a->rel_kw);
    prm.rel_staged = a->rel_kh + a->rel_kw <= kRelStageWords - 1;
    // The 64-wide form reads both tables with 16-byte loads: aligned rows, and rel_h in whole groups of eight.
    const auto rows16 = [](const void* ptr, const int64_t s[3]) {
      return aligned16(ptr) && s[0] % 8 == 0 && s[1] % 8 == 0 && s[2] % 8 == 0;
    };
    if (a->rel_kw == 64 && a->rel_kh % 8 == 0 && a->rel_dtype != B200_ATTN_F32 && rows16(a->rel_w, a->rel_w_stride) &&
        rows16(a->rel_h, a->rel_h_stride))
      bias_mode = kBiasDecomposed64;
    else if (a->rel_kh == 14 && a->rel_kw == 14)
      bias_mode = kBiasDecomposed14;
  }
  DeviceState* dev = nullptr;
  if ((rc = device_state(&dev))) return rc;
  prm.status = dev->status;

  if (bias_shared_by_the_batch(a)) {
    prm.batch_fastest = 1;  // one bias for every image: the images of a head run side by side (see decode_item)
    prm.magic_heads = div_magic(a->batch);
  }
  CUtensorMap mb = mq;  // only the dense-tile bias form looks at it
  if (bias_mode == kBiasDenseTiles && (rc = cached_bias_map(&mb, a))) return rc;
  const unsigned grid = plan_work(prm, a, dev->sms);
  const bool f16 = a->dtype == B200_ATTN_F16;
  const bool short_sched = sched == B200_ATTN_SCHED_SHORT;
  switch (bias_mode) {
    case kBiasNone:
      return f16 ? launch_sched<__half, kBiasNone>(short_sched, prm, grid, *dev, mq, mk, mv, mo, mb, stream)
                 : launch_sched<__nv_bfloat16, kBiasNone>(short_sched, prm, grid, *dev, mq, mk, mv, mo, mb, stream);
    case kBiasDenseTiles:
      return f16 ? launch_sched<__half, kBiasDenseTiles>(short_sched, prm, grid, *dev, mq, mk, mv, mo, mb, stream)
                 : launch_sched<__nv_bfloat16, kBiasDenseTiles>(short_sched, prm, grid, *dev, mq, mk, mv, mo, mb, stream);
    case kBiasDense:
      return f16 ? launch_sched<__half, kBiasDense>(short_sched, prm, grid, *dev, mq, mk, mv, mo, mb, stream)
                 : launch_sched<__nv_bfloat16, kBiasDense>(short_sched, prm, grid, *dev, mq, mk, mv, mo, mb, stream);
    case kBiasDecomposed64:
      return f16 ? launch_sched<__half, kBiasDecomposed64>(short_sched, prm, grid, *dev, mq, mk, mv, mo, mb, stream)
                 : launch_sched<__nv_bfloat16, kBiasDecomposed64>(short_sched, prm, grid, *dev, mq, mk, mv, mo, mb, stream);
    case kBiasDecomposed14:
      return f16 ? launch_sched<__half, kBiasDecomposed14>(short_sched, prm, grid, *dev, mq, mk, mv, mo, mb, stream)
                 : launch_sched<__nv_bfloat16, kBiasDecomposed14>(short_sched, prm, grid, *dev, mq, mk, mv, mo, mb, stream);
    default:
      return f16 ? launch_sched<__half, kBiasDecomposed>(short_sched, prm, grid, *dev, mq, mk, mv, mo, mb, stream)
                 : launch_sched<__nv_bfloat16, kBiasDecomposed>(short_sched, prm, grid, *dev, mq, mk, mv, mo, mb, stream);
  }
}

int b200_attn_plan(const B200AttnArgs* a, int32_t sms, int32_t cta, int32_t* grid_out, int32_t* items_out,
                   int32_t max_items, int32_t* n_items_out, int32_t* later_parts_out) {
  int bias_mode = 0, sched = 0;
  int rc = validate(a, &bias_mode, &sched);
  if (rc != B200_ATTN_OK) return rc;
  if (sms < 1 || grid_out == nullptr || n_items_out == nullptr || later_parts_out == nullptr || (items_out == nullptr && max_items > 0))
    return fail(B200_ATTN_BAD_CONFIG, "b200_attn_plan: sms must be positive and the output pointers not NULL");
  AttnParams prm;
  std::memset(&prm, 0, sizeof(prm));
  prm.batch = a->batch;
  prm.heads = a->heads;
  prm.q_tokens = a->q_tokens;
  prm.kv_tokens = a->kv_tokens;
  prm.q_tiles = (a->q_tokens + kTileRows - 1) / kTileRows;
  prm.kv_tiles = (a->kv_tokens + kTileRows - 1) / kTileRows;
  prm.magic_heads = div_magic(a->heads);
  if (bias_shared_by_the_batch(a)) {  // as b200_attn_fwd
    prm.batch_fastest = 1;
    prm.magic_heads = div_magic(a->batch);
  }
  B200AttnArgs with_ws = *a;
  if (with_ws.workspace != nullptr && static_cast<size_t>(with_ws.workspace_bytes) < workspace_bytes_for(sms)) {
    with_ws.workspace = nullptr;  // as b200_attn_fwd: too small a workspace is not used
    with_ws.workspace_bytes = 0;
  }
  const int grid = static_cast<int>(plan_work(prm, &with_ws, sms));
  *grid_out = grid;
  if (cta < 0 || cta >= grid) return fail(B200_ATTN_BAD_CONFIG, "b200_attn_plan: cta %d outside the grid of %d", cta, grid);
  const CtaWork cw = cta_work(prm, cta, grid);
  const int n = cw.pairs + cw.singles;
  *n_items_out = n;
  *later_parts_out = cw.last_parts;
  for (int it = 0; it < n && it < max_items; ++it) {
    const WorkItem w = prm.chunked ? decode_item<true>(prm, cw, it) : decode_item<false>(prm, cw, it);
    int32_t* o = items_out + 7 * it;
    o[0] = w.b; o[1] = w.h; o[2] = w.q_row0; o[3] = w.n_tiles; o[4] = w.ja; o[5] = w.jb; o[6] = w.kind;
  }
  return B200_ATTN_OK;
}

int b200_attn_workspace_size(int64_t* bytes) {
  if (bytes == nullptr) return fail(B200_ATTN_BAD_CONFIG, "bytes is NULL");
  DeviceState* dev = nullptr;
  if (const int rc = device_state(&dev)) return rc;
  *bytes = static_cast<int64_t>(workspace_bytes_for(dev->sms));
  return B200_ATTN_OK;
}

int b200_attn_fwd_static(const B200AttnArgs* a, void* stream_ptr) {
  if (a == nullptr) return fail(B200_ATTN_BAD_CONFIG, "args is NULL");
  DeviceState* dev = nullptr;
  if (const int rc = device_state(&dev)) return rc;
  if (dev->sms > kStaticMaxSms)
    return fail(B200_ATTN_UNSUPPORTED,
                "b200_attn_fwd_static: this device has %d SMs, the built-in scratch array holds the partial results of "
                "at most %d; use b200_attn_fwd with a workspace of b200_attn_workspace_size() bytes",
                dev->sms, kStaticMaxSms);
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  // Set-up, once per device and with that device current: in host code the array's name is only a handle for the
  // runtime, the address a kernel can use has to be asked for.
  StaticScratch& scratch = g_static_scratch[device];
  if (!scratch.ready.load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> lock(g_devices_mutex);
    if (!scratch.ready.load(std::memory_order_relaxed)) {
      void* ptr = nullptr;
      e = cudaGetSymbolAddress(&ptr, g_static_workspace);
      if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(built-in scratch array)");
      scratch.ptr = ptr;
      scratch.ready.store(true, std::memory_order_release);
    }
  }
  B200AttnArgs with_scratch = *a;
  with_scratch.workspace = scratch.ptr;
  with_scratch.workspace_bytes = static_cast<int64_t>(workspace_bytes_for(dev->sms));
  // The array keeps what the last call left. The partial results are written before they are read; the counters
  // must start at zero, and a call that was cut short may have left some raised: clear them, in stream order.
  e = cudaMemsetAsync(static_cast<char*>(scratch.ptr) + workspace_flags_offset(dev->sms), 0,
                      static_cast<size_t>(dev->sms) * 2 * sizeof(uint32_t), static_cast<cudaStream_t>(stream_ptr));
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(counters of the built-in scratch array)");
  return b200_attn_fwd(&with_scratch, stream_ptr);
}

// Per SM and clock: what the tensor pipe delivers in a GEMM under the power cap (measured with cuBLAS: 1.4 PFLOP/s
// over 148 SMs at 1.9 GHz) and what the L2 delivers to one SM when all of them pull (about 10 TB/s).
constexpr double kGemmPipeFlopsPerClock = 5000.0, kGemmL2BytesPerClock = 36.0;

int b200_gemm(const B200GemmArgs* a, void* stream_ptr) {
  if (a == nullptr) return fail(B200_ATTN_BAD_CONFIG, "args is NULL");
  if (a->struct_size != sizeof(B200GemmArgs))
    return fail(B200_ATTN_BAD_CONFIG, "struct_size %u does not match this library's B200GemmArgs (%zu bytes)", a->struct_size,
                sizeof(B200GemmArgs));
  if (a->dtype != B200_ATTN_F16 && a->dtype != B200_ATTN_BF16)
    return fail(B200_ATTN_BAD_CONFIG, "dtype %u: x, w, bias, res, y must be fp16 (0) or bf16 (1)", a->dtype);
  if (a->act != kActNone && a->act != kActRelu && a->act != kActGelu && a->act != kActGeluTanh)
    return fail(B200_ATTN_BAD_CONFIG, "act %d: 0 none, 1 relu, 5 gelu (erf), 6 gelu (tanh form)", a->act);
  if (a->m < 1 || a->n < 1 || a->k < 1 || a->n % 8 != 0 || a->k % 8 != 0)
    return fail(B200_ATTN_UNSUPPORTED, "m %d n %d k %d: all positive, n and k multiples of 8", a->m, a->n, a->k);
  if (a->lda < a->k || a->lda % 8 != 0 || a->ldy < a->n || a->ldy % 8 != 0 || (a->res != nullptr && (a->lres < a->n || a->lres % 8 != 0)))
    return fail(B200_ATTN_UNSUPPORTED, "row strides lda %lld ldy %lld lres %lld must cover their rows and be multiples of 8",
                static_cast<long long>(a->lda), static_cast<long long>(a->ldy), static_cast<long long>(a->lres));
  if (a->lda >= (int64_t(1) << 38)) return fail(B200_ATTN_UNSUPPORTED, "lda too large for a tensor map");
  const struct { const char* name; const void* ptr; bool required; } ptrs[] = {
      {"x", a->x, true}, {"w", a->w, true}, {"y", a->y, true}, {"bias", a->bias, false}, {"scale", a->scale, false}, {"res", a->res, false}};
  for (const auto& x : ptrs) {
    if (x.ptr == nullptr && x.required) return fail(B200_ATTN_BAD_CONFIG, "%s is NULL", x.name);
    if (!aligned16(x.ptr)) return fail(B200_ATTN_UNSUPPORTED, "%s is not 16-byte aligned", x.name);
  }
  DeviceState* dev = nullptr;
  if (int rc = device_state(&dev)) return rc;
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return fail(B200_ATTN_CUDA_ERROR_BASE, "cuTensorMapEncodeTiled is not available from this driver");
  const CUtensorMapDataType dt = a->dtype == B200_ATTN_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap mx, mw;
  const cuuint32_t box[2] = {kGemmBK, 128}, elem[2] = {1, 1};
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(a->k), static_cast<cuuint64_t>(a->m)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(a->lda) * 2};
    const CUresult r = enc(&mx, dt, 2, const_cast<void*>(a->x), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B200_ATTN_UNSUPPORTED, "tensor map for x rejected by the driver (CUresult %d)", static_cast<int>(r));
  }
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(a->k), static_cast<cuuint64_t>(a->n)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(a->k) * 2};
    const CUresult r = enc(&mw, dt, 2, const_cast<void*>(a->w), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B200_ATTN_UNSUPPORTED, "tensor map for w rejected by the driver (CUresult %d)", static_cast<int>(r));
  }
  GemmParams prm{};
  prm.m = a->m; prm.n = a->n; prm.k = a->k;
  prm.bias = a->bias; prm.scale = a->scale; prm.res = a->res; prm.lres = a->lres;
  prm.y = a->y; prm.ldy = a->ldy; prm.act = a->act;
  prm.status = dev->status;
  // Tile shape: of 128 x 128, 128 x 256 and 256 x 256 the one with the shortest estimated time. A tile's time is its
  // flops over the rate its shape allows - the tensor pipe, or the L2 bandwidth times the flops the tile gets out of
  // a byte (2 BM BN / (2 (BM + BN)) per k-value) - and the tiles run in rounds of one per SM.
  struct Shape { int bm, bn; } shapes[3] = {{128, 128}, {128, 256}, {256, 256}};
  int best = 0;
  double best_time = 0;
  for (int i = 0; i < 3; ++i) {
    if (shapes[i].bn > 128 && a->n <= 128) continue;
    if (shapes[i].bm > 128 && a->m <= 128) continue;
    const long long tm = (a->m + shapes[i].bm - 1) / shapes[i].bm, tn = (a->n + shapes[i].bn - 1) / shapes[i].bn;
    const double rounds = static_cast<double>((tm * tn + dev->sms - 1) / dev->sms);
    const double flops_per_byte = static_cast<double>(shapes[i].bm) * shapes[i].bn / (shapes[i].bm + shapes[i].bn);
    const double rate = std::min(kGemmPipeFlopsPerClock, kGemmL2BytesPerClock * flops_per_byte);
    const double time = rounds * (2.0 * shapes[i].bm * shapes[i].bn) / rate;
    if (i == 0 || time < best_time) {
      best = i;
      best_time = time;
    }
  }
  const int bm = shapes[best].bm, bn = shapes[best].bn;
  prm.tiles_m = (a->m + bm - 1) / bm;
  prm.tiles_n = (a->n + bn - 1) / bn;
  const long long tiles = static_cast<long long>(prm.tiles_m) * prm.tiles_n;
  if (tiles > 0x7fffffffLL) return fail(B200_ATTN_UNSUPPORTED, "problem too large for one launch");
  const unsigned grid = static_cast<unsigned>(std::min<long long>(tiles, dev->sms));
  const bool f16 = a->dtype == B200_ATTN_F16;
  const int form = (f16 ? 0 : 1) * 3 + best;
  const void* kernels[6] = {
      reinterpret_cast<const void*>(gemm_epilogue_kernel<__half, 128, 128>), reinterpret_cast<const void*>(gemm_epilogue_kernel<__half, 128, 256>),
      reinterpret_cast<const void*>(gemm_epilogue_kernel<__half, 256, 256>), reinterpret_cast<const void*>(gemm_epilogue_kernel<__nv_bfloat16, 128, 128>),
      reinterpret_cast<const void*>(gemm_epilogue_kernel<__nv_bfloat16, 128, 256>), reinterpret_cast<const void*>(gemm_epilogue_kernel<__nv_bfloat16, 256, 256>)};
  const void* kernel = kernels[form];
  const size_t smem_of[3] = {sizeof(GemmSmem<128, 128>), sizeof(GemmSmem<128, 256>), sizeof(GemmSmem<256, 256>)};
  const int smem = static_cast<int>(smem_of[best]) + 1024;
  if (!dev->gemm_opted_in[form].load(std::memory_order_acquire)) {
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(shared memory)");
    dev->gemm_opted_in[form].store(true, std::memory_order_release);
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(grid);
  config.blockDim = dim3(kGemmThreads);
  config.dynamicSmemBytes = smem;
  config.stream = static_cast<cudaStream_t>(stream_ptr);
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  void* kargs[] = {&mx, &mw, &prm};
  cudaError_t e = cudaLaunchKernelExC(&config, kernel, kargs);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "gemm kernel launch");
  tl_error[0] = '\0';
  return B200_ATTN_OK;
}

int b200_sam_rel_terms(const B200RelTermsArgs* a, void* stream_ptr) {
  if (a == nullptr) return fail(B200_ATTN_BAD_CONFIG, "args is NULL");
  if (a->struct_size != sizeof(B200RelTermsArgs))
    return fail(B200_ATTN_BAD_CONFIG, "struct_size %u does not match this library's B200RelTermsArgs (%zu bytes)",
                a->struct_size, sizeof(B200RelTermsArgs));
  if (a->dtype != B200_ATTN_F16 && a->dtype != B200_ATTN_BF16)
    return fail(B200_ATTN_BAD_CONFIG, "dtype %u: q, the tables and the results must be fp16 (0) or bf16 (1)", a->dtype);
  if (a->head_dim != kHeadDim) return fail(B200_ATTN_UNSUPPORTED, "head_dim %d: only head dim 64 is built", a->head_dim);
  if (a->batch < 1 || a->heads < 1 || a->side < 2 || a->side > kRelMaxSide || a->side % 2 != 0)
    return fail(B200_ATTN_UNSUPPORTED, "batch %d heads %d side %d: side must be even, 2 .. %d", a->batch, a->heads, a->side, kRelMaxSide);
  if (static_cast<int64_t>(a->batch) * a->side > 0x7fffffffLL) return fail(B200_ATTN_UNSUPPORTED, "batch too large for one launch");
  const int tokens = a->side * a->side;
  if (int rc = check_view("q", a->q, a->q_stride, a->batch, a->heads, tokens)) return rc;
  const struct { const char* name; const void* ptr; int align; } ptrs[] = {
      {"rel_pos_h", a->rel_pos_h, 4}, {"rel_pos_w", a->rel_pos_w, 4}, {"rel_h", a->rel_h, 4}, {"rel_w", a->rel_w, 4}};
  for (const auto& x : ptrs) {
    if (x.ptr == nullptr) return fail(B200_ATTN_BAD_CONFIG, "%s is NULL", x.name);
    if (reinterpret_cast<uintptr_t>(x.ptr) % x.align != 0) return fail(B200_ATTN_UNSUPPORTED, "%s is not 4-byte aligned", x.name);
  }
  RelTermsParams prm{};
  prm.q = a->q;
  prm.q_sb = a->q_stride[0];
  prm.q_sn = a->q_stride[1];
  prm.q_sh = a->q_stride[2];
  prm.rel_pos_h = a->rel_pos_h;
  prm.rel_pos_w = a->rel_pos_w;
  prm.rel_h = a->rel_h;
  prm.rel_w = a->rel_w;
  prm.batch = a->batch;
  prm.heads = a->heads;
  prm.side = a->side;
  const int rows = a->side * a->heads;
  const dim3 grid(static_cast<unsigned>(a->batch * a->side), 2, static_cast<unsigned>(std::min(8, (rows + kRelThreads - 1) / kRelThreads)));
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  if (a->dtype == B200_ATTN_F16) sam_rel_terms_kernel<__half><<<grid, kRelThreads, 0, stream>>>(prm);
  else sam_rel_terms_kernel<__nv_bfloat16><<<grid, kRelThreads, 0, stream>>>(prm);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "sam_rel_terms kernel launch");
  tl_error[0] = '\0';
  return B200_ATTN_OK;
}

int b200_rope_qk(const B200RopeArgs* a, void* stream_ptr) {
  if (a == nullptr) return fail(B200_ATTN_BAD_CONFIG, "args is NULL");
  if (a->struct_size != sizeof(B200RopeArgs))
    return fail(B200_ATTN_BAD_CONFIG, "struct_size %u does not match this library's B200RopeArgs (%zu bytes)",
                a->struct_size, sizeof(B200RopeArgs));
  if (a->dtype != B200_ATTN_F16 && a->dtype != B200_ATTN_BF16)
    return fail(B200_ATTN_BAD_CONFIG, "dtype %u: q and k must be fp16 (0) or bf16 (1)", a->dtype);
  if (a->head_dim != kHeadDim) return fail(B200_ATTN_UNSUPPORTED, "head_dim %d: only head dim 64 is built", a->head_dim);
  if (a->batch < 1 || a->heads < 1 || a->tokens < 1 || a->prefix < 0 || a->prefix > a->tokens)
    return fail(B200_ATTN_BAD_CONFIG, "batch %d heads %d tokens %d prefix %d", a->batch, a->heads, a->tokens, a->prefix);
  if (!(a->q_scale > 0.f) || !std::isfinite(a->q_scale)) return fail(B200_ATTN_BAD_CONFIG, "q_scale must be positive and finite");
  if (int rc = check_view("q", a->q, a->q_stride, a->batch, a->heads, a->tokens)) return rc;
  if (int rc = check_view("k", a->k, a->k_stride, a->batch, a->heads, a->tokens)) return rc;
  if (a->prefix < a->tokens) {
    if (a->cs == nullptr) return fail(B200_ATTN_BAD_CONFIG, "cs is NULL");
    if (!aligned16(a->cs)) return fail(B200_ATTN_UNSUPPORTED, "cs is not 16-byte aligned");
  }
  DeviceState* dev = nullptr;
  if (int rc = device_state(&dev)) return rc;
  RopeParams prm{};
  prm.q = a->q;
  prm.k = a->k;
  prm.q_sb = a->q_stride[0];
  prm.q_sn = a->q_stride[1];
  prm.q_sh = a->q_stride[2];
  prm.k_sb = a->k_stride[0];
  prm.k_sn = a->k_stride[1];
  prm.k_sh = a->k_stride[2];
  prm.cs = a->cs;
  prm.batch = a->batch;
  prm.heads = a->heads;
  prm.tokens = a->tokens;
  prm.prefix = a->prefix;
  prm.q_scale = a->q_scale;
  // One token per CTA and pass; enough CTAs to fill every SM sixteen times over (128 threads each), no more.
  const long long rows = static_cast<long long>(a->batch) * a->tokens;
  const unsigned grid = static_cast<unsigned>(std::min<long long>(rows, static_cast<long long>(dev->sms) * 16));
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  if (a->dtype == B200_ATTN_F16) rope_qk_kernel<__half><<<grid, kRopeThreads, 0, stream>>>(prm);
  else rope_qk_kernel<__nv_bfloat16><<<grid, kRopeThreads, 0, stream>>>(prm);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "rope_qk kernel launch");
  tl_error[0] = '\0';
  return B200_ATTN_OK;
}

int b200_attn_status(uint32_t* status) {
  if (status == nullptr) return fail(B200_ATTN_BAD_CONFIG, "status is NULL");
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceSynchronize");
  uint32_t word = 0, zero = 0;
  e = cudaMemcpyFromSymbol(&word, g_status_word, sizeof(word));
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyFromSymbol(status word)");
  if (word != 0) {
    e = cudaMemcpyToSymbol(g_status_word, &zero, sizeof(zero));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyToSymbol(status word)");
  }
  *status = word;
  return B200_ATTN_OK;
}


int b200_attn_selftest_wait_limit(uint32_t limit_us, void* stream_ptr) {
  if (limit_us == 0 || limit_us > 100000)
    return fail(B200_ATTN_BAD_CONFIG, "limit_us %u must be between 1 and 100000", limit_us);
  uint32_t* status = nullptr;
  cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_status_word);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(status word)");
  wait_limit_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_ptr)>>>(uint64_t(limit_us) * 1000, status);
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "self-test kernel launch");
  return B200_ATTN_OK;
}

const char* b200_attn_last_error(void) { return tl_error; }

// The build passes the digest of the sources (fastforks_b200/_lib.py: source_hash); the loader compares it with the
// sources beside the binary and refuses a binary of other sources.
#ifndef B200_SOURCE_HASH
#define B200_SOURCE_HASH "0000000000000000"
#endif
const char* b200_attn_version(void) { return "b200attn 0.2 (sm_100a, tcgen05 + TMA) b200attn-src:" B200_SOURCE_HASH; }

}  // extern "C"
