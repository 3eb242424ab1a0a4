/*
 * b200_attn.h - C ABI of the B200 (sm_100a) attention-forward library `libb200attn.so`.
 *
 * The library computes  O = softmax(scale * Q K^T + bias) V  for head dim 64, fp16 or bf16, non-causal,
 * with fp32 accumulation, on hand-written tcgen05 / TMA kernels.  It is the replacement for the two
 * forms the reference's kernels backend uses for this operation:
 *
 *   - the `flash64_r{1,2}_{hh,fh,ff}` kernels (src/fastforks/kernels/fastbb/fastbb_kernels.cu:58-307)
 *     launched by `Flash64._run` (src/fastforks/kernels/fastbb/__init__.py:124-136) on strided
 *     `[B, N, heads, 64]` views of a packed qkv tensor;
 *   - the `F.scaled_dot_product_attention(q, k, v, attn_mask=..., scale=...)` calls on `[B, heads, N, 64]`
 *     views in the kernels-mode block forwards (src/fastforks/_optimize/transformer.py:286-289, 476-479)
 *     and in the SAM encoder, where the decomposed relative-position bias is folded into widened q / k
 *     (src/fastforks/promptable_segmentation/models/sam/fast.py:92-113, fused.py:80-86).
 *
 * Conventions follow the reference's `shared`-kind kernel libraries
 * (src/fastforks/_core/kernels.py:481-494, src/fastforks/kernels/dpt_fused/dpt_fused.cu:17-18):
 * plain pointers and sizes, the caller owns every buffer, the launch goes to the stream the caller
 * passes and never synchronises, the return value is a status code.
 *
 * All pointers are device pointers.  Strides are in ELEMENTS of the tensor's own dtype.
 */
#ifndef B200_ATTN_H_
#define B200_ATTN_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Return codes (the reference's convention: 0 = ran, 1 = geometry / alignment unsupported,
 * -1 = unknown configuration, anything else = CUDA error). CUDA errors are 1000 + cudaError_t. */
#define B200_ATTN_OK 0
#define B200_ATTN_UNSUPPORTED 1
#define B200_ATTN_BAD_CONFIG (-1)
#define B200_ATTN_CUDA_ERROR_BASE 1000

/* Element types. */
#define B200_ATTN_F16 0
#define B200_ATTN_BF16 1
#define B200_ATTN_F32 2 /* bias tensors only */

/* Tile schedule hints. Both schedules are the same persistent kernel (one CTA per SM walks work items of one or two
 * 128-row query tiles of one head, the next item's tiles prefetched while the current one computes). The short one
 * skips the exponentials of the last 32 columns of a ragged last key tile when they hold no key at all, which pays
 * for sequences of at most two key tiles (197 tokens: 69 keys in the second tile) and costs the long sequences a
 * little. AUTO picks SHORT for at most 256 keys whose last tile holds at most 96, else LONG; b200_attn_query
 * reports the choice. Results are identical bit for bit. */
#define B200_ATTN_SCHED_AUTO 0
#define B200_ATTN_SCHED_LONG 1
#define B200_ATTN_SCHED_SHORT 2

/*
 * One attention call.  Element (b, n, h, d) of q lives at q + b*q_stride[0] + n*q_stride[1] + h*q_stride[2] + d
 * (same for k, v, o), exactly the addressing of the reference kernel (fastbb_kernels.cu:52-54), so both the
 * `[B, N, heads, 64]` views of packed qkv and the `[B, heads, N, 64]` SDPA layout are described without a copy.
 * Requirements: head_dim == 64, unit stride along d, base pointers 16-byte aligned, strides multiples of 8.
 */
typedef struct B200AttnArgs {
  uint32_t struct_size; /* sizeof(B200AttnArgs): lets the library reject a caller built against another layout */
  uint32_t dtype;       /* B200_ATTN_F16 or B200_ATTN_BF16: type of q, k, v and o */

  const void* q;
  const void* k;
  const void* v;
  void* o;
  int64_t q_stride[3]; /* batch, token, head */
  int64_t k_stride[3];
  int64_t v_stride[3];
  int64_t o_stride[3];

  int32_t batch;
  int32_t heads;
  int32_t q_tokens;  /* N of q and o */
  int32_t kv_tokens; /* N of k and v (== q_tokens for self-attention) */
  int32_t head_dim;  /* must be 64 */
  float scale;       /* softmax scale, > 0 (the reference passes head_dim ** -0.5) */

  /* Optional dense additive bias (an SDPA `attn_mask` of floating type), added to scale * q k^T.
   * Element (b, h, i, j) at bias + b*bias_stride[0] + h*bias_stride[1] + i*bias_stride[2] + j.
   * A stride of 0 broadcasts that dimension.  NULL = none.
   * A 16-bit bias whose base is 16-byte aligned and whose strides (of the dimensions with more than one entry) are
   * multiples of 8 elements is fetched tile by tile through the tensor memory accelerator, like K and V; this is the
   * layout the reference builds for its windowed blocks (rows padded to a multiple of 8 and sliced,
   * src/fastforks/_optimize/transformer.py:463-466).  Any other layout, and fp32, is read row by row: same results,
   * several times slower. */
  const void* bias;
  uint32_t bias_dtype; /* B200_ATTN_F16 / BF16 / F32 */
  int64_t bias_stride[3];

  /* Optional decomposed bias (SAM's relative-position term, sam/net/image_encoder.py:326-362):
   * bias(i, j) = rel_h[b, h, i, j / rel_kw] + rel_w[b, h, i, j % rel_kw], with kv_tokens == rel_kh * rel_kw.
   * Element (b, h, i, c) at rel_h + b*rel_h_stride[0] + h*rel_h_stride[1] + i*rel_h_stride[2] + c.
   * Both NULL = none.  Mutually exclusive with `bias`. */
  const void* rel_h;
  const void* rel_w;
  uint32_t rel_dtype; /* B200_ATTN_F16 / BF16 / F32 */
  int32_t rel_kh;
  int32_t rel_kw;
  int64_t rel_h_stride[3];
  int64_t rel_w_stride[3];

  int32_t schedule;   /* B200_ATTN_SCHED_* */
  int32_t test_flags; /* 0.  For tests: 1 makes every merge of a split launch (see `workspace`) take its general,
                       * slower route, which otherwise only runs when parts complete in an unusual order. */

  /* Optional scratch memory for long sequences: `workspace_bytes` bytes of device memory, 256-byte aligned, at
   * least b200_attn_workspace_size() of them, ZEROED once when it is allocated and then left to the library (the
   * kernel leaves it ready for the next launch).  With it, sequences of more than two key tiles are split along the
   * keys where whole query tiles are too coarse to keep every SM busy to the end of the launch (1370 tokens x 48 heads is
   * 3.6 query tiles per SM): the CTAs that share a tile leave partial results (unnormalised output, row maxima, row
   * sums) there and are counted; the CTA with the tile's first keys folds them in when they are all there, as they
   * are as a rule, else whichever part is counted last does.
   * No CTA waits for another, so grids of several streams may share the GPU in any way.  NULL / 0 = never split (every call then works as it does without
   * scratch memory, only slower where the split would have paid).  Launches that may run at the same time (other
   * streams) need workspaces of their own; the reference keys its workspaces by (device, stream) the same way
   * (src/fastforks/_optimize/ops.py:248-296).  After a launch that b200_attn_status reports as failed, zero it again. */
  void* workspace;
  int64_t workspace_bytes;
} B200AttnArgs;

/*
 * Launches the attention forward on `stream` (a cudaStream_t / CUstream; NULL = the legacy default stream)
 * of the current device and returns without synchronising.  Replaces the `flash64_*` launch
 * (fastbb/__init__.py:130-135) and the SDPA call sites named above.
 * Arguments are checked before anything is launched; a non-zero return means nothing ran.
 * The kernel is launched with programmatic stream serialisation: its set-up may overlap the tail of the kernel
 * before it in the stream, and it waits on the device for that kernel's completion before it reads or writes
 * global memory, so stream order holds for every buffer.  Thread-safe: per-device values are looked up once under
 * a mutex, nothing else is shared between calls.
 */
int b200_attn_fwd(const B200AttnArgs* args, void* stream);

/*
 * b200_attn_fwd for callers that have no device memory to give: the same call, but long sequences are split with
 * scratch memory that is built into the library (`args->workspace` and `workspace_bytes` are ignored) and nothing
 * is allocated, by this call or on its behalf.  It is meant for hosts that cannot call cudaMalloc where they call
 * attention: a serving loop that handed all device memory to a pool of its own at start-up, a pipeline that must
 * not take the device-wide synchronisation an allocation or a free implies, a plain C or ctypes caller that only
 * holds the pointers of its inputs and outputs.  It has no counterpart in the reference, whose callers always
 * have torch's allocator at hand (src/fastforks/_optimize/ops.py:248-296).
 *
 * The price and the limits:
 *   - the scratch array is sized for devices of up to 160 SMs (a B200 has 148): 21.6 MB, held on every GPU that
 *     loads the library until the process ends.  On a device with more SMs the call returns
 *     B200_ATTN_UNSUPPORTED and the message says so; use b200_attn_fwd with a workspace there;
 *   - there is ONE array per device and every call uses it: calls that may overlap on the GPU (two streams, two
 *     threads) race on it and give wrong results.  Calls on one stream are safe.  The array keeps the last call's
 *     contents; the call clears, in stream order, the counters that must start from zero;
 *   - the first call on a device looks up the array's device address (cudaGetSymbolAddress, once per device, with
 *     that device current).  Make that first call before any stream capture begins.
 * Return codes, argument checks, stream and status-word behaviour are those of b200_attn_fwd, and so is the result.
 */
int b200_attn_fwd_static(const B200AttnArgs* args, void* stream);

/*
 * Reports whether `args` describes a call the library can run, without launching: returns the code
 * `b200_attn_fwd` would return from its argument checks, and stores the schedule it would pick
 * (B200_ATTN_SCHED_LONG / SHORT) in *schedule when that pointer is not NULL.  Pointers in `args` are
 * only inspected for alignment.  Counterpart of `check_flash64` (fastbb/__init__.py:51-67).
 */
int b200_attn_query(const B200AttnArgs* args, int32_t* schedule);

/*
 * GEMM with a fused epilogue for the layers around attention (qkv, projection, MLP):
 *     y[p, n] = act((sum_k x[p, k] * w[n, k] + bias[n]) * scale[n] + res[p, n])        bias, scale, res optional
 * x is [m, k] with row stride lda, w is [n, k] row-major and contiguous, y is [m, n] with row stride ldy and may alias
 * res (row stride lres): a LayerScale + residual block output `x += gamma * (o w^T + b)` is one call with
 * scale = gamma, res = y = x.  x, w, bias, res, y are of `dtype`, scale is fp32, accumulation is fp32.
 * act: 0 none, 1 relu, 5 gelu (erf), 6 gelu (tanh form).  Requirements: n, k, lda, ldy, lres multiples of 8, pointers
 * 16-byte aligned.  It replaces `dpt_gemm(cfg, M, N, K, x, lda, w, EpiArgs*, stream)` of the reference's `dpt_fused`
 * library (src/fastforks/kernels/dpt_fused/dpt_fused.cu:7-18, 20-34; caller `DptFused.gemm`,
 * src/fastforks/kernels/dpt_fused/__init__.py:179-220) with the same epilogue formula, operand layouts and return
 * codes; not carried over: the second residual / second output (res2, y2), the pixel-shuffle store of the DPT
 * head's deconvolutions, and the tile-configuration argument (the library picks its tile itself).  bf16 is new.
 * Launch, stream and status-word behaviour are those of b200_attn_fwd (status bits 64 / 128 / 256: the GEMM's
 * loader, MMA issuer, epilogue).
 */
typedef struct B200GemmArgs {
  uint32_t struct_size; /* sizeof(B200GemmArgs) */
  uint32_t dtype;       /* B200_ATTN_F16 or B200_ATTN_BF16 */
  int32_t m;
  int32_t n;
  int32_t k;
  int32_t act;
  const void* x;
  int64_t lda;
  const void* w;
  const void* bias;   /* [n] or NULL */
  const float* scale; /* [n] fp32 or NULL */
  const void* res;    /* [m, lres] or NULL */
  int64_t lres;
  void* y;
  int64_t ldy;
} B200GemmArgs;

int b200_gemm(const B200GemmArgs* args, void* stream);

/*
 * The producer of SAM's decomposed bias: for every query (y, x) of a `side` x `side` grid and k = 0 .. side - 1
 *     rel_h[b, head, (y, x), k] = q[b, (y, x), head, :] . rel_pos_h[y - k + side - 1, :]
 *     rel_w[b, head, (y, x), k] = q[b, (y, x), head, :] . rel_pos_w[x - k + side - 1, :]
 * which are the `rel_h` / `rel_w` arguments of B200AttnArgs.  It replaces the two einsums of the reference's
 * `augmented` (src/fastforks/promptable_segmentation/models/sam/fast.py:104-106) together with the table gather in
 * front of them (`get_rel_pos`, sam/net/image_encoder.py:293-323): q is the UNSCALED query, read in place from the
 * packed qkv tensor (element (b, n, head, d) at q + b*q_stride[0] + n*q_stride[1] + head*q_stride[2] + d, strides in
 * elements, multiples of 8, base 16-byte aligned), `rel_pos_h` / `rel_pos_w` are the module's parameters themselves,
 * `[2 * side - 1, 64]` contiguous, and the results are `[batch, heads, side * side, side]` contiguous, all of `dtype`.
 * `side` must be even and at most 64 (SAM: 14 for the windows, 64 for the global blocks).
 */
typedef struct B200RelTermsArgs {
  uint32_t struct_size; /* sizeof(B200RelTermsArgs) */
  uint32_t dtype;       /* B200_ATTN_F16 or B200_ATTN_BF16 */
  const void* q;
  int64_t q_stride[3]; /* batch, token, head */
  const void* rel_pos_h;
  const void* rel_pos_w;
  void* rel_h;
  void* rel_w;
  int32_t batch;
  int32_t heads;
  int32_t side;
  int32_t head_dim; /* must be 64 */
} B200RelTermsArgs;

int b200_sam_rel_terms(const B200RelTermsArgs* args, void* stream);

/*
 * DINOv3's rotary position embedding, in place on q and k (head dim 64) before the attention call:
 *     out[j]      = (x[j] cos[j] - x[j + 32] sin[j]) * m
 *     out[j + 32] = (x[j + 32] cos[j] + x[j] sin[j]) * m        j = 0 .. 31,  m = q_scale for q, 1 for k
 * computed in fp32 and rounded once.  It replaces the reference's `rope_qk_h` kernel
 * (src/fastforks/kernels/fastbb/fastbb_kernels.cu:793-818; launched from src/fastforks/features/models/dinov3/model.py:199-201
 * with q_scale = 64 ** -0.5, after which attention is called with scale 1.0).  q and k are views of the packed qkv
 * tensor (element (b, n, head, d) at ptr + b*stride[0] + n*stride[1] + head*stride[2] + d, strides in elements,
 * multiples of 8, base 16-byte aligned); `cs` is the reference's table, fp32 `[tokens - prefix, 2, 32]` = cos | sin of
 * the patch tokens (model.py:185-188); the first `prefix` tokens of each sequence (class token and registers) are not
 * rotated: their q is scaled, their k is left as it is.  Unlike the reference's kernel, bf16 is accepted too.
 */
typedef struct B200RopeArgs {
  uint32_t struct_size; /* sizeof(B200RopeArgs) */
  uint32_t dtype;       /* B200_ATTN_F16 or B200_ATTN_BF16 */
  void* q;
  void* k;
  int64_t q_stride[3]; /* batch, token, head */
  int64_t k_stride[3];
  const float* cs;
  int32_t batch;
  int32_t heads;
  int32_t tokens;
  int32_t prefix;   /* 0 .. tokens */
  int32_t head_dim; /* must be 64 */
  float q_scale;
} B200RopeArgs;

int b200_rope_qk(const B200RopeArgs* args, void* stream);

/*
 * Describes, without launching and without a GPU, the work the kernel's CTA number `cta` would do for `args` on a
 * device with `sms` SMs (148 on a B200): the grid size in *grid, the CTA's item count in *n_items, up to `max_items`
 * items as 7 integers each in `items` - batch, head, first query row, query tiles (1 or 2), first key tile, end key
 * tile, kind (0 whole item, 1 a part whose result goes to the workspace, 2 the part that merges the later ones) -
 * and in *later_parts how many following CTAs hold later parts of its last item.  The plan is computed by the very
 * functions the kernel runs, so tests can check on a CPU that every (query tile, key tile) of a problem is covered
 * exactly once.  `args->workspace` only matters as NULL / not NULL (with a workspace long sequences may be split).
 * The reference has no counterpart: its grid is (query tiles, batch * heads), fastbb/__init__.py:130-135.
 */
int b200_attn_plan(const B200AttnArgs* args, int32_t sms, int32_t cta, int32_t* grid, int32_t* items, int32_t max_items,
                   int32_t* n_items, int32_t* later_parts);

/*
 * Stores in *bytes the workspace size that is enough for any call on the current device (it depends on the
 * device's SM count only: four partial tiles of 33 KB and two counters per SM, about 20 MB on a B200).
 * The reference sizes the workspace of its GEMM library with a constant and keeps one per (device, stream)
 * (`_PW_WS`, src/fastforks/_optimize/ops.py:248-296); a caller of this library should do the same.
 */
int b200_attn_workspace_size(int64_t* bytes);

/*
 * Reads and clears the device-side error word of the current device (synchronises that device).
 * 0 = every wait inside the kernels completed.  Non-zero: a kernel gave up a bounded wait on a barrier and
 * returned early, its output is invalid; the bits say which role (1 loader, 2 MMA issuer, 4 softmax, 16 output store).
 * The reference has no counterpart: its kernels contain no waits on asynchronous units.
 */
int b200_attn_status(uint32_t* status);

/*
 * Launches a one-warp kernel that waits, for at most `limit_us` microseconds (1..100000), on a barrier that nothing
 * ever completes, then gives up the way every wait in the attention kernels does: it sets bit 8 of the device
 * status word and returns normally.  `b200_attn_status` must then report 8, and the context stays usable.
 * It exists so that the give-up path can be tested without faulting, trapping or hanging a GPU.
 * The reference has no counterpart.
 */
int b200_attn_selftest_wait_limit(uint32_t limit_us, void* stream);

/* Human-readable reason of the calling thread's last non-zero return. Never NULL. */
const char* b200_attn_last_error(void);

/* Library version string, e.g. "b200attn 0.1 (sm_100a)". */
const char* b200_attn_version(void);

#ifdef __cplusplus
}
#endif

#endif /* B200_ATTN_H_ */
