// TEST INFRASTRUCTURE ONLY: host launcher around the reference's own `flash64_*` kernels, for side-by-side checks.
//
// The kernels themselves are not in this repository. The build recipe (oracle/Makefile, target `_ref`) compiles this
// file with -DREF_FLASH64_SOURCE="<path of the reference's src/fastforks/kernels/fastbb/fastbb_kernels.cu>", so the
// reference source is read where it lies, with the reference's own flags and target (plain sm_100, as its
// build.toml lists), and the result goes to oracle/_ref/, which is never committed. Only tests may load it.
//
// The launch rule below restates `Flash64._run` (src/fastforks/kernels/fastbb/__init__.py:124-136):
// rm = 2 when n * b * heads >= 36864 else 1 (chosen by the caller), 64 * rm query rows per CTA,
// grid ((n + br - 1) / br, b * heads), 128 threads; the kernels' shared memory is static.
#include REF_FLASH64_SOURCE

#include <cuda_runtime.h>

namespace {
using Kernel = void (*)(const __half*, const __half*, const __half*, __half*, int, int, long long, int, int, long long,
                        int, int, long long, int, int, long long, int, int, float);

Kernel pick(int rm, int variant) {
  // variant: 0 = "hh" (fp16 accumulation in both products), 1 = "fh", 2 = "ff" (fp32 in both)
  if (rm == 2) return variant == 0 ? flash64_r2_hh : variant == 1 ? flash64_r2_fh : flash64_r2_ff;
  return variant == 0 ? flash64_r1_hh : variant == 1 ? flash64_r1_fh : flash64_r1_ff;
}
}  // namespace

// Returns 0 or the CUDA error code. Strides in elements: batch (64-bit), token, head for each of q, k, v, o.
extern "C" int ref_flash64_launch(int variant, int rm, const void* q, const void* k, const void* v,
                                  void* o, int batch, int tokens, int heads, const long long* strides /* 12 */,
                                  float scale_log2, void* stream) {
  if (variant < 0 || variant > 2 || (rm != 1 && rm != 2)) return -1;
  Kernel fn = pick(rm, variant);
  const int br = 64 * rm;
  dim3 grid((tokens + br - 1) / br, batch * heads, 1);
  fn<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __half*>(q), static_cast<const __half*>(k), static_cast<const __half*>(v),
      static_cast<__half*>(o), tokens, heads, strides[0], static_cast<int>(strides[1]), static_cast<int>(strides[2]),
      strides[3], static_cast<int>(strides[4]), static_cast<int>(strides[5]), strides[6], static_cast<int>(strides[7]),
      static_cast<int>(strides[8]), strides[9], static_cast<int>(strides[10]), static_cast<int>(strides[11]),
      scale_log2);
  return static_cast<int>(cudaGetLastError());
}
