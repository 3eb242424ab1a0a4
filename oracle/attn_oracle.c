/*
 * CPU oracle of the attention path in plain C: TEST INFRASTRUCTURE ONLY.
 *
 * Restates, independently of numpy / torch, the arithmetic of the reference's portable attention
 * (DINOv2 Attention.forward, src/fastforks/shared/depth_anything_v2/net/dinov2_layers/attention.py:46-60:
 * q*scale, q k^T, softmax over keys, attn v) with SAM's decomposed relative-position term added to the logits
 * (add_decomposed_rel_pos, src/fastforks/promptable_segmentation/models/sam/net/image_encoder.py:357-360).
 * Only tests, the smoke check and bench.py's CPU-baseline leg may link or call it; the product never does.
 *
 * All arrays are contiguous fp32: q, out [B, H, Nq, d]; k, v [B, H, Nk, d]; bias (may be NULL) [B, H, Nq, Nk];
 * rel_h [B, H, Nq, kh] and rel_w [B, H, Nq, kw] (may both be NULL) with kh * kw == Nk.
 * The call computes output rows [row_begin, row_end) of the B*H*Nq rows, so a caller can split rows over threads.
 * Logits and sums are accumulated in double so that the oracle's own rounding stays far below the tolerances.
 */
#include <math.h>
#include <stddef.h>
#include <stdlib.h>

int attn_oracle_f32(const float* q, const float* k, const float* v, const float* bias, const float* rel_h,
                    const float* rel_w, int kh, int kw, float* out, int batch, int heads, int nq, int nk, int d,
                    float scale, long row_begin, long row_end) {
  if (batch < 1 || heads < 1 || nq < 1 || nk < 1 || d < 1) return 1;
  if ((rel_h == NULL) != (rel_w == NULL)) return 1;
  if (rel_h != NULL && (long)kh * kw != nk) return 1;
  const long rows = (long)batch * heads * nq;
  if (row_begin < 0 || row_end > rows || row_begin > row_end) return 1;
  double* logit = (double*)malloc(sizeof(double) * (size_t)nk);
  double* acc = (double*)malloc(sizeof(double) * (size_t)d);
  if (logit == NULL || acc == NULL) {
    free(logit);
    free(acc);
    return 2;
  }
  for (long r = row_begin; r < row_end; ++r) {
    const long bh = r / nq;
    const float* qr = q + r * d;
    const float* kb = k + bh * (long)nk * d;
    const float* vb = v + bh * (long)nk * d;
    double mx = -INFINITY;
    for (int j = 0; j < nk; ++j) {
      double s = 0.0;
      for (int c = 0; c < d; ++c) s += (double)(qr[c] * scale) * (double)kb[(long)j * d + c];
      if (bias != NULL) s += (double)bias[r * nk + j];
      if (rel_h != NULL) s += (double)rel_h[r * kh + j / kw] + (double)rel_w[r * kw + j % kw];
      logit[j] = s;
      if (s > mx) mx = s;
    }
    double sum = 0.0;
    for (int c = 0; c < d; ++c) acc[c] = 0.0;
    for (int j = 0; j < nk; ++j) {
      const double p = exp(logit[j] - mx);
      sum += p;
      for (int c = 0; c < d; ++c) acc[c] += p * (double)vb[(long)j * d + c];
    }
    for (int c = 0; c < d; ++c) out[r * d + c] = (float)(acc[c] / sum);
  }
  free(logit);
  free(acc);
  return 0;
}
