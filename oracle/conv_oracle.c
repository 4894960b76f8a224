/*
 * TEST INFRASTRUCTURE — not part of the product.  Only tests/, the smoke check
 * and the CPU-baseline legs of bench.py may build or call this file.
 *
 * CPU restatement of the reference's convolution arithmetic for the fused
 * conv -> (scale) -> bias -> ReLU path, written as plain loops:
 *
 *   index math      src/flag_dnn/graph/kernels/fused_conv.py:249-299
 *                   m -> (n, oh, ow); k -> (c, kh, kw);
 *                   ih = oh*stride_h + kh*dil_h - pad_top,
 *                   iw = ow*stride_w + kw*dil_w - pad_left; zero outside the image
 *   bias and ReLU   src/flag_dnn/graph/kernels/fused_conv.py:297-299
 *   output size     src/flag_dnn/ops/conv2d.py:52-62
 *   groups          src/flag_dnn/ops/conv2d.py:90-135 (channel/group split)
 *
 * The reference has no CPU convolution of its own: on CPU tensors its graph
 * executor calls torch.nn.functional.conv2d (src/flag_dnn/graph/registry.py:
 * 1357-1365).  This file is the second, independent oracle; it accumulates in
 * double so that it can judge fp32 results.  Parity is pinned against outputs
 * of the reference itself stored under tests/golden/.
 */
#include <stddef.h>
#include <stdint.h>

typedef struct {
  int n, c, h, w, k, r, s;
  int stride_h, stride_w, pad_top, pad_left, dil_h, dil_w, groups;
  int oh, ow, relu;
  int64_t xs[4], ws[4], ys[4]; /* element strides, logical NCHW / KCRS / NKHW order */
} oracle_conv_desc;

#define ORACLE_CONV_BODY(T)                                                                      \
  const int cg = d->c / d->groups, kg = d->k / d->groups;                                        \
  for (int n = 0; n < d->n; ++n)                                                                 \
    for (int k = 0; k < d->k; ++k) {                                                             \
      const int g = k / kg;                                                                      \
      for (int oh = 0; oh < d->oh; ++oh)                                                         \
        for (int ow = 0; ow < d->ow; ++ow) {                                                     \
          double acc = 0.0;                                                                      \
          for (int c = 0; c < cg; ++c)                                                           \
            for (int r = 0; r < d->r; ++r) {                                                     \
              const int ih = oh * d->stride_h + r * d->dil_h - d->pad_top;                       \
              if (ih < 0 || ih >= d->h) continue;                                                \
              for (int s = 0; s < d->s; ++s) {                                                   \
                const int iw = ow * d->stride_w + s * d->dil_w - d->pad_left;                    \
                if (iw < 0 || iw >= d->w) continue;                                              \
                acc += (double)x[n * d->xs[0] + (int64_t)(g * cg + c) * d->xs[1] + ih * d->xs[2] + \
                                 iw * d->xs[3]] *                                                \
                       (double)w[k * d->ws[0] + c * d->ws[1] + r * d->ws[2] + s * d->ws[3]];     \
              }                                                                                  \
            }                                                                                    \
          if (scale) acc *= (double)scale[k];                                                    \
          if (bias) acc += (double)bias[k];                                                      \
          if (d->relu && acc < 0.0) acc = 0.0;                                                   \
          y[n * d->ys[0] + k * d->ys[1] + oh * d->ys[2] + ow * d->ys[3]] = (T)acc;               \
        }                                                                                        \
    }                                                                                            \
  return 0;

int oracle_conv2d_f32(const oracle_conv_desc* d, const float* x, const float* w, const float* bias,
                      const float* scale, float* y) {
  ORACLE_CONV_BODY(float)
}

int oracle_conv2d_f64(const oracle_conv_desc* d, const double* x, const double* w,
                      const double* bias, const double* scale, double* y) {
  ORACLE_CONV_BODY(double)
}

/* Output-size rule of src/flag_dnn/ops/conv2d.py:52-62 (Python floor division). */
int oracle_conv_out_dim(int in, int pad_before, int pad_after, int dil, int kernel, int stride) {
  long num = (long)in + pad_before + pad_after - (long)dil * (kernel - 1) - 1;
  long q = num / stride;
  if ((num % stride != 0) && ((num < 0) != (stride < 0))) --q;
  return (int)(q + 1);
}
