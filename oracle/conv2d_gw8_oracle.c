/* CPU oracle for the group-width-8 convolution path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker, never the product: only tests/, __graft_entry__.smoke()
 * and bench.py's CPU-baseline leg may build, load or call it.  The shipped operators
 * run CUDA kernels and fail when the native library is missing.
 *
 * It restates, as plain loops, the arithmetic contract of the reference's three
 * kernels: fp16 operands, products and sums in fp32, one rounding to fp16 at the end
 * (fp32 result for the weight gradient).
 *
 *   fprop  reference spio/src/conv2d_gw8.cu:10-224   (taps :160-166, bias :27-33,139,
 *          rounding spio/include/spio/fragment.cuh:156-158)
 *   dgrad  same source with Mode::igrad, :94-107     (filter flip and transpose)
 *   wgrad  reference spio/src/conv2d_gw8_wgrad.cu:10-226 (fp32 output, :207-224)
 *   shapes reference spio/kernels/conv2d_gw8_params.py:140-209 (P, Q, padding)
 *
 * The reference's own tests do not hold golden vectors; they compare the kernels with
 * torch.nn.functional.conv2d on fp32 copies of the fp16 tensors
 * (spio/src_tests/run_test.py:43-50, 84-102).  Parity of this file is pinned the same
 * way: tests/test_oracle.py checks it against that function and against the fixtures
 * in tests/golden/ that tests/golden/make_golden.py produced with it.
 *
 * Layouts: activations NHWC, weights [K][R][S][8], K == C, group g owns channels
 * [8g, 8g+8) on both sides.  fp16 values are passed as uint16_t bit patterns.
 */
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

typedef _Float16 f16;

static inline float h2f(uint16_t bits) {
  f16 h;
  memcpy(&h, &bits, sizeof h);
  return (float)h;
}

static inline uint16_t f2h(float v) {
  f16 h = (f16)v; /* round to nearest even, as __float22half2_rn */
  uint16_t bits;
  memcpy(&bits, &h, sizeof bits);
  return bits;
}

int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* y[n][p][q][k] = bias[k] + sum_{r,s,c<8} x[n][p+r-pad_h][q+s-pad_w][8g+c] * w[k][r][s][c],
 * g = k / 8.  Terms are added in (r, s, c) order starting from the bias. */
void oracle_conv2d_gw8_fprop(uint16_t* y, const uint16_t* x, const uint16_t* w, const float* bias,
                             int n, int c, int h, int wd, int r, int s, int pad_h, int pad_w) {
  const int p = h + 2 * pad_h - r + 1, q = wd + 2 * pad_w - s + 1;
  const long rows = (long)n * p;
#pragma omp parallel for schedule(static)
  for (long row = 0; row < rows; ++row) {
    const int in = (int)(row / p), ip = (int)(row % p);
    for (int iq = 0; iq < q; ++iq) {
      for (int k = 0; k < c; ++k) {
        const int g = k / 8;
        float acc = bias ? bias[k] : 0.0f;
        for (int ir = 0; ir < r; ++ir) {
          const int ih = ip + ir - pad_h;
          if (ih < 0 || ih >= h) continue;
          for (int is = 0; is < s; ++is) {
            const int iw = iq + is - pad_w;
            if (iw < 0 || iw >= wd) continue;
            const uint16_t* xp = x + (((size_t)in * h + ih) * wd + iw) * c + 8 * g;
            const uint16_t* wp = w + (((size_t)k * r + ir) * s + is) * 8;
            for (int ic = 0; ic < 8; ++ic) acc += h2f(xp[ic]) * h2f(wp[ic]);
          }
        }
        y[(((size_t)in * p + ip) * q + iq) * c + k] = f2h(acc);
      }
    }
  }
}

/* dx[n][h][w][8g+c] = sum_{r,s,k in group g} dy[n][h+pad_h-r][w+pad_w-s][k] * w[k][r][s][c]. */
void oracle_conv2d_gw8_dgrad(uint16_t* dx, const uint16_t* dy, const uint16_t* w, int n, int c,
                             int h, int wd, int r, int s, int pad_h, int pad_w) {
  const int p = h + 2 * pad_h - r + 1, q = wd + 2 * pad_w - s + 1;
  const long rows = (long)n * h;
#pragma omp parallel for schedule(static)
  for (long row = 0; row < rows; ++row) {
    const int in = (int)(row / h), ih = (int)(row % h);
    for (int iw = 0; iw < wd; ++iw) {
      for (int ch = 0; ch < c; ++ch) {
        const int g = ch / 8, ic = ch % 8;
        float acc = 0.0f;
        for (int ir = 0; ir < r; ++ir) {
          const int ip = ih + pad_h - ir;
          if (ip < 0 || ip >= p) continue;
          for (int is = 0; is < s; ++is) {
            const int iq = iw + pad_w - is;
            if (iq < 0 || iq >= q) continue;
            const uint16_t* dp = dy + (((size_t)in * p + ip) * q + iq) * c + 8 * g;
            for (int kk = 0; kk < 8; ++kk) {
              const int k = 8 * g + kk;
              acc += h2f(dp[kk]) * h2f(w[(((size_t)k * r + ir) * s + is) * 8 + ic]);
            }
          }
        }
        dx[(((size_t)in * h + ih) * wd + iw) * c + ch] = f2h(acc);
      }
    }
  }
}

/* dw[k][r][s][c] = sum_{n,p,q} x[n][p+r-pad_h][q+s-pad_w][8g+c] * dy[n][p][q][k], fp32 result.
 * Each thread owns whole output channels, so the sum order is fixed: (n, p, q).  The sum
 * runs over up to millions of pixels; the checker keeps it in double so that its own
 * rounding does not use up the tolerance the kernels are held to. */
void oracle_conv2d_gw8_wgrad(float* dw, const uint16_t* x, const uint16_t* dy, int n, int c, int h,
                             int wd, int r, int s, int pad_h, int pad_w) {
  const int p = h + 2 * pad_h - r + 1, q = wd + 2 * pad_w - s + 1;
#pragma omp parallel for schedule(dynamic, 1)
  for (int k = 0; k < c; ++k) {
    const int g = k / 8;
    double out[5 * 5 * 8];
    for (int i = 0; i < r * s * 8; ++i) out[i] = 0.0;
    for (int in = 0; in < n; ++in)
      for (int ip = 0; ip < p; ++ip)
        for (int iq = 0; iq < q; ++iq) {
          const double d = (double)h2f(dy[(((size_t)in * p + ip) * q + iq) * c + k]);
          for (int ir = 0; ir < r; ++ir) {
            const int ih = ip + ir - pad_h;
            if (ih < 0 || ih >= h) continue;
            for (int is = 0; is < s; ++is) {
              const int iw = iq + is - pad_w;
              if (iw < 0 || iw >= wd) continue;
              const uint16_t* xp = x + (((size_t)in * h + ih) * wd + iw) * c + 8 * g;
              double* o = out + (ir * s + is) * 8;
              for (int ic = 0; ic < 8; ++ic) o[ic] += (double)h2f(xp[ic]) * d;
            }
          }
        }
    for (int i = 0; i < r * s * 8; ++i) dw[(size_t)k * r * s * 8 + i] = (float)out[i];
  }
}
