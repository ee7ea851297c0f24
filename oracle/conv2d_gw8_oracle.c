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
#include <pthread.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

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

/* ---- a minimal parallel-for over independent work items (pthreads) ---- */

static int g_threads = 0; /* 0 = all online cores */

void oracle_set_num_threads(int n) { g_threads = n > 0 ? n : 0; }

int oracle_num_threads(void) {
  if (g_threads > 0) return g_threads;
  const char* env = getenv("ORACLE_THREADS");
  if (env && atoi(env) > 0) return atoi(env);
  long n = sysconf(_SC_NPROCESSORS_ONLN);
  return n > 0 ? (int)n : 1;
}

typedef struct {
  uint16_t* y16;
  float* y32;
  const uint16_t* a;
  const uint16_t* b;
  const float* bias;
  int n, c, h, wd, r, s, pad_h, pad_w, p, q;
} conv_args;

typedef void (*item_fn)(const conv_args*, long item);

typedef struct {
  const conv_args* args;
  item_fn fn;
  long begin, end;
} work_span;

static void* run_span(void* vp) {
  work_span* w = (work_span*)vp;
  for (long i = w->begin; i < w->end; ++i) w->fn(w->args, i);
  return NULL;
}

static void parallel_for(const conv_args* args, item_fn fn, long items) {
  int nt = oracle_num_threads();
  if (nt > items) nt = (int)items;
  if (nt <= 1) {
    work_span w = {args, fn, 0, items};
    run_span(&w);
    return;
  }
  pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)nt);
  work_span* sp = (work_span*)malloc(sizeof(work_span) * (size_t)nt);
  for (int t = 0; t < nt; ++t) {
    sp[t].args = args;
    sp[t].fn = fn;
    sp[t].begin = items * t / nt;
    sp[t].end = items * (t + 1) / nt;
    pthread_create(&th[t], NULL, run_span, &sp[t]);
  }
  for (int t = 0; t < nt; ++t) pthread_join(th[t], NULL);
  free(th);
  free(sp);
}

/* ---- fprop: one item = one output row (n, p) ---- */

/* y[n][p][q][k] = bias[k] + sum_{r,s,c<8} x[n][p+r-pad_h][q+s-pad_w][8g+c] * w[k][r][s][c],
 * g = k / 8.  Terms are added in (r, s, c) order starting from the bias. */
static void fprop_row(const conv_args* a, long row) {
  const int in = (int)(row / a->p), ip = (int)(row % a->p);
  const int c = a->c, h = a->h, wd = a->wd, r = a->r, s = a->s;
  for (int iq = 0; iq < a->q; ++iq) {
    for (int k = 0; k < c; ++k) {
      const int g = k / 8;
      float acc = a->bias ? a->bias[k] : 0.0f;
      for (int ir = 0; ir < r; ++ir) {
        const int ih = ip + ir - a->pad_h;
        if (ih < 0 || ih >= h) continue;
        for (int is = 0; is < s; ++is) {
          const int iw = iq + is - a->pad_w;
          if (iw < 0 || iw >= wd) continue;
          const uint16_t* xp = a->a + (((size_t)in * h + ih) * wd + iw) * c + 8 * g;
          const uint16_t* wp = a->b + (((size_t)k * r + ir) * s + is) * 8;
          for (int ic = 0; ic < 8; ++ic) acc += h2f(xp[ic]) * h2f(wp[ic]);
        }
      }
      a->y16[(((size_t)in * a->p + ip) * a->q + iq) * c + k] = f2h(acc);
    }
  }
}

void oracle_conv2d_gw8_fprop(uint16_t* y, const uint16_t* x, const uint16_t* w, const float* bias,
                             int n, int c, int h, int wd, int r, int s, int pad_h, int pad_w) {
  conv_args a = {y, NULL, x, w, bias, n, c, h, wd, r, s, pad_h, pad_w,
                 h + 2 * pad_h - r + 1, wd + 2 * pad_w - s + 1};
  parallel_for(&a, fprop_row, (long)n * a.p);
}

/* ---- dgrad: one item = one input row (n, h) ---- */

/* dx[n][h][w][8g+c] = sum_{r,s,k in group g} dy[n][h+pad_h-r][w+pad_w-s][k] * w[k][r][s][c]. */
static void dgrad_row(const conv_args* a, long row) {
  const int in = (int)(row / a->h), ih = (int)(row % a->h);
  const int c = a->c, r = a->r, s = a->s, p = a->p, q = a->q;
  for (int iw = 0; iw < a->wd; ++iw) {
    for (int ch = 0; ch < c; ++ch) {
      const int g = ch / 8, ic = ch % 8;
      float acc = 0.0f;
      for (int ir = 0; ir < r; ++ir) {
        const int ip = ih + a->pad_h - ir;
        if (ip < 0 || ip >= p) continue;
        for (int is = 0; is < s; ++is) {
          const int iq = iw + a->pad_w - is;
          if (iq < 0 || iq >= q) continue;
          const uint16_t* dp = a->a + (((size_t)in * p + ip) * q + iq) * c + 8 * g;
          for (int kk = 0; kk < 8; ++kk) {
            const int k = 8 * g + kk;
            acc += h2f(dp[kk]) * h2f(a->b[(((size_t)k * r + ir) * s + is) * 8 + ic]);
          }
        }
      }
      a->y16[(((size_t)in * a->h + ih) * a->wd + iw) * c + ch] = f2h(acc);
    }
  }
}

void oracle_conv2d_gw8_dgrad(uint16_t* dx, const uint16_t* dy, const uint16_t* w, int n, int c,
                             int h, int wd, int r, int s, int pad_h, int pad_w) {
  conv_args a = {dx, NULL, dy, w, NULL, n, c, h, wd, r, s, pad_h, pad_w,
                 h + 2 * pad_h - r + 1, wd + 2 * pad_w - s + 1};
  parallel_for(&a, dgrad_row, (long)n * h);
}

/* ---- wgrad: one item = one output channel k ---- */

/* dw[k][r][s][c] = sum_{n,p,q} x[n][p+r-pad_h][q+s-pad_w][8g+c] * dy[n][p][q][k], fp32 result.
 * A thread owns whole output channels, so the sum order is fixed: (n, p, q).  The sum
 * runs over up to millions of pixels; the checker keeps it in double so that its own
 * rounding does not use up the tolerance the kernels are held to. */
static void wgrad_channel(const conv_args* a, long item) {
  const int k = (int)item, g = k / 8;
  const int c = a->c, h = a->h, wd = a->wd, r = a->r, s = a->s, p = a->p, q = a->q;
  double out[5 * 5 * 8];
  for (int i = 0; i < r * s * 8; ++i) out[i] = 0.0;
  for (int in = 0; in < a->n; ++in)
    for (int ip = 0; ip < p; ++ip)
      for (int iq = 0; iq < q; ++iq) {
        const double d = (double)h2f(a->b[(((size_t)in * p + ip) * q + iq) * c + k]);
        for (int ir = 0; ir < r; ++ir) {
          const int ih = ip + ir - a->pad_h;
          if (ih < 0 || ih >= h) continue;
          for (int is = 0; is < s; ++is) {
            const int iw = iq + is - a->pad_w;
            if (iw < 0 || iw >= wd) continue;
            const uint16_t* xp = a->a + (((size_t)in * h + ih) * wd + iw) * c + 8 * g;
            double* o = out + (ir * s + is) * 8;
            for (int ic = 0; ic < 8; ++ic) o[ic] += (double)h2f(xp[ic]) * d;
          }
        }
      }
  for (int i = 0; i < r * s * 8; ++i) a->y32[(size_t)k * r * s * 8 + i] = (float)out[i];
}

void oracle_conv2d_gw8_wgrad(float* dw, const uint16_t* x, const uint16_t* dy, int n, int c, int h,
                             int wd, int r, int s, int pad_h, int pad_w) {
  conv_args a = {NULL, dw, x, dy, NULL, n, c, h, wd, r, s, pad_h, pad_w,
                 h + 2 * pad_h - r + 1, wd + 2 * pad_w - s + 1};
  parallel_for(&a, wgrad_channel, (long)c);
}
