/* conv2d_oracle.c -- CPU restatement of the reference's Conv2d, for checking only.
 *
 * TEST INFRASTRUCTURE. Nothing that ships links, imports or calls this file: it is used by tests/,
 * by the smoke check and by the CPU-baseline leg of the benchmark, always as the checker or the
 * timed baseline, never as a compute path of the library.
 *
 * What it restates (paths relative to the reference project's root):
 *   - oracle_conv2d: the 7-deep loop nest, index formulas, zero padding and fp32 accumulation of
 *     `cpu_conv2d` in examples/verify_conv2d.rs:8-44, with the output-size formula of
 *     src/emitter/cuda/conv.rs:40-41, generalised from (NHWC, RSCK) to arbitrary element strides
 *     over the logical NCHW / OIHW index space and to separate h / w stride, padding and dilation.
 *   - the epilogue: bias -> residual -> activation in fp32, formulas of
 *     src/kernels/gpu/epilogue.cuh:12-63, op order of src/interface/c_bindings.rs:144-197 and
 *     src/interface/python.rs:41-87.
 *   - oracle_conv2d_gemm: the reference's SIMD CPU engine (src/kernels/cpu/gemm.rs:12-180, 208-298:
 *     Mc x Kc blocking, A and B panel packing, 6 x 16 AVX2/FMA register tile, one parallel task
 *     per Mc block) fed by an im2col gather, because the reference has no CPU conv kernel of its
 *     own (src/emitter/cpu.rs:53-55 rejects Conv2d).
 *
 * Pinning: the reference's tests hold no golden vectors for conv (its conv checks draw unseeded
 * random inputs). This file is pinned instead against fixtures produced by
 * torch.nn.functional.conv2d -- the reference's own comparison target
 * (examples/jit_conv_verify.py:20-26) and the result its Python op returns
 * (tracea-python/src/conv2d.rs:80-136) -- see tests/golden/.
 */
#include <immintrin.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

enum { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU = 2, ACT_SILU = 3 };

static inline float act_apply(float x, int act) {
  switch (act) {
    case ACT_RELU: return fmaxf(0.0f, x);
    case ACT_GELU: return 0.5f * x * (1.0f + tanhf(0.79788456f * (x + 0.044715f * x * x * x)));
    case ACT_SILU: return x / (1.0f + expf(-x));
    default: return x;
  }
}

typedef struct {
  long long N, C, H, W;      /* input, logical NCHW */
  long long K, R, S;         /* filter, logical OIHW = [K, C, R, S] */
  long long stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
  long long xs[4];           /* element strides of x   for (n, c, h, w) */
  long long ws[4];           /* element strides of w   for (k, c, r, s) */
  long long os[4];           /* element strides of out for (n, k, ho, wo) */
  long long rs[4];           /* element strides of residual, same index space as out */
  int act;                   /* ACT_* */
  int acc_double;            /* 1: accumulate the dot product in double (sampled high-precision checks) */
} OracleConvDesc;

long long oracle_out_extent(long long in, long long pad, long long dil, long long filt, long long stride) {
  return (in + 2 * pad - dil * (filt - 1) - 1) / stride + 1;
}

/* Scalar direct convolution. bias / residual may be NULL. All data fp32 (callers round inputs to
 * the storage type first and round the result afterwards). Returns 0. */
int oracle_conv2d(const OracleConvDesc* d, const float* x, const float* w, const float* bias,
                  const float* residual, float* out) {
  const long long Ho = oracle_out_extent(d->H, d->pad_h, d->dil_h, d->R, d->stride_h);
  const long long Wo = oracle_out_extent(d->W, d->pad_w, d->dil_w, d->S, d->stride_w);
#pragma omp parallel for collapse(2) schedule(static)
  for (long long n = 0; n < d->N; ++n) {
    for (long long ho = 0; ho < Ho; ++ho) {
      for (long long wo = 0; wo < Wo; ++wo) {
        for (long long k = 0; k < d->K; ++k) {
          float acc = 0.0f;
          double acc_d = 0.0;
          for (long long r = 0; r < d->R; ++r) {
            const long long hi = ho * d->stride_h - d->pad_h + r * d->dil_h;
            if (hi < 0 || hi >= d->H) continue;
            for (long long s = 0; s < d->S; ++s) {
              const long long wi = wo * d->stride_w - d->pad_w + s * d->dil_w;
              if (wi < 0 || wi >= d->W) continue;
              const float* xp = x + n * d->xs[0] + hi * d->xs[2] + wi * d->xs[3];
              const float* wp = w + k * d->ws[0] + r * d->ws[2] + s * d->ws[3];
              if (d->acc_double) {
                for (long long c = 0; c < d->C; ++c)
                  acc_d += (double)xp[c * d->xs[1]] * (double)wp[c * d->ws[1]];
              } else {
                for (long long c = 0; c < d->C; ++c) acc += xp[c * d->xs[1]] * wp[c * d->ws[1]];
              }
            }
          }
          float v = d->acc_double ? (float)acc_d : acc;
          if (bias) v += bias[k];
          if (residual)
            v += residual[n * d->rs[0] + k * d->rs[1] + ho * d->rs[2] + wo * d->rs[3]];
          v = act_apply(v, d->act);
          out[n * d->os[0] + k * d->os[1] + ho * d->os[2] + wo * d->os[3]] = v;
        }
      }
    }
  }
  return 0;
}

/* Same arithmetic for a list of output points only: idx[4*i..] = (n, k, ho, wo); result in vals[i].
 * Used to spot-check full-size tensors the scalar loop cannot finish. */
int oracle_conv2d_points(const OracleConvDesc* d, const float* x, const float* w, const float* bias,
                         const float* residual, const long long* idx, long long count, float* vals) {
#pragma omp parallel for schedule(static)
  for (long long i = 0; i < count; ++i) {
    const long long n = idx[4 * i], k = idx[4 * i + 1], ho = idx[4 * i + 2], wo = idx[4 * i + 3];
    double acc = 0.0;
    float accf = 0.0f;
    for (long long r = 0; r < d->R; ++r) {
      const long long hi = ho * d->stride_h - d->pad_h + r * d->dil_h;
      if (hi < 0 || hi >= d->H) continue;
      for (long long s = 0; s < d->S; ++s) {
        const long long wi = wo * d->stride_w - d->pad_w + s * d->dil_w;
        if (wi < 0 || wi >= d->W) continue;
        const float* xp = x + n * d->xs[0] + hi * d->xs[2] + wi * d->xs[3];
        const float* wp = w + k * d->ws[0] + r * d->ws[2] + s * d->ws[3];
        for (long long c = 0; c < d->C; ++c) {
          if (d->acc_double) acc += (double)xp[c * d->xs[1]] * (double)wp[c * d->ws[1]];
          else accf += xp[c * d->xs[1]] * wp[c * d->ws[1]];
        }
      }
    }
    float v = d->acc_double ? (float)acc : accf;
    if (bias) v += bias[k];
    if (residual) v += residual[n * d->rs[0] + k * d->rs[1] + ho * d->rs[2] + wo * d->rs[3]];
    vals[i] = act_apply(v, d->act);
  }
  return 0;
}

/* ------------------------------------------------------------------------------------------
 * im2col + packed GEMM: the reference's CPU SIMD engine applied to conv.
 * x must be dense NHWC (xs = {H*W*C, 1, W*C, C}); w is read through its strides and packed as the
 * B matrix [Kgemm = (r, s, c)][K]; out / residual through their strides. fp32 throughout.
 * ------------------------------------------------------------------------------------------ */
#define MR 6
#define NR 16

#if defined(__AVX2__) && defined(__FMA__)
static void micro_6x16(const float* a, const float* b, long long kc, float* c, long long ldc, int first) {
  __m256 c00, c01, c10, c11, c20, c21, c30, c31, c40, c41, c50, c51;
  if (first) {
    c00 = c01 = c10 = c11 = c20 = c21 = c30 = c31 = c40 = c41 = c50 = c51 = _mm256_setzero_ps();
  } else {
    c00 = _mm256_loadu_ps(c + 0 * ldc); c01 = _mm256_loadu_ps(c + 0 * ldc + 8);
    c10 = _mm256_loadu_ps(c + 1 * ldc); c11 = _mm256_loadu_ps(c + 1 * ldc + 8);
    c20 = _mm256_loadu_ps(c + 2 * ldc); c21 = _mm256_loadu_ps(c + 2 * ldc + 8);
    c30 = _mm256_loadu_ps(c + 3 * ldc); c31 = _mm256_loadu_ps(c + 3 * ldc + 8);
    c40 = _mm256_loadu_ps(c + 4 * ldc); c41 = _mm256_loadu_ps(c + 4 * ldc + 8);
    c50 = _mm256_loadu_ps(c + 5 * ldc); c51 = _mm256_loadu_ps(c + 5 * ldc + 8);
  }
  for (long long l = 0; l < kc; ++l) {
    const __m256 b0 = _mm256_loadu_ps(b), b1 = _mm256_loadu_ps(b + 8);
    __m256 av;
    av = _mm256_broadcast_ss(a + 0); c00 = _mm256_fmadd_ps(av, b0, c00); c01 = _mm256_fmadd_ps(av, b1, c01);
    av = _mm256_broadcast_ss(a + 1); c10 = _mm256_fmadd_ps(av, b0, c10); c11 = _mm256_fmadd_ps(av, b1, c11);
    av = _mm256_broadcast_ss(a + 2); c20 = _mm256_fmadd_ps(av, b0, c20); c21 = _mm256_fmadd_ps(av, b1, c21);
    av = _mm256_broadcast_ss(a + 3); c30 = _mm256_fmadd_ps(av, b0, c30); c31 = _mm256_fmadd_ps(av, b1, c31);
    av = _mm256_broadcast_ss(a + 4); c40 = _mm256_fmadd_ps(av, b0, c40); c41 = _mm256_fmadd_ps(av, b1, c41);
    av = _mm256_broadcast_ss(a + 5); c50 = _mm256_fmadd_ps(av, b0, c50); c51 = _mm256_fmadd_ps(av, b1, c51);
    a += MR;
    b += NR;
  }
  _mm256_storeu_ps(c + 0 * ldc, c00); _mm256_storeu_ps(c + 0 * ldc + 8, c01);
  _mm256_storeu_ps(c + 1 * ldc, c10); _mm256_storeu_ps(c + 1 * ldc + 8, c11);
  _mm256_storeu_ps(c + 2 * ldc, c20); _mm256_storeu_ps(c + 2 * ldc + 8, c21);
  _mm256_storeu_ps(c + 3 * ldc, c30); _mm256_storeu_ps(c + 3 * ldc + 8, c31);
  _mm256_storeu_ps(c + 4 * ldc, c40); _mm256_storeu_ps(c + 4 * ldc + 8, c41);
  _mm256_storeu_ps(c + 5 * ldc, c50); _mm256_storeu_ps(c + 5 * ldc + 8, c51);
}
#else
static void micro_6x16(const float* a, const float* b, long long kc, float* c, long long ldc, int first) {
  float acc[MR][NR];
  for (int i = 0; i < MR; ++i)
    for (int j = 0; j < NR; ++j) acc[i][j] = first ? 0.0f : c[i * ldc + j];
  for (long long l = 0; l < kc; ++l)
    for (int i = 0; i < MR; ++i)
      for (int j = 0; j < NR; ++j) acc[i][j] += a[l * MR + i] * b[l * NR + j];
  for (int i = 0; i < MR; ++i)
    for (int j = 0; j < NR; ++j) c[i * ldc + j] = acc[i][j];
}
#endif

int oracle_conv2d_gemm(const OracleConvDesc* d, const float* x, const float* w, const float* bias,
                       const float* residual, float* out, int num_threads) {
  const long long Ho = oracle_out_extent(d->H, d->pad_h, d->dil_h, d->R, d->stride_h);
  const long long Wo = oracle_out_extent(d->W, d->pad_w, d->dil_w, d->S, d->stride_w);
  const long long M = d->N * Ho * Wo, Kg = d->R * d->S * d->C, Nn = d->K;
  const long long Np = (Nn + NR - 1) / NR * NR;
  const long long MC = 96, KC = 384;
  /* dense NHWC memory; the stride of an extent-1 axis carries no information and is not checked */
  if ((d->C > 1 && d->xs[1] != 1) || (d->W > 1 && d->xs[3] != d->C) || (d->H > 1 && d->xs[2] != d->W * d->C) ||
      (d->N > 1 && d->xs[0] != d->H * d->W * d->C))
    return -1;
#ifdef _OPENMP
  if (num_threads > 0) omp_set_num_threads(num_threads);
#else
  (void)num_threads;
#endif
  /* B packed once: for each Kc block, panels of [kc][16] */
  float* bp = (float*)aligned_alloc(64, sizeof(float) * (size_t)(Kg * Np));
  if (!bp) return -2;
#pragma omp parallel for schedule(static)
  for (long long k0 = 0; k0 < Kg; k0 += KC) {
    const long long kc = (Kg - k0 < KC) ? Kg - k0 : KC;
    float* dst = bp + k0 * Np;
    for (long long nb = 0; nb < Np; nb += NR) {
      for (long long l = 0; l < kc; ++l) {
        const long long kk = k0 + l;
        const long long c = kk % d->C, rs = kk / d->C, s = rs % d->S, r = rs / d->S;
        for (long long j = 0; j < NR; ++j) {
          const long long n = nb + j;
          *dst++ = (n < Nn) ? w[n * d->ws[0] + c * d->ws[1] + r * d->ws[2] + s * d->ws[3]] : 0.0f;
        }
      }
    }
  }
  int fail = 0;
#pragma omp parallel
  {
    float* ap = (float*)aligned_alloc(64, sizeof(float) * (size_t)((MC + MR) * KC));
    float* cb = (float*)aligned_alloc(64, sizeof(float) * (size_t)((MC + MR) * Np));
    if (!ap || !cb) {
#pragma omp atomic write
      fail = 1;
    }
#pragma omp barrier
    if (!fail) {
#pragma omp for schedule(dynamic, 1)
      for (long long m0 = 0; m0 < M; m0 += MC) {
        const long long mc = (M - m0 < MC) ? M - m0 : MC;
        for (long long k0 = 0; k0 < Kg; k0 += KC) {
          const long long kc = (Kg - k0 < KC) ? Kg - k0 : KC;
          /* pack A: im2col gather straight into Mr-row panels [kc][6] */
          for (long long mi = 0; mi < mc; mi += MR) {
            float* dst = ap + mi * kc;
            const float* rowp[MR];
            long long hb[MR], wb[MR];
            for (int i = 0; i < MR; ++i) {
              const long long m = m0 + mi + i;
              if (m < M) {
                const long long wo = m % Wo, t = m / Wo, ho = t % Ho, n = t / Ho;
                rowp[i] = x + n * d->xs[0];
                hb[i] = ho * d->stride_h - d->pad_h;
                wb[i] = wo * d->stride_w - d->pad_w;
              } else {
                rowp[i] = NULL; hb[i] = wb[i] = 0;
              }
            }
            for (long long l = 0; l < kc; ++l) {
              const long long kk = k0 + l;
              const long long c = kk % d->C, rs = kk / d->C, s = rs % d->S, r = rs / d->S;
              for (int i = 0; i < MR; ++i) {
                float v = 0.0f;
                if (rowp[i]) {
                  const long long hi = hb[i] + r * d->dil_h, wi = wb[i] + s * d->dil_w;
                  if (hi >= 0 && hi < d->H && wi >= 0 && wi < d->W)
                    v = rowp[i][(hi * d->W + wi) * d->C + c];
                }
                dst[l * MR + i] = v;
              }
            }
          }
          const float* bblk = bp + k0 * Np;
          for (long long mi = 0; mi < mc; mi += MR)
            for (long long nb = 0; nb < Np; nb += NR)
              micro_6x16(ap + mi * kc, bblk + nb * kc, kc, cb + mi * Np + nb, Np, k0 == 0);
        }
        /* epilogue for this Mc block */
        for (long long mi = 0; mi < mc; ++mi) {
          const long long m = m0 + mi;
          const long long wo = m % Wo, t = m / Wo, ho = t % Ho, n = t / Ho;
          for (long long k = 0; k < Nn; ++k) {
            float v = cb[mi * Np + k];
            if (bias) v += bias[k];
            if (residual) v += residual[n * d->rs[0] + k * d->rs[1] + ho * d->rs[2] + wo * d->rs[3]];
            out[n * d->os[0] + k * d->os[1] + ho * d->os[2] + wo * d->os[3]] = act_apply(v, d->act);
          }
        }
      }
    }
    free(ap);
    free(cb);
  }
  free(bp);
  return fail ? -2 : 0;
}

int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
