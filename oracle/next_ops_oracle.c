/* next_ops_oracle.c -- CPU restatements of the two operators either side of the conv path:
 * ConvTranspose2d and GEMM with the conv epilogue. For checking only.
 *
 * TEST INFRASTRUCTURE. Nothing that ships links, imports or calls this file.
 *
 * What it restates (paths relative to the reference project's root):
 *   - oracle_conv_transpose2d: the scatter loop nest of `cpu_conv_transpose2d` in
 *     examples/verify_conv_transpose.rs:12-52 (ho = hi*stride - pad + r; every input pixel adds
 *     x * w to the outputs it reaches; fp32 accumulation in the output), with the output-size
 *     formula (h_in - 1)*stride - 2*pad + r + output_padding of src/interface/c_bindings.rs:343-344,
 *     generalised from (NHWC input, [C*R*S][K] weights) to element strides over the index spaces
 *     x[n, h, w, c], w[k, r, s, c], out[n, ho, wo, k] (the shapes tracea-python/python/tracea/ops.py:72-88
 *     passes) and to separate h / w stride and padding. The gather form the reference's CUDA kernel uses
 *     (src/emitter/conv_transpose.rs:208-229: ho_adj = ho + pad - r must be a multiple of stride)
 *     selects the same (hi, r) pairs.
 *   - oracle_gemm: C = epilogue(A[M,K] * B[K,N]) with fp32 accumulation, the contract of
 *     tracea_gemm (include/tracea.hpp:139-144; src/interface/c_bindings.rs:375-440), checked in the
 *     reference by tests of the same shape (tests/numerical_parity.rs, examples/verify_epilogue.rs).
 *   - the epilogue: bias -> residual -> activation (src/kernels/gpu/epilogue.cuh:12-63;
 *     src/interface/c_bindings.rs:144-197).
 *
 * Pinning: the reference holds no golden vectors for these operators (its checks draw unseeded random
 * inputs); this file is pinned against fixtures produced by torch.nn.functional.conv_transpose2d and
 * torch.matmul, see tests/golden/.
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

enum { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU = 2, ACT_SILU = 3 };

static inline float act_apply2(float x, int act) {
  switch (act) {
    case ACT_RELU: return fmaxf(0.0f, x);
    case ACT_GELU: return 0.5f * x * (1.0f + tanhf(0.79788456f * (x + 0.044715f * x * x * x)));
    case ACT_SILU: return x / (1.0f + expf(-x));
    default: return x;
  }
}

typedef struct {
  long long N, H, W, C;      /* input  x[n, h, w, c] */
  long long K, R, S;         /* filter w[k, r, s, c] */
  long long stride_h, stride_w, pad_h, pad_w, opad_h, opad_w;
  long long xs[4];           /* element strides of x   for (n, h, w, c) */
  long long ws[4];           /* element strides of w   for (k, r, s, c) */
  long long os[4];           /* element strides of out for (n, ho, wo, k) */
  long long rs[4];           /* element strides of residual, same index space as out */
  int act;
} OracleConvTDesc;

long long oracle_conv_transpose_extent(long long in, long long pad, long long filt, long long stride, long long opad) {
  return (in - 1) * stride - 2 * pad + filt + opad;
}

/* Accumulates into a dense fp32 scratch of N*Ho*Wo*K values, then applies the epilogue. bias / residual may
 * be NULL. Returns 0, or non-zero when the output would be empty or the scratch cannot be had. */
int oracle_conv_transpose2d(const OracleConvTDesc* d, const float* x, const float* w, const float* bias,
                            const float* residual, float* out) {
  const long long Ho = oracle_conv_transpose_extent(d->H, d->pad_h, d->R, d->stride_h, d->opad_h);
  const long long Wo = oracle_conv_transpose_extent(d->W, d->pad_w, d->S, d->stride_w, d->opad_w);
  if (Ho <= 0 || Wo <= 0) return 1;
  float* acc = (float*)calloc((size_t)(d->N * Ho * Wo * d->K), sizeof(float));
  if (!acc) return 2;
#pragma omp parallel for schedule(static)
  for (long long n = 0; n < d->N; ++n) {
    for (long long hi = 0; hi < d->H; ++hi)
      for (long long wi = 0; wi < d->W; ++wi)
        for (long long c = 0; c < d->C; ++c) {
          const float xv = x[n * d->xs[0] + hi * d->xs[1] + wi * d->xs[2] + c * d->xs[3]];
          for (long long r = 0; r < d->R; ++r) {
            const long long ho = hi * d->stride_h - d->pad_h + r;
            if (ho < 0 || ho >= Ho) continue;
            for (long long s = 0; s < d->S; ++s) {
              const long long wo = wi * d->stride_w - d->pad_w + s;
              if (wo < 0 || wo >= Wo) continue;
              float* ap = acc + ((n * Ho + ho) * Wo + wo) * d->K;
              const float* wp = w + r * d->ws[1] + s * d->ws[2] + c * d->ws[3];
              for (long long k = 0; k < d->K; ++k) ap[k] += xv * wp[k * d->ws[0]];
            }
          }
        }
  }
  for (long long n = 0; n < d->N; ++n)
    for (long long ho = 0; ho < Ho; ++ho)
      for (long long wo = 0; wo < Wo; ++wo)
        for (long long k = 0; k < d->K; ++k) {
          float v = acc[((n * Ho + ho) * Wo + wo) * d->K + k];
          if (bias) v += bias[k];
          if (residual) v += residual[n * d->rs[0] + ho * d->rs[1] + wo * d->rs[2] + k * d->rs[3]];
          out[n * d->os[0] + ho * d->os[1] + wo * d->os[2] + k * d->os[3]] = act_apply2(v, d->act);
        }
  free(acc);
  return 0;
}

typedef struct {
  long long M, N, K;
  long long as[2], bs[2], cs[2], rs[2];   /* element strides of A[m,k], B[k,n], C[m,n], residual[m,n] */
  int act;
} OracleGemmDesc;

int oracle_gemm(const OracleGemmDesc* d, const float* a, const float* b, const float* bias, const float* residual,
                float* c) {
#pragma omp parallel for schedule(static)
  for (long long m = 0; m < d->M; ++m)
    for (long long n = 0; n < d->N; ++n) {
      float acc = 0.0f;
      for (long long k = 0; k < d->K; ++k) acc += a[m * d->as[0] + k * d->as[1]] * b[k * d->bs[0] + n * d->bs[1]];
      if (bias) acc += bias[n];
      if (residual) acc += residual[m * d->rs[0] + n * d->rs[1]];
      c[m * d->cs[0] + n * d->cs[1]] = act_apply2(acc, d->act);
    }
  return 0;
}
