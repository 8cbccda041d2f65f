/*
 * CPU oracle for the LiteNN op-layer hot path.  TEST INFRASTRUCTURE ONLY: it may be
 * called from tests/, from __graft_entry__.smoke() and from bench.py's cpu_baseline /
 * reference arm, never from the product (litenn_b200/).
 *
 * Each function restates, in plain C, what one family of the reference's generated
 * OpenCL kernels computes (iperov/litenn, file:line cited per function), with the same
 * operand order, single-precision literals (the reference builds with
 * -cl-single-precision-constant, litenn/core/minicl/CLDevice.py:93) and one rounding per
 * source-level operation: compile with -ffp-contract=off.  OpenCL's float exp/log/sin/cos
 * are restated as the double libm function rounded once to float.
 *
 * Parity pinned: tests/test_oracle_golden.py checks every function here against outputs
 * of the reference's own Python op layer and kernel text (the .npz files under tests/golden, produced by
 * tests/golden/make_golden.py).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define MAXD 6
typedef int64_t i64;

/* ---- element-wise: litenn/core/op/element_wise_op.py:112-364 ------------------------- */
enum { EW_ABS, EW_ADD_CONST, EW_CLIP, EW_COS, EW_EXP, EW_LEAKY_RELU, EW_LOG, EW_MUL_CONST,
       EW_RDIV_CONST, EW_RSUB_CONST, EW_RELU, EW_SIGMOID, EW_SIN, EW_SQRT, EW_SQUARE, EW_TANH };

static float f_exp(float x) { return (float)exp((double)x); }
static float f_log(float x) { return (float)log((double)x); }
static float f_sin(float x) { return (float)sin((double)x); }
static float f_cos(float x) { return (float)cos((double)x); }

static float ew_f(int op, float I, float p0, float p1) {
  switch (op) {
    case EW_ABS: return fabsf(I);                                              /* :113 */
    case EW_ADD_CONST: return I + p0;                                          /* :124 */
    case EW_CLIP: return I * (float)((I >= p0) & (I <= p1)) + p0 * (float)(I < p0) + p1 * (float)(I > p1); /* :137 */
    case EW_COS: return f_cos(I);                                              /* :180 */
    case EW_EXP: return f_exp(I);                                              /* :194 */
    case EW_LEAKY_RELU: return I * (float)(I >= 0.0f) + p0 * I * (float)(I < 0.0f); /* :210 */
    case EW_LOG: return f_log(I);                                              /* :225 */
    case EW_MUL_CONST: return I * p0;                                          /* :243 */
    case EW_RDIV_CONST: return p0 / I;                                         /* :253 */
    case EW_RSUB_CONST: return p0 - I;                                         /* :263 */
    case EW_RELU: return I * (float)(I >= 0.0f);                               /* :272 */
    case EW_SIGMOID: return 1.0f / (1.0f + f_exp(-I));                         /* :287 */
    case EW_SIN: return f_sin(I);                                              /* :302 */
    case EW_SQRT: return sqrtf(I);                                             /* :317 */
    case EW_SQUARE: return I * I;                                              /* :332 */
    case EW_TANH: return 2.0f / (1.0f + f_exp(-2.0f * I)) - 1.0f;              /* :352 */
  }
  return 0.0f;
}

static float ew_g(int op, float I, float O, float dO, float p0, float p1, int flag) {
  switch (op) {
    case EW_ABS: return dO * (I / fabsf(I));
    case EW_ADD_CONST: return dO;
    case EW_CLIP: return flag ? dO : dO * (float)((I >= p0) & (I <= p1));
    case EW_COS: return dO * -f_sin(I);
    case EW_EXP: return dO * f_exp(I);
    case EW_LEAKY_RELU: return dO * ((float)(I >= 0.0f) + p0 * (float)(I < 0.0f));
    case EW_LOG: return dO * (1.0f / I);
    case EW_MUL_CONST: return dO * p0;
    case EW_RDIV_CONST: return dO * (-(p0 / (I * I)));
    case EW_RSUB_CONST: return -dO;
    case EW_RELU: return dO * (float)(I >= 0.0f);
    case EW_SIGMOID: return dO * (O * (1.0f - O));
    case EW_SIN: return dO * f_cos(I);
    case EW_SQRT: return dO * (1.0f / (2.0f * sqrtf(I)));
    case EW_SQUARE: return dO * 2.0f * I;
    case EW_TANH: return dO * (1.0f - O * O);
  }
  return 0.0f;
}

/* forward template element_wise_op.py:88-96 */
void lnn_o_eltwise_fwd(int op, float* O, const float* I, i64 n, float p0, float p1, int flag, int acc) {
  (void)flag;
#pragma omp parallel for
  for (i64 i = 0; i < n; ++i) {
    float r = ew_f(op, I[i], p0, p1);
    if (acc) O[i] += r; else O[i] = r;
  }
}

/* backward template element_wise_op.py:98-110 */
void lnn_o_eltwise_bwd(int op, float* dI, const float* I, const float* O, const float* dO, i64 n,
                       float p0, float p1, int flag) {
#pragma omp parallel for
  for (i64 i = 0; i < n; ++i) dI[i] += ew_g(op, I[i], O[i], dO[i], p0, p1, flag);
}

/* ---- broadcast binary: litenn/core/op/dual_wise_op.py:132-312 ------------------------ */
enum { BIN_ADD, BIN_SUB, BIN_MUL, BIN_DIV, BIN_MAX, BIN_MIN, BIN_BCE };

static float bin_f(int op, float A, float B) {
  switch (op) {
    case BIN_ADD: return A + B;
    case BIN_SUB: return A - B;
    case BIN_MUL: return A * B;
    case BIN_DIV: return A / B;
    case BIN_MAX: return fmaxf(A, B);
    case BIN_MIN: return fminf(A, B);
    case BIN_BCE: return -B * f_log(A) - (1.0f - B) * f_log(1.0f - A);          /* :207 */
  }
  return 0.0f;
}

static float bin_g(int op, int which, float A, float B, float O, float dO) {
  (void)O;
  if (which == 0) {
    switch (op) {
      case BIN_ADD: case BIN_SUB: return dO;
      case BIN_MUL: return dO * B;
      case BIN_DIV: return dO / B;
      case BIN_MAX: return dO * (float)(A >= B);
      case BIN_MIN: return dO * (float)(A <= B);
      case BIN_BCE: return dO * (A - B) / (A * (1.0f - A));
    }
  } else {
    switch (op) {
      case BIN_ADD: return dO;
      case BIN_SUB: return -dO;
      case BIN_MUL: return dO * A;
      case BIN_DIV: return dO * (-(A / (B * B)));
      case BIN_MAX: return dO * (float)(A < B);
      case BIN_MIN: return dO * (float)(A > B);
      case BIN_BCE: return dO;
    }
  }
  return 0.0f;
}

/* index-modulus broadcasting: CLKernelHelper.py:8-72 (X_idx_mod) */
static void bc_off(int rank, const i64* o, const i64* a, const i64* b, i64 gid, i64* ao, i64* bo) {
  i64 idx[MAXD];
  for (int k = rank - 1; k >= 0; --k) { idx[k] = gid % o[k]; gid /= o[k]; }
  i64 x = 0, y = 0;
  for (int k = 0; k < rank; ++k) { x = x * a[k] + idx[k] % a[k]; y = y * b[k] + idx[k] % b[k]; }
  *ao = x; *bo = y;
}

void lnn_o_binary_fwd(int op, float* O, const float* A, const float* B, int rank, const i64* o,
                      const i64* a, const i64* b, int acc) {
  i64 n = 1;
  for (int k = 0; k < rank; ++k) n *= o[k];
#pragma omp parallel for
  for (i64 i = 0; i < n; ++i) {
    i64 ao, bo;
    bc_off(rank, o, a, b, i, &ao, &bo);
    float r = bin_f(op, A[ao], B[bo]);
    if (acc) O[i] += r; else O[i] = r;
  }
}

void lnn_o_binary_bwd(int op, int which, float* dX, const float* A, const float* B, const float* O,
                      const float* dO, int rank, const i64* o, const i64* a, const i64* b) {
  i64 n = 1;
  for (int k = 0; k < rank; ++k) n *= o[k];
#pragma omp parallel for
  for (i64 i = 0; i < n; ++i) {
    i64 ao, bo;
    bc_off(rank, o, a, b, i, &ao, &bo);
    dX[i] += bin_g(op, which, A[ao], B[bo], O[i], dO[i]);
  }
}

/* y (+)= leaky_relu(x*g + b): the chain mul, add, leaky_relu as three rounded steps
 * (dual_wise_op.py:283-295,194-204; element_wise_op.py:207-221) */
void lnn_o_scale_bias_lrelu(float* Y, const float* X, const float* G, const float* Bv, i64 n, i64 c,
                            i64 hw, float alpha, int acc) {
  i64 total = n * c * hw;
#pragma omp parallel for
  for (i64 i = 0; i < total; ++i) {
    i64 ch = (i / hw) % c;
    float m = X[i] * G[ch];
    float t = m + Bv[ch];
    float r = t * (float)(t >= 0.0f) + alpha * t * (float)(t < 0.0f);
    if (acc) Y[i] += r; else Y[i] = r;
  }
}

/* ---- pooling: litenn/core/op/pool2D.py:111-230 ---------------------------------------- */
void lnn_o_pool2d_fwd(int mode, float* O, const float* I, i64 n, i64 c, int IH, int IW, int OH, int OW,
                      int P, int S, int PADL, int PADT) {
  i64 total = n * c * OH * OW;
#pragma omp parallel for
  for (i64 gid = 0; gid < total; ++gid) {
    int ow = (int)(gid % OW); i64 t = gid / OW; int oh = (int)(t % OH); i64 plane = t / OH;
    const float* ip = I + plane * IH * IW;
    float v = mode == 0 ? 0.0f : (mode == 1 ? -INFINITY : INFINITY);
    int cnt = 0;
    for (int ph = 0; ph < P; ++ph)
      for (int pw = 0; pw < P; ++pw) {
        int ih = -PADT + ph + oh * S, iw = -PADL + pw + ow * S;
        if ((iw >= 0) & (ih >= 0) & (iw < IW) & (ih < IH)) {
          float x = ip[(i64)ih * IW + iw];
          if (mode == 0) { v += x; ++cnt; } else if (mode == 1) v = fmaxf(v, x); else v = fminf(v, x);
        }
      }
    if (mode == 0) { if (cnt != 0) v /= cnt; }
    else if (mode == 1) { if (v == -INFINITY) v = 0.0f; }
    else { if (v == INFINITY) v = 0.0f; }
    O[gid] = v;
  }
}

void lnn_o_pool2d_bwd(int mode, float* dI, const float* I, const float* dO, const float* O, i64 n, i64 c,
                      int IH, int IW, int OH, int OW, int P, int S, int PADL, int PADT) {
  i64 total = n * c * IH * IW;
#pragma omp parallel for
  for (i64 gid = 0; gid < total; ++gid) {
    int iw = (int)(gid % IW); i64 t = gid / IW; int ih = (int)(t % IH); i64 plane = t / IH;
    const float* ip = I ? I + plane * IH * IW : 0;
    const float* op = O ? O + plane * OH * OW : 0;
    const float* dop = dO + plane * OH * OW;
    float v = 0.0f;
    for (int ph = 0; ph < P; ++ph)
      for (int pw = 0; pw < P; ++pw) {
        int oh = (PADT + ih - ph) / S, ow = (PADL + iw - pw) / S;
        if ((ow >= 0) & (oh >= 0) & (ow < OW) & (oh < OH) & (iw == (-PADL + pw + ow * S)) &
            (ih == (-PADT + ph + oh * S))) {
          if (mode == 0) {                                                       /* :147-180 */
            int d = 0;
            for (int dph = 0; dph < P; ++dph)
              for (int dpw = 0; dpw < P; ++dpw) {
                int dih = -PADT + dph + oh * S, diw = -PADL + dpw + ow * S;
                d += (diw >= 0) & (dih >= 0) & (diw < IW) & (dih < IH);
              }
            v += dop[(i64)oh * OW + ow] / d;
          } else {                                                               /* :181-230 */
            float Ov = op[(i64)oh * OW + ow];
            for (int k = 0; k < P * P; ++k) {
              int dih = -PADT + (k / P) + oh * S, diw = -PADL + (k % P) + ow * S;
              if ((diw >= 0) & (dih >= 0) & (diw < IW) & (dih < IH) && ip[(i64)dih * IW + diw] == Ov) {
                if ((dih == ih) & (diw == iw)) v += dop[(i64)oh * OW + ow];
                break;
              }
            }
          }
        }
      }
    dI[gid] += v;
  }
}

/* ---- reductions: litenn/core/op/reduce.py:166-205, stage kernel :279-293 ------------- */
/* Input [outer][r0][mid][r1][inner]; r0 and r1 reduced.  Each row is gathered (the
 * reference's transpose), reduced IN PLACE by the halving stages, divided for mean (:295-301)
 * and column 0 is stored (the reference's slice). */
void lnn_o_reduce(int op, float* O, const float* I, i64 outer, i64 r0, i64 mid, i64 r1, i64 inner, int acc) {
  i64 rows = outer * mid * inner, cols = r0 * r1;
#pragma omp parallel
  {
    float* row = (float*)malloc(sizeof(float) * (size_t)cols);
#pragma omp for
    for (i64 r = 0; r < rows; ++r) {
      i64 in_i = r % inner, t = r / inner, mid_i = t % mid, out_i = t / mid;
      for (i64 c = 0; c < cols; ++c) {
        i64 a = c / r1, b = c % r1;
        row[c] = I[(((out_i * r0 + a) * mid + mid_i) * r1 + b) * inner + in_i];
      }
      i64 valid = cols;
      while (valid > 1) {
        i64 half = (valid + 1) / 2;            /* STAGE_COLS = ceil(valid/2) */
        for (i64 c = 0; c < half; ++c) {
          i64 other = c + half;
          if (other < valid) {
            if (op == 2) row[c] = fmaxf(row[c], row[other]);
            else if (op == 3) row[c] = fminf(row[c], row[other]);
            else row[c] = row[c] + row[other];
          }
        }
        valid = half;
      }
      float v = row[0];
      if (op == 1) v /= (float)cols;
      if (acc) O[r] += v; else O[r] = v;
    }
    free(row);
  }
}

/* reduce.py:250-276; ties of max/min: lowest column index (the reference's winner is
 * thread-order dependent; a serial launch gives the lowest index) */
void lnn_o_reduce_bwd(int op, float* dI, const float* I, const float* dO, const float* O, i64 outer,
                      i64 r0, i64 mid, i64 r1, i64 inner) {
  i64 rows = outer * mid * inner, cols = r0 * r1;
#pragma omp parallel for
  for (i64 r = 0; r < rows; ++r) {
    i64 in_i = r % inner, t = r / inner, mid_i = t % mid, out_i = t / mid;
    int done = 0;
    for (i64 c = 0; c < cols; ++c) {
      i64 a = c / r1, b = c % r1;
      i64 off = (((out_i * r0 + a) * mid + mid_i) * r1 + b) * inner + in_i;
      if (op == 0) dI[off] += dO[r];
      else if (op == 1) dI[off] += dO[r] / (float)cols;
      else if (!done && I[off] == O[r]) { dI[off] += dO[r]; done = 1; }
    }
  }
}

/* ---- transpose / slice: op/transpose.py:94-103, op/slice.py:168-190 ------------------ */
void lnn_o_transpose(float* O, const float* I, int rank, const i64* shape, const int* axes, int acc) {
  i64 n = 1, ostr[MAXD], oshape[MAXD];
  for (int k = 0; k < rank; ++k) { n *= shape[k]; oshape[k] = shape[axes[k]]; }
  i64 s = 1;
  for (int k = rank - 1; k >= 0; --k) { ostr[k] = s; s *= oshape[k]; }
  for (i64 gid = 0; gid < n; ++gid) {
    i64 idx[MAXD], x = gid;
    for (int k = rank - 1; k >= 0; --k) { idx[k] = x % shape[k]; x /= shape[k]; }
    i64 o = 0;
    for (int k = 0; k < rank; ++k) o += idx[axes[k]] * ostr[k];
    if (acc) O[o] += I[gid]; else O[o] = I[gid];
  }
}

void lnn_o_slice(float* O, float* I_or_dI, int rank, const i64* in_shape, const i64* out_shape,
                 const i64* begin, const i64* step, int acc, int backward) {
  i64 n = 1, istr[MAXD];
  i64 s = 1;
  for (int k = rank - 1; k >= 0; --k) { istr[k] = s; s *= in_shape[k]; n *= out_shape[k]; }
  for (i64 gid = 0; gid < n; ++gid) {
    i64 x = gid, off = 0;
    for (int k = rank - 1; k >= 0; --k) { i64 o = x % out_shape[k]; x /= out_shape[k]; off += (begin[k] + o * step[k]) * istr[k]; }
    if (backward) I_or_dI[off] += O[gid];
    else if (acc) O[gid] += I_or_dI[off];
    else O[gid] = I_or_dI[off];
  }
}

/* ---- matmul: op/matmul.py:115-164 (k strictly ascending, fp32 accumulate from 0) ------- */
/* C[b] (+)= op(A[b]) op(B[b]); accum64 != 0 accumulates in double (accuracy yardstick). */
void lnn_o_gemm(float* C, const float* A, const float* B, const float* bias, i64 batch, i64 m, i64 n, i64 k,
                int ta, int tb, int acc, int accum64) {
#pragma omp parallel for collapse(2)
  for (i64 b = 0; b < batch; ++b)
    for (i64 i = 0; i < m; ++i) {
      const float* Ab = A + b * m * k;
      const float* Bb = B + b * k * n;
      for (i64 j = 0; j < n; ++j) {
        float r;
        if (accum64) {
          double s = 0.0;
          for (i64 x = 0; x < k; ++x)
            s += (double)(ta ? Ab[x * m + i] : Ab[i * k + x]) * (double)(tb ? Bb[j * k + x] : Bb[x * n + j]);
          r = (float)s;
        } else {
          float s = 0.0f;
          for (i64 x = 0; x < k; ++x)
            s += (ta ? Ab[x * m + i] : Ab[i * k + x]) * (tb ? Bb[j * k + x] : Bb[x * n + j]);
          r = s;
        }
        if (bias) r = r + bias[j];
        float* dst = C + (b * m + i) * n + j;
        if (acc) *dst += r; else *dst = r;
      }
    }
}

/* ---- conv2D: op/conv2D.py:32-54 + op/unfold2D.py:84-138 ------------------------------- */
typedef struct { int n, ic, ih, iw, oc, kh, kw, oh, ow, stride, dilation, padl, padt; } conv_geom;

/* forward: GEMM of kernel[OC][IC*KH*KW] with im2col, contraction index (ic, kh, kw)
 * ascending, zero for taps outside the image; optional bias added afterwards (module/
 * Conv2D.py:61) and leaky_relu (element_wise_op.py:210). */
void lnn_o_conv2d_fwd(const conv_geom* g, float* Y, const float* X, const float* W, const float* bias,
                      int act, float alpha, int acc, int accum64) {
  i64 total = (i64)g->n * g->oc * g->oh * g->ow;
#pragma omp parallel for
  for (i64 gid = 0; gid < total; ++gid) {
    int ow = (int)(gid % g->ow); i64 t = gid / g->ow; int oh = (int)(t % g->oh); t /= g->oh;
    int oc = (int)(t % g->oc); i64 n = t / g->oc;
    float s = 0.0f; double s64 = 0.0;
    for (int ic = 0; ic < g->ic; ++ic)
      for (int kh = 0; kh < g->kh; ++kh)
        for (int kw = 0; kw < g->kw; ++kw) {
          int ih = oh * g->stride + kh * g->dilation - g->padt;
          int iw = ow * g->stride + kw * g->dilation - g->padl;
          float x = 0.0f;
          if (ih >= 0 && iw >= 0 && ih < g->ih && iw < g->iw) x = X[((n * g->ic + ic) * g->ih + ih) * g->iw + iw];
          float w = W[(((i64)oc * g->ic + ic) * g->kh + kh) * g->kw + kw];
          if (accum64) s64 += (double)w * (double)x; else s += w * x;
        }
    float r = accum64 ? (float)s64 : s;
    if (bias) r = r + bias[oc];
    if (act == 1) r = r * (float)(r >= 0.0f) + alpha * r * (float)(r < 0.0f);
    if (acc) Y[gid] += r; else Y[gid] = r;
  }
}

/* input gradient: dX += GEMM(im2rowT(dY)[N*IH*IW][OC*KH*KW], K'[OC*KH*KW][IC]); contraction
 * index (oc, kh, kw) ascending (conv2D.py:46-50, unfold2D.py:112-138). */
void lnn_o_conv2d_dx(const conv_geom* g, float* dX, const float* dY, const float* W, int accum64) {
  i64 total = (i64)g->n * g->ic * g->ih * g->iw;
#pragma omp parallel for
  for (i64 gid = 0; gid < total; ++gid) {
    int iw = (int)(gid % g->iw); i64 t = gid / g->iw; int ih = (int)(t % g->ih); t /= g->ih;
    int ic = (int)(t % g->ic); i64 n = t / g->ic;
    float s = 0.0f; double s64 = 0.0;
    for (int oc = 0; oc < g->oc; ++oc)
      for (int kh = 0; kh < g->kh; ++kh)
        for (int kw = 0; kw < g->kw; ++kw) {
          int ny = ih + g->padt - kh * g->dilation, nx = iw + g->padl - kw * g->dilation;
          float d = 0.0f;
          if (ny >= 0 && nx >= 0 && ny % g->stride == 0 && nx % g->stride == 0) {
            int oh = ny / g->stride, ow = nx / g->stride;
            if (oh < g->oh && ow < g->ow) d = dY[((n * g->oc + oc) * g->oh + oh) * g->ow + ow];
          }
          float w = W[(((i64)oc * g->ic + ic) * g->kh + kh) * g->kw + kw];
          if (accum64) s64 += (double)d * (double)w; else s += d * w;
        }
    dX[gid] += accum64 ? (float)s64 : s;
  }
}

/* kernel gradient: dW += GEMM(dY^T[OC][N*OH*OW], im2row(X)[N*OH*OW][IC*KH*KW]); contraction
 * index (n, oh, ow) ascending (conv2D.py:52-54). */
void lnn_o_conv2d_dw(const conv_geom* g, float* dW, const float* dY, const float* X, int accum64) {
  i64 total = (i64)g->oc * g->ic * g->kh * g->kw;
#pragma omp parallel for
  for (i64 gid = 0; gid < total; ++gid) {
    int kw = (int)(gid % g->kw); i64 t = gid / g->kw; int kh = (int)(t % g->kh); t /= g->kh;
    int ic = (int)(t % g->ic); int oc = (int)(t / g->ic);
    float s = 0.0f; double s64 = 0.0;
    for (i64 n = 0; n < g->n; ++n)
      for (int oh = 0; oh < g->oh; ++oh)
        for (int ow = 0; ow < g->ow; ++ow) {
          int ih = oh * g->stride + kh * g->dilation - g->padt;
          int iw = ow * g->stride + kw * g->dilation - g->padl;
          float x = 0.0f;
          if (ih >= 0 && iw >= 0 && ih < g->ih && iw < g->iw) x = X[((n * g->ic + ic) * g->ih + ih) * g->iw + iw];
          float d = dY[((n * g->oc + oc) * g->oh + oh) * g->ow + ow];
          if (accum64) s64 += (double)d * (double)x; else s += d * x;
        }
    dW[gid] += accum64 ? (float)s64 : s;
  }
}

/* ---- conv2DTranspose: op/conv2DTranspose.py:33-46, op/unfold2D.py:112-138 ----------------
 * g describes the transposed convolution itself: input X[n][ic][ih][iw], kernel K[oc][ic][kh][kw],
 * output Y[n][oc][oh][ow] with oh = ih*stride + kh*dilation - padt.  The "transposed unfold" of
 * the reference gathers, for output pixel (oh, ow) and tap (kh, kw), input pixel
 * ((oh + padt - kh*d) / s, ...) when that division is exact and inside the image, else 0. */
static float convt_gather(const conv_geom* g, const float* X, i64 n, int ic, int oh, int ow, int kh, int kw) {
  int ny = oh + g->padt - kh * g->dilation, nx = ow + g->padl - kw * g->dilation;
  if (ny < 0 || nx < 0 || ny % g->stride != 0 || nx % g->stride != 0) return 0.0f;
  int ih = ny / g->stride, iw = nx / g->stride;
  if (ih >= g->ih || iw >= g->iw) return 0.0f;
  return X[((n * g->ic + ic) * g->ih + ih) * g->iw + iw];
}
/* forward: GEMM of kernel[OC][IC*KH*KW] with im2colT(X); contraction index (ic, kh, kw) ascending */
void lnn_o_convt_fwd(const conv_geom* g, float* Y, const float* X, const float* K, int accum64) {
  i64 total = (i64)g->n * g->oc * g->oh * g->ow;
#pragma omp parallel for
  for (i64 gid = 0; gid < total; ++gid) {
    int ow = (int)(gid % g->ow); i64 t = gid / g->ow; int oh = (int)(t % g->oh); t /= g->oh;
    int oc = (int)(t % g->oc); i64 n = t / g->oc;
    float s = 0.0f; double s64 = 0.0;
    for (int ic = 0; ic < g->ic; ++ic)
      for (int kh = 0; kh < g->kh; ++kh)
        for (int kw = 0; kw < g->kw; ++kw) {
          float k = K[(((i64)oc * g->ic + ic) * g->kh + kh) * g->kw + kw];
          float x = convt_gather(g, X, n, ic, oh, ow, kh, kw);
          if (accum64) s64 += (double)k * (double)x; else s += k * x;
        }
    Y[gid] = accum64 ? (float)s64 : s;
  }
}
/* input gradient: dX += GEMM(im2row(dY)[N*IH*IW][OC*KH*KW], K'[OC*KH*KW][IC]); index (oc, kh, kw) ascending */
void lnn_o_convt_dx(const conv_geom* g, float* dX, const float* dY, const float* K, int accum64) {
  i64 total = (i64)g->n * g->ic * g->ih * g->iw;
#pragma omp parallel for
  for (i64 gid = 0; gid < total; ++gid) {
    int iw = (int)(gid % g->iw); i64 t = gid / g->iw; int ih = (int)(t % g->ih); t /= g->ih;
    int ic = (int)(t % g->ic); i64 n = t / g->ic;
    float s = 0.0f; double s64 = 0.0;
    for (int oc = 0; oc < g->oc; ++oc)
      for (int kh = 0; kh < g->kh; ++kh)
        for (int kw = 0; kw < g->kw; ++kw) {
          int oh = ih * g->stride + kh * g->dilation - g->padt, ow = iw * g->stride + kw * g->dilation - g->padl;
          float d = 0.0f;
          if (oh >= 0 && ow >= 0 && oh < g->oh && ow < g->ow) d = dY[((n * g->oc + oc) * g->oh + oh) * g->ow + ow];
          float k = K[(((i64)oc * g->ic + ic) * g->kh + kh) * g->kw + kw];
          if (accum64) s64 += (double)d * (double)k; else s += d * k;
        }
    dX[gid] += accum64 ? (float)s64 : s;
  }
}
/* kernel gradient: dK += GEMM(dY^T[OC][N*OH*OW], im2rowT(X)[N*OH*OW][IC*KH*KW]); index (n, oh, ow) ascending */
void lnn_o_convt_dk(const conv_geom* g, float* dK, const float* dY, const float* X, int accum64) {
  i64 total = (i64)g->oc * g->ic * g->kh * g->kw;
#pragma omp parallel for
  for (i64 gid = 0; gid < total; ++gid) {
    int kw = (int)(gid % g->kw); i64 t = gid / g->kw; int kh = (int)(t % g->kh); t /= g->kh;
    int ic = (int)(t % g->ic); int oc = (int)(t / g->ic);
    float s = 0.0f; double s64 = 0.0;
    for (i64 n = 0; n < g->n; ++n)
      for (int oh = 0; oh < g->oh; ++oh)
        for (int ow = 0; ow < g->ow; ++ow) {
          float d = dY[((n * g->oc + oc) * g->oh + oh) * g->ow + ow];
          float x = convt_gather(g, X, n, ic, oh, ow, kh, kw);
          if (accum64) s64 += (double)d * (double)x; else s += d * x;
        }
    dK[gid] += accum64 ? (float)s64 : s;
  }
}

/* ---- depthwise_conv2D: op/depthwise_conv2D.py:78-123 (g->oc == g->ic, K[c][kh][kw]) ------- */
void lnn_o_depthwise_fwd(const conv_geom* g, float* O, const float* I, const float* K) {
  i64 total = (i64)g->n * g->ic * g->oh * g->ow;
#pragma omp parallel for
  for (i64 gid = 0; gid < total; ++gid) {
    int ow = (int)(gid % g->ow); i64 t = gid / g->ow; int oh = (int)(t % g->oh); t /= g->oh;
    int c = (int)(t % g->ic);
    float v = 0.0f;
    for (int kh = 0; kh < g->kh; ++kh) {
      int ih = -g->padt + kh * g->dilation + oh * g->stride;
      if (ih >= 0 && ih < g->ih)
        for (int kw = 0; kw < g->kw; ++kw) {
          int iw = -g->padl + kw * g->dilation + ow * g->stride;
          if (iw >= 0 && iw < g->iw) v += I[(t * g->ih + ih) * g->iw + iw] * K[((i64)c * g->kh + kh) * g->kw + kw];
        }
    }
    O[gid] = v;
  }
}
void lnn_o_depthwise_dx(const conv_geom* g, float* dI, const float* K, const float* dO) {
  i64 total = (i64)g->n * g->ic * g->ih * g->iw;
#pragma omp parallel for
  for (i64 gid = 0; gid < total; ++gid) {
    int iw = (int)(gid % g->iw); i64 t = gid / g->iw; int ih = (int)(t % g->ih); t /= g->ih;
    int c = (int)(t % g->ic);
    float v = 0.0f;
    for (int kh = 0; kh < g->kh; ++kh) {
      int oh = (g->padt + ih - kh * g->dilation) / g->stride;
      if (oh >= 0 && oh < g->oh)
        for (int kw = 0; kw < g->kw; ++kw) {
          int ow = (g->padl + iw - kw * g->dilation) / g->stride;
          if (ow >= 0 && ow < g->ow && iw == (-g->padl + kw * g->dilation + ow * g->stride) &&
              ih == (-g->padt + kh * g->dilation + oh * g->stride))
            v += dO[(t * g->oh + oh) * g->ow + ow] * K[((i64)c * g->kh + kh) * g->kw + kw];
        }
    }
    dI[gid] += v;
  }
}
/* products of the kernel gradient: P[(c, kh, kw)][(n, oh, ow)] = im2col(I) * dO; the caller sums the
 * rows with lnn_o_reduce (the reference's reduce_sum over the last axis, += into dK) */
void lnn_o_depthwise_dk_products(const conv_geom* g, float* P, const float* I, const float* dO) {
  i64 cols = (i64)g->n * g->oh * g->ow, total = (i64)g->ic * g->kh * g->kw * cols;
#pragma omp parallel for
  for (i64 gid = 0; gid < total; ++gid) {
    i64 col = gid % cols, row = gid / cols;
    int kw = (int)(row % g->kw); row /= g->kw; int kh = (int)(row % g->kh); int c = (int)(row / g->kh);
    int ow = (int)(col % g->ow); i64 t = col / g->ow; int oh = (int)(t % g->oh); i64 n = t / g->oh;
    int ih = -g->padt + kh * g->dilation + oh * g->stride, iw = -g->padl + kw * g->dilation + ow * g->stride;
    float x = 0.0f;
    if (ih >= 0 && ih < g->ih && iw >= 0 && iw < g->iw) x = I[((n * g->ic + c) * g->ih + ih) * g->iw + iw];
    P[gid] = x * dO[((n * g->ic + c) * g->oh + oh) * g->ow + ow];
  }
}

/* ---- SGD, momentum 0: optimizer/SGD.py:42-74 (A = 0*A - lr*G ; V += A) ---------------- */
void lnn_o_sgd(float* V, const float* G, i64 n, float lr, float gscale) {
#pragma omp parallel for
  for (i64 i = 0; i < n; ++i) {
    float g = G[i];
    if (gscale != 1.0f) g = g * gscale;
    float a = -(lr * g);
    V[i] += a;
  }
}

/* ---- random initializers --------------------------------------------------------------- */
/* The reference fills a tensor on the device from a counter-based hash of the element index
 * (litenn/core/initializer/RandomUniform.py:12-20, RandomNormal.py:10-24) with the PCG output
 * functions of litenn/core/CLKernelHelper.py:210-233 (the "pcg" and "pcg2d" hashes published
 * by Jarzynski & Olano, "Hash Functions for GPU Rendering").  Restated here from the
 * published algorithm; UIF = 1 / (float)0xffffffff = 2^-32 in single precision. */
static uint32_t pcg_hash(uint32_t v) {
  const uint32_t state = v * 747796405u + 2891336453u;
  const uint32_t word = ((state >> ((state >> 28) + 4u)) ^ state) * 277803737u;
  return (word >> 22) ^ word;
}
static void pcg2d_hash(uint32_t* x, uint32_t* y) {
  uint32_t a = *x * 1664525u + 1013904223u, b = *y * 1664525u + 1013904223u;
  a += b * 1664525u; b += a * 1664525u;
  a ^= a >> 16; b ^= b >> 16;
  a += b * 1664525u; b += a * 1664525u;
  a ^= a >> 16; b ^= b >> 16;
  *x = a; *y = b;
}
static const float kUIF = 1.0f / 4294967296.0f;

/* O[i] = hash(i + seed) * (high - low) + low            (RandomUniform.py:16-19) */
void lnn_o_init_uniform(float* O, i64 n, uint32_t seed, float low, float high) {
  const float range = high - low;
  for (i64 i = 0; i < n; ++i) {
    const float h = (float)pcg_hash((uint32_t)((uint64_t)i + seed)) * kUIF;
    O[i] = h * range + low;
  }
}

/* Box-Muller on the two outputs of the 2-D hash of (i + seed, 1):
 * O[i] = mean + sqrt(-2 log(rx)) * cos(2 PI ry) * stddev      (RandomNormal.py:14-23) */
void lnn_o_init_normal(float* O, i64 n, uint32_t seed, float mean, float stddev) {
  const float two_pi = 2.0f * 3.14159274101257f;
  for (i64 i = 0; i < n; ++i) {
    uint32_t a = (uint32_t)((uint64_t)i + seed), b = 1u;
    pcg2d_hash(&a, &b);
    const float rx = (float)a * kUIF, ry = (float)b * kUIF;
    const float r = sqrtf(-2.0f * (float)log((double)rx)) * (float)cos((double)(two_pi * ry));
    O[i] = mean + r * stddev;
  }
}

/* ---- threading ----------------------------------------------------------------------------- */
#ifdef _OPENMP
#include <omp.h>
/* Launchers such as torchrun export OMP_NUM_THREADS=1; the timed CPU baseline asks for the host
 * threads it is allowed to use explicitly. */
void lnn_o_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }
int lnn_o_get_max_threads(void) { return omp_get_max_threads(); }
#else
void lnn_o_set_threads(int n) { (void)n; }
int lnn_o_get_max_threads(void) { return 1; }
#endif
