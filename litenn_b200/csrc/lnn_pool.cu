// 2-D pooling forward/backward (avg, max, min) on NCHW fp32.
// Semantics follow litenn/core/op/pool2D.py:111-230: taps are visited in row-major
// window order; avg divides the ordered sum by the number of in-bounds taps; max/min of
// an empty window is 0; the max/min gradient goes to the FIRST tap (row-major) equal to
// the pooled value.  HBM-bound: the 2x2/stride-2 even-width case reads two float4 rows
// per two outputs and writes float2; everything else uses the generic kernels, which clip each
// window to the image once instead of testing every tap.
#include "lnn_common.cuh"
#include <math_constants.h>

namespace {

constexpr int kThreads = 256;

struct PoolGeom {
  int ih, iw, oh, ow, pool, stride, padl, padt;
};

// The part of window (oh, ow) that lies inside the image: rows [h0, h1), columns [w0, w1).
struct Window { int h0, h1, w0, w1; };
__device__ __forceinline__ Window window_of(const PoolGeom& g, int oh, int ow) {
  Window w;
  const int top = oh * g.stride - g.padt, left = ow * g.stride - g.padl;
  w.h0 = max(top, 0); w.h1 = min(top + g.pool, g.ih);
  w.w0 = max(left, 0); w.w1 = min(left + g.pool, g.iw);
  return w;
}

// Generic forward: one thread per output.  The window is clipped to the image once, then its
// elements are combined in row-major order, which is the order in which the reference visits
// the taps it does not skip (pool2D.py:111-146): sum / (number of in-image taps), or max / min
// with 0 for a window that lies entirely outside.
template <int MODE>
__global__ void __launch_bounds__(kThreads)
pool_fwd_kernel(float* __restrict__ O, const float* __restrict__ I, int64_t total, PoolGeom g) {
  for (int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gid < total; gid += (int64_t)gridDim.x * blockDim.x) {
    const int ow = (int)(gid % g.ow);
    const int64_t rest = gid / g.ow;
    const int oh = (int)(rest % g.oh);
    const float* plane = I + (rest / g.oh) * g.ih * g.iw;
    const Window w = window_of(g, oh, ow);
    float acc = MODE == LNN_POOL_AVG ? 0.0f : (MODE == LNN_POOL_MAX ? -CUDART_INF_F : CUDART_INF_F);
    for (int h = w.h0; h < w.h1; ++h) {
      const float* row = plane + (int64_t)h * g.iw;
      for (int x = w.w0; x < w.w1; ++x) {
        const float v = row[x];
        acc = MODE == LNN_POOL_AVG ? __fadd_rn(acc, v) : (MODE == LNN_POOL_MAX ? fmaxf(acc, v) : fminf(acc, v));
      }
    }
    const int count = max(w.h1 - w.h0, 0) * max(w.w1 - w.w0, 0);
    if (MODE == LNN_POOL_AVG) { if (count > 0) acc = __fdiv_rn(acc, (float)count); }
    else if (acc == (MODE == LNN_POOL_MAX ? -CUDART_INF_F : CUDART_INF_F)) acc = 0.0f;
    O[gid] = acc;
  }
}

// 2x2 / stride 2 / no left-top padding / even IW, OW == IW/2, IW % 4 == 0: every thread
// produces two horizontally adjacent outputs from two float4 loads.  All taps in bounds
// except possibly the bottom row when IH is odd (padded bottom).
template <int MODE>
__global__ void __launch_bounds__(kThreads)
pool2x2_fwd_kernel(float2* __restrict__ O, const float* __restrict__ I, int64_t total2, int ih,
                   int iw, int oh, int ow2) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t gid = tid; gid < total2; gid += nthreads) {
    const int x2 = (int)(gid % ow2);
    const int64_t t = gid / ow2;
    const int y = (int)(t % oh);
    const int64_t plane = t / oh;
    const float* row0 = I + (plane * ih + 2 * y) * (int64_t)iw + 4 * x2;
    const float4 a = __ldcs(reinterpret_cast<const float4*>(row0));
    const bool has1 = (2 * y + 1) < ih;
    float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
    if (has1) b = __ldcs(reinterpret_cast<const float4*>(row0 + iw));
    float2 r;
    if (MODE == LNN_POOL_AVG) {
      // ordered sum ((0 + t00) + t01) + t10) + t11 ; 0 + t00 == t00 except for -0
      float s0 = __fadd_rn(__fadd_rn(0.0f, a.x), a.y);
      float s1 = __fadd_rn(__fadd_rn(0.0f, a.z), a.w);
      if (has1) {
        s0 = __fadd_rn(__fadd_rn(s0, b.x), b.y);
        s1 = __fadd_rn(__fadd_rn(s1, b.z), b.w);
      }
      const float cnt = has1 ? 4.0f : 2.0f;
      r.x = __fdiv_rn(s0, cnt);
      r.y = __fdiv_rn(s1, cnt);
    } else if (MODE == LNN_POOL_MAX) {
      float m0 = fmaxf(fmaxf(-CUDART_INF_F, a.x), a.y), m1 = fmaxf(fmaxf(-CUDART_INF_F, a.z), a.w);
      if (has1) { m0 = fmaxf(fmaxf(m0, b.x), b.y); m1 = fmaxf(fmaxf(m1, b.z), b.w); }
      r.x = (m0 == -CUDART_INF_F) ? 0.0f : m0;
      r.y = (m1 == -CUDART_INF_F) ? 0.0f : m1;
    } else {
      float m0 = fminf(fminf(CUDART_INF_F, a.x), a.y), m1 = fminf(fminf(CUDART_INF_F, a.z), a.w);
      if (has1) { m0 = fminf(fminf(m0, b.x), b.y); m1 = fminf(fminf(m1, b.z), b.w); }
      r.x = (m0 == CUDART_INF_F) ? 0.0f : m0;
      r.y = (m1 == CUDART_INF_F) ? 0.0f : m1;
    }
    __stcs(O + gid, r);
  }
}

// Backward of the 2x2 / stride 2 / no left-top padding case: every input element lies in
// exactly one window, so a thread takes one window pair (two horizontally adjacent outputs),
// finds the first tap (row-major) equal to the pooled value and adds dO there; avg spreads
// dO / count.  Same results as the gather form below, one pass, 128-bit accesses.
template <int MODE>
__global__ void __launch_bounds__(kThreads)
pool2x2_bwd_kernel(float* __restrict__ dI, const float* __restrict__ I, const float2* __restrict__ dO,
                   const float2* __restrict__ O, int64_t total2, int ih, int iw, int oh, int ow2) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t gid = tid; gid < total2; gid += nthreads) {
    const int x2 = (int)(gid % ow2);
    const int64_t t = gid / ow2;
    const int y = (int)(t % oh);
    const int64_t plane = t / oh;
    const int64_t off0 = (plane * ih + 2 * y) * (int64_t)iw + 4 * x2;
    const bool has1 = (2 * y + 1) < ih;
    const float2 g = dO[gid];
    float4 ga = make_float4(0.f, 0.f, 0.f, 0.f), gb = ga;       // gradient of the two input rows
    if (MODE == LNN_POOL_AVG) {
      const float cnt = has1 ? 4.0f : 2.0f;
      const float q0 = __fdiv_rn(g.x, cnt), q1 = __fdiv_rn(g.y, cnt);
      ga = make_float4(q0, q0, q1, q1);
      gb = ga;
    } else {
      const float4 a = *reinterpret_cast<const float4*>(I + off0);
      float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
      if (has1) b = *reinterpret_cast<const float4*>(I + off0 + iw);
      const float2 o = O[gid];
      // window 0: taps a.x, a.y, b.x, b.y in row-major order; window 1: a.z, a.w, b.z, b.w
      if (a.x == o.x) ga.x = g.x; else if (a.y == o.x) ga.y = g.x;
      else if (has1 && b.x == o.x) gb.x = g.x; else if (has1 && b.y == o.x) gb.y = g.x;
      if (a.z == o.y) ga.z = g.y; else if (a.w == o.y) ga.w = g.y;
      else if (has1 && b.z == o.y) gb.z = g.y; else if (has1 && b.w == o.y) gb.w = g.y;
    }
    float4* d0 = reinterpret_cast<float4*>(dI + off0);
    float4 v = *d0;
    // the reference adds 0.0 + dO to its accumulator first, then accumulator to dI
    v.x = __fadd_rn(v.x, __fadd_rn(0.0f, ga.x)); v.y = __fadd_rn(v.y, __fadd_rn(0.0f, ga.y));
    v.z = __fadd_rn(v.z, __fadd_rn(0.0f, ga.z)); v.w = __fadd_rn(v.w, __fadd_rn(0.0f, ga.w));
    *d0 = v;
    if (has1) {
      float4* d1 = reinterpret_cast<float4*>(dI + off0 + iw);
      float4 w = *d1;
      w.x = __fadd_rn(w.x, __fadd_rn(0.0f, gb.x)); w.y = __fadd_rn(w.y, __fadd_rn(0.0f, gb.y));
      w.z = __fadd_rn(w.z, __fadd_rn(0.0f, gb.z)); w.w = __fadd_rn(w.w, __fadd_rn(0.0f, gb.w));
      *d1 = w;
    }
  }
}

// Generic backward: one thread per INPUT element (so "+=" needs no atomics).  The windows that
// contain element (ih, iw) form a rectangle of outputs, oh in [oh_lo, oh_hi], ow likewise; their
// contributions are added from the highest (oh, ow) down, the order in which the reference meets
// them while it walks its taps upwards (pool2D.py:147-230), so overlapping windows accumulate
// identically.  avg: dO / (in-image size of the window).  max / min: dO if this element is the
// first one of the window, in row-major order, that equals the pooled value.
template <int MODE>
__global__ void __launch_bounds__(kThreads)
pool_bwd_kernel(float* __restrict__ dI, const float* __restrict__ I, const float* __restrict__ dO,
                const float* __restrict__ O, int64_t total, PoolGeom g) {
  for (int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gid < total; gid += (int64_t)gridDim.x * blockDim.x) {
    const int iw = (int)(gid % g.iw);
    const int64_t rest = gid / g.iw;
    const int ih = (int)(rest % g.ih);
    const int64_t pl = rest / g.ih;
    const float* iplane = I ? I + pl * g.ih * g.iw : nullptr;
    const float* oplane = O ? O + pl * g.oh * g.ow : nullptr;
    const float* gplane = dO + pl * g.oh * g.ow;
    // windows covering the element: oh*stride - padt <= ih < oh*stride - padt + pool
    const int ah = ih + g.padt, aw = iw + g.padl;
    const int oh_hi = min(ah / g.stride, g.oh - 1), ow_hi = min(aw / g.stride, g.ow - 1);
    const int oh_lo = max((ah - g.pool + g.stride) / g.stride, 0), ow_lo = max((aw - g.pool + g.stride) / g.stride, 0);
    float sum = 0.0f;
    for (int oh = oh_hi; oh >= oh_lo; --oh)
      for (int ow = ow_hi; ow >= ow_lo; --ow) {
        const Window w = window_of(g, oh, ow);
        const float go = gplane[(int64_t)oh * g.ow + ow];
        if (MODE == LNN_POOL_AVG) {
          sum = __fadd_rn(sum, __fdiv_rn(go, (float)((w.h1 - w.h0) * (w.w1 - w.w0))));
        } else {
          const float pooled = oplane[(int64_t)oh * g.ow + ow];
          if (iplane[(int64_t)ih * g.iw + iw] != pooled) continue;
          // is an earlier element of the window equal to the pooled value too?
          bool first = true;
          for (int h = w.h0; h <= ih && first; ++h) {
            const int stop = h == ih ? iw : w.w1;
            for (int x = w.w0; x < stop; ++x)
              if (iplane[(int64_t)h * g.iw + x] == pooled) { first = false; break; }
          }
          if (first) sum = __fadd_rn(sum, go);
        }
      }
    dI[gid] = __fadd_rn(dI[gid], sum);
  }
}

inline int grid_for(const lnn::Device* d, int64_t work_items) {
  int64_t blocks = lnn_ceil_div(work_items, kThreads);
  int64_t cap = (int64_t)d->sm_count * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

// Gradient of max_pool2D(2, 2) followed by the gradient of leaky_relu in one pass, WRITING dZ
// (the chain of the two un-fused gradient kernels reads and re-writes two zero-filled
// full-resolution tensors).  Y = leaky_relu(Z) is the pooled tensor's input, P its output, dP the
// gradient of P.  Per element exactly the roundings of the un-fused chain: the pooling gradient
// 0 + (0 + dP) at the first window position equal to P in row-major order (pool2D.py:147-230),
// then 0 + that * ((Y >= 0) + alpha * (Y < 0)) (element_wise_op.py:207-221; sign(Y) == sign(Z)).
__global__ void __launch_bounds__(kThreads)
pool2x2_lrelu_bwd_kernel(float* __restrict__ dZ, const float* __restrict__ Y, const float2* __restrict__ dP,
                         const float2* __restrict__ P, int64_t total2, int ih, int iw, int oh, int ow2,
                         float alpha, int act) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t gid = tid; gid < total2; gid += nthreads) {
    const int x2 = (int)(gid % ow2);
    const int64_t t = gid / ow2;
    const int y = (int)(t % oh);
    const int64_t plane = t / oh;
    const int64_t off0 = (plane * ih + 2 * y) * (int64_t)iw + 4 * x2;
    const float4 a = __ldcs(reinterpret_cast<const float4*>(Y + off0));
    const float4 b = __ldcs(reinterpret_cast<const float4*>(Y + off0 + iw));
    const float2 g = dP[gid];
    const float2 o = P[gid];
    float ga[4] = {0.f, 0.f, 0.f, 0.f}, gb[4] = {0.f, 0.f, 0.f, 0.f};
    if (a.x == o.x) ga[0] = g.x; else if (a.y == o.x) ga[1] = g.x;
    else if (b.x == o.x) gb[0] = g.x; else if (b.y == o.x) gb[1] = g.x;
    if (a.z == o.y) ga[2] = g.y; else if (a.w == o.y) ga[3] = g.y;
    else if (b.z == o.y) gb[2] = g.y; else if (b.w == o.y) gb[3] = g.y;
    const float ya[4] = {a.x, a.y, a.z, a.w}, yb[4] = {b.x, b.y, b.z, b.w};
    float ra[4], rb[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float ua = __fadd_rn(0.0f, __fadd_rn(0.0f, ga[e]));
      float ub = __fadd_rn(0.0f, __fadd_rn(0.0f, gb[e]));
      if (act) {
        const float fa = __fadd_rn(ya[e] >= 0.0f ? 1.0f : 0.0f, __fmul_rn(alpha, ya[e] < 0.0f ? 1.0f : 0.0f));
        const float fb = __fadd_rn(yb[e] >= 0.0f ? 1.0f : 0.0f, __fmul_rn(alpha, yb[e] < 0.0f ? 1.0f : 0.0f));
        ua = __fadd_rn(0.0f, __fmul_rn(ua, fa));
        ub = __fadd_rn(0.0f, __fmul_rn(ub, fb));
      }
      ra[e] = ua; rb[e] = ub;
    }
    __stcs(reinterpret_cast<float4*>(dZ + off0), make_float4(ra[0], ra[1], ra[2], ra[3]));
    __stcs(reinterpret_cast<float4*>(dZ + off0 + iw), make_float4(rb[0], rb[1], rb[2], rb[3]));
  }
}

// The same gradient from the map of winning window positions a fused forward epilogue wrote
// (0..3 in row-major order, 4 = no position matched) instead of the full-resolution activation:
// the winner holds the pooled value itself, so leaky_relu' is taken from the sign of P, and every
// other position is +0 whatever its activation was.  T (optional, pooled size) receives the
// winner's value: its sum over (n, h, w) is the bias gradient.
__global__ void __launch_bounds__(kThreads)
pool2x2_idx_lrelu_bwd_kernel(float* __restrict__ dZ, float2* __restrict__ T, const uchar2* __restrict__ IDX,
                             const float2* __restrict__ dP, const float2* __restrict__ P, int64_t total2, int ih,
                             int iw, int oh, int ow2, float alpha, int act) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t gid = tid; gid < total2; gid += nthreads) {
    const int x2 = (int)(gid % ow2);
    const int64_t t = gid / ow2;
    const int y = (int)(t % oh);
    const int64_t plane = t / oh;
    const int64_t off0 = (plane * ih + 2 * y) * (int64_t)iw + 4 * x2;
    const uchar2 w = IDX[gid];
    const float2 g = dP[gid];
    const float2 o = P[gid];
    float u[2] = {__fadd_rn(0.0f, __fadd_rn(0.0f, g.x)), __fadd_rn(0.0f, __fadd_rn(0.0f, g.y))};
    if (act) {
      const float f0 = __fadd_rn(o.x >= 0.0f ? 1.0f : 0.0f, __fmul_rn(alpha, o.x < 0.0f ? 1.0f : 0.0f));
      const float f1 = __fadd_rn(o.y >= 0.0f ? 1.0f : 0.0f, __fmul_rn(alpha, o.y < 0.0f ? 1.0f : 0.0f));
      u[0] = __fadd_rn(0.0f, __fmul_rn(u[0], f0));
      u[1] = __fadd_rn(0.0f, __fmul_rn(u[1], f1));
    }
    if (w.x > 3) u[0] = 0.0f;
    if (w.y > 3) u[1] = 0.0f;
    float ra[4] = {0.f, 0.f, 0.f, 0.f}, rb[4] = {0.f, 0.f, 0.f, 0.f};
    if (w.x == 0) ra[0] = u[0]; else if (w.x == 1) ra[1] = u[0]; else if (w.x == 2) rb[0] = u[0]; else if (w.x == 3) rb[1] = u[0];
    if (w.y == 0) ra[2] = u[1]; else if (w.y == 1) ra[3] = u[1]; else if (w.y == 2) rb[2] = u[1]; else if (w.y == 3) rb[3] = u[1];
    __stcs(reinterpret_cast<float4*>(dZ + off0), make_float4(ra[0], ra[1], ra[2], ra[3]));
    __stcs(reinterpret_cast<float4*>(dZ + off0 + iw), make_float4(rb[0], rb[1], rb[2], rb[3]));
    if (T) T[gid] = make_float2(u[0], u[1]);
  }
}

}  // namespace

extern "C" {

int lnn_pool2d_fwd(int dev, int mode, uint64_t O, uint64_t I, int64_t n, int64_t c, int ih, int iw,
                   int oh, int ow, int pool, int stride, int padl, int padt) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(O && I, "null buffer");
  LNN_REQUIRE(n > 0 && c > 0 && ih > 0 && iw > 0 && oh > 0 && ow > 0, "bad extents");
  LNN_REQUIRE(pool >= 2 && stride >= 1, "pool_size must be >= 2 and stride >= 1");
  LNN_REQUIRE(mode >= 0 && mode <= 2, "unknown pool mode %d", mode);
  const int64_t total = n * c * oh * ow;
  float* o = (float*)(uintptr_t)O;
  const float* i = (const float*)(uintptr_t)I;
  const bool fast = pool == 2 && stride == 2 && padl == 0 && padt == 0 && (iw % 4) == 0 &&
                    ow == iw / 2 && oh == (ih + 1) / 2 && (O & 7) == 0 && (I & 15) == 0;
  if (fast) {
    const int64_t total2 = total / 2;
    const int grid = grid_for(d, total2);
    if (mode == LNN_POOL_AVG)
      pool2x2_fwd_kernel<LNN_POOL_AVG><<<grid, kThreads, 0, d->stream>>>((float2*)o, i, total2, ih, iw, oh, ow / 2);
    else if (mode == LNN_POOL_MAX)
      pool2x2_fwd_kernel<LNN_POOL_MAX><<<grid, kThreads, 0, d->stream>>>((float2*)o, i, total2, ih, iw, oh, ow / 2);
    else
      pool2x2_fwd_kernel<LNN_POOL_MIN><<<grid, kThreads, 0, d->stream>>>((float2*)o, i, total2, ih, iw, oh, ow / 2);
  } else {
    PoolGeom g{ih, iw, oh, ow, pool, stride, padl, padt};
    const int grid = grid_for(d, total);
    if (mode == LNN_POOL_AVG)
      pool_fwd_kernel<LNN_POOL_AVG><<<grid, kThreads, 0, d->stream>>>(o, i, total, g);
    else if (mode == LNN_POOL_MAX)
      pool_fwd_kernel<LNN_POOL_MAX><<<grid, kThreads, 0, d->stream>>>(o, i, total, g);
    else
      pool_fwd_kernel<LNN_POOL_MIN><<<grid, kThreads, 0, d->stream>>>(o, i, total, g);
  }
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

int lnn_pool2d_bwd(int dev, int mode, uint64_t dI, uint64_t I, uint64_t dO, uint64_t O, int64_t n,
                   int64_t c, int ih, int iw, int oh, int ow, int pool, int stride, int padl,
                   int padt) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(dI && dO, "null buffer");
  LNN_REQUIRE(mode >= 0 && mode <= 2, "unknown pool mode %d", mode);
  LNN_REQUIRE(mode == LNN_POOL_AVG || (I && O), "max/min backward needs I and O");
  LNN_REQUIRE(n > 0 && c > 0 && ih > 0 && iw > 0 && oh > 0 && ow > 0, "bad extents");
  LNN_REQUIRE(pool >= 2 && stride >= 1, "pool_size must be >= 2 and stride >= 1");
  const int64_t total = n * c * ih * iw;
  PoolGeom g{ih, iw, oh, ow, pool, stride, padl, padt};
  float* di = (float*)(uintptr_t)dI;
  const float* i = (const float*)(uintptr_t)I;
  const float* dout = (const float*)(uintptr_t)dO;
  const float* o = (const float*)(uintptr_t)O;
  const bool fast = pool == 2 && stride == 2 && padl == 0 && padt == 0 && (iw % 4) == 0 &&
                    ow == iw / 2 && oh == (ih + 1) / 2 && (dI & 15) == 0 && (dO & 7) == 0 &&
                    (mode == LNN_POOL_AVG || ((I & 15) == 0 && (O & 7) == 0));
  if (fast) {
    const int64_t total2 = n * c * oh * (ow / 2);
    const int grid2 = grid_for(d, total2);
    if (mode == LNN_POOL_AVG)
      pool2x2_bwd_kernel<LNN_POOL_AVG><<<grid2, kThreads, 0, d->stream>>>(di, i, (const float2*)dout, (const float2*)o, total2, ih, iw, oh, ow / 2);
    else if (mode == LNN_POOL_MAX)
      pool2x2_bwd_kernel<LNN_POOL_MAX><<<grid2, kThreads, 0, d->stream>>>(di, i, (const float2*)dout, (const float2*)o, total2, ih, iw, oh, ow / 2);
    else
      pool2x2_bwd_kernel<LNN_POOL_MIN><<<grid2, kThreads, 0, d->stream>>>(di, i, (const float2*)dout, (const float2*)o, total2, ih, iw, oh, ow / 2);
    LNN_CHECK_LAUNCH(d);
    return LNN_OK;
  }
  const int grid = grid_for(d, total);
  if (mode == LNN_POOL_AVG)
    pool_bwd_kernel<LNN_POOL_AVG><<<grid, kThreads, 0, d->stream>>>(di, i, dout, o, total, g);
  else if (mode == LNN_POOL_MAX)
    pool_bwd_kernel<LNN_POOL_MAX><<<grid, kThreads, 0, d->stream>>>(di, i, dout, o, total, g);
  else
    pool_bwd_kernel<LNN_POOL_MIN><<<grid, kThreads, 0, d->stream>>>(di, i, dout, o, total, g);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}


int lnn_pool2x2_idx_lrelu_bwd(int dev, uint64_t dZ, uint64_t T, uint64_t IDX, uint64_t P, uint64_t dP, int64_t n,
                              int64_t c, int ih, int iw, float alpha, int act) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(dZ && IDX && P && dP, "null buffer");
  LNN_REQUIRE(n > 0 && c > 0 && ih > 0 && iw > 0, "bad extents");
  LNN_REQUIRE(act == 0 || act == 1, "unknown activation %d", act);
  if ((ih & 1) || (iw & 3) || (dZ & 15) || ((P | dP | T) & 7) || (IDX & 1))
    return lnn::set_error(LNN_E_UNSUPPORTED,
                          "fused pooling gradient needs an even height, a width that is a multiple of 4 and aligned buffers");
  const int oh = ih / 2, ow = iw / 2;
  const int64_t total2 = n * c * oh * (ow / 2);
  pool2x2_idx_lrelu_bwd_kernel<<<grid_for(d, total2), kThreads, 0, d->stream>>>(
      (float*)(uintptr_t)dZ, (float2*)(uintptr_t)T, (const uchar2*)(uintptr_t)IDX, (const float2*)(uintptr_t)dP,
      (const float2*)(uintptr_t)P, total2, ih, iw, oh, ow / 2, alpha, act);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

int lnn_pool2x2_lrelu_bwd(int dev, uint64_t dZ, uint64_t Y, uint64_t P, uint64_t dP, int64_t n, int64_t c,
                          int ih, int iw, float alpha, int act) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(dZ && Y && P && dP, "null buffer");
  LNN_REQUIRE(n > 0 && c > 0 && ih > 0 && iw > 0, "bad extents");
  LNN_REQUIRE(act == 0 || act == 1, "unknown activation %d", act);
  if ((ih & 1) || (iw & 3) || ((dZ | Y) & 15) || ((P | dP) & 7))
    return lnn::set_error(LNN_E_UNSUPPORTED,
                          "fused pooling gradient needs an even height, a width that is a multiple of 4 and aligned buffers");
  const int oh = ih / 2, ow = iw / 2;
  const int64_t total2 = n * c * oh * (ow / 2);
  pool2x2_lrelu_bwd_kernel<<<grid_for(d, total2), kThreads, 0, d->stream>>>(
      (float*)(uintptr_t)dZ, (const float*)(uintptr_t)Y, (const float2*)(uintptr_t)dP,
      (const float2*)(uintptr_t)P, total2, ih, iw, oh, ow / 2, alpha, act);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

}  // extern "C"
