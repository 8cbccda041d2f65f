// depthwise_conv2D and its gradients (litenn/core/op/depthwise_conv2D.py:9-123): one filter of
// KH x KW taps per channel, no contraction over channels -- a few multiply-adds per element
// read, so HBM bandwidth bounds all three passes.  One thread per output element, taps walked
// in the reference's (kh, kw) order with one rounding per product and per addition, so forward
// and input gradient are bit-identical to the reference's kernels.  The kernel gradient follows
// the reference's two steps: the products X_patch * dO as a [C*KH*KW, N*OH*OW] matrix, then the
// row sums in the halving-tree order of its reduce_sum (lnn_reduce), accumulated into dK.
#include "lnn_common.cuh"

namespace {

constexpr int kThreads = 256;

struct DwGeom {
  int n, c, ih, iw, oh, ow, kh, kw, stride, dilation, padl, padt;
};

inline int grid_for(const lnn::Device* d, int64_t work_items) {
  int64_t blocks = lnn_ceil_div(work_items, kThreads);
  const int64_t cap = (int64_t)d->sm_count * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

// O[n,c,oh,ow] = sum over (kh, kw) of I[n,c,oh*s + kh*d - padt, ow*s + kw*d - padl] * K[c,kh,kw]
__global__ void __launch_bounds__(kThreads)
depthwise_fwd_kernel(float* __restrict__ O, const float* __restrict__ I, const float* __restrict__ K, DwGeom g,
                     int64_t total, int accumulate) {
  for (int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gid < total; gid += (int64_t)gridDim.x * blockDim.x) {
    const int ow = (int)(gid % g.ow);
    int64_t t = gid / g.ow;
    const int oh = (int)(t % g.oh);
    t /= g.oh;
    const int c = (int)(t % g.c);
    const float* ip = I + t * g.ih * g.iw;            // plane (n, c)
    const float* kp = K + (int64_t)c * g.kh * g.kw;
    float v = 0.0f;
    for (int kh = 0; kh < g.kh; ++kh) {
      const int ih = -g.padt + kh * g.dilation + oh * g.stride;
      if (ih < 0 || ih >= g.ih) continue;
      for (int kw = 0; kw < g.kw; ++kw) {
        const int iw = -g.padl + kw * g.dilation + ow * g.stride;
        if (iw >= 0 && iw < g.iw) v = __fadd_rn(v, __fmul_rn(__ldg(ip + (int64_t)ih * g.iw + iw), __ldg(kp + kh * g.kw + kw)));
      }
    }
    O[gid] = accumulate ? __fadd_rn(O[gid], v) : v;
  }
}

// dI[n,c,ih,iw] += sum over the taps (kh, kw) that reach (ih, iw) of dO[n,c,oh,ow] * K[c,kh,kw]
__global__ void __launch_bounds__(kThreads)
depthwise_dx_kernel(float* __restrict__ dI, const float* __restrict__ K, const float* __restrict__ dO, DwGeom g,
                    int64_t total) {
  for (int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gid < total; gid += (int64_t)gridDim.x * blockDim.x) {
    const int iw = (int)(gid % g.iw);
    int64_t t = gid / g.iw;
    const int ih = (int)(t % g.ih);
    t /= g.ih;
    const int c = (int)(t % g.c);
    const float* op = dO + t * g.oh * g.ow;
    const float* kp = K + (int64_t)c * g.kh * g.kw;
    float v = 0.0f;
    for (int kh = 0; kh < g.kh; ++kh) {
      const int nh = g.padt + ih - kh * g.dilation;
      if (nh < 0 || nh % g.stride != 0) continue;
      const int oh = nh / g.stride;
      if (oh >= g.oh) continue;
      for (int kw = 0; kw < g.kw; ++kw) {
        const int nw = g.padl + iw - kw * g.dilation;
        if (nw < 0 || nw % g.stride != 0) continue;
        const int ow = nw / g.stride;
        if (ow < g.ow) v = __fadd_rn(v, __fmul_rn(__ldg(op + (int64_t)oh * g.ow + ow), __ldg(kp + kh * g.kw + kw)));
      }
    }
    dI[gid] = __fadd_rn(dI[gid], v);
  }
}

// P[(c, kh, kw)][(n, oh, ow)] = I[n,c,ih,iw] * dO[n,c,oh,ow]  (zero outside the image)
__global__ void __launch_bounds__(kThreads)
depthwise_dk_product_kernel(float* __restrict__ P, const float* __restrict__ I, const float* __restrict__ dO,
                            DwGeom g, int64_t total) {
  const int64_t cols = (int64_t)g.n * g.oh * g.ow;
  for (int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gid < total; gid += (int64_t)gridDim.x * blockDim.x) {
    const int64_t col = gid % cols;
    int64_t row = gid / cols;
    const int kw = (int)(row % g.kw); row /= g.kw;
    const int kh = (int)(row % g.kh);
    const int c = (int)(row / g.kh);
    const int ow = (int)(col % g.ow);
    const int64_t t = col / g.ow;
    const int oh = (int)(t % g.oh);
    const int64_t n = t / g.oh;
    const int ih = -g.padt + kh * g.dilation + oh * g.stride;
    const int iw = -g.padl + kw * g.dilation + ow * g.stride;
    float x = 0.0f;
    if (ih >= 0 && ih < g.ih && iw >= 0 && iw < g.iw) x = __ldg(I + ((n * g.c + c) * g.ih + ih) * g.iw + iw);
    P[gid] = __fmul_rn(x, __ldg(dO + ((n * g.c + c) * g.oh + oh) * g.ow + ow));
  }
}

int to_geom(DwGeom* g, const lnn_conv_geom* c) {
  LNN_REQUIRE(c, "geometry is null");
  LNN_REQUIRE(c->n > 0 && c->ic > 0 && c->ih > 0 && c->iw > 0 && c->kh > 0 && c->kw > 0 && c->oh > 0 && c->ow > 0 &&
              c->stride >= 1 && c->dilation >= 1, "bad depthwise convolution extents");
  LNN_REQUIRE(c->oc == c->ic, "a depthwise convolution keeps the channel count");
  g->n = c->n; g->c = c->ic; g->ih = c->ih; g->iw = c->iw; g->oh = c->oh; g->ow = c->ow; g->kh = c->kh; g->kw = c->kw;
  g->stride = c->stride; g->dilation = c->dilation; g->padl = c->padl; g->padt = c->padt;
  return LNN_OK;
}

}  // namespace

extern "C" {

int lnn_reduce(int dev, int op, uint64_t O, uint64_t I, int64_t outer, int64_t r0, int64_t mid, int64_t r1,
               int64_t inner, int accumulate);

int lnn_depthwise_conv2d_fwd(int dev, const lnn_conv_geom* cg, uint64_t Y, uint64_t X, uint64_t K, int accumulate) {
  LNN_DEV(d, dev);
  DwGeom g;
  int rc = to_geom(&g, cg);
  if (rc) return rc;
  LNN_REQUIRE(Y && X && K, "null buffer");
  const int64_t total = (int64_t)g.n * g.c * g.oh * g.ow;
  depthwise_fwd_kernel<<<grid_for(d, total), kThreads, 0, d->stream>>>(
      (float*)(uintptr_t)Y, (const float*)(uintptr_t)X, (const float*)(uintptr_t)K, g, total, accumulate);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

int lnn_depthwise_conv2d_dx(int dev, const lnn_conv_geom* cg, uint64_t dX, uint64_t dY, uint64_t K) {
  LNN_DEV(d, dev);
  DwGeom g;
  int rc = to_geom(&g, cg);
  if (rc) return rc;
  LNN_REQUIRE(dX && dY && K, "null buffer");
  const int64_t total = (int64_t)g.n * g.c * g.ih * g.iw;
  depthwise_dx_kernel<<<grid_for(d, total), kThreads, 0, d->stream>>>(
      (float*)(uintptr_t)dX, (const float*)(uintptr_t)K, (const float*)(uintptr_t)dY, g, total);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

int lnn_depthwise_conv2d_dk(int dev, const lnn_conv_geom* cg, uint64_t dK, uint64_t dY, uint64_t X) {
  LNN_DEV(d, dev);
  DwGeom g;
  int rc = to_geom(&g, cg);
  if (rc) return rc;
  LNN_REQUIRE(dK && dY && X, "null buffer");
  const int64_t rows = (int64_t)g.c * g.kh * g.kw, cols = (int64_t)g.n * g.oh * g.ow;
  lnn::Scratch prod(d);
  rc = prod.get((uint64_t)rows * cols * 4);
  if (rc) return rc;
  depthwise_dk_product_kernel<<<grid_for(d, rows * cols), kThreads, 0, d->stream>>>(
      prod.as<float>(), (const float*)(uintptr_t)X, (const float*)(uintptr_t)dY, g, rows * cols);
  LNN_CHECK_LAUNCH(d);
  // row sums over the trailing axis, accumulated: reduce_sum(dK_products, -1, output_t=dK, is_add_to_output)
  return lnn_reduce(dev, LNN_RED_SUM, dK, (uint64_t)(uintptr_t)prod.p, rows, 1, 1, cols, 1, 1);
}

}  // extern "C"
