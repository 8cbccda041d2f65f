// Direct convolution for layers with very few input channels (IC <= 4, e.g. the RGB input
// layer of a CNN).  With K = IC*KH*KW <= ~100 an implicit GEMM wastes the tensor cores on
// zero padding and is bound by writing / re-reading the big activation, so this layer runs
// on the FP32 pipes instead: one thread produces a 2x2 quad of output pixels for 16 output
// channels at a time, weights come from shared memory as broadcast 128-bit loads, the input
// is read from NCHW as it is (no repack, exact fp32 products, fmaf accumulation), and bias,
// leaky_relu and an optional 2x2/stride-2 max-pool are applied before the only store.
// Semantics: litenn/core/op/conv2D.py:9-44 (+ module/Conv2D.py:61 bias,
// op/element_wise_op.py:210 leaky_relu, op/pool2D.py:111-146 max pool).
#include "lnn_common.cuh"
#include <math_constants.h>

namespace {

constexpr int kThreads = 256;
constexpr int kOcChunk = 16;
constexpr int kMaxWeights = 11 * 1024;     // floats of shared memory for one launch's kernel taps

__device__ __forceinline__ float act_apply(float v, int act, float alpha) {
  if (act == 1) {
    const float pos = __fmul_rn(v, v >= 0.0f ? 1.0f : 0.0f);
    const float neg = __fmul_rn(__fmul_rn(alpha, v), v < 0.0f ? 1.0f : 0.0f);
    return __fadd_rn(pos, neg);
  }
  return v;
}

// W is OIHW.  Shared layout: [ic][kh][kw][ocp] with ocp = OC rounded up to 16.
// pool != 0: Y is [N][OC][ceil(OH/2)][ceil(OW/2)] = max_pool2D(act(conv + bias), 2, 2, 'same').
__global__ void __launch_bounds__(kThreads)
conv_direct_fwd_kernel(float* __restrict__ Y, const float* __restrict__ X, const float* __restrict__ W,
                       const float* __restrict__ bias, lnn_conv_geom g, int act, float alpha,
                       int accumulate, int pool) {
  extern __shared__ float wsm[];
  const int taps = g.ic * g.kh * g.kw;
  const int ocp = (g.oc + kOcChunk - 1) / kOcChunk * kOcChunk;
  for (int i = threadIdx.x; i < taps * ocp; i += blockDim.x) {
    const int o = i % ocp, t = i / ocp;
    wsm[i] = o < g.oc ? W[(int64_t)o * taps + t] : 0.0f;
  }
  __syncthreads();

  const int qw = (g.ow + 1) >> 1, qh = (g.oh + 1) >> 1;
  const int64_t quads = (int64_t)g.n * qh * qw;
  const int64_t in_plane = (int64_t)g.ih * g.iw, out_plane = (int64_t)g.oh * g.ow;
  const int64_t pool_plane = (int64_t)qh * qw;
  for (int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q < quads;
       q += (int64_t)gridDim.x * blockDim.x) {
    const int qx = (int)(q % qw);
    const int64_t t2 = q / qw;
    const int qy = (int)(t2 % qh);
    const int64_t n = t2 / qh;
    const int oh0 = 2 * qy, ow0 = 2 * qx;
    const bool v01 = ow0 + 1 < g.ow, v10 = oh0 + 1 < g.oh;
    const float* xin = X + n * g.ic * in_plane;
    for (int oc0 = 0; oc0 < g.oc; oc0 += kOcChunk) {
      float a00[kOcChunk], a01[kOcChunk], a10[kOcChunk], a11[kOcChunk];
#pragma unroll
      for (int o = 0; o < kOcChunk; ++o) { a00[o] = 0.f; a01[o] = 0.f; a10[o] = 0.f; a11[o] = 0.f; }
      int tap = 0;
      for (int ic = 0; ic < g.ic; ++ic) {
        const float* xp = xin + ic * in_plane;
        for (int kh = 0; kh < g.kh; ++kh) {
          const int ih0 = oh0 * g.stride + kh * g.dilation - g.padt;
          const int ih1 = ih0 + g.stride;
          const bool r0 = ih0 >= 0 && ih0 < g.ih, r1 = ih1 >= 0 && ih1 < g.ih;
          for (int kw = 0; kw < g.kw; ++kw, ++tap) {
            const int iw0 = ow0 * g.stride + kw * g.dilation - g.padl;
            const int iw1 = iw0 + g.stride;
            const bool c0 = iw0 >= 0 && iw0 < g.iw, c1 = iw1 >= 0 && iw1 < g.iw;
            const float x00 = (r0 && c0) ? __ldg(xp + (int64_t)ih0 * g.iw + iw0) : 0.0f;
            const float x01 = (r0 && c1) ? __ldg(xp + (int64_t)ih0 * g.iw + iw1) : 0.0f;
            const float x10 = (r1 && c0) ? __ldg(xp + (int64_t)ih1 * g.iw + iw0) : 0.0f;
            const float x11 = (r1 && c1) ? __ldg(xp + (int64_t)ih1 * g.iw + iw1) : 0.0f;
            const float4* wv = reinterpret_cast<const float4*>(wsm + tap * ocp + oc0);
#pragma unroll
            for (int j = 0; j < kOcChunk / 4; ++j) {
              const float4 w4 = wv[j];
              const float ww[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                a00[4 * j + e] = fmaf(x00, ww[e], a00[4 * j + e]);
                a01[4 * j + e] = fmaf(x01, ww[e], a01[4 * j + e]);
                a10[4 * j + e] = fmaf(x10, ww[e], a10[4 * j + e]);
                a11[4 * j + e] = fmaf(x11, ww[e], a11[4 * j + e]);
              }
            }
          }
        }
      }
#pragma unroll
      for (int o = 0; o < kOcChunk; ++o) {
        const int oc = oc0 + o;
        if (oc < g.oc) {
          const float b = bias ? __ldg(bias + oc) : 0.0f;
          float y00 = a00[o], y01 = a01[o], y10 = a10[o], y11 = a11[o];
          if (bias) { y00 = __fadd_rn(y00, b); y01 = __fadd_rn(y01, b); y10 = __fadd_rn(y10, b); y11 = __fadd_rn(y11, b); }
          y00 = act_apply(y00, act, alpha); y01 = act_apply(y01, act, alpha);
          y10 = act_apply(y10, act, alpha); y11 = act_apply(y11, act, alpha);
          if (pool) {
            float m = fmaxf(-CUDART_INF_F, y00);
            if (v01) m = fmaxf(m, y01);
            if (v10) m = fmaxf(m, y10);
            if (v01 && v10) m = fmaxf(m, y11);
            float* dst = Y + (n * g.oc + oc) * pool_plane + (int64_t)qy * qw + qx;
            *dst = accumulate ? __fadd_rn(*dst, m) : m;
          } else {
            float* dst = Y + (n * g.oc + oc) * out_plane + (int64_t)oh0 * g.ow + ow0;
            if (accumulate) {
              dst[0] = __fadd_rn(dst[0], y00);
              if (v01) dst[1] = __fadd_rn(dst[1], y01);
              if (v10) dst[g.ow] = __fadd_rn(dst[g.ow], y10);
              if (v01 && v10) dst[g.ow + 1] = __fadd_rn(dst[g.ow + 1], y11);
            } else if (v01 && ((g.ow & 1) == 0) && ((((uintptr_t)dst) & 7) == 0)) {
              *reinterpret_cast<float2*>(dst) = make_float2(y00, y01);
              if (v10) *reinterpret_cast<float2*>(dst + g.ow) = make_float2(y10, y11);
            } else {
              dst[0] = y00;
              if (v01) dst[1] = y01;
              if (v10) dst[g.ow] = y10;
              if (v01 && v10) dst[g.ow + 1] = y11;
            }
          }
        }
      }
    }
  }
}

}  // namespace

namespace lnn {

// true when the direct kernel handles this geometry
bool conv_direct_applicable(const lnn_conv_geom* g) {
  const int ocp = (g->oc + kOcChunk - 1) / kOcChunk * kOcChunk;
  return g->ic <= 4 && (int64_t)g->ic * g->kh * g->kw * ocp <= kMaxWeights;
}

int conv_direct_fwd(Device* d, const lnn_conv_geom* g, float* Y, const float* X, const float* W,
                    const float* bias, int act, float alpha, int accumulate, int pool) {
  const int ocp = (g->oc + kOcChunk - 1) / kOcChunk * kOcChunk;
  const size_t smem = (size_t)g->ic * g->kh * g->kw * ocp * sizeof(float);
  const int64_t quads = (int64_t)g->n * ((g->oh + 1) / 2) * ((g->ow + 1) / 2);
  int64_t blocks = lnn_ceil_div(quads, kThreads);
  const int64_t cap = (int64_t)d->sm_count * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  conv_direct_fwd_kernel<<<(unsigned)blocks, kThreads, smem, d->stream>>>(Y, X, W, bias, *g, act, alpha,
                                                                         accumulate, pool);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

}  // namespace lnn
