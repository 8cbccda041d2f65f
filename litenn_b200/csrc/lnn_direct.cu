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
#include <algorithm>

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
// FAST_IC > 0: 3x3 taps, stride 1, dilation 1 and exactly FAST_IC input channels, everything
// unrolled (the quad's 4x4 input patch is read once per channel, validity of its rows and columns
// is decided once per quad); FAST_IC == 0: any geometry.  Same accumulation order in both.
template <int FAST_IC>
__global__ void __launch_bounds__(kThreads, 2)
conv_direct_fwd_kernel(float* __restrict__ Y, const float* __restrict__ X, const float* __restrict__ W,
                       const float* __restrict__ bias, lnn_conv_geom g, int act, float alpha,
                       int accumulate, int pool, int packed, float* __restrict__ Ylo, int ocp_out) {
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
  uint32_t amax = 0u;                       // packed == 2: largest magnitude this thread wrote
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
      if (FAST_IC > 0) {
        const int py = oh0 - g.padt, px = ow0 - g.padl;
        bool rok[4], cok[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          rok[r] = py + r >= 0 && py + r < g.ih;
          cok[r] = px + r >= 0 && px + r < g.iw;
        }
#pragma unroll 1
        for (int ic = 0; ic < FAST_IC; ++ic) {     // one channel's patch in registers at a time
          const float* xp = xin + ic * in_plane + (int64_t)py * g.iw + px;
          float xv[4][4];
#pragma unroll
          for (int r = 0; r < 4; ++r) {
#pragma unroll
            for (int c = 0; c < 4; ++c) xv[r][c] = (rok[r] && cok[c]) ? __ldg(xp + r * g.iw + c) : 0.0f;
          }
#pragma unroll
          for (int kh = 0; kh < 3; ++kh) {
#pragma unroll
            for (int kw = 0; kw < 3; ++kw) {
              const float4* wv = reinterpret_cast<const float4*>(wsm + ((ic * 3 + kh) * 3 + kw) * ocp + oc0);
#pragma unroll
              for (int j = 0; j < kOcChunk / 4; ++j) {
                const float4 w4 = wv[j];
                const float ww[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  a00[4 * j + e] = fmaf(xv[kh][kw], ww[e], a00[4 * j + e]);
                  a01[4 * j + e] = fmaf(xv[kh][kw + 1], ww[e], a01[4 * j + e]);
                  a10[4 * j + e] = fmaf(xv[kh + 1][kw], ww[e], a10[4 * j + e]);
                  a11[4 * j + e] = fmaf(xv[kh + 1][kw + 1], ww[e], a11[4 * j + e]);
                }
              }
            }
          }
        }
      }
      int tap = 0;
      for (int ic = 0; ic < (FAST_IC > 0 ? 0 : g.ic); ++ic) {
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
      if (packed) {
        // pooled result written channel-innermost and pre-split for the next convolution:
        // Y / Ylo are [n][qh][qw][ocp_out], this thread owns 16 consecutive channels of one pixel
        // (packed == 2: the fp32 values themselves go to Y and their largest magnitude, as a bit
        // pattern, to the word Ylo points at -- the fp16 split needs it before it can run)
        float hi[kOcChunk], lo[kOcChunk];
#pragma unroll
        for (int o = 0; o < kOcChunk; ++o) {
          const int oc = oc0 + o;
          float m = 0.0f;
          if (oc < g.oc) {
            const float b = bias ? __ldg(bias + oc) : 0.0f;
            float y00 = a00[o], y01 = a01[o], y10 = a10[o], y11 = a11[o];
            if (bias) { y00 = __fadd_rn(y00, b); y01 = __fadd_rn(y01, b); y10 = __fadd_rn(y10, b); y11 = __fadd_rn(y11, b); }
            y00 = act_apply(y00, act, alpha); y01 = act_apply(y01, act, alpha);
            y10 = act_apply(y10, act, alpha); y11 = act_apply(y11, act, alpha);
            m = fmaxf(-CUDART_INF_F, y00);
            if (v01) m = fmaxf(m, y01);
            if (v10) m = fmaxf(m, y10);
            if (v01 && v10) m = fmaxf(m, y11);
            if (m == -CUDART_INF_F) m = 0.0f;      // a window of NaNs, as the pooling kernel
          }
          if (packed == 2) {
            hi[o] = m; lo[o] = 0.0f;
            amax = max(amax, __float_as_uint(m) & 0x7fffffffu);
          } else {
            uint32_t r;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(m));
            hi[o] = __uint_as_float(r);
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(__fsub_rn(m, hi[o])));
            lo[o] = __uint_as_float(r);
          }
        }
        const int64_t pix = (n * qh + qy) * qw + qx;
#pragma unroll
        for (int o = 0; o < kOcChunk; o += 4) {
          if (oc0 + o < ocp_out) {
            *reinterpret_cast<float4*>(Y + pix * ocp_out + oc0 + o) = make_float4(hi[o], hi[o + 1], hi[o + 2], hi[o + 3]);
            if (Ylo && packed == 1)
              *reinterpret_cast<float4*>(Ylo + pix * ocp_out + oc0 + o) = make_float4(lo[o], lo[o + 1], lo[o + 2], lo[o + 3]);
          }
        }
        continue;
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
            if (m == -CUDART_INF_F) m = 0.0f;      // a window of NaNs, as the pooling kernel
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
  if (packed == 2) {
    // one atomic per warp for the whole launch
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0 && amax != 0u) atomicMax(reinterpret_cast<unsigned int*>(Ylo), amax);
  }
}

// -----------------------------------------------------------------------------------------
// Kernel gradient of the same layers (IC <= 4, 3x3 taps): dW[oc][ic][kh][kw] += sum over
// (n, oh, ow) of dY[n][oc][oh][ow] * X[n][ic][oh*s + kh*d - padt][ow*s + kw*d - padl]
// (litenn/core/op/conv2D.py:52-54).  The contraction runs over tens of millions of pixels
// but has only OC x IC*9 outputs, so a tensor-core tile would be almost all padding: each
// lane owns one output channel and keeps its IC*9 sums in registers, a warp walks groups of
// four pixels of a tile staged in shared memory (dY tile read as one 128-bit load per lane,
// X values as warp-wide broadcasts), and a block keeps accumulating over all the tiles it
// visits.  Block partials are combined in a fixed order by dw_direct_finalize_kernel, so the
// result does not depend on scheduling.
constexpr int kDwOc = 32;          // output channels per block (one per lane)
constexpr int kDwTilePix = 128;    // output pixels per tile

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
// asynchronous global -> shared copies; bytes beyond src_bytes are written as zeros
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int kDwXPer = 6;         // X-tile elements per thread whose position is precomputed

template <int IC, bool UNIT>
__global__ void __launch_bounds__(kThreads, 2)
conv_direct_dw_kernel(float* __restrict__ partial, const float* __restrict__ dY,
                      const float* __restrict__ X, lnn_conv_geom g, int tw, int th, int pp, int xr,
                      int xwp, int tiles_w, int tiles_h, int oc_chunks, int slots) {
  constexpr int T = IC * 9;
  extern __shared__ __align__(16) float sm[];
  const int buf_floats = kDwOc * pp + IC * xr * xwp;      // one stage: dY tile [32][pp], X tile [IC][xr][xwp]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunk = blockIdx.x % oc_chunks, slot = blockIdx.x / oc_chunks;
  const int oc0 = chunk * kDwOc;
  const int tile_pix = th * tw;                            // <= 128: at most one group of four per lane
  const int s = g.stride, dl = g.dilation;
  const bool vec_ok = (g.ow % 4 == 0) && ((((uintptr_t)dY) & 15) == 0);
  const int64_t in_plane = (int64_t)g.ih * g.iw, out_plane = (int64_t)g.oh * g.ow;
  float acc[T];
#pragma unroll
  for (int i = 0; i < T; ++i) acc[i] = 0.0f;

  // positions this thread copies for every tile
  const int my_p4 = lane * 4;
  const int my_r = my_p4 / tw, my_c = my_p4 - my_r * tw;
  const int x_elems = IC * xr * xwp;
  int x_pos[kDwXPer], x_off[kDwXPer];                      // (row << 16 | column), offset inside the image
#pragma unroll
  for (int k = 0; k < kDwXPer; ++k) {
    const int i = threadIdx.x + k * kThreads;
    const int cc = i % xwp, t3 = i / xwp;
    const int rr = t3 % xr, ic = t3 / xr;
    x_pos[k] = (rr << 16) | cc;
    x_off[k] = (int)(ic * in_plane) + rr * g.iw + cc;
  }

  const int64_t items = (int64_t)g.n * tiles_h * tiles_w;
  auto issue = [&](int64_t item, int b) {
    const int twi = (int)(item % tiles_w);
    const int64_t t2 = item / tiles_w;
    const int thi = (int)(t2 % tiles_h);
    const int64_t n = t2 / tiles_h;
    const int oh0 = thi * th, ow0 = twi * tw;
    float* dys = sm + b * buf_floats;
    float* xs = dys + kDwOc * pp;
    if (my_p4 < tile_pix) {
      const int oh = oh0 + my_r, ow = ow0 + my_c;
      const int nvalid = (oh < g.oh) ? max(0, min(4, g.ow - ow)) : 0;
#pragma unroll
      for (int k = 0; k < kDwOc / (kThreads / 32); ++k) {
        const int o = warp + k * (kThreads / 32);
        const int nv = (oc0 + o < g.oc) ? nvalid : 0;
        const float* q = nv ? dY + (n * g.oc + (oc0 + o)) * out_plane + (int64_t)oh * g.ow + ow : dY;
        const uint32_t dst = smem_addr(dys + o * pp + my_p4);
        if (vec_ok) cp_async_16(dst, q, nv * 4);
        else {
#pragma unroll
          for (int e = 0; e < 4; ++e) cp_async_4(dst + 4 * e, e < nv ? q + e : dY, e < nv ? 4 : 0);
        }
      }
    }
    const int ih0 = oh0 * s - g.padt, iw0 = ow0 * s - g.padl;
    const float* xn = X + n * g.ic * in_plane + (int64_t)ih0 * g.iw + iw0;
#pragma unroll
    for (int k = 0; k < kDwXPer; ++k) {
      const int i = threadIdx.x + k * kThreads;
      if (i < x_elems) {
        const int ih = ih0 + (x_pos[k] >> 16), iw = iw0 + (x_pos[k] & 0xffff);
        const bool ok = ih >= 0 && ih < g.ih && iw >= 0 && iw < g.iw;
        cp_async_4(smem_addr(xs + i), ok ? xn + x_off[k] : X, ok ? 4 : 0);
      }
    }
    for (int i = threadIdx.x + kDwXPer * kThreads; i < x_elems; i += kThreads) {
      const int cc = i % xwp, t3 = i / xwp;
      const int rr = t3 % xr, ic = t3 / xr;
      const int ih = ih0 + rr, iw = iw0 + cc;
      const bool ok = ih >= 0 && ih < g.ih && iw >= 0 && iw < g.iw;
      cp_async_4(smem_addr(xs + i), ok ? xn + ic * in_plane + (int64_t)rr * g.iw + cc : X, ok ? 4 : 0);
    }
    cp_async_commit();
  };

  int b = 0;
  if (slot < items) issue(slot, 0);
  for (int64_t item = slot; item < items; item += slots, b ^= 1) {
    const int64_t next = item + slots;
    if (next < items) { issue(next, b ^ 1); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();                          // this tile has landed for every thread
    const float* dys = sm + b * buf_floats;
    const float* xs = dys + kDwOc * pp;
    for (int p4 = warp * 4; p4 < tile_pix; p4 += (kThreads / 32) * 4) {
      const int r = p4 / tw, c = p4 - r * tw;
      const float4 dy = *reinterpret_cast<const float4*>(dys + lane * pp + p4);
#pragma unroll
      for (int ic = 0; ic < IC; ++ic) {
#pragma unroll
        for (int kh = 0; kh < 3; ++kh) {
          const float* xrow = xs + (ic * xr + r * s + kh * dl) * xwp;
          if (UNIT) {
            const float4 a = *reinterpret_cast<const float4*>(xrow + c);
            const float2 b2 = *reinterpret_cast<const float2*>(xrow + c + 4);
            const float xv[6] = {a.x, a.y, a.z, a.w, b2.x, b2.y};
#pragma unroll
            for (int kw = 0; kw < 3; ++kw) {
              float t = acc[(ic * 3 + kh) * 3 + kw];
              t = fmaf(dy.x, xv[kw], t);
              t = fmaf(dy.y, xv[kw + 1], t);
              t = fmaf(dy.z, xv[kw + 2], t);
              t = fmaf(dy.w, xv[kw + 3], t);
              acc[(ic * 3 + kh) * 3 + kw] = t;
            }
          } else {
#pragma unroll
            for (int kw = 0; kw < 3; ++kw) {
              const float* xq = xrow + c * s + kw * dl;
              float t = acc[(ic * 3 + kh) * 3 + kw];
              t = fmaf(dy.x, xq[0], t);
              t = fmaf(dy.y, xq[s], t);
              t = fmaf(dy.z, xq[2 * s], t);
              t = fmaf(dy.w, xq[3 * s], t);
              acc[(ic * 3 + kh) * 3 + kw] = t;
            }
          }
        }
      }
    }
    __syncthreads();                          // stage b may be refilled by the next iteration's issue
  }
  // combine the eight warps in warp order, then publish this block's partial
  float* red = sm;                            // [warps][T][32]
#pragma unroll
  for (int i = 0; i < T; ++i) red[(warp * T + i) * 32 + lane] = acc[i];
  __syncthreads();
  for (int i = threadIdx.x; i < T * 32; i += kThreads) {
    float v = red[i];
    for (int w = 1; w < kThreads / 32; ++w) v = __fadd_rn(v, red[w * T * 32 + i]);
    const int t = i >> 5, o = i & 31;
    partial[((int64_t)slot * oc_chunks * kDwOc + oc0 + o) * T + t] = v;
  }
}

// dW[oc][t] += partial[0][oc][t] + partial[1][oc][t] + ... (slot order)
__global__ void __launch_bounds__(kThreads)
dw_direct_finalize_kernel(float* __restrict__ dW, const float* __restrict__ partial, int oc, int T,
                          int ocp, int slots) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= oc * T) return;
  float v = 0.0f;
  for (int k = 0; k < slots; ++k) v = __fadd_rn(v, partial[(int64_t)k * ocp * T + i]);
  dW[i] = __fadd_rn(dW[i], v);
}

// Kernel gradient of a pooled block (conv -> leaky_relu -> max_pool2D(2,2)) with few input
// channels, 3x3, unit stride, from the WINNERS: the gradient of the convolution output is zero
// except at one position per pooling window, so instead of walking every pixel of a
// full-resolution dZ (three quarters zeros) a lane (= output channel) walks the windows: T holds
// the winner's gradient, IDX its position (0..3 row-major, 4 = none).  Per window 27 broadcast-free
// shared-memory loads (four distinct addresses per warp, in distinct banks: the X row pitch is
// 4 mod 32) and 27 FMAs, a quarter of the full-resolution kernel's.  One tile = 4 window rows x 32
// window columns (8 x 64 pixels); accumulation order is fixed (deterministic), block partials are
// added in slot order by dw_direct_finalize_kernel.
constexpr int kWinRows = 4, kWinCols = 32, kWinTile = kWinRows * kWinCols;   // windows per tile
constexpr int kWinTPitch = kWinTile + 4;          // floats per channel row of the T tile (pitch / 4 odd)
constexpr int kWinIPitch = kWinTile + 4;          // bytes per channel row of the IDX tile (33 words)
constexpr int kWinXRows = 2 * kWinRows + 2, kWinXPitch = 2 * kWinCols + 4;   // 10 x 68 (66 used)

template <int IC>
__global__ void __launch_bounds__(kThreads)
conv_dw_winners_kernel(float* __restrict__ partial, const float* __restrict__ T, const uint8_t* __restrict__ IDX,
                       const float* __restrict__ X, lnn_conv_geom g, int tiles_w, int tiles_h, int oc_chunks,
                       int slots) {
  constexpr int NT = IC * 9;
  extern __shared__ __align__(16) uint8_t smw[];
  constexpr int kTBytes = kDwOc * kWinTPitch * 4, kIBytes = kDwOc * kWinIPitch;
  constexpr int kXFloats = IC * kWinXRows * kWinXPitch;
  constexpr int kStage = kTBytes + kIBytes + kXFloats * 4;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunk = blockIdx.x % oc_chunks, slot = blockIdx.x / oc_chunks;
  const int oc0 = chunk * kDwOc;
  const int ohp = g.oh >> 1, owp = g.ow >> 1;
  const int64_t in_plane = (int64_t)g.ih * g.iw, pool_plane = (int64_t)ohp * owp;
  float acc[NT];
#pragma unroll
  for (int i = 0; i < NT; ++i) acc[i] = 0.0f;

  const int64_t items = (int64_t)g.n * tiles_h * tiles_w;
  auto issue = [&](int64_t item, int b) {
    const int twi = (int)(item % tiles_w);
    const int64_t t2 = item / tiles_w;
    const int thi = (int)(t2 % tiles_h);
    const int64_t n = t2 / tiles_h;
    const int py0 = thi * kWinRows, px0 = twi * kWinCols;
    uint8_t* st = smw + (size_t)b * kStage;
    // T: 32 channels x 4 window rows x 32 floats = 1024 pieces of 16 bytes; IDX: as many of 4 bytes
    for (int i = threadIdx.x; i < kDwOc * kWinRows * 8; i += kThreads) {
      const int piece = i & 7, rw = (i >> 3) % kWinRows, o = i / (8 * kWinRows);
      const bool ok = oc0 + o < g.oc && py0 + rw < ohp;
      const int64_t off = ((n * g.oc + oc0 + o) * ohp + py0 + rw) * (int64_t)owp + px0 + 4 * piece;
      cp_async_16(smem_addr(st + (o * kWinTPitch + rw * kWinCols + 4 * piece) * 4), ok ? T + off : T, ok ? 16 : 0);
      cp_async_4(smem_addr(st + kTBytes + o * kWinIPitch + rw * kWinCols + 4 * piece), ok ? IDX + off : IDX, ok ? 4 : 0);
    }
    const int ih0 = 2 * py0 - 1, iw0 = 2 * px0 - 1;
    float* xs = reinterpret_cast<float*>(st + kTBytes + kIBytes);
    const float* xn = X + n * g.ic * in_plane;
    for (int i = threadIdx.x; i < IC * kWinXRows * (2 * kWinCols + 2); i += kThreads) {
      const int cc = i % (2 * kWinCols + 2), t3 = i / (2 * kWinCols + 2);
      const int rr = t3 % kWinXRows, ic = t3 / kWinXRows;
      const int ih = ih0 + rr, iw = iw0 + cc;
      const bool ok = ih >= 0 && ih < g.ih && iw >= 0 && iw < g.iw;
      cp_async_4(smem_addr(xs + (ic * kWinXRows + rr) * kWinXPitch + cc),
                 ok ? xn + ic * in_plane + (int64_t)ih * g.iw + iw : X, ok ? 4 : 0);
    }
    cp_async_commit();
  };

  int b = 0;
  if (slot < items) issue(slot, 0);
  for (int64_t item = slot; item < items; item += slots, b ^= 1) {
    const int64_t next = item + slots;
    if (next < items) { issue(next, b ^ 1); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();
    const uint8_t* st = smw + (size_t)b * kStage;
    const float* ts = reinterpret_cast<const float*>(st) + lane * kWinTPitch;
    const uint8_t* is = st + kTBytes + lane * kWinIPitch;
    const float* xs = reinterpret_cast<const float*>(st + kTBytes + kIBytes);
    for (int grp = warp; grp < kWinTile / 4; grp += kThreads / 32) {
      const float4 t4 = *reinterpret_cast<const float4*>(ts + 4 * grp);
      const uint32_t w4 = *reinterpret_cast<const uint32_t*>(is + 4 * grp);
      const float tv[4] = {t4.x, t4.y, t4.z, t4.w};
      const int rw = (4 * grp) / kWinCols, pw0 = (4 * grp) % kWinCols;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int wi = (int)((w4 >> (8 * e)) & 0xffu);
        const float t = wi > 3 ? 0.0f : tv[e];
        const int wy = (wi >> 1) & 1, wx = wi & 1;
        const float* xb = xs + (2 * rw + wy) * kWinXPitch + 2 * (pw0 + e) + wx;
#pragma unroll
        for (int ic = 0; ic < IC; ++ic)
#pragma unroll
          for (int kh = 0; kh < 3; ++kh)
#pragma unroll
            for (int kw = 0; kw < 3; ++kw)
              acc[(ic * 3 + kh) * 3 + kw] = fmaf(t, xb[(ic * kWinXRows + kh) * kWinXPitch + kw], acc[(ic * 3 + kh) * 3 + kw]);
      }
    }
    __syncthreads();
  }
  float* red = reinterpret_cast<float*>(smw);      // [warps][NT][32]
#pragma unroll
  for (int i = 0; i < NT; ++i) red[(warp * NT + i) * 32 + lane] = acc[i];
  __syncthreads();
  for (int i = threadIdx.x; i < NT * 32; i += kThreads) {
    float v = red[i];
    for (int w = 1; w < kThreads / 32; ++w) v = __fadd_rn(v, red[w * NT * 32 + i]);
    const int t = i >> 5, o = i & 31;
    partial[((int64_t)slot * oc_chunks * kDwOc + oc0 + o) * NT + t] = v;
  }
}

struct DwPlan { int tw, th, pp, xr, xwp, tiles_w, tiles_h; size_t smem; };

DwPlan plan_dw(const lnn_conv_geom* g) {
  DwPlan q;
  q.tw = std::min(kDwTilePix, (g->ow + 3) & ~3);
  q.th = std::max(1, std::min(g->oh, kDwTilePix / q.tw));
  q.pp = ((q.th * q.tw + 7) & ~7) + 4;                   // pitch / 4 odd: conflict-free 128-bit reads
  q.xr = (q.th - 1) * g->stride + 2 * g->dilation + 1;
  q.xwp = ((q.tw - 1) * g->stride + 2 * g->dilation + 1 + 3) & ~3;
  q.tiles_w = (g->ow + q.tw - 1) / q.tw;
  q.tiles_h = (g->oh + q.th - 1) / q.th;
  const size_t tile = 2 * (size_t)(kDwOc * q.pp + g->ic * q.xr * q.xwp) * sizeof(float);   // two stages
  const size_t red = (size_t)(kThreads / 32) * g->ic * 9 * 32 * sizeof(float);
  q.smem = std::max(tile, red);
  return q;
}

}  // namespace

namespace lnn {

bool conv_direct_dw_applicable(const lnn_conv_geom* g) {
  if (g->ic > 4 || g->kh != 3 || g->kw != 3) return false;
  return plan_dw(g).smem <= 96 * 1024;
}

int conv_direct_dw(Device* d, const lnn_conv_geom* g, float* dW, const float* dY, const float* X) {
  const DwPlan q = plan_dw(g);
  const int oc_chunks = (g->oc + kDwOc - 1) / kDwOc;
  const int64_t items = (int64_t)g->n * q.tiles_h * q.tiles_w;
  int slots = (int)std::min<int64_t>(items, std::max(1, d->sm_count * 2 / oc_chunks));
  const int T = g->ic * 9;
  Scratch part(d);
  int rc = part.get((uint64_t)slots * oc_chunks * kDwOc * T * sizeof(float));
  if (rc) return rc;
  const bool unit = g->stride == 1 && g->dilation == 1;
  const unsigned grid = (unsigned)(slots * oc_chunks);
#define LNN_DW_CASE(IC_, U_)                                                                        \
  do {                                                                                              \
    auto kern = conv_direct_dw_kernel<IC_, U_>;                                                     \
    if (q.smem > 48 * 1024)                                                                         \
      LNN_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)q.smem)); \
    kern<<<grid, kThreads, q.smem, d->stream>>>(part.as<float>(), dY, X, *g, q.tw, q.th, q.pp, q.xr, \
                                                q.xwp, q.tiles_w, q.tiles_h, oc_chunks, slots);     \
  } while (0)
  switch (g->ic * 2 + (unit ? 1 : 0)) {
    case 2: LNN_DW_CASE(1, false); break;
    case 3: LNN_DW_CASE(1, true); break;
    case 4: LNN_DW_CASE(2, false); break;
    case 5: LNN_DW_CASE(2, true); break;
    case 6: LNN_DW_CASE(3, false); break;
    case 7: LNN_DW_CASE(3, true); break;
    case 8: LNN_DW_CASE(4, false); break;
    default: LNN_DW_CASE(4, true); break;
  }
#undef LNN_DW_CASE
  LNN_CHECK_LAUNCH(d);
  dw_direct_finalize_kernel<<<(g->oc * T + kThreads - 1) / kThreads, kThreads, 0, d->stream>>>(
      dW, part.as<float>(), g->oc, T, oc_chunks * kDwOc, slots);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

// the pooled block's kernel gradient from winners: 3x3, unit stride and dilation, 'same' padding,
// whole tiles of pooled columns
bool conv_dw_winners_applicable(const lnn_conv_geom* g) {
  return g->ic <= 4 && g->kh == 3 && g->kw == 3 && g->stride == 1 && g->dilation == 1 && g->padl == 1 &&
         g->padt == 1 && g->oh == g->ih && g->ow == g->iw && (g->oh & 1) == 0 && g->ow % (2 * kWinCols) == 0;
}

int conv_dw_winners(Device* d, const lnn_conv_geom* g, float* dW, const float* T, const uint8_t* IDX, const float* X) {
  const int oc_chunks = (g->oc + kDwOc - 1) / kDwOc;
  const int tiles_w = (g->ow / 2) / kWinCols, tiles_h = (g->oh / 2 + kWinRows - 1) / kWinRows;
  const int64_t items = (int64_t)g->n * tiles_h * tiles_w;
  const int slots = (int)std::min<int64_t>(items, std::max(1, d->sm_count * 2 / oc_chunks));
  const int NT = g->ic * 9;
  Scratch part(d);
  int rc = part.get((uint64_t)slots * oc_chunks * kDwOc * NT * sizeof(float));
  if (rc) return rc;
  const size_t stage = (size_t)kDwOc * kWinTPitch * 4 + (size_t)kDwOc * kWinIPitch +
                       (size_t)g->ic * kWinXRows * kWinXPitch * 4;
  const size_t smem = std::max(2 * stage, (size_t)(kThreads / 32) * NT * 32 * sizeof(float));
  const unsigned grid = (unsigned)(slots * oc_chunks);
#define LNN_WIN_CASE(IC_)                                                                           \
  do {                                                                                              \
    auto kern = conv_dw_winners_kernel<IC_>;                                                        \
    LNN_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));   \
    kern<<<grid, kThreads, smem, d->stream>>>(part.as<float>(), T, IDX, X, *g, tiles_w, tiles_h, oc_chunks, slots); \
  } while (0)
  switch (g->ic) {
    case 1: LNN_WIN_CASE(1); break;
    case 2: LNN_WIN_CASE(2); break;
    case 3: LNN_WIN_CASE(3); break;
    default: LNN_WIN_CASE(4); break;
  }
#undef LNN_WIN_CASE
  LNN_CHECK_LAUNCH(d);
  dw_direct_finalize_kernel<<<(g->oc * NT + kThreads - 1) / kThreads, kThreads, 0, d->stream>>>(
      dW, part.as<float>(), g->oc, NT, oc_chunks * kDwOc, slots);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

// true when the direct kernel handles this geometry
bool conv_direct_applicable(const lnn_conv_geom* g) {
  const int ocp = (g->oc + kOcChunk - 1) / kOcChunk * kOcChunk;
  return g->ic <= 4 && (int64_t)g->ic * g->kh * g->kw * ocp <= kMaxWeights;
}

int conv_direct_fwd(Device* d, const lnn_conv_geom* g, float* Y, const float* X, const float* W,
                    const float* bias, int act, float alpha, int accumulate, int pool, int packed,
                    float* Ylo, int ocp_out) {
  const int ocp = (g->oc + kOcChunk - 1) / kOcChunk * kOcChunk;
  const size_t smem = (size_t)g->ic * g->kh * g->kw * ocp * sizeof(float);
  const int64_t quads = (int64_t)g->n * ((g->oh + 1) / 2) * ((g->ow + 1) / 2);
  int64_t blocks = lnn_ceil_div(quads, kThreads);
  const int64_t cap = (int64_t)d->sm_count * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  const bool fast = g->kh == 3 && g->kw == 3 && g->stride == 1 && g->dilation == 1;
#define LNN_FWD_LAUNCH(F_)                                                                               \
  conv_direct_fwd_kernel<F_><<<(unsigned)blocks, kThreads, smem, d->stream>>>(Y, X, W, bias, *g, act, alpha, \
                                                                              accumulate, pool, packed, Ylo, ocp_out)
  switch (fast ? g->ic : 0) {
    case 1: LNN_FWD_LAUNCH(1); break;
    case 2: LNN_FWD_LAUNCH(2); break;
    case 3: LNN_FWD_LAUNCH(3); break;
    case 4: LNN_FWD_LAUNCH(4); break;
    default: LNN_FWD_LAUNCH(0); break;
  }
#undef LNN_FWD_LAUNCH
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

}  // namespace lnn
