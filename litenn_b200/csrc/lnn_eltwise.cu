// HBM-bound element-wise, broadcast-binary, fused scale+bias+leaky_relu, fill and SGD
// kernels.  Arithmetic follows the OpenCL C text the reference generates, with every
// literal single precision (the reference builds with -cl-single-precision-constant,
// litenn/core/minicl/CLDevice.py:93), comparisons converted int->float and multiplied
// in, and no fused multiply-add: each reference operator is its own rounding step, so
// the intrinsics __fmul_rn/__fadd_rn/__fsub_rn/__fdiv_rn are used throughout.
#include "lnn_common.cuh"
#include <algorithm>

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float fmul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float fadd(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float fsub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float fdiv(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ float b2f(bool c) { return c ? 1.0f : 0.0f; }

// ---- element-wise bodies (litenn/core/op/element_wise_op.py:112-364) -------------------

template <int OP>
__device__ __forceinline__ float ew_fwd(float I, float p0, float p1) {
  if (OP == LNN_EW_ABS) return fabsf(I);
  if (OP == LNN_EW_ADD_CONST) return fadd(I, p0);
  if (OP == LNN_EW_CLIP)
    return fadd(fadd(fmul(I, b2f((I >= p0) & (I <= p1))), fmul(p0, b2f(I < p0))),
                fmul(p1, b2f(I > p1)));
  if (OP == LNN_EW_COS) return cosf(I);
  if (OP == LNN_EW_EXP) return expf(I);
  if (OP == LNN_EW_LEAKY_RELU)
    return fadd(fmul(I, b2f(I >= 0.0f)), fmul(fmul(p0, I), b2f(I < 0.0f)));
  if (OP == LNN_EW_LOG) return logf(I);
  if (OP == LNN_EW_MUL_CONST) return fmul(I, p0);
  if (OP == LNN_EW_RDIV_CONST) return fdiv(p0, I);
  if (OP == LNN_EW_RSUB_CONST) return fsub(p0, I);
  if (OP == LNN_EW_RELU) return fmul(I, b2f(I >= 0.0f));
  if (OP == LNN_EW_SIGMOID) return fdiv(1.0f, fadd(1.0f, expf(-I)));
  if (OP == LNN_EW_SIN) return sinf(I);
  if (OP == LNN_EW_SQRT) return __fsqrt_rn(I);
  if (OP == LNN_EW_SQUARE) return fmul(I, I);
  if (OP == LNN_EW_TANH)
    return fsub(fdiv(2.0f, fadd(1.0f, expf(fmul(-2.0f, I)))), 1.0f);
  return 0.0f;
}

template <int OP>
__device__ __forceinline__ float ew_bwd(float I, float O, float dO, float p0, float p1, int flag) {
  if (OP == LNN_EW_ABS) return fmul(dO, fdiv(I, fabsf(I)));
  if (OP == LNN_EW_ADD_CONST) return dO;
  if (OP == LNN_EW_CLIP) return flag ? dO : fmul(dO, b2f((I >= p0) & (I <= p1)));
  if (OP == LNN_EW_COS) return fmul(dO, -sinf(I));
  if (OP == LNN_EW_EXP) return fmul(dO, expf(I));
  if (OP == LNN_EW_LEAKY_RELU)
    return fmul(dO, fadd(b2f(I >= 0.0f), fmul(p0, b2f(I < 0.0f))));
  if (OP == LNN_EW_LOG) return fmul(dO, fdiv(1.0f, I));
  if (OP == LNN_EW_MUL_CONST) return fmul(dO, p0);
  if (OP == LNN_EW_RDIV_CONST) return fmul(dO, -fdiv(p0, fmul(I, I)));
  if (OP == LNN_EW_RSUB_CONST) return -dO;
  if (OP == LNN_EW_RELU) return fmul(dO, b2f(I >= 0.0f));
  if (OP == LNN_EW_SIGMOID) return fmul(dO, fmul(O, fsub(1.0f, O)));
  if (OP == LNN_EW_SIN) return fmul(dO, cosf(I));
  if (OP == LNN_EW_SQRT) return fmul(dO, fdiv(1.0f, fmul(2.0f, __fsqrt_rn(I))));
  if (OP == LNN_EW_SQUARE) return fmul(fmul(dO, 2.0f), I);
  if (OP == LNN_EW_TANH) return fmul(dO, fsub(1.0f, fmul(O, O)));
  return 0.0f;
}

template <int OP>
__global__ void __launch_bounds__(kThreads)
ew_fwd_kernel(float* __restrict__ O, const float* __restrict__ I, int64_t n, float p0, float p1,
              int acc, int vec) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  if (vec) {
    const int64_t n4 = n >> 2;
    const float4* I4 = reinterpret_cast<const float4*>(I);
    float4* O4 = reinterpret_cast<float4*>(O);
    for (int64_t i = tid; i < n4; i += nthreads) {
      float4 v = __ldcs(I4 + i);
      float4 r;
      r.x = ew_fwd<OP>(v.x, p0, p1); r.y = ew_fwd<OP>(v.y, p0, p1);
      r.z = ew_fwd<OP>(v.z, p0, p1); r.w = ew_fwd<OP>(v.w, p0, p1);
      if (acc) {
        float4 o = O4[i];
        r.x = fadd(o.x, r.x); r.y = fadd(o.y, r.y); r.z = fadd(o.z, r.z); r.w = fadd(o.w, r.w);
      }
      O4[i] = r;
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += nthreads) {
      float r = ew_fwd<OP>(I[i], p0, p1);
      O[i] = acc ? fadd(O[i], r) : r;
    }
  } else {
    for (int64_t i = tid; i < n; i += nthreads) {
      float r = ew_fwd<OP>(I[i], p0, p1);
      O[i] = acc ? fadd(O[i], r) : r;
    }
  }
}

template <int OP>
__global__ void __launch_bounds__(kThreads)
ew_bwd_kernel(float* __restrict__ dI, const float* __restrict__ I, const float* __restrict__ O,
              const float* __restrict__ dO, int64_t n, float p0, float p1, int flag, int vec) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  if (vec) {
    const int64_t n4 = n >> 2;
    for (int64_t i = tid; i < n4; i += nthreads) {
      float4 vi = reinterpret_cast<const float4*>(I)[i];
      float4 vo = reinterpret_cast<const float4*>(O)[i];
      float4 vd = reinterpret_cast<const float4*>(dO)[i];
      float4 g = reinterpret_cast<float4*>(dI)[i];
      g.x = fadd(g.x, ew_bwd<OP>(vi.x, vo.x, vd.x, p0, p1, flag));
      g.y = fadd(g.y, ew_bwd<OP>(vi.y, vo.y, vd.y, p0, p1, flag));
      g.z = fadd(g.z, ew_bwd<OP>(vi.z, vo.z, vd.z, p0, p1, flag));
      g.w = fadd(g.w, ew_bwd<OP>(vi.w, vo.w, vd.w, p0, p1, flag));
      reinterpret_cast<float4*>(dI)[i] = g;
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += nthreads)
      dI[i] = fadd(dI[i], ew_bwd<OP>(I[i], O[i], dO[i], p0, p1, flag));
  } else {
    for (int64_t i = tid; i < n; i += nthreads)
      dI[i] = fadd(dI[i], ew_bwd<OP>(I[i], O[i], dO[i], p0, p1, flag));
  }
}

// ---- broadcast binary bodies (litenn/core/op/dual_wise_op.py:194-312) ------------------

template <int OP>
__device__ __forceinline__ float bin_fwd(float A, float B) {
  if (OP == LNN_BIN_ADD) return fadd(A, B);
  if (OP == LNN_BIN_SUB) return fsub(A, B);
  if (OP == LNN_BIN_MUL) return fmul(A, B);
  if (OP == LNN_BIN_DIV) return fdiv(A, B);
  if (OP == LNN_BIN_MAX) return fmaxf(A, B);
  if (OP == LNN_BIN_MIN) return fminf(A, B);
  if (OP == LNN_BIN_BCE)
    return fsub(fmul(-B, logf(A)), fmul(fsub(1.0f, B), logf(fsub(1.0f, A))));
  return 0.0f;
}

template <int OP, int WHICH>
__device__ __forceinline__ float bin_bwd(float A, float B, float O, float dO) {
  if (WHICH == 0) {
    if (OP == LNN_BIN_ADD || OP == LNN_BIN_SUB) return dO;
    if (OP == LNN_BIN_MUL) return fmul(dO, B);
    if (OP == LNN_BIN_DIV) return fdiv(dO, B);
    if (OP == LNN_BIN_MAX) return fmul(dO, b2f(A >= B));
    if (OP == LNN_BIN_MIN) return fmul(dO, b2f(A <= B));
    if (OP == LNN_BIN_BCE) return fdiv(fmul(dO, fsub(A, B)), fmul(A, fsub(1.0f, A)));
  } else {
    if (OP == LNN_BIN_ADD) return dO;
    if (OP == LNN_BIN_SUB) return -dO;
    if (OP == LNN_BIN_MUL) return fmul(dO, A);
    if (OP == LNN_BIN_DIV) return fmul(dO, -fdiv(A, fmul(B, B)));
    if (OP == LNN_BIN_MAX) return fmul(dO, b2f(A < B));
    if (OP == LNN_BIN_MIN) return fmul(dO, b2f(A > B));
    if (OP == LNN_BIN_BCE) return dO;
  }
  return 0.0f;
}

struct BcastDims {
  int rank;
  int64_t o[LNN_MAX_DIMS];     // output extents
  int64_t as[LNN_MAX_DIMS];    // element strides of A (0 where broadcast)
  int64_t bs[LNN_MAX_DIMS];
};

__device__ __forceinline__ void bcast_offsets(const BcastDims& d, int64_t gid, int64_t& ao,
                                              int64_t& bo) {
  ao = 0; bo = 0;
#pragma unroll
  for (int k = LNN_MAX_DIMS - 1; k >= 0; --k) {
    if (k < d.rank) {
      int64_t q = gid / d.o[k];
      int64_t r = gid - q * d.o[k];
      ao += r * d.as[k];
      bo += r * d.bs[k];
      gid = q;
    }
  }
}

// mode 0: forward; 1: dA; 2: dB.  same=1: no broadcasting at all (flat indexing).
template <int OP, int MODE>
__global__ void __launch_bounds__(kThreads)
bin_kernel(float* __restrict__ X, const float* __restrict__ A, const float* __restrict__ B,
           const float* __restrict__ O, const float* __restrict__ dO, int64_t n, BcastDims d,
           int acc, int same) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = tid; i < n; i += nthreads) {
    int64_t ao = i, bo = i;
    if (!same) bcast_offsets(d, i, ao, bo);
    float a = A[ao], b = B[bo];
    float r;
    if (MODE == 0) {
      r = bin_fwd<OP>(a, b);
      X[i] = acc ? fadd(X[i], r) : r;
    } else {
      r = bin_bwd<OP, MODE - 1>(a, b, O[i], dO[i]);
      X[i] = fadd(X[i], r);
    }
  }
}

// Fast broadcast path: every operand is the full tensor, one element, or varies along a
// single contiguous run of axes, so its element index is i, 0 or (i / inner) % size -- no
// per-axis index decomposition.  With vec != 0 a thread handles four consecutive outputs.
enum { OPM_FULL = 0, OPM_SCALAR = 1, OPM_AXIS = 2, OPM_GENERIC = 3 };
struct Operand { int mode; int64_t inner, size; };

__device__ __forceinline__ float op_load1(const float* __restrict__ p, const Operand& o, int64_t i) {
  if (o.mode == OPM_FULL) return p[i];
  if (o.mode == OPM_SCALAR) return __ldg(p);
  return __ldg(p + (i / o.inner) % o.size);
}
__device__ __forceinline__ float4 op_load4(const float* __restrict__ p, const Operand& o, int64_t i) {
  if (o.mode == OPM_FULL) return *reinterpret_cast<const float4*>(p + i);
  if (o.mode == OPM_SCALAR) { const float v = __ldg(p); return make_float4(v, v, v, v); }
  if (o.inner == 1) return __ldg(reinterpret_cast<const float4*>(p + i % o.size));
  const float v = __ldg(p + (i / o.inner) % o.size);
  return make_float4(v, v, v, v);
}

template <int OP, int MODE>
__global__ void __launch_bounds__(kThreads)
bin_fast_kernel(float* __restrict__ X, const float* __restrict__ A, const float* __restrict__ B,
                const float* __restrict__ O, const float* __restrict__ dO, int64_t n, Operand oa,
                Operand ob, int acc, int vec) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  if (vec) {
    const int64_t n4 = n >> 2;
    for (int64_t q = tid; q < n4; q += nthreads) {
      const int64_t i = q << 2;
      const float4 a = op_load4(A, oa, i), b = op_load4(B, ob, i);
      float4 r;
      if (MODE == 0) {
        r.x = bin_fwd<OP>(a.x, b.x); r.y = bin_fwd<OP>(a.y, b.y);
        r.z = bin_fwd<OP>(a.z, b.z); r.w = bin_fwd<OP>(a.w, b.w);
      } else {
        const float4 o = *reinterpret_cast<const float4*>(O + i);
        const float4 g = *reinterpret_cast<const float4*>(dO + i);
        r.x = bin_bwd<OP, MODE - 1>(a.x, b.x, o.x, g.x); r.y = bin_bwd<OP, MODE - 1>(a.y, b.y, o.y, g.y);
        r.z = bin_bwd<OP, MODE - 1>(a.z, b.z, o.z, g.z); r.w = bin_bwd<OP, MODE - 1>(a.w, b.w, o.w, g.w);
      }
      float4* dst = reinterpret_cast<float4*>(X + i);
      if (acc || MODE != 0) {
        const float4 x = *dst;
        r.x = fadd(x.x, r.x); r.y = fadd(x.y, r.y); r.z = fadd(x.z, r.z); r.w = fadd(x.w, r.w);
      }
      *dst = r;
    }
    return;
  }
  for (int64_t i = tid; i < n; i += nthreads) {
    const float a = op_load1(A, oa, i), b = op_load1(B, ob, i);
    float r;
    if (MODE == 0) {
      r = bin_fwd<OP>(a, b);
      X[i] = acc ? fadd(X[i], r) : r;
    } else {
      r = bin_bwd<OP, MODE - 1>(a, b, O[i], dO[i]);
      X[i] = fadd(X[i], r);
    }
  }
}

// y (+)= leaky_relu(x*g + b): x[N,C,HW]; each (n,c) plane is contiguous.  One float4 per
// thread per step; the channel index is recovered per vector (HW % 4 == 0 on this path).
__global__ void __launch_bounds__(kThreads)
scale_bias_lrelu_vec_kernel(float4* __restrict__ Y, const float4* __restrict__ X,
                            const float* __restrict__ G, const float* __restrict__ Bv,
                            int64_t n4, int64_t hw4, int64_t c, float alpha, int acc) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = tid; i < n4; i += nthreads) {
    const int64_t ch = (i / hw4) % c;
    const float g = __ldg(G + ch), b = __ldg(Bv + ch);
    float4 v = __ldcs(X + i);
    float4 r;
    float t;
    t = fadd(fmul(v.x, g), b); r.x = fadd(fmul(t, b2f(t >= 0.0f)), fmul(fmul(alpha, t), b2f(t < 0.0f)));
    t = fadd(fmul(v.y, g), b); r.y = fadd(fmul(t, b2f(t >= 0.0f)), fmul(fmul(alpha, t), b2f(t < 0.0f)));
    t = fadd(fmul(v.z, g), b); r.z = fadd(fmul(t, b2f(t >= 0.0f)), fmul(fmul(alpha, t), b2f(t < 0.0f)));
    t = fadd(fmul(v.w, g), b); r.w = fadd(fmul(t, b2f(t >= 0.0f)), fmul(fmul(alpha, t), b2f(t < 0.0f)));
    if (acc) {
      float4 o = Y[i];
      r.x = fadd(o.x, r.x); r.y = fadd(o.y, r.y); r.z = fadd(o.z, r.z); r.w = fadd(o.w, r.w);
      Y[i] = r;
    } else {
      __stcs(Y + i, r);
    }
  }
}

__global__ void __launch_bounds__(kThreads)
scale_bias_lrelu_kernel(float* __restrict__ Y, const float* __restrict__ X,
                        const float* __restrict__ G, const float* __restrict__ Bv, int64_t n,
                        int64_t hw, int64_t c, float alpha, int acc) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = tid; i < n; i += nthreads) {
    const int64_t ch = (i / hw) % c;
    float t = fadd(fmul(X[i], G[ch]), Bv[ch]);
    float r = fadd(fmul(t, b2f(t >= 0.0f)), fmul(fmul(alpha, t), b2f(t < 0.0f)));
    Y[i] = acc ? fadd(Y[i], r) : r;
  }
}

__global__ void __launch_bounds__(kThreads)
fill_kernel(float* __restrict__ p, int64_t n, float v, int vec) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  if (vec) {
    const int64_t n4 = n >> 2;
    float4 v4 = make_float4(v, v, v, v);
    for (int64_t i = tid; i < n4; i += nthreads) reinterpret_cast<float4*>(p)[i] = v4;
    for (int64_t i = (n4 << 2) + tid; i < n; i += nthreads) p[i] = v;
  } else {
    for (int64_t i = tid; i < n; i += nthreads) p[i] = v;
  }
}

// A = -lr*G ; V += A  (litenn/core/optimizer/SGD.py:42-74 with momentum 0: the product
// is rounded, then added -- two kernels in the reference, two roundings here).
__global__ void __launch_bounds__(kThreads)
sgd_kernel(float* __restrict__ V, const float* __restrict__ G, int64_t n, float lr, float gscale,
           int use_scale) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = tid; i < n; i += nthreads) {
    float g = G[i];
    if (use_scale) g = fmul(g, gscale);
    V[i] = fadd(V[i], fmul(-lr, g));
  }
}

inline int grid_for(const lnn::Device* d, int64_t work_items) {
  int64_t blocks = lnn_ceil_div(work_items, kThreads);
  int64_t cap = (int64_t)d->sm_count * 8;   // 8 resident blocks of 256 threads per SM
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

inline bool aligned16(uint64_t p) { return (p & 15) == 0; }

}  // namespace

#define EW_DISPATCH(OPV, CALL)                                                            \
  switch (OPV) {                                                                          \
    case LNN_EW_ABS: { CALL(LNN_EW_ABS); break; }                                         \
    case LNN_EW_ADD_CONST: { CALL(LNN_EW_ADD_CONST); break; }                             \
    case LNN_EW_CLIP: { CALL(LNN_EW_CLIP); break; }                                       \
    case LNN_EW_COS: { CALL(LNN_EW_COS); break; }                                         \
    case LNN_EW_EXP: { CALL(LNN_EW_EXP); break; }                                         \
    case LNN_EW_LEAKY_RELU: { CALL(LNN_EW_LEAKY_RELU); break; }                           \
    case LNN_EW_LOG: { CALL(LNN_EW_LOG); break; }                                         \
    case LNN_EW_MUL_CONST: { CALL(LNN_EW_MUL_CONST); break; }                             \
    case LNN_EW_RDIV_CONST: { CALL(LNN_EW_RDIV_CONST); break; }                           \
    case LNN_EW_RSUB_CONST: { CALL(LNN_EW_RSUB_CONST); break; }                           \
    case LNN_EW_RELU: { CALL(LNN_EW_RELU); break; }                                       \
    case LNN_EW_SIGMOID: { CALL(LNN_EW_SIGMOID); break; }                                 \
    case LNN_EW_SIN: { CALL(LNN_EW_SIN); break; }                                         \
    case LNN_EW_SQRT: { CALL(LNN_EW_SQRT); break; }                                       \
    case LNN_EW_SQUARE: { CALL(LNN_EW_SQUARE); break; }                                   \
    case LNN_EW_TANH: { CALL(LNN_EW_TANH); break; }                                       \
    default: return lnn::set_error(LNN_E_INVALID, "unknown element-wise op %d", OPV);     \
  }

#define BIN_DISPATCH(OPV, CALL)                                                           \
  switch (OPV) {                                                                          \
    case LNN_BIN_ADD: { CALL(LNN_BIN_ADD); break; }                                       \
    case LNN_BIN_SUB: { CALL(LNN_BIN_SUB); break; }                                       \
    case LNN_BIN_MUL: { CALL(LNN_BIN_MUL); break; }                                       \
    case LNN_BIN_DIV: { CALL(LNN_BIN_DIV); break; }                                       \
    case LNN_BIN_MAX: { CALL(LNN_BIN_MAX); break; }                                       \
    case LNN_BIN_MIN: { CALL(LNN_BIN_MIN); break; }                                       \
    case LNN_BIN_BCE: { CALL(LNN_BIN_BCE); break; }                                       \
    default: return lnn::set_error(LNN_E_INVALID, "unknown binary op %d", OPV);           \
  }

static int make_bcast(BcastDims& bd, int rank, const int64_t* o_shape, const int64_t* a_shape,
                      const int64_t* b_shape, int64_t* n_out, int* same) {
  LNN_REQUIRE(rank >= 1 && rank <= LNN_MAX_DIMS, "rank %d out of range", rank);
  LNN_REQUIRE(o_shape && a_shape && b_shape, "null shape");
  bd.rank = rank;
  int64_t n = 1, astr = 1, bstr = 1;
  *same = 1;
  for (int k = rank - 1; k >= 0; --k) {
    LNN_REQUIRE(o_shape[k] >= 1, "bad extent");
    LNN_REQUIRE(a_shape[k] == o_shape[k] || a_shape[k] == 1, "A axis %d not broadcastable", k);
    LNN_REQUIRE(b_shape[k] == o_shape[k] || b_shape[k] == 1, "B axis %d not broadcastable", k);
    bd.o[k] = o_shape[k];
    bd.as[k] = (a_shape[k] == 1) ? 0 : astr;
    bd.bs[k] = (b_shape[k] == 1) ? 0 : bstr;
    if (a_shape[k] != o_shape[k] || b_shape[k] != o_shape[k]) *same = 0;
    astr *= a_shape[k];
    bstr *= b_shape[k];
    n *= o_shape[k];
  }
  for (int k = rank; k < LNN_MAX_DIMS; ++k) { bd.o[k] = 1; bd.as[k] = 0; bd.bs[k] = 0; }
  *n_out = n;
  return LNN_OK;
}

// Classify one operand of a broadcast: FULL (same shape as the output), SCALAR (one element)
// or AXIS (its non-broadcast axes are one contiguous run: element = (i / inner) % size).
static void classify_operand(int rank, const int64_t* o_shape, const int64_t* x_shape, Operand& op) {
  int64_t x_size = 1, o_size = 1;
  for (int k = 0; k < rank; ++k) { x_size *= x_shape[k]; o_size *= o_shape[k]; }
  op.inner = 1; op.size = 1;
  if (x_size == o_size) { op.mode = OPM_FULL; return; }
  if (x_size == 1) { op.mode = OPM_SCALAR; return; }
  // find the run of axes where the operand is not broadcast (ignoring size-1 output axes)
  int first = -1, last = -1;
  for (int k = 0; k < rank; ++k)
    if (x_shape[k] != 1) { if (first < 0) first = k; last = k; }
  for (int k = first; k <= last; ++k)
    if (x_shape[k] != o_shape[k]) { op.mode = OPM_GENERIC; return; }
  for (int k = first; k <= last; ++k) op.size *= o_shape[k];
  for (int k = last + 1; k < rank; ++k) op.inner *= o_shape[k];
  op.mode = OPM_AXIS;
}

static bool operand_vec_ok(const Operand& op, uint64_t ptr) {
  if (op.mode == OPM_FULL) return (ptr & 15) == 0;
  if (op.mode == OPM_SCALAR) return true;
  if (op.mode == OPM_AXIS) return (op.inner % 4 == 0) || (op.inner == 1 && op.size % 4 == 0 && (ptr & 15) == 0);
  return false;
}

namespace {

__device__ __forceinline__ uint32_t pcg_hash(uint32_t v);

// ---- softmax and categorical cross-entropy over the rows of a [rows, cols] matrix -------------
// The reference composes them from exp, reduce_sum, div (softmax, element_wise_op.py:309-314) and
// clip, log, mul_const, mul, reduce_sum (categorical_crossentropy, dual_wise_op.py:228-250), nine
// launches and as many gradient launches.  Here one block owns a row: same operations in the
// same order per element (no max-subtraction, clip to [1e-7, 1 - 1e-7]) and the row sums in the
// reference's ceil-halving tree order (reduce.py:285-291), so forward values are identical.
constexpr int kRowThreads = 256;
constexpr int kRowMax = 8192;        // columns a block keeps in shared memory (32 KB)

// In-place ceil-halving tree over v[0..n): v[i] += v[i + ceil(n/2)], n = ceil(n/2), ... ; result in v[0].
__device__ __forceinline__ float row_tree_sum(float* v, int n) {
  while (n > 1) {
    const int h = (n + 1) >> 1;
    __syncthreads();
    for (int i = threadIdx.x; i + h < n; i += blockDim.x) v[i] = fadd(v[i], v[i + h]);
    n = h;
  }
  __syncthreads();
  return v[0];
}

__global__ void __launch_bounds__(kRowThreads)
softmax_fwd_kernel(float* __restrict__ P, const float* __restrict__ X, int64_t rows, int cols) {
  __shared__ float e[kRowMax];
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const float* x = X + r * cols;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) e[i] = expf(x[i]);
    const float s = row_tree_sum(e, cols);
    __syncthreads();
    // the tree consumed e: the quotient uses a fresh exp of the same input (same value)
    for (int i = threadIdx.x; i < cols; i += blockDim.x) P[r * cols + i] = fdiv(expf(x[i]), s);
    __syncthreads();
  }
}

// dX += (dP / s - sum_j(dP_j * e_j / s^2)) * e : the gradients of div (both operands), of the
// keepdims sum and of exp, in that association (dual_wise_op.py:268-281, reduce.py:250-260,
// element_wise_op.py:181-188)
__global__ void __launch_bounds__(kRowThreads)
softmax_bwd_kernel(float* __restrict__ dX, const float* __restrict__ X, const float* __restrict__ dP,
                   int64_t rows, int cols) {
  __shared__ float e[kRowMax];
  __shared__ float s_sh;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const float* x = X + r * cols;
    const float* dp = dP + r * cols;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) e[i] = expf(x[i]);
    const float s = row_tree_sum(e, cols);
    __syncthreads();
    if (threadIdx.x == 0) s_sh = s;
    // ds = sum_j dP_j * (-e_j / (s * s))
    const float ss = fmul(s, s);
    for (int i = threadIdx.x; i < cols; i += blockDim.x) e[i] = fmul(dp[i], fdiv(-expf(x[i]), ss));
    const float ds = row_tree_sum(e, cols);
    __syncthreads();
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
      const float de = fadd(fdiv(dp[i], s), ds);
      dX[r * cols + i] = fadd(dX[r * cols + i], fmul(de, expf(x[i])));
    }
    __syncthreads();
  }
}

// L[r] = sum_j (-T[r][j]) * log(clip(P[r][j], 1e-7, 1 - 1e-7)); T is [rows, cols] or one row (stride 0)
__global__ void __launch_bounds__(kRowThreads)
cce_fwd_kernel(float* __restrict__ L, const float* __restrict__ P, const float* __restrict__ T, int64_t rows,
               int cols, int64_t t_row_stride) {
  __shared__ float v[kRowMax];
  const float lo = 1e-7f, hi = fsub(1.0f, 1e-7f);
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const float* p = P + r * cols;
    const float* t = T + r * t_row_stride;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
      const float c = fminf(fmaxf(p[i], lo), hi);
      v[i] = fmul(fmul(t[i], -1.0f), logf(c));
    }
    const float s = row_tree_sum(v, cols);
    if (threadIdx.x == 0) L[r] = s;
    __syncthreads();
  }
}

// dP += dL[r] * (-T) * (1 / c) where the clip passed the value through (element_wise_op.py:133-139)
__global__ void __launch_bounds__(kThreads)
cce_bwd_kernel(float* __restrict__ dP, const float* __restrict__ P, const float* __restrict__ T,
               const float* __restrict__ dL, int64_t total, int64_t cols, int64_t t_row_stride) {
  const float lo = 1e-7f, hi = fsub(1.0f, 1e-7f);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / cols, j = i - r * cols;
    const float p = P[i];
    const float c = fminf(fmaxf(p, lo), hi);
    // reduce_sum' broadcasts dL; mul' gives dL * (-T); log' gives * (1 / c); clip' passes inside [lo, hi]
    const float dlog = fmul(dL[r], fmul(T[r * t_row_stride + j], -1.0f));
    const float dc = fmul(dlog, fdiv(1.0f, c));
    dP[i] = fadd(dP[i], fmul(dc, (p >= lo && p <= hi) ? 1.0f : 0.0f));
  }
}

// One optimizer update per element, the reference's two or three kernels per tensor in one pass
// with the same operations in the same order (litenn/core/optimizer/SGD.py:42-83,
// RMSprop.py:37-69, Adam.py:43-84) and its learning-rate prologue (Optimizer.py:186-203):
// decay by 1 / (1 + lr_decay * iteration), then dropout of the step where the hash of
// (element index + seed) is <= lr_dropout.  SGD evaluates that prologue in both of its kernels,
// each with its own seed.  g is G * gscale when gscale != 1 (gradient averaging over replicas).
template <int KIND>
__global__ void __launch_bounds__(kThreads)
opt_kernel(float* __restrict__ V, const float* __restrict__ G, float* __restrict__ S1, float* __restrict__ S2,
           int64_t n, const lnn_opt_params p) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  float lr0 = p.lr;
  if (p.lr_decay != 0.0f) lr0 = fmul(lr0, fdiv(1.0f, fadd(1.0f, fmul(p.lr_decay, __uint2float_rn(p.iteration)))));
  const float uif = 1.0f / 4294967296.0f;
  for (int64_t i = tid; i < n; i += nthreads) {
    float g = G[i];
    if (p.gscale != 1.0f) g = fmul(g, p.gscale);
    float lr_a = lr0, lr_b = lr0;
    if (p.lr_dropout != 0.0f) {
      if (fmul(__uint2float_rn(pcg_hash((uint32_t)i + p.seed_a)), uif) <= p.lr_dropout) lr_a = 0.0f;
      if (fmul(__uint2float_rn(pcg_hash((uint32_t)i + p.seed_b)), uif) <= p.lr_dropout) lr_b = 0.0f;
    }
    if (KIND == LNN_OPT_SGD) {
      // A = momentum*A - lr*G ; V += A   (nesterov: V += momentum*A - lr*G with the new A)
      const float a = fsub(fmul(p.beta1, S1[i]), fmul(lr_a, g));
      S1[i] = a;
      V[i] = fadd(V[i], p.nesterov ? fsub(fmul(p.beta1, a), fmul(lr_b, g)) : a);
    } else if (KIND == LNN_OPT_RMSPROP) {
      // A = rho*A + (1-rho)*g*g ; V += -lr*G / (sqrt(A) + 1e-7)
      const float a = fadd(fmul(p.beta1, S1[i]), fmul(fmul(fsub(1.0f, p.beta1), g), g));
      S1[i] = a;
      V[i] = fadd(V[i], fdiv(fmul(-lr_b, g), fadd(__fsqrt_rn(a), 1e-7f)));
    } else {
      // M = b1*M + (1-b1)*G ; U = b2*U + (1-b2)*g*g ; V += -lr*M / (sqrt(U) + 1e-7)
      const float m = fadd(fmul(p.beta1, S1[i]), fmul(fsub(1.0f, p.beta1), g));
      const float u = fadd(fmul(p.beta2, S2[i]), fmul(fmul(fsub(1.0f, p.beta2), g), g));
      S1[i] = m; S2[i] = u;
      V[i] = fadd(V[i], fdiv(fmul(-lr_b, m), fadd(__fsqrt_rn(u), 1e-7f)));
    }
  }
}

// Random initializers: counter-based, one hash of (element index + seed) per element, so the
// result does not depend on the launch geometry.  PCG output functions as the reference uses
// them (litenn/core/CLKernelHelper.py:210-233; initializer/RandomUniform.py:12-20,
// RandomNormal.py:10-24); 2^-32 is the reference's 1 / (float)0xffffffff in single precision.
__device__ __forceinline__ uint32_t pcg_hash(uint32_t v) {
  const uint32_t state = v * 747796405u + 2891336453u;
  const uint32_t word = ((state >> ((state >> 28) + 4u)) ^ state) * 277803737u;
  return (word >> 22) ^ word;
}
__device__ __forceinline__ void pcg2d_hash(uint32_t& a, uint32_t& b) {
  a = a * 1664525u + 1013904223u; b = b * 1664525u + 1013904223u;
  a += b * 1664525u; b += a * 1664525u;
  a ^= a >> 16; b ^= b >> 16;
  a += b * 1664525u; b += a * 1664525u;
  a ^= a >> 16; b ^= b >> 16;
}
constexpr float kUIF = 1.0f / 4294967296.0f;

__global__ void __launch_bounds__(kThreads)
init_uniform_kernel(float* __restrict__ O, int64_t n, uint32_t seed, float low, float high) {
  const float range = fsub(high, low);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float h = fmul(__uint2float_rn(pcg_hash((uint32_t)((uint64_t)i + seed))), kUIF);
    O[i] = fadd(fmul(h, range), low);
  }
}

__global__ void __launch_bounds__(kThreads)
init_normal_kernel(float* __restrict__ O, int64_t n, uint32_t seed, float mean, float stddev) {
  const float two_pi = 2.0f * 3.14159274101257f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    uint32_t a = (uint32_t)((uint64_t)i + seed), b = 1u;
    pcg2d_hash(a, b);
    const float rx = fmul(__uint2float_rn(a), kUIF), ry = fmul(__uint2float_rn(b), kUIF);
    const float r = fmul(sqrtf(fmul(-2.0f, logf(rx))), cosf(fmul(two_pi, ry)));
    O[i] = fadd(mean, fmul(r, stddev));
  }
}

}  // namespace

extern "C" {

int lnn_init_uniform(int dev, uint64_t dst, int64_t count, uint32_t seed, float low, float high) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(dst && count > 0, "bad arguments");
  init_uniform_kernel<<<grid_for(d, count), kThreads, 0, d->stream>>>((float*)(uintptr_t)dst, count, seed, low, high);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

int lnn_init_normal(int dev, uint64_t dst, int64_t count, uint32_t seed, float mean, float stddev) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(dst && count > 0, "bad arguments");
  init_normal_kernel<<<grid_for(d, count), kThreads, 0, d->stream>>>((float*)(uintptr_t)dst, count, seed, mean, stddev);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

int lnn_fill_f32(int dev, uint64_t dst, int64_t count, float value) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(dst && count > 0, "bad arguments");
  int vec = aligned16(dst);
  fill_kernel<<<grid_for(d, vec ? count / 4 + 1 : count), kThreads, 0, d->stream>>>(
      (float*)(uintptr_t)dst, count, value, vec);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

int lnn_eltwise_fwd(int dev, int op, uint64_t O, uint64_t I, int64_t n, float p0, float p1,
                    int flag, int accumulate) {
  LNN_DEV(d, dev);
  (void)flag;
  LNN_REQUIRE(O && I && n > 0, "bad arguments");
  int vec = aligned16(O) && aligned16(I);
  int grid = grid_for(d, vec ? n / 4 + 1 : n);
#define CALL(OPC)                                                                         \
  ew_fwd_kernel<OPC><<<grid, kThreads, 0, d->stream>>>((float*)(uintptr_t)O,              \
      (const float*)(uintptr_t)I, n, p0, p1, accumulate, vec)
  EW_DISPATCH(op, CALL)
#undef CALL
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

int lnn_eltwise_bwd(int dev, int op, uint64_t dI, uint64_t I, uint64_t O, uint64_t dO, int64_t n,
                    float p0, float p1, int flag) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(dI && I && O && dO && n > 0, "bad arguments");
  int vec = aligned16(dI) && aligned16(I) && aligned16(O) && aligned16(dO);
  int grid = grid_for(d, vec ? n / 4 + 1 : n);
#define CALL(OPC)                                                                         \
  ew_bwd_kernel<OPC><<<grid, kThreads, 0, d->stream>>>((float*)(uintptr_t)dI,             \
      (const float*)(uintptr_t)I, (const float*)(uintptr_t)O, (const float*)(uintptr_t)dO, \
      n, p0, p1, flag, vec)
  EW_DISPATCH(op, CALL)
#undef CALL
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

int lnn_binary_fwd(int dev, int op, uint64_t O, uint64_t A, uint64_t B, int rank,
                   const int64_t* o_shape, const int64_t* a_shape, const int64_t* b_shape,
                   int accumulate) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(O && A && B, "null buffer");
  BcastDims bd; int64_t n; int same;
  int rc = make_bcast(bd, rank, o_shape, a_shape, b_shape, &n, &same);
  if (rc) return rc;
  Operand oa, ob;
  classify_operand(rank, o_shape, a_shape, oa);
  classify_operand(rank, o_shape, b_shape, ob);
  if (oa.mode != OPM_GENERIC && ob.mode != OPM_GENERIC) {
    const int vec = (n % 4 == 0) && aligned16(O) && operand_vec_ok(oa, A) && operand_vec_ok(ob, B);
    const int grid = grid_for(d, vec ? n / 4 : n);
#define CALL(OPC)                                                                         \
  bin_fast_kernel<OPC, 0><<<grid, kThreads, 0, d->stream>>>((float*)(uintptr_t)O,         \
      (const float*)(uintptr_t)A, (const float*)(uintptr_t)B, nullptr, nullptr, n, oa, ob, \
      accumulate, vec)
    BIN_DISPATCH(op, CALL)
#undef CALL
    LNN_CHECK_LAUNCH(d);
    return LNN_OK;
  }
  int grid = grid_for(d, n);
#define CALL(OPC)                                                                         \
  bin_kernel<OPC, 0><<<grid, kThreads, 0, d->stream>>>((float*)(uintptr_t)O,              \
      (const float*)(uintptr_t)A, (const float*)(uintptr_t)B, nullptr, nullptr, n, bd,    \
      accumulate, same)
  BIN_DISPATCH(op, CALL)
#undef CALL
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

int lnn_binary_bwd(int dev, int op, int which, uint64_t dX, uint64_t A, uint64_t B, uint64_t O,
                   uint64_t dO, int rank, const int64_t* o_shape, const int64_t* a_shape,
                   const int64_t* b_shape) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(dX && A && B && O && dO, "null buffer");
  LNN_REQUIRE(which == 0 || which == 1, "which must be 0 or 1");
  BcastDims bd; int64_t n; int same;
  int rc = make_bcast(bd, rank, o_shape, a_shape, b_shape, &n, &same);
  if (rc) return rc;
  Operand oa, ob;
  classify_operand(rank, o_shape, a_shape, oa);
  classify_operand(rank, o_shape, b_shape, ob);
  if (oa.mode != OPM_GENERIC && ob.mode != OPM_GENERIC) {
    const int vec = (n % 4 == 0) && aligned16(dX) && aligned16(O) && aligned16(dO) &&
                    operand_vec_ok(oa, A) && operand_vec_ok(ob, B);
    const int grid = grid_for(d, vec ? n / 4 : n);
#define CALL(OPC)                                                                         \
  if (which == 0)                                                                         \
    bin_fast_kernel<OPC, 1><<<grid, kThreads, 0, d->stream>>>((float*)(uintptr_t)dX,      \
        (const float*)(uintptr_t)A, (const float*)(uintptr_t)B, (const float*)(uintptr_t)O, \
        (const float*)(uintptr_t)dO, n, oa, ob, 1, vec);                                  \
  else                                                                                    \
    bin_fast_kernel<OPC, 2><<<grid, kThreads, 0, d->stream>>>((float*)(uintptr_t)dX,      \
        (const float*)(uintptr_t)A, (const float*)(uintptr_t)B, (const float*)(uintptr_t)O, \
        (const float*)(uintptr_t)dO, n, oa, ob, 1, vec)
    BIN_DISPATCH(op, CALL)
#undef CALL
    LNN_CHECK_LAUNCH(d);
    return LNN_OK;
  }
  int grid = grid_for(d, n);
#define CALL(OPC)                                                                         \
  if (which == 0)                                                                         \
    bin_kernel<OPC, 1><<<grid, kThreads, 0, d->stream>>>((float*)(uintptr_t)dX,           \
        (const float*)(uintptr_t)A, (const float*)(uintptr_t)B, (const float*)(uintptr_t)O, \
        (const float*)(uintptr_t)dO, n, bd, 1, same);                                     \
  else                                                                                    \
    bin_kernel<OPC, 2><<<grid, kThreads, 0, d->stream>>>((float*)(uintptr_t)dX,           \
        (const float*)(uintptr_t)A, (const float*)(uintptr_t)B, (const float*)(uintptr_t)O, \
        (const float*)(uintptr_t)dO, n, bd, 1, same)
  BIN_DISPATCH(op, CALL)
#undef CALL
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

int lnn_scale_bias_lrelu(int dev, uint64_t y, uint64_t x, uint64_t g, uint64_t b, int64_t n,
                         int64_t c, int64_t hw, float alpha, int accumulate) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(y && x && g && b && n > 0 && c > 0 && hw > 0, "bad arguments");
  int64_t total = n * c * hw;
  if ((hw & 3) == 0 && aligned16(y) && aligned16(x)) {
    int64_t n4 = total >> 2;
    scale_bias_lrelu_vec_kernel<<<grid_for(d, n4), kThreads, 0, d->stream>>>(
        (float4*)(uintptr_t)y, (const float4*)(uintptr_t)x, (const float*)(uintptr_t)g,
        (const float*)(uintptr_t)b, n4, hw >> 2, c, alpha, accumulate);
  } else {
    scale_bias_lrelu_kernel<<<grid_for(d, total), kThreads, 0, d->stream>>>(
        (float*)(uintptr_t)y, (const float*)(uintptr_t)x, (const float*)(uintptr_t)g,
        (const float*)(uintptr_t)b, total, hw, c, alpha, accumulate);
  }
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

int lnn_softmax_fwd(int dev, uint64_t P, uint64_t X, int64_t rows, int64_t cols) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(P && X && rows > 0 && cols > 0, "bad arguments");
  LNN_REQUIRE(cols <= kRowMax, "rows longer than %d elements are not supported by the fused softmax", kRowMax);
  softmax_fwd_kernel<<<(unsigned)std::min<int64_t>(rows, (int64_t)d->sm_count * 8), kRowThreads, 0, d->stream>>>(
      (float*)(uintptr_t)P, (const float*)(uintptr_t)X, rows, (int)cols);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

int lnn_softmax_bwd(int dev, uint64_t dX, uint64_t X, uint64_t dP, int64_t rows, int64_t cols) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(dX && X && dP && rows > 0 && cols > 0 && cols <= kRowMax, "bad arguments");
  softmax_bwd_kernel<<<(unsigned)std::min<int64_t>(rows, (int64_t)d->sm_count * 8), kRowThreads, 0, d->stream>>>(
      (float*)(uintptr_t)dX, (const float*)(uintptr_t)X, (const float*)(uintptr_t)dP, rows, (int)cols);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

int lnn_cce_fwd(int dev, uint64_t L, uint64_t P, uint64_t T, int64_t rows, int64_t cols, int64_t t_row_stride) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(L && P && T && rows > 0 && cols > 0 && cols <= kRowMax, "bad arguments");
  cce_fwd_kernel<<<(unsigned)std::min<int64_t>(rows, (int64_t)d->sm_count * 8), kRowThreads, 0, d->stream>>>(
      (float*)(uintptr_t)L, (const float*)(uintptr_t)P, (const float*)(uintptr_t)T, rows, (int)cols, t_row_stride);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

int lnn_cce_bwd(int dev, uint64_t dP, uint64_t P, uint64_t T, uint64_t dL, int64_t rows, int64_t cols,
                int64_t t_row_stride) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(dP && P && T && dL && rows > 0 && cols > 0, "bad arguments");
  cce_bwd_kernel<<<grid_for(d, rows * cols), kThreads, 0, d->stream>>>(
      (float*)(uintptr_t)dP, (const float*)(uintptr_t)P, (const float*)(uintptr_t)T, (const float*)(uintptr_t)dL,
      rows * cols, cols, t_row_stride);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

int lnn_optimizer_step(int dev, int kind, uint64_t V, uint64_t G, uint64_t S1, uint64_t S2, int64_t n,
                       const lnn_opt_params* p) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(V && G && n > 0 && p, "bad arguments");
  LNN_REQUIRE(kind >= LNN_OPT_SGD && kind <= LNN_OPT_ADAM, "unknown optimizer kind %d", kind);
  LNN_REQUIRE(S1 && (kind != LNN_OPT_ADAM || S2), "optimizer state buffer missing");
  float* v = (float*)(uintptr_t)V;
  const float* g = (const float*)(uintptr_t)G;
  float* s1 = (float*)(uintptr_t)S1;
  float* s2 = (float*)(uintptr_t)S2;
  const unsigned grid = (unsigned)grid_for(d, n);
  if (kind == LNN_OPT_SGD) opt_kernel<LNN_OPT_SGD><<<grid, kThreads, 0, d->stream>>>(v, g, s1, s2, n, *p);
  else if (kind == LNN_OPT_RMSPROP) opt_kernel<LNN_OPT_RMSPROP><<<grid, kThreads, 0, d->stream>>>(v, g, s1, s2, n, *p);
  else opt_kernel<LNN_OPT_ADAM><<<grid, kThreads, 0, d->stream>>>(v, g, s1, s2, n, *p);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

int lnn_sgd_step(int dev, uint64_t V, uint64_t G, int64_t n, float lr, float gscale) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(V && G && n > 0, "bad arguments");
  sgd_kernel<<<grid_for(d, n), kThreads, 0, d->stream>>>(
      (float*)(uintptr_t)V, (const float*)(uintptr_t)G, n, lr, gscale, gscale != 1.0f);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

}  // extern "C"
