// Reductions (sum, mean, max, min) with the reference's summation tree, one read of the
// input instead of the reference's transpose + log2(COLS) in-place stages + slice
// (litenn/core/op/reduce.py:166-205, stage kernel :279-293).
//
// The reference reduces a row of n values in stages: h = ceil(n/2); x[c] = x[c] (+) x[c+h]
// for every c with c+h < n; n = h; until n == 1.  With n_0 = COLS and n_j = ceil(n_{j-1}/2)
// the value at stage s, column c is V_s(c) = V_{s-1}(c) (+) V_{s-1}(c + n_s) when that
// partner exists, else V_{s-1}(c).  Here one thread evaluates a whole subtree V_s(c0) by a
// depth-first walk (a stack of one partial value per level), so the operand pairing, and
// therefore every rounding, is the reference's.  A row is finished either inside a block
// (shared-memory stages for the last levels) or, when a row is split over many threads
// to fill the GPU, by running the same routine again on the partial values -- the tree
// over n_s partials is by construction the tail of the tree over n_0 values.
#include "lnn_common.cuh"
#include <math_constants.h>

namespace {

constexpr int kThreads = 256;
constexpr int kMaxLevels = 40;

struct Levels {
  int S;                       // number of stages: n[S] == 1
  int64_t n[kMaxLevels + 1];   // n[0] = COLS, n[j] = ceil(n[j-1]/2)
};

struct RedGeom {
  int64_t outer, r0, mid, r1, inner;
  int64_t rows;        // outer*mid*inner
  int64_t stride_r0;   // mid*r1*inner
  int64_t stride_r1;   // inner
  int64_t stride_outer;// r0*mid*r1*inner
  int64_t stride_mid;  // r1*inner
};

template <int OP>
__device__ __forceinline__ float comb(float a, float b) {
  if (OP == LNN_RED_MAX) return fmaxf(a, b);
  if (OP == LNN_RED_MIN) return fminf(a, b);
  return __fadd_rn(a, b);
}

__device__ __forceinline__ int64_t row_base(const RedGeom& g, int64_t row) {
  const int64_t inner_i = row % g.inner;
  const int64_t t = row / g.inner;
  const int64_t mid_i = t % g.mid;
  const int64_t outer_i = t / g.mid;
  return outer_i * g.stride_outer + mid_i * g.stride_mid + inner_i;
}

// V_s(c0) of one row (base points at the row's column 0).
template <int OP>
__device__ float subtree(const float* __restrict__ base, int64_t c0, int s, const Levels& L,
                         const RedGeom& g) {
  float acc[kMaxLevels];
  int64_t leaf = c0;
  uint64_t m = 0;
  const bool one_group = (g.r0 == 1);
  for (;;) {
    int64_t off;
    if (one_group) {
      off = leaf * g.stride_r1;
    } else {
      const int64_t q = leaf / g.r1;
      off = q * g.stride_r0 + (leaf - q * g.r1) * g.stride_r1;
    }
    float v = __ldcs(base + off);
    int64_t cur = leaf;
    int j = 1;
    for (; j <= s; ++j) {
      if ((m >> (j - 1)) & 1ull) {
        v = comb<OP>(acc[j], v);
        cur -= L.n[j];
      } else if (cur + L.n[j] < L.n[j - 1]) {
        acc[j] = v;
        break;
      }
    }
    if (j > s) return v;
    m = ((m >> (j - 1)) | 1ull) << (j - 1);
    leaf = cur + L.n[j];
  }
}

// inner == 1, n[s] <= 256: tpr consecutive threads share a row, thread t owns subtree
// c0 = t, and the remaining stages s+1..S run in shared memory.
template <int OP>
__global__ void __launch_bounds__(kThreads)
reduce_rowcoop_kernel(float* __restrict__ O, const float* __restrict__ I, RedGeom g, Levels L,
                      int s, int tpr, int acc, float mean_div) {
  __shared__ float vals[kThreads];
  const int rows_per_block = kThreads / tpr;
  const int t = threadIdx.x % tpr;
  const int lr = threadIdx.x / tpr;
  const int64_t row = (int64_t)blockIdx.x * rows_per_block + lr;
  const int64_t parts = L.n[s];
  const bool active = row < g.rows && t < parts;
  float v = 0.0f;
  if (active) v = subtree<OP>(I + row_base(g, row), t, s, L, g);
  vals[threadIdx.x] = v;
  __syncthreads();
  for (int j = s + 1; j <= L.S; ++j) {
    const int64_t nj = L.n[j];
    float nv = v;
    const bool doit = active && t < nj && (t + nj) < L.n[j - 1];
    if (doit) nv = comb<OP>(vals[threadIdx.x], vals[threadIdx.x + nj]);
    __syncthreads();
    if (doit) vals[threadIdx.x] = nv;
    __syncthreads();
  }
  if (active && t == 0) {
    float r = vals[threadIdx.x];
    if (mean_div != 0.0f) r = __fdiv_rn(r, mean_div);
    O[row] = acc ? __fadd_rn(O[row], r) : r;
  }
}

// One thread per (row, c0) pair evaluating V_s(c0); parts = n[s].  c0_fastest selects which
// index varies between neighbouring threads (columns when the reduced axis is the
// contiguous one, rows when an inner kept axis is).  parts == 1 finishes rows and writes
// O; otherwise partials go to P laid out [outer][parts][mid*inner].
template <int OP>
__global__ void __launch_bounds__(kThreads)
reduce_parts_kernel(float* __restrict__ O, float* __restrict__ P, const float* __restrict__ I,
                    RedGeom g, Levels L, int s, int c0_fastest, int acc, float mean_div) {
  const int64_t parts = L.n[s];
  const int64_t total = g.rows * parts;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  const int64_t mi = g.mid * g.inner;
  for (int64_t gid = tid; gid < total; gid += nthreads) {
    int64_t c0, row;
    if (c0_fastest) { row = gid / parts; c0 = gid - row * parts; }
    else { c0 = gid / g.rows; row = gid - c0 * g.rows; }
    float v = subtree<OP>(I + row_base(g, row), c0, s, L, g);
    if (parts == 1) {
      if (mean_div != 0.0f) v = __fdiv_rn(v, mean_div);
      O[row] = acc ? __fadd_rn(O[row], v) : v;
    } else {
      const int64_t outer_i = row / mi;
      const int64_t rem = row - outer_i * mi;
      P[(outer_i * parts + c0) * mi + rem] = v;
    }
  }
}

// dI += dO[row] (/ COLS)   (reduce.py:250-260)
__global__ void __launch_bounds__(kThreads)
reduce_bwd_bcast_kernel(float* __restrict__ dI, const float* __restrict__ dO, int64_t total,
                        RedGeom g, float mean_div) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t gid = tid; gid < total; gid += nthreads) {
    int64_t x = gid;
    const int64_t inner_i = x % g.inner; x /= g.inner;
    x /= g.r1;
    const int64_t mid_i = x % g.mid; x /= g.mid;
    x /= g.r0;
    const int64_t outer_i = x;
    float v = dO[(outer_i * g.mid + mid_i) * g.inner + inner_i];
    if (mean_div != 0.0f) v = __fdiv_rn(v, mean_div);
    dI[gid] = __fadd_rn(dI[gid], v);
  }
}

// max/min: the gradient goes to the lowest column whose value equals the reduced value
// (reduce.py:262-276 gives it to whichever work-item wins an atomic; on tie-free data
// both agree).  One thread per row.
__global__ void __launch_bounds__(kThreads)
reduce_bwd_select_kernel(float* __restrict__ dI, const float* __restrict__ I,
                         const float* __restrict__ dO, const float* __restrict__ O, RedGeom g) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  const int64_t cols = g.r0 * g.r1;
  for (int64_t row = tid; row < g.rows; row += nthreads) {
    const int64_t base = row_base(g, row);
    const float o = O[row];
    for (int64_t c = 0; c < cols; ++c) {
      const int64_t q = c / g.r1;
      const int64_t off = base + q * g.stride_r0 + (c - q * g.r1) * g.stride_r1;
      if (I[off] == o) {
        dI[off] = __fadd_rn(dI[off], dO[row]);
        break;
      }
    }
  }
}

int make_geom(RedGeom& g, int64_t outer, int64_t r0, int64_t mid, int64_t r1, int64_t inner) {
  LNN_REQUIRE(outer >= 1 && r0 >= 1 && mid >= 1 && r1 >= 1 && inner >= 1, "bad reduce extents");
  g.outer = outer; g.r0 = r0; g.mid = mid; g.r1 = r1; g.inner = inner;
  g.rows = outer * mid * inner;
  g.stride_r1 = inner;
  g.stride_mid = r1 * inner;
  g.stride_r0 = mid * r1 * inner;
  g.stride_outer = r0 * mid * r1 * inner;
  return LNN_OK;
}

void make_levels(Levels& L, int64_t cols) {
  L.n[0] = cols;
  int s = 0;
  while (L.n[s] > 1) {
    L.n[s + 1] = (L.n[s] + 1) / 2;
    ++s;
  }
  L.S = s;
  for (int j = s + 1; j <= kMaxLevels; ++j) L.n[j] = 1;
}

inline int grid_for(const lnn::Device* d, int64_t work_items) {
  int64_t blocks = lnn_ceil_div(work_items, kThreads);
  int64_t cap = (int64_t)d->sm_count * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

// Plans one reduction as 1..3 launches.  mean_div is the ORIGINAL column count (as float)
// for mean, 0 otherwise; it is applied only where a row is finished.
template <int OP>
int reduce_impl(lnn::Device* d, float* O, const float* I, int64_t outer, int64_t r0, int64_t mid,
                int64_t r1, int64_t inner, int acc, float mean_div) {
  RedGeom g;
  int rc = make_geom(g, outer, r0, mid, r1, inner);
  if (rc) return rc;
  Levels L;
  make_levels(L, r0 * r1);
  const int64_t cols = r0 * r1;
  const int64_t kTargetThreads = 1 << 19;
  if (inner == 1) {
    int s_block = 0;                       // smallest s with n[s] <= 256
    while (L.n[s_block] > kThreads) ++s_block;
    const bool split = (g.rows * kThreads < kTargetThreads / 2) && cols > 65536;
    if (!split) {
      int tpr = 1;
      while (tpr < L.n[s_block]) tpr <<= 1;
      const int rows_per_block = kThreads / tpr;
      const int64_t blocks = lnn_ceil_div(g.rows, rows_per_block);
      LNN_REQUIRE(blocks < (1ll << 31), "too many rows");
      reduce_rowcoop_kernel<OP><<<(unsigned)blocks, kThreads, 0, d->stream>>>(
          O, I, g, L, s_block, tpr, acc, mean_div);
      LNN_CHECK_LAUNCH(d);
      return LNN_OK;
    }
    int s = 6;                             // at least 64 leaves per thread
    while (s < L.S && g.rows * L.n[s] > kTargetThreads) ++s;
    const int64_t parts = L.n[s];
    lnn::Scratch scratch(d);
    rc = scratch.get((uint64_t)(g.rows * parts) * sizeof(float));
    if (rc) return rc;
    reduce_parts_kernel<OP><<<grid_for(d, g.rows * parts), kThreads, 0, d->stream>>>(
        nullptr, scratch.as<float>(), I, g, L, s, 1, 0, 0.0f);
    LNN_CHECK_LAUNCH(d);
    return reduce_impl<OP>(d, O, scratch.as<float>(), outer, parts, mid, 1, 1, acc, mean_div);
  }
  // inner > 1: coalesce along the inner axis, one thread per output when there are enough
  int s = L.S;
  if (g.rows < 65536 && cols > 256) {
    s = 4;
    while (s < L.S && g.rows * L.n[s] > kTargetThreads) ++s;
  }
  const int64_t parts = L.n[s];
  if (parts == 1) {
    reduce_parts_kernel<OP><<<grid_for(d, g.rows), kThreads, 0, d->stream>>>(
        O, nullptr, I, g, L, L.S, 0, acc, mean_div);
    LNN_CHECK_LAUNCH(d);
    return LNN_OK;
  }
  lnn::Scratch scratch(d);
  rc = scratch.get((uint64_t)(g.rows * parts) * sizeof(float));
  if (rc) return rc;
  reduce_parts_kernel<OP><<<grid_for(d, g.rows * parts), kThreads, 0, d->stream>>>(
      nullptr, scratch.as<float>(), I, g, L, s, 0, 0, 0.0f);
  LNN_CHECK_LAUNCH(d);
  return reduce_impl<OP>(d, O, scratch.as<float>(), outer, parts, 1, 1, mid * inner, acc, mean_div);
}


// ---- reduction without any allocation ---------------------------------------------------------
// Partial results of split rows live in this fixed device array instead of pooled memory.
// Every device that loads the library holds its own 1 MiB copy until the process exits.
constexpr int64_t kStaticScratchFloats = 1 << 18;
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

// Device address of g_static_scratch per device slot, resolved once per device.  In host
// code the symbol itself is only a stand-in; kernels must be given this address.
float* g_static_scratch_ptr[LNN_MAX_DEVICES] = {nullptr};

int static_scratch_for(lnn::Device* d, int dev, float** out) {
  if (!g_static_scratch_ptr[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);   // d's device is current
    if (e != cudaSuccess || !p)
      return lnn::set_error(LNN_E_CUDA, "cudaGetSymbolAddress(static scratch) failed on device %d: %s",
                            d->ordinal, cudaGetErrorString(e));
    g_static_scratch_ptr[dev] = (float*)p;
  }
  *out = g_static_scratch_ptr[dev];
  return LNN_OK;
}

// Same plan as reduce_impl, with the partial buffers carved from [scratch, scratch + cap).
template <int OP>
int reduce_impl_static(lnn::Device* d, float* O, const float* I, int64_t outer, int64_t r0, int64_t mid,
                       int64_t r1, int64_t inner, int acc, float mean_div, float* scratch, int64_t cap) {
  RedGeom g;
  int rc = make_geom(g, outer, r0, mid, r1, inner);
  if (rc) return rc;
  Levels L;
  make_levels(L, r0 * r1);
  const int64_t cols = r0 * r1;
  const int64_t kTargetThreads = 1 << 19;
  if (inner == 1) {
    int s_block = 0;
    while (L.n[s_block] > kThreads) ++s_block;
    const bool split = (g.rows * kThreads < kTargetThreads / 2) && cols > 65536;
    if (!split) {
      int tpr = 1;
      while (tpr < L.n[s_block]) tpr <<= 1;
      const int rows_per_block = kThreads / tpr;
      const int64_t blocks = lnn_ceil_div(g.rows, rows_per_block);
      LNN_REQUIRE(blocks < (1ll << 31), "too many rows");
      reduce_rowcoop_kernel<OP><<<(unsigned)blocks, kThreads, 0, d->stream>>>(O, I, g, L, s_block, tpr, acc, mean_div);
      LNN_CHECK_LAUNCH(d);
      return LNN_OK;
    }
    int s = 6;
    while (s < L.S && g.rows * L.n[s] > kTargetThreads) ++s;
    const int64_t parts = L.n[s];
    const int64_t need = (g.rows * parts + 63) & ~63ll;
    if (need > cap)
      return lnn::set_error(LNN_E_UNSUPPORTED,
                            "reduction needs %lld floats of scratch but the static scratch holds %lld "
                            "(1 MiB in total): use lnn_reduce", (long long)need, (long long)cap);
    reduce_parts_kernel<OP><<<grid_for(d, g.rows * parts), kThreads, 0, d->stream>>>(
        nullptr, scratch, I, g, L, s, 1, 0, 0.0f);
    LNN_CHECK_LAUNCH(d);
    return reduce_impl_static<OP>(d, O, scratch, outer, parts, mid, 1, 1, acc, mean_div, scratch + need, cap - need);
  }
  int s = L.S;
  if (g.rows < 65536 && cols > 256) {
    s = 4;
    while (s < L.S && g.rows * L.n[s] > kTargetThreads) ++s;
  }
  const int64_t parts = L.n[s];
  if (parts == 1) {
    reduce_parts_kernel<OP><<<grid_for(d, g.rows), kThreads, 0, d->stream>>>(O, nullptr, I, g, L, L.S, 0, acc, mean_div);
    LNN_CHECK_LAUNCH(d);
    return LNN_OK;
  }
  const int64_t need = (g.rows * parts + 63) & ~63ll;
  if (need > cap)
    return lnn::set_error(LNN_E_UNSUPPORTED,
                          "reduction needs %lld floats of scratch but the static scratch holds %lld "
                          "(1 MiB in total): use lnn_reduce", (long long)need, (long long)cap);
  reduce_parts_kernel<OP><<<grid_for(d, g.rows * parts), kThreads, 0, d->stream>>>(
      nullptr, scratch, I, g, L, s, 0, 0, 0.0f);
  LNN_CHECK_LAUNCH(d);
  return reduce_impl_static<OP>(d, O, scratch, outer, parts, 1, 1, mid * inner, acc, mean_div, scratch + need, cap - need);
}

}  // namespace

extern "C" {

int lnn_reduce(int dev, int op, uint64_t O, uint64_t I, int64_t outer, int64_t r0, int64_t mid,
               int64_t r1, int64_t inner, int accumulate) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(O && I, "null buffer");
  LNN_REQUIRE(outer >= 1 && r0 >= 1 && mid >= 1 && r1 >= 1 && inner >= 1, "bad reduce extents");
  float* o = (float*)(uintptr_t)O;
  const float* i = (const float*)(uintptr_t)I;
  const float cols_f = (float)(r0 * r1);
  switch (op) {
    case LNN_RED_SUM: return reduce_impl<LNN_RED_SUM>(d, o, i, outer, r0, mid, r1, inner, accumulate, 0.0f);
    case LNN_RED_MEAN: return reduce_impl<LNN_RED_SUM>(d, o, i, outer, r0, mid, r1, inner, accumulate, cols_f);
    case LNN_RED_MAX: return reduce_impl<LNN_RED_MAX>(d, o, i, outer, r0, mid, r1, inner, accumulate, 0.0f);
    case LNN_RED_MIN: return reduce_impl<LNN_RED_MIN>(d, o, i, outer, r0, mid, r1, inner, accumulate, 0.0f);
  }
  return lnn::set_error(LNN_E_INVALID, "unknown reduce op %d", op);
}

int lnn_reduce_bwd(int dev, int op, uint64_t dI, uint64_t I, uint64_t dO, uint64_t O, int64_t outer,
                   int64_t r0, int64_t mid, int64_t r1, int64_t inner) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(dI && dO, "null buffer");
  RedGeom g;
  int rc = make_geom(g, outer, r0, mid, r1, inner);
  if (rc) return rc;
  const int64_t total = g.rows * r0 * r1;
  if (op == LNN_RED_SUM || op == LNN_RED_MEAN) {
    reduce_bwd_bcast_kernel<<<grid_for(d, total), kThreads, 0, d->stream>>>(
        (float*)(uintptr_t)dI, (const float*)(uintptr_t)dO, total, g,
        op == LNN_RED_MEAN ? (float)(r0 * r1) : 0.0f);
  } else if (op == LNN_RED_MAX || op == LNN_RED_MIN) {
    LNN_REQUIRE(I && O, "max/min backward needs I and O");
    reduce_bwd_select_kernel<<<grid_for(d, g.rows), kThreads, 0, d->stream>>>(
        (float*)(uintptr_t)dI, (const float*)(uintptr_t)I, (const float*)(uintptr_t)dO,
        (const float*)(uintptr_t)O, g);
  } else {
    return lnn::set_error(LNN_E_INVALID, "unknown reduce op %d", op);
  }
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

// Reduction for callers that must not allocate device memory: a host thread inside a
// latency-critical serving loop, a library embedded in an application that has handed the
// whole GPU heap to its own allocator, or code running after memory has been exhausted --
// cudaMalloc there either stalls the device or fails.  Same arguments and bit-identical
// results as lnn_reduce; the partial sums of rows that are split across thread blocks are
// kept in a fixed 1 MiB device array that belongs to the library (one copy per device,
// held until the process exits) instead of pooled memory.
//  * Reductions whose partials do not fit (more than 2^18 floats) are refused with
//    LNN_E_UNSUPPORTED; nothing is launched in that case.
//  * The first call on a device resolves the array's device address (one
//    cudaGetSymbolAddress, no allocation); make that first call before any stream capture.
//  * All calls share the one array and it keeps whatever the previous call left; every
//    partial a launch reads has been written by the launch before it, so nothing needs
//    clearing.  Calls follow each other on the device's single stream; two calls made to
//    overlap on the GPU (by driving the same device from two threads) would race on it.
int lnn_reduce_noalloc(int dev, int op, uint64_t O, uint64_t I, int64_t outer, int64_t r0, int64_t mid,
                       int64_t r1, int64_t inner, int accumulate) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(O && I, "null buffer");
  LNN_REQUIRE(outer >= 1 && r0 >= 1 && mid >= 1 && r1 >= 1 && inner >= 1, "bad reduce extents");
  float* scratch = nullptr;
  int rc = static_scratch_for(d, dev, &scratch);
  if (rc) return rc;
  float* o = (float*)(uintptr_t)O;
  const float* i = (const float*)(uintptr_t)I;
  const float cols_f = (float)(r0 * r1);
  const int64_t cap = kStaticScratchFloats;
  switch (op) {
    case LNN_RED_SUM: return reduce_impl_static<LNN_RED_SUM>(d, o, i, outer, r0, mid, r1, inner, accumulate, 0.0f, scratch, cap);
    case LNN_RED_MEAN: return reduce_impl_static<LNN_RED_SUM>(d, o, i, outer, r0, mid, r1, inner, accumulate, cols_f, scratch, cap);
    case LNN_RED_MAX: return reduce_impl_static<LNN_RED_MAX>(d, o, i, outer, r0, mid, r1, inner, accumulate, 0.0f, scratch, cap);
    case LNN_RED_MIN: return reduce_impl_static<LNN_RED_MIN>(d, o, i, outer, r0, mid, r1, inner, accumulate, 0.0f, scratch, cap);
  }
  return lnn::set_error(LNN_E_INVALID, "unknown reduce op %d", op);
}

}  // extern "C"
