// Reductions (sum, mean, max, min) with the reference's summation tree, one read of the
// input instead of the reference's transpose + log2(COLS) in-place stages + slice
// (litenn/core/op/reduce.py:166-205, stage kernel :279-293).
//
// The reference reduces a row of n values in stages: h = ceil(n/2); x[c] = x[c] (+) x[c+h]
// for every c with c+h < n; n = h; until n == 1.  With n_0 = COLS and n_j = ceil(n_{j-1}/2)
// the value at stage s, column c is V_s(c) = V_{s-1}(c) (+) V_{s-1}(c + n_s) when that
// partner exists, else V_{s-1}(c).  Here one thread evaluates a whole subtree V_s(c0), so
// the operand pairing, and therefore every rounding, is the reference's:
//   * any COLS: a depth-first walk with a stack of one partial value per level;
//   * power-of-two COLS (every benchmark shape): the 2^s leaves c0 + m*n_s form a plain
//     halving tree over m, evaluated with 16 independent loads in flight per thread.
// A row is finished inside a warp (shuffles), inside a block (shared memory), or, when a
// row is split over many threads to fill the GPU, by running the same routine again on the
// partial values -- the tree over n_s partials is the tail of the tree over n_0 values.
#include "lnn_common.cuh"
#include <math_constants.h>
#include <utility>
#include <algorithm>

namespace {

constexpr int kThreads = 256;
constexpr int kMaxLevels = 40;
constexpr int kMaxPow2Levels = 9;      // fast subtree: up to 2^9 leaves per thread

struct Levels {
  int S;                       // number of stages: n[S] == 1
  int pow2;                    // COLS is a power of two
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

__device__ __forceinline__ int64_t leaf_offset(const RedGeom& g, int64_t leaf) {
  if (g.r0 == 1) return leaf * g.stride_r1;
  const int64_t q = leaf / g.r1;
  return q * g.stride_r0 + (leaf - q * g.r1) * g.stride_r1;
}

// V_s(c0) of one row for any COLS (base points at the row's column 0).
template <int OP>
__device__ float subtree_dfs(const float* __restrict__ base, int64_t c0, int s, const Levels& L,
                             const RedGeom& g) {
  float acc[kMaxLevels];
  int64_t leaf = c0;
  uint64_t m = 0;
  for (;;) {
    float v = __ldcs(base + leaf_offset(g, leaf));
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

__host__ __device__ constexpr int bit_reverse(int t, int bits) {
  int r = 0;
  for (int i = 0; i < bits; ++i) r |= ((t >> i) & 1) << (bits - 1 - i);
  return r;
}

// Power-of-two COLS: leaf m of V_s(c0) is column c0 + m*ns (ns = COLS >> s) and the tree is
// the halving tree over m.  m = a*B + b: the A = 2^LOG_A leaves of one b are loaded together
// and halved in registers (the high bits of m go first); b then runs in bit-reversed order so
// that a binary-counter stack, fully unrolled into registers, pairs b with b + B/2 first.
template <int OP, int LOG_A, int LOG_B>
__device__ __forceinline__ float subtree_pow2(const float* __restrict__ base, int64_t c0, int64_t ns,
                                              const RedGeom& g) {
  constexpr int A = 1 << LOG_A, B = 1 << LOG_B;
  float stack[LOG_B + 1];
  float result = 0.0f;
#pragma unroll
  for (int t = 0; t < B; ++t) {
    const int b = bit_reverse(t, LOG_B);
    float v[A];
#pragma unroll
    for (int a = 0; a < A; ++a) v[a] = __ldcs(base + leaf_offset(g, c0 + (int64_t)(a * B + b) * ns));
#pragma unroll
    for (int h = A / 2; h >= 1; h >>= 1) {
#pragma unroll
      for (int i = 0; i < h; ++i) v[i] = comb<OP>(v[i], v[i + h]);
    }
    float w = v[0];
    bool stored = false;
#pragma unroll
    for (int level = 0; level < LOG_B; ++level) {
      if (!stored) {
        if ((t >> level) & 1) w = comb<OP>(stack[level], w);
        else { stack[level] = w; stored = true; }
      }
    }
    if (t == B - 1) result = w;
  }
  return result;
}

template <int OP>
__device__ __forceinline__ float4 comb4(const float4& a, const float4& b) {
  return make_float4(comb<OP>(a.x, b.x), comb<OP>(a.y, b.y), comb<OP>(a.z, b.z), comb<OP>(a.w, b.w));
}

// Four independent subtrees at once from 128-bit loads: the four lanes of a float4 are four
// adjacent kept rows (inner axis) or four adjacent columns c0..c0+3, whichever is contiguous
// in memory.  Same tree per lane as subtree_pow2.
template <int OP, int LOG_A, int LOG_B>
__device__ __forceinline__ float4 subtree_pow2_v4(const float* __restrict__ base, int64_t c0, int64_t ns,
                                                  const RedGeom& g) {
  constexpr int A = 1 << LOG_A, B = 1 << LOG_B;
  float4 stack[LOG_B + 1];
  float4 result = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int t = 0; t < B; ++t) {
    const int b = bit_reverse(t, LOG_B);
    float4 v[A];
#pragma unroll
    for (int a = 0; a < A; ++a)
      v[a] = __ldcs(reinterpret_cast<const float4*>(base + leaf_offset(g, c0 + (int64_t)(a * B + b) * ns)));
#pragma unroll
    for (int h = A / 2; h >= 1; h >>= 1) {
#pragma unroll
      for (int i = 0; i < h; ++i) v[i] = comb4<OP>(v[i], v[i + h]);
    }
    float4 w = v[0];
    bool stored = false;
#pragma unroll
    for (int level = 0; level < LOG_B; ++level) {
      if (!stored) {
        if ((t >> level) & 1) w = comb4<OP>(stack[level], w);
        else { stack[level] = w; stored = true; }
      }
    }
    if (t == B - 1) result = w;
  }
  return result;
}

// s <= 8 keeps the unrolled body within the register budget (A = 8 float4 loads in flight)
template <int OP>
__device__ __forceinline__ float4 subtree_v4(const float* __restrict__ base, int64_t c0, int s,
                                             const Levels& L, const RedGeom& g) {
  const int64_t ns = L.n[s];
  switch (s) {
    case 0: return subtree_pow2_v4<OP, 0, 0>(base, c0, ns, g);
    case 1: return subtree_pow2_v4<OP, 1, 0>(base, c0, ns, g);
    case 2: return subtree_pow2_v4<OP, 2, 0>(base, c0, ns, g);
    case 3: return subtree_pow2_v4<OP, 3, 0>(base, c0, ns, g);
    case 4: return subtree_pow2_v4<OP, 3, 1>(base, c0, ns, g);
    case 5: return subtree_pow2_v4<OP, 3, 2>(base, c0, ns, g);
    case 6: return subtree_pow2_v4<OP, 3, 3>(base, c0, ns, g);
    case 7: return subtree_pow2_v4<OP, 3, 4>(base, c0, ns, g);
    case 8: return subtree_pow2_v4<OP, 3, 5>(base, c0, ns, g);
    default: return subtree_pow2_v4<OP, 3, 6>(base, c0, ns, g);
  }
}

template <int OP>
__device__ __forceinline__ float subtree(const float* __restrict__ base, int64_t c0, int s,
                                         const Levels& L, const RedGeom& g) {
  if (L.pow2 && s <= kMaxPow2Levels) {
    const int64_t ns = L.n[s];
    switch (s) {
      case 0: return subtree_pow2<OP, 0, 0>(base, c0, ns, g);
      case 1: return subtree_pow2<OP, 1, 0>(base, c0, ns, g);
      case 2: return subtree_pow2<OP, 2, 0>(base, c0, ns, g);
      case 3: return subtree_pow2<OP, 3, 0>(base, c0, ns, g);
      case 4: return subtree_pow2<OP, 4, 0>(base, c0, ns, g);
      case 5: return subtree_pow2<OP, 4, 1>(base, c0, ns, g);
      case 6: return subtree_pow2<OP, 4, 2>(base, c0, ns, g);
      case 7: return subtree_pow2<OP, 4, 3>(base, c0, ns, g);
      case 8: return subtree_pow2<OP, 4, 4>(base, c0, ns, g);
      default: return subtree_pow2<OP, 4, 5>(base, c0, ns, g);
    }
  }
  return subtree_dfs<OP>(base, c0, s, L, g);
}

// inner == 1, power-of-two COLS, n[s] <= 32: one warp per row.  Lane t owns subtree c0 = t
// (coalesced: neighbouring lanes read neighbouring columns) and the last stages are
// shuffles: lane t takes lane t+h for h = n[s]/2 ... 1.
template <int OP>
__global__ void __launch_bounds__(kThreads)
reduce_warp_kernel(float* __restrict__ O, const float* __restrict__ I, RedGeom g, Levels L, int s,
                   int acc, float mean_div) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int parts = (int)L.n[s];
  for (int64_t row = warp0; row < g.rows; row += nwarps) {
    float v = 0.0f;
    if (lane < parts) v = subtree<OP>(I + row_base(g, row), lane, s, L, g);
    for (int h = parts >> 1; h >= 1; h >>= 1) {
      const float other = __shfl_down_sync(0xffffffffu, v, h);
      if (lane < h) v = comb<OP>(v, other);
    }
    if (lane == 0) {
      if (mean_div != 0.0f) v = __fdiv_rn(v, mean_div);
      O[row] = acc ? __fadd_rn(O[row], v) : v;
    }
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
    } else if (c0_fastest) {
      P[row * parts + c0] = v;                    // inner == 1: partials of a row are contiguous
    } else {
      const int64_t outer_i = row / mi;
      const int64_t rem = row - outer_i * mi;
      P[(outer_i * parts + c0) * mi + rem] = v;
    }
  }
}

// inner == 1, power-of-two COLS >= 128, contiguous columns: one warp per row with 128-bit
// loads.  Lane t owns the four subtrees c0 = 4t..4t+3 of the n[s] = 128 partials; the last
// stages pair c with c+64 ... c+4 by shuffles (lane t with t+16 ... t+1), then c with c+2
// and c with c+1 inside the lane.
template <int OP>
__global__ void __launch_bounds__(kThreads)
reduce_warp4_kernel(float* __restrict__ O, const float* __restrict__ I, RedGeom g, Levels L, int s,
                    int acc, float mean_div) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t row = warp0; row < g.rows; row += nwarps) {
    float4 v = subtree_v4<OP>(I + row_base(g, row), 4 * lane, s, L, g);
#pragma unroll
    for (int h = 16; h >= 1; h >>= 1) {
      float4 o;
      o.x = __shfl_down_sync(0xffffffffu, v.x, h); o.y = __shfl_down_sync(0xffffffffu, v.y, h);
      o.z = __shfl_down_sync(0xffffffffu, v.z, h); o.w = __shfl_down_sync(0xffffffffu, v.w, h);
      if (lane < h) v = comb4<OP>(v, o);
    }
    if (lane == 0) {
      float r = comb<OP>(comb<OP>(v.x, v.z), comb<OP>(v.y, v.w));
      if (mean_div != 0.0f) r = __fdiv_rn(r, mean_div);
      O[row] = acc ? __fadd_rn(O[row], r) : r;
    }
  }
}

// The same for short rows (128 ... 1024 columns, S = s known at compile time): a warp works on four
// rows at a time so that the loads of all four are in flight before the first shuffle (one row
// per iteration left the kernel latency-bound at 2.7 TB/s on rows of 256 columns).
template <int OP, int S>
__global__ void __launch_bounds__(kThreads)
reduce_warp4_short_kernel(float* __restrict__ O, const float* __restrict__ I, RedGeom g, Levels L, int acc,
                          float mean_div) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int64_t ns = L.n[S];
  for (int64_t row0 = warp0 * 4; row0 < g.rows; row0 += nwarps * 4) {
    float4 v[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int64_t row = row0 + q < g.rows ? row0 + q : g.rows - 1;      // the tail repeats the last row
      v[q] = subtree_pow2_v4<OP, S, 0>(I + row_base(g, row), 4 * lane, ns, g);
    }
#pragma unroll
    for (int h = 16; h >= 1; h >>= 1) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float4 o;
        o.x = __shfl_down_sync(0xffffffffu, v[q].x, h); o.y = __shfl_down_sync(0xffffffffu, v[q].y, h);
        o.z = __shfl_down_sync(0xffffffffu, v[q].z, h); o.w = __shfl_down_sync(0xffffffffu, v[q].w, h);
        if (lane < h) v[q] = comb4<OP>(v[q], o);
      }
    }
    if (lane == 0) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (row0 + q < g.rows) {
          float r = comb<OP>(comb<OP>(v[q].x, v[q].z), comb<OP>(v[q].y, v[q].w));
          if (mean_div != 0.0f) r = __fdiv_rn(r, mean_div);
          O[row0 + q] = acc ? __fadd_rn(O[row0 + q], r) : r;
        }
      }
    }
  }
}

// Number of blocks of a single-row reduction that have stored their partials; the block that
// finds itself last finishes the row and resets the counter for the next launch.
static __device__ unsigned int g_blocks_done;

// The halving tree over x[i] = P[first + stride * i], i < m (m a power of two): stage after stage
// element i is combined with element i + m/2.  Leaves are visited in bit-reversed order so that
// a binary-counter stack meets them in exactly that pairing; eight loads are in flight at a time.
// P was written by other blocks of the same launch: the loads go to L2.
template <int OP>
__device__ float strided_halving_tree(const float* P, int64_t first, int64_t stride, int m) {
  float stack[24];
  const int bits = 31 - __clz(m);
  float w = 0.0f;
  for (int k0 = 0; k0 < m; k0 += 8) {
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int k = k0 + u;
      const int i = bits ? (int)(__brev((unsigned)k) >> (32 - bits)) : 0;
      v[u] = k < m ? __ldcg(P + first + stride * i) : 0.0f;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int k = k0 + u;
      if (k < m) {
        w = v[u];
        int level = 0;
        for (int kk = k; kk & 1; kk >>= 1, ++level) w = comb<OP>(stack[level], w);
        stack[level] = w;
      }
    }
  }
  return w;
}

// 128-bit variant of reduce_parts_kernel.  rows_vec != 0: a thread owns four adjacent kept
// rows (inner % 4 == 0) of one c0; else four adjacent columns c0..c0+3 of one row (inner == 1,
// mid == 1).  Either way its four results are adjacent in O / P.
template <int OP>
// 4 blocks per SM (64 registers): the few spills of the counter stack cost less than the lost
// occupancy (measured: 0.67 -> 0.76 of the copy bandwidth on the axis-1 case; 6 blocks: 0.59)
__global__ void __launch_bounds__(kThreads, 4)
reduce_parts4_kernel(float* __restrict__ O, float* __restrict__ P, const float* __restrict__ I,
                     RedGeom g, Levels L, int s, int rows_vec, int acc, float mean_div, int finish_row = 0) {
  __shared__ float tail_vals[kThreads];
  __shared__ int is_last;
  const int64_t parts = L.n[s];
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  if (rows_vec) {
    const int64_t rows4 = g.rows >> 2;
    const int64_t total = rows4 * parts;
    const int64_t mi = g.mid * g.inner;
    for (int64_t gid = tid; gid < total; gid += nthreads) {
      const int64_t c0 = gid / rows4;
      const int64_t row = (gid - c0 * rows4) << 2;
      float4 v = subtree_v4<OP>(I + row_base(g, row), c0, s, L, g);
      if (parts == 1) {
        if (mean_div != 0.0f) {
          v.x = __fdiv_rn(v.x, mean_div); v.y = __fdiv_rn(v.y, mean_div);
          v.z = __fdiv_rn(v.z, mean_div); v.w = __fdiv_rn(v.w, mean_div);
        }
        float4* dst = reinterpret_cast<float4*>(O + row);
        if (acc) { const float4 o = *dst; v.x = __fadd_rn(o.x, v.x); v.y = __fadd_rn(o.y, v.y); v.z = __fadd_rn(o.z, v.z); v.w = __fadd_rn(o.w, v.w); }
        *dst = v;
      } else {
        const int64_t outer_i = row / mi;
        const int64_t rem = row - outer_i * mi;
        *reinterpret_cast<float4*>(P + (outer_i * parts + c0) * mi + rem) = v;
      }
    }
  } else {
    const int64_t parts4 = parts >> 2;
    const int64_t total = g.rows * parts4;
    for (int64_t gid = tid; gid < total; gid += nthreads) {
      const int64_t row = gid / parts4;
      const int64_t c0 = (gid - row * parts4) << 2;
      const float4 v = subtree_v4<OP>(I + row_base(g, row), c0, s, L, g);
      *reinterpret_cast<float4*>(P + row * parts + c0) = v;     // partials of a row are contiguous
    }
    if (finish_row) {
      // One kept row, power-of-two column count, few partials: the last block to arrive runs the
      // rest of the same tree over them instead of two more dependent launches.
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) {
        const unsigned int prev = atomicAdd(&g_blocks_done, 1u);
        is_last = prev == gridDim.x - 1;
      }
      __syncthreads();
      if (!is_last) return;
      __threadfence();
      const int width = parts < kThreads ? (int)parts : kThreads;      // a power of two
      if ((int)threadIdx.x < width)
        tail_vals[threadIdx.x] = strided_halving_tree<OP>(P, threadIdx.x, width, (int)(parts / width));
      __syncthreads();
      for (int h = width >> 1; h >= 1; h >>= 1) {
        float nv = 0.0f;
        if ((int)threadIdx.x < h) nv = comb<OP>(tail_vals[threadIdx.x], tail_vals[threadIdx.x + h]);
        __syncthreads();
        if ((int)threadIdx.x < h) tail_vals[threadIdx.x] = nv;
        __syncthreads();
      }
      if (threadIdx.x == 0) {
        float r = tail_vals[0];
        if (mean_div != 0.0f) r = __fdiv_rn(r, mean_div);
        O[0] = acc ? __fadd_rn(O[0], r) : r;
        g_blocks_done = 0u;
      }
    }
  }
}

// dI += dO[row] (/ COLS)   (reduce.py:250-260)
// The common case of the same gradient: the reduced axes are the trailing ones (inner == 1,
// r0 == 1), so I is [rows][cols] and four consecutive elements share a row (cols % 4 == 0).
__global__ void __launch_bounds__(kThreads)
reduce_bwd_bcast_rows4_kernel(float4* __restrict__ dI, const float* __restrict__ dO, int64_t total4,
                              int64_t cols4, float mean_div) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t gid = tid; gid < total4; gid += nthreads) {
    float v = __ldg(dO + gid / cols4);
    if (mean_div != 0.0f) v = __fdiv_rn(v, mean_div);
    float4 o = dI[gid];
    o.x = __fadd_rn(o.x, v); o.y = __fadd_rn(o.y, v); o.z = __fadd_rn(o.z, v); o.w = __fadd_rn(o.w, v);
    dI[gid] = o;
  }
}

// The same gradient when kept axes follow the reduced ones (inner > 1): four consecutive elements
// of dI share every index but the innermost, so dO is read as float4 too (inner % 4 == 0).
__global__ void __launch_bounds__(kThreads)
reduce_bwd_bcast_inner4_kernel(float4* __restrict__ dI, const float4* __restrict__ dO, int64_t total4,
                               RedGeom g, float mean_div) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  const int64_t inner4 = g.inner >> 2;
  for (int64_t gid = tid; gid < total4; gid += nthreads) {
    int64_t x = gid;
    const int64_t inner_i = x % inner4; x /= inner4;
    x /= g.r1;
    const int64_t mid_i = x % g.mid; x /= g.mid;
    x /= g.r0;
    float4 v = __ldg(dO + (x * g.mid + mid_i) * inner4 + inner_i);
    if (mean_div != 0.0f) {
      v.x = __fdiv_rn(v.x, mean_div); v.y = __fdiv_rn(v.y, mean_div);
      v.z = __fdiv_rn(v.z, mean_div); v.w = __fdiv_rn(v.w, mean_div);
    }
    float4 o = dI[gid];
    o.x = __fadd_rn(o.x, v.x); o.y = __fadd_rn(o.y, v.y); o.z = __fadd_rn(o.z, v.z); o.w = __fadd_rn(o.w, v.w);
    dI[gid] = o;
  }
}

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
      const int64_t off = base + leaf_offset(g, c);
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
  L.pow2 = (cols & (cols - 1)) == 0;
  for (int j = s + 1; j <= kMaxLevels; ++j) L.n[j] = 1;
}

inline int grid_for(const lnn::Device* d, int64_t work_items) {
  int64_t blocks = lnn_ceil_div(work_items, kThreads);
  int64_t cap = (int64_t)d->sm_count * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

// Where the partial values of split rows live: pooled memory (lnn_reduce) or a caller-given
// fixed region (lnn_reduce_noalloc).
struct PartialSpace {
  lnn::Device* d;
  float* fixed = nullptr;       // non-null: bump-allocate from [fixed, fixed + cap)
  int64_t cap = 0;
  std::vector<std::pair<void*, uint64_t>> pooled;
  explicit PartialSpace(lnn::Device* dev) : d(dev) {}
  ~PartialSpace() { for (auto& b : pooled) lnn::free_bytes(d, b.first, b.second); }
  int get(int64_t floats, float** out) {
    if (fixed) {
      const int64_t need = (floats + 63) & ~63ll;
      if (need > cap)
        return lnn::set_error(LNN_E_UNSUPPORTED,
                              "reduction needs %lld more floats of scratch but the static scratch has %lld "
                              "left (1 MiB in total): use lnn_reduce", (long long)need, (long long)cap);
      *out = fixed; fixed += need; cap -= need;
      return LNN_OK;
    }
    void* p = nullptr;
    int rc = lnn::alloc_bytes(d, (uint64_t)floats * 4, &p);
    if (rc) return rc;
    pooled.push_back({p, (uint64_t)floats * 4});
    *out = (float*)p;
    return LNN_OK;
  }
};

// Plans one reduction as 1..3 launches.  mean_div is the ORIGINAL column count (as float)
// for mean, 0 otherwise; it is applied only where a row is finished.
template <int OP>
int reduce_impl(lnn::Device* d, PartialSpace& space, float* O, const float* I, int64_t outer,
                int64_t r0, int64_t mid, int64_t r1, int64_t inner, int acc, float mean_div) {
  RedGeom g;
  int rc = make_geom(g, outer, r0, mid, r1, inner);
  if (rc) return rc;
  Levels L;
  make_levels(L, r0 * r1);
  const int64_t cols = r0 * r1;
  const int64_t kTargetThreads = 1 << 19;
  if (inner == 1) {
    const bool split = ((g.rows * kThreads < kTargetThreads / 2) && cols > 65536) ||
                       (g.rows == 1 && L.pow2 && cols >= 8192);
    // 128-bit paths need contiguous, 16-byte aligned columns
    const bool cols_vec = L.pow2 && ((((uintptr_t)I) & 15) == 0) &&
                          (r0 == 1 || (r1 % 4 == 0 && g.stride_r0 % 4 == 0)) && g.stride_mid % 4 == 0 &&
                          g.stride_outer % 4 == 0;
    // a handful of long rows (the last pass of an all-axes reduction): one warp per row would be a
    // single latency-bound chain, so those take the block-per-row kernel below
    const bool few_long_rows = g.rows <= 32 && cols >= 2048;
    if (!split) {
      if (!few_long_rows && cols_vec && cols >= 128 && L.S - 7 <= kMaxPow2Levels) {
        const int s = L.S - 7;                           // 128 partials per row, four per lane
        int64_t blocks = lnn_ceil_div(g.rows, kThreads / 32);
        const int64_t cap = (int64_t)d->sm_count * 16;
        if (blocks > cap) blocks = cap;
        if (s <= 3 && g.rows >= 4096) {
          blocks = std::min<int64_t>(lnn_ceil_div(g.rows, 4 * (kThreads / 32)), cap);
          switch (s) {
            case 0: reduce_warp4_short_kernel<OP, 0><<<(unsigned)blocks, kThreads, 0, d->stream>>>(O, I, g, L, acc, mean_div); break;
            case 1: reduce_warp4_short_kernel<OP, 1><<<(unsigned)blocks, kThreads, 0, d->stream>>>(O, I, g, L, acc, mean_div); break;
            case 2: reduce_warp4_short_kernel<OP, 2><<<(unsigned)blocks, kThreads, 0, d->stream>>>(O, I, g, L, acc, mean_div); break;
            default: reduce_warp4_short_kernel<OP, 3><<<(unsigned)blocks, kThreads, 0, d->stream>>>(O, I, g, L, acc, mean_div); break;
          }
        } else {
          reduce_warp4_kernel<OP><<<(unsigned)blocks, kThreads, 0, d->stream>>>(O, I, g, L, s, acc, mean_div);
        }
        LNN_CHECK_LAUNCH(d);
        return LNN_OK;
      }
      if (!few_long_rows && L.pow2 && L.S - 5 <= kMaxPow2Levels) {
        const int s = L.S > 5 ? L.S - 5 : 0;           // n[s] = min(cols, 32) partials per row
        int64_t blocks = lnn_ceil_div(g.rows, kThreads / 32);
        const int64_t cap = (int64_t)d->sm_count * 16;
        if (blocks > cap) blocks = cap;
        reduce_warp_kernel<OP><<<(unsigned)blocks, kThreads, 0, d->stream>>>(O, I, g, L, s, acc, mean_div);
        LNN_CHECK_LAUNCH(d);
        return LNN_OK;
      }
      int s_block = 0;                       // smallest s with n[s] <= 256
      while (L.n[s_block] > kThreads) ++s_block;
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
    // enough threads to fill the GPU (a 128-bit thread covers four partials), at least 64 leaves each
    int64_t target_vals = cols_vec ? 4 * kTargetThreads / 2 : kTargetThreads;
    if (space.fixed) target_vals = std::min<int64_t>(target_vals, std::max<int64_t>(space.cap / 2, 1024));
    int s = 6;
    while (s < L.S && g.rows * L.n[s] > target_vals) ++s;
    if (L.pow2 && s > kMaxPow2Levels) s = kMaxPow2Levels;   // stay on the unrolled subtree (more partials)
    // A single row of a few hundred thousand columns (the partials of an all-axes reduction): 16
    // leaves per thread and at most 2^14 partials, which the last block of the same launch finishes.
    const bool finish_here = g.rows == 1 && L.pow2 && cols_vec && cols <= (1ll << 18) && cols >= (1ll << 12);
    if (finish_here) s = 4;
    const int64_t parts = L.n[s];
    float* part = nullptr;
    rc = space.get(g.rows * parts, &part);
    if (rc) return rc;
    // the partials of one kept row are stored contiguously, [row][parts], whatever the position of
    // the kept axes: the second pass is then a plain row reduction over `parts` columns, the tail
    // of the same tree
    if (cols_vec && s <= kMaxPow2Levels && parts % 4 == 0 && ((((uintptr_t)part) & 15) == 0)) {
      if (finish_here) {
        reduce_parts4_kernel<OP><<<grid_for(d, parts / 4), kThreads, 0, d->stream>>>(
            O, part, I, g, L, s, 0, acc, mean_div, 1);
        LNN_CHECK_LAUNCH(d);
        return LNN_OK;
      }
      reduce_parts4_kernel<OP><<<grid_for(d, g.rows * parts / 4), kThreads, 0, d->stream>>>(
          nullptr, part, I, g, L, s, 0, 0, 0.0f);
    } else {
      reduce_parts_kernel<OP><<<grid_for(d, g.rows * parts), kThreads, 0, d->stream>>>(
          nullptr, part, I, g, L, s, 1, 0, 0.0f);
    }
    LNN_CHECK_LAUNCH(d);
    return reduce_impl<OP>(d, space, O, part, g.rows, 1, 1, parts, 1, acc, mean_div);
  }
  // inner > 1: coalesce along the inner axis, one thread per output when there are enough
  // four adjacent kept rows per thread when the inner axis allows 128-bit loads
  const bool vec_possible = L.pow2 && inner % 4 == 0 && ((((uintptr_t)I) & 15) == 0) && ((((uintptr_t)O) & 15) == 0);
  int s = L.S;
  // one thread per kept row (or per four) leaves most of the GPU idle when there are few rows:
  // split the columns as well, down to 16 leaves per thread
  if (g.rows / (vec_possible ? 4 : 1) < kTargetThreads / 4 && cols > 256) {
    int64_t target_vals = vec_possible ? 4 * kTargetThreads / 2 : kTargetThreads;
    if (space.fixed) target_vals = std::min<int64_t>(target_vals, std::max<int64_t>(space.cap / 2, 1024));
    s = 4;
    while (s < L.S && g.rows * L.n[s] > target_vals) ++s;
  }
  const int64_t parts = L.n[s];
  const bool rows_vec = vec_possible && s <= kMaxPow2Levels;
  if (parts == 1) {
    if (rows_vec)
      reduce_parts4_kernel<OP><<<grid_for(d, g.rows / 4), kThreads, 0, d->stream>>>(
          O, nullptr, I, g, L, L.S, 1, acc, mean_div);
    else
      reduce_parts_kernel<OP><<<grid_for(d, g.rows), kThreads, 0, d->stream>>>(
          O, nullptr, I, g, L, L.S, 0, acc, mean_div);
    LNN_CHECK_LAUNCH(d);
    return LNN_OK;
  }
  float* part = nullptr;
  rc = space.get(g.rows * parts, &part);
  if (rc) return rc;
  if (rows_vec && ((((uintptr_t)part) & 15) == 0))
    reduce_parts4_kernel<OP><<<grid_for(d, g.rows * parts / 4), kThreads, 0, d->stream>>>(
        nullptr, part, I, g, L, s, 1, 0, 0.0f);
  else
    reduce_parts_kernel<OP><<<grid_for(d, g.rows * parts), kThreads, 0, d->stream>>>(
        nullptr, part, I, g, L, s, 0, 0, 0.0f);
  LNN_CHECK_LAUNCH(d);
  return reduce_impl<OP>(d, space, O, part, outer, parts, 1, 1, mid * inner, acc, mean_div);
}

int reduce_dispatch(lnn::Device* d, PartialSpace& space, int op, uint64_t O, uint64_t I, int64_t outer,
                    int64_t r0, int64_t mid, int64_t r1, int64_t inner, int accumulate) {
  float* o = (float*)(uintptr_t)O;
  const float* i = (const float*)(uintptr_t)I;
  const float cols_f = (float)(r0 * r1);
  switch (op) {
    case LNN_RED_SUM: return reduce_impl<LNN_RED_SUM>(d, space, o, i, outer, r0, mid, r1, inner, accumulate, 0.0f);
    case LNN_RED_MEAN: return reduce_impl<LNN_RED_SUM>(d, space, o, i, outer, r0, mid, r1, inner, accumulate, cols_f);
    case LNN_RED_MAX: return reduce_impl<LNN_RED_MAX>(d, space, o, i, outer, r0, mid, r1, inner, accumulate, 0.0f);
    case LNN_RED_MIN: return reduce_impl<LNN_RED_MIN>(d, space, o, i, outer, r0, mid, r1, inner, accumulate, 0.0f);
  }
  return lnn::set_error(LNN_E_INVALID, "unknown reduce op %d", op);
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

}  // namespace

extern "C" {

int lnn_reduce(int dev, int op, uint64_t O, uint64_t I, int64_t outer, int64_t r0, int64_t mid,
               int64_t r1, int64_t inner, int accumulate) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(O && I, "null buffer");
  LNN_REQUIRE(outer >= 1 && r0 >= 1 && mid >= 1 && r1 >= 1 && inner >= 1, "bad reduce extents");
  PartialSpace space(d);
  return reduce_dispatch(d, space, op, O, I, outer, r0, mid, r1, inner, accumulate);
}

int lnn_reduce_bwd(int dev, int op, uint64_t dI, uint64_t I, uint64_t dO, uint64_t O, int64_t outer,
                   int64_t r0, int64_t mid, int64_t r1, int64_t inner) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(dI && dO, "null buffer");
  RedGeom g;
  int rc = make_geom(g, outer, r0, mid, r1, inner);
  if (rc) return rc;
  const int64_t total = g.rows * r0 * r1;
  if ((op == LNN_RED_SUM || op == LNN_RED_MEAN) && inner == 1 && r0 == 1 && r1 % 4 == 0 && (dI & 15) == 0) {
    const float mean_div_rows = op == LNN_RED_MEAN ? (float)(r0 * r1) : 0.0f;
    reduce_bwd_bcast_rows4_kernel<<<grid_for(d, total / 4), kThreads, 0, d->stream>>>(
        (float4*)(uintptr_t)dI, (const float*)(uintptr_t)dO, total / 4, r1 / 4, mean_div_rows);
    LNN_CHECK_LAUNCH(d);
    return LNN_OK;
  }
  if ((op == LNN_RED_SUM || op == LNN_RED_MEAN) && inner % 4 == 0 && ((dI | dO) & 15) == 0) {
    reduce_bwd_bcast_inner4_kernel<<<grid_for(d, total / 4), kThreads, 0, d->stream>>>(
        (float4*)(uintptr_t)dI, (const float4*)(uintptr_t)dO, total / 4, g,
        op == LNN_RED_MEAN ? (float)(r0 * r1) : 0.0f);
    LNN_CHECK_LAUNCH(d);
    return LNN_OK;
  }
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
//    LNN_E_UNSUPPORTED; nothing more is launched once that is found.
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
  PartialSpace space(d);
  space.fixed = scratch;
  space.cap = kStaticScratchFloats;
  return reduce_dispatch(d, space, op, O, I, outer, r0, mid, r1, inner, accumulate);
}

}  // extern "C"
