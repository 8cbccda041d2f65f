// Data movement: axis permutation and strided slicing, each with the "=" / "+=" output
// convention of the reference (litenn/core/op/transpose.py:94-103, op/slice.py:168-190).
// Threads enumerate the OUTPUT (coalesced stores) and gather from the input; when the
// permutation swaps the innermost axis a 32x32 shared-memory tile keeps both sides
// coalesced.
#include "lnn_common.cuh"

namespace {

constexpr int kThreads = 256;

struct MoveDims {
  int rank;
  int64_t o[LNN_MAX_DIMS];        // output extents
  int64_t istride[LNN_MAX_DIMS];  // input element stride of each OUTPUT axis
  int64_t ibase;                  // input element offset of output index 0
};

// out[gid] (+)= in[ibase + sum_k idx_k * istride_k]
__global__ void __launch_bounds__(kThreads)
gather_kernel(float* __restrict__ O, const float* __restrict__ I, int64_t total, MoveDims d, int acc) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t gid = tid; gid < total; gid += nthreads) {
    int64_t x = gid, off = d.ibase;
#pragma unroll
    for (int k = LNN_MAX_DIMS - 1; k >= 0; --k) {
      if (k < d.rank) {
        const int64_t q = x / d.o[k];
        off += (x - q * d.o[k]) * d.istride[k];
        x = q;
      }
    }
    const float v = I[off];
    O[gid] = acc ? __fadd_rn(O[gid], v) : v;
  }
}

// in[ibase + sum idx_k*istride_k] += src[gid]   (slice backward: scatter-add, indices unique)
__global__ void __launch_bounds__(kThreads)
scatter_add_kernel(float* __restrict__ D, const float* __restrict__ S, int64_t total, MoveDims d) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t gid = tid; gid < total; gid += nthreads) {
    int64_t x = gid, off = d.ibase;
#pragma unroll
    for (int k = LNN_MAX_DIMS - 1; k >= 0; --k) {
      if (k < d.rank) {
        const int64_t q = x / d.o[k];
        off += (x - q * d.o[k]) * d.istride[k];
        x = q;
      }
    }
    D[off] = __fadd_rn(D[off], S[gid]);
  }
}

// Batched 2-D transpose O[b][c][r] (+)= I[b][r][c] through a padded 32x32 tile.
__global__ void __launch_bounds__(256)
transpose2d_kernel(float* __restrict__ O, const float* __restrict__ I, int64_t rows, int64_t cols,
                   int64_t tiles_r, int64_t tiles_c, int64_t total_tiles, int acc) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
  for (int64_t tidx = blockIdx.x; tidx < total_tiles; tidx += gridDim.x) {
    const int64_t tc = tidx % tiles_c;
    const int64_t t2 = tidx / tiles_c;
    const int64_t tr = t2 % tiles_r;
    const int64_t b = t2 / tiles_r;
    const float* ip = I + b * rows * cols;
    float* op = O + b * rows * cols;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int64_t r = tr * 32 + ty + k * 8, c = tc * 32 + tx;
      if (r < rows && c < cols) tile[ty + k * 8][tx] = ip[r * cols + c];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int64_t c = tc * 32 + ty + k * 8, r = tr * 32 + tx;
      if (r < rows && c < cols) {
        const float v = tile[tx][ty + k * 8];
        float* dst = op + c * rows + r;
        *dst = acc ? __fadd_rn(*dst, v) : v;
      }
    }
    __syncthreads();
  }
}

inline int grid_for(const lnn::Device* d, int64_t work_items) {
  int64_t blocks = lnn_ceil_div(work_items, kThreads);
  int64_t cap = (int64_t)d->sm_count * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace

extern "C" {

int lnn_transpose(int dev, uint64_t O, uint64_t I, int rank, const int64_t* in_shape, const int* axes,
                  int accumulate) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(O && I && in_shape && axes, "null argument");
  LNN_REQUIRE(rank >= 1 && rank <= LNN_MAX_DIMS, "rank %d out of range", rank);
  int64_t in_stride[LNN_MAX_DIMS];
  int64_t s = 1;
  bool seen[LNN_MAX_DIMS] = {false};
  for (int k = rank - 1; k >= 0; --k) {
    LNN_REQUIRE(in_shape[k] >= 1, "bad extent");
    in_stride[k] = s;
    s *= in_shape[k];
  }
  const int64_t total = s;
  for (int k = 0; k < rank; ++k) {
    LNN_REQUIRE(axes[k] >= 0 && axes[k] < rank && !seen[axes[k]], "axes is not a permutation");
    seen[axes[k]] = true;
  }
  // Collapse to (batch, rows, cols) -> (batch, cols, rows) when the permutation is a
  // rotation of two contiguous axis groups behind an untouched prefix.
  int prefix = 0;
  while (prefix < rank && axes[prefix] == prefix) ++prefix;
  if (prefix == rank) {   // identity
    if (accumulate) {
      MoveDims md; md.rank = 1; md.o[0] = total; md.istride[0] = 1; md.ibase = 0;
      for (int k = 1; k < LNN_MAX_DIMS; ++k) { md.o[k] = 1; md.istride[k] = 0; }
      gather_kernel<<<grid_for(d, total), kThreads, 0, d->stream>>>(
          (float*)(uintptr_t)O, (const float*)(uintptr_t)I, total, md, 1);
      LNN_CHECK_LAUNCH(d);
      return LNN_OK;
    }
    return lnn_d2d(dev, O, I, (uint64_t)total * 4);
  }
  {
    // axes = [0..prefix-1, p..rank-1, prefix..p-1] ?
    int p = axes[prefix];
    bool rot = p > prefix;
    for (int k = prefix; rot && k < rank; ++k) {
      int expect = (k - prefix) + p;
      if (expect >= rank) expect = expect - rank + prefix;
      if (axes[k] != expect) rot = false;
    }
    if (rot) {
      int64_t batch = 1, rows = 1, cols = 1;
      for (int k = 0; k < prefix; ++k) batch *= in_shape[k];
      for (int k = prefix; k < p; ++k) rows *= in_shape[k];
      for (int k = p; k < rank; ++k) cols *= in_shape[k];
      if (rows >= 8 && cols >= 8) {
        const int64_t tiles_r = lnn_ceil_div(rows, 32), tiles_c = lnn_ceil_div(cols, 32);
        const int64_t total_tiles = batch * tiles_r * tiles_c;
        int64_t grid = total_tiles;
        const int64_t cap = (int64_t)d->sm_count * 16;
        if (grid > cap) grid = cap;
        transpose2d_kernel<<<(unsigned)grid, 256, 0, d->stream>>>(
            (float*)(uintptr_t)O, (const float*)(uintptr_t)I, rows, cols, tiles_r, tiles_c,
            total_tiles, accumulate);
        LNN_CHECK_LAUNCH(d);
        return LNN_OK;
      }
    }
  }
  MoveDims md;
  md.rank = rank;
  md.ibase = 0;
  for (int k = 0; k < LNN_MAX_DIMS; ++k) { md.o[k] = 1; md.istride[k] = 0; }
  for (int k = 0; k < rank; ++k) {
    md.o[k] = in_shape[axes[k]];
    md.istride[k] = in_stride[axes[k]];
  }
  gather_kernel<<<grid_for(d, total), kThreads, 0, d->stream>>>(
      (float*)(uintptr_t)O, (const float*)(uintptr_t)I, total, md, accumulate);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

static int slice_dims(MoveDims& md, int64_t* total, int rank, const int64_t* in_shape,
                      const int64_t* out_shape, const int64_t* begin, const int64_t* step) {
  LNN_REQUIRE(rank >= 1 && rank <= LNN_MAX_DIMS, "rank %d out of range", rank);
  LNN_REQUIRE(in_shape && out_shape && begin && step, "null argument");
  md.rank = rank;
  md.ibase = 0;
  for (int k = 0; k < LNN_MAX_DIMS; ++k) { md.o[k] = 1; md.istride[k] = 0; }
  int64_t s = 1, n = 1;
  for (int k = rank - 1; k >= 0; --k) {
    LNN_REQUIRE(in_shape[k] >= 1 && out_shape[k] >= 1, "bad extent");
    const int64_t last = begin[k] + (out_shape[k] - 1) * step[k];
    LNN_REQUIRE(begin[k] >= 0 && begin[k] < in_shape[k] && last >= 0 && last < in_shape[k],
                "slice of axis %d leaves the tensor", k);
    md.o[k] = out_shape[k];
    md.istride[k] = step[k] * s;
    md.ibase += begin[k] * s;
    s *= in_shape[k];
    n *= out_shape[k];
  }
  *total = n;
  return LNN_OK;
}

int lnn_slice_fwd(int dev, uint64_t O, uint64_t I, int rank, const int64_t* in_shape,
                  const int64_t* out_shape, const int64_t* begin, const int64_t* step,
                  int accumulate) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(O && I, "null buffer");
  MoveDims md; int64_t total;
  int rc = slice_dims(md, &total, rank, in_shape, out_shape, begin, step);
  if (rc) return rc;
  gather_kernel<<<grid_for(d, total), kThreads, 0, d->stream>>>(
      (float*)(uintptr_t)O, (const float*)(uintptr_t)I, total, md, accumulate);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

int lnn_slice_bwd(int dev, uint64_t dI, uint64_t dO, int rank, const int64_t* in_shape,
                  const int64_t* out_shape, const int64_t* begin, const int64_t* step) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(dI && dO, "null buffer");
  MoveDims md; int64_t total;
  int rc = slice_dims(md, &total, rank, in_shape, out_shape, begin, step);
  if (rc) return rc;
  scatter_add_kernel<<<grid_for(d, total), kThreads, 0, d->stream>>>(
      (float*)(uintptr_t)dI, (const float*)(uintptr_t)dO, total, md);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

}  // extern "C"
