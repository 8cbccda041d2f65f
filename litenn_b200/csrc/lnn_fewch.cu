// 3x3 unit-stride convolution of an image with at most four channels (a network's first layer)
// on the tensor cores, split-FP16 precision.
//
// With K = IC*9 <= 36 an im2col tile is almost all padding and a TMA-fed pipeline has nothing
// to stream, so this kernel builds its operand itself.  Producer warps read the NCHW fp32 input
// and write a halo patch into shared memory as a flat array of 16-byte "slots": slot (r, s)
// holds the fp16 values of input pixel (r, s) AND of its right neighbour (r, s + 1), 2*IC <= 8
// halves, scaled and split into hi / lo.  In the un-swizzled K-major layout of tcgen05 an
// operand row is one 16-byte chunk per 8 elements of K, rows of a group of 8 are contiguous and
// the byte distance between the two K chunks of an instruction (LBO) and between row groups
// (SBO) are free parameters.  So one MMA (K = 16) reads, for 128 output pixels at once,
//     chunk 0 = slot (oh + dy, ow)     -> taps (dy, 0) and (dy, 1)
//     chunk 1 = slot (oh + dy, ow + 2) -> tap  (dy, 2)  (its second half meets zero weights)
// with LBO = 2 slots, and SBO = one patch row makes the 16 row groups of M = 128 sixteen
// consecutive image rows: an MMA tile is 16 rows x 8 columns of output pixels, and a whole 3x3
// convolution is 3 instructions per split product instead of 9 taps.  A CTA works on super-tiles of
// 16 rows x 8*nsub columns that share one patch; their accumulators (oc columns each) sit side
// by side in TMEM, two sets, so that the epilogue of one super-tile overlaps the MMAs of the next.
//
//   warps 0-3  : patch producers (global fp32 -> scaled fp16 hi/lo slots, generic-proxy stores
//                made visible to the tensor core by fence.proxy.async)
//   warp  4    : MMA issuer, TMEM owner
//   warps 5-12 : epilogue, two warps per TMEM lane quarter taking alternate MMA tiles: lane =
//                output pixel (4 rows x 8 columns per warp), columns = channels; scale, bias,
//                leaky_relu, optional 2x2 max pool across lanes (two shuffles), store
// With 27 products per output the epilogue, not the MMA stream, is the long pole (16 outputs per
// thread and MMA), hence its eight warps and the short instruction sequences below.
//
// Same values as the FP32-pipe kernel of lnn_direct.cu up to the split's rounding; every wait is
// bounded like in the tile engine.  ref: litenn/core/op/conv2D.py:9-44, module/Conv2D.py:58-62,
// op/element_wise_op.py:207-221, op/pool2D.py:47-146
#include "lnn_tc_dev.cuh"
#include <stdlib.h>
#include <string.h>
#include <algorithm>

using namespace lnn_tc;

// timing experiments (wrong results by design) exist only in builds made with -DLNN_TC_EXPERIMENTS
#ifdef LNN_TC_EXPERIMENTS
#define FC_DBG(p, bit) (((p).debug & (bit)) != 0)
#else
#define FC_DBG(p, bit) false
#endif

namespace {

constexpr int kFcThreads = 416;
constexpr int kFcEpiWarps = 8;
constexpr int kFcProducers = 128;
constexpr int kFcEpilogueWarps = 8;         // warps 5..12
constexpr int kRows = 16;                 // image rows of a tile (row groups of M = 128)

struct FcParams {
  const float* X; const float* W; const float* bias; float* out;
  int n, ic, ih, iw, oc, oh, ow, padl, padt;
  int ocn;                                // MMA N: oc rounded up to 32
  int nsub, pws;                          // MMA tiles per super-tile, slots per patch row (8*nsub + 2)
  int tiles_w, tiles_h;
  int act; float alpha;
  int ep_mode;                            // 0 NCHW, 1 pooled NCHW,
                                          // 4 pooled channel-innermost split fp16 (scale from the bound in amax_out[-1])
  float* out_lo;
  uint8_t* idx_out;                       // ep_mode 1, optional: winning window position of every pooled value
  int ocp;                                // channel pitch of the ep_mode 4 output
  const uint32_t* amax_x; uint32_t* amax_out;
  int* status;
  uint32_t idesc;
  int patch_bytes;                        // one (hi or lo) patch buffer, 1024-byte multiple
  int w_bytes;                            // one (hi or lo) weight image: 6 * ocn * 16
  int debug;                              // experiments: 1 no MMAs, 2 no patch fill, 4 no epilogue math / stores
};

__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// leaky_relu with the reference's value for every input (I*(I>=0) + alpha*I*(I<0),
// element_wise_op.py:210) in five instructions: for finite v that expression equals
// v >= 0 ? v : alpha*v, signed zeros included, and v*0 is a zero of v's sign, so adding it changes
// nothing; for infinities and NaN the reference's products with 0 give NaN, and so does v*0.
__device__ __forceinline__ float lrelu_as_reference(float v, float alpha) {
  const float r = v >= 0.0f ? v : __fmul_rn(alpha, v);
  return __fadd_rn(r, __fmul_rn(v, 0.0f));
}

// multiplication by 2^k: one exact product when 2^k is a normal number, else two
struct FastPow2 {
  float f1, f2; bool one;
  __device__ __forceinline__ explicit FastPow2(int k) {
    one = k >= -126 && k <= 127;
    const int k1 = one ? k : k / 2;
    f1 = pow2f_int(k1); f2 = pow2f_int(k - k1);
  }
  __device__ __forceinline__ float operator()(float v) const {
    const float t = __fmul_rn(v, f1);
    if (one) return t;                    // uniform over the launch
    return __fmul_rn(t, f2);
  }
};

// One slot: the pixel at xp and its right neighbour, IC channels each: load, then scale, split, store.
template <int IC>
__device__ __forceinline__ void load_slot(float* v, const float* xp, int64_t plane, bool c0ok, bool c1ok) {
#pragma unroll
  for (int k = 0; k < 2 * IC; ++k) {
    const int c = k % IC, nb = k / IC;              // compile-time: nb 0 = this pixel, 1 = its right neighbour
    v[k] = (nb ? c1ok : c0ok) ? __ldg(xp + (int64_t)c * plane + nb) : 0.0f;
  }
}
template <int IC>
__device__ __forceinline__ void store_slot(uint8_t* dst_hi, uint8_t* dst_lo, const float* v, const FastPow2& sc) {
  __align__(16) __half h[8];
  __align__(16) __half l[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    if (k < 2 * IC) split_half(sc(v[k]), h[k], l[k]);
    else { h[k] = __float2half_rn(0.0f); l[k] = h[k]; }
  }
  *reinterpret_cast<uint4*>(dst_hi) = *reinterpret_cast<const uint4*>(h);
  *reinterpret_cast<uint4*>(dst_lo) = *reinterpret_cast<const uint4*>(l);
}

// WANT_IDX: the instance that also writes the map of winning pool positions (training); kept apart
// so that its extra registers do not touch the inference instances.
template <int IC, bool WANT_IDX>
__global__ void __launch_bounds__(kFcThreads, 1)
fewch_conv_kernel(const __grid_constant__ FcParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t patch_full[2];
  __shared__ uint64_t patch_empty[2];
  __shared__ uint64_t tmem_full[2];
  __shared__ uint64_t tmem_empty[2];
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag_smem;
  __shared__ uint32_t wmax_smem;
  __shared__ float bias_s[256];

  if (threadIdx.x == 0) { abort_flag_smem = (*(volatile int*)p.status != 0) ? 2 : 0; wmax_smem = 0u; }
  __syncthreads();
  if (abort_flag_smem == 2) return;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &abort_flag_smem;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t w_hi = base;
  const uint32_t patch0 = base + 2u * (uint32_t)p.w_bytes;          // [stage][hi, lo]
  uint8_t* const gen_base = smem_raw + (base - smem_u32(smem_raw)); // generic pointer to the same place
  const int num_tiles = p.n * p.tiles_h * p.tiles_w;
  const int set_cols = p.nsub * p.ocn;

  // ---- set-up: barriers, TMEM, the kernel's largest magnitude, weight images, bias -------------
  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&patch_full[s]), kFcProducers);
      mbar_init(smem_u32(&patch_empty[s]), 1);
      mbar_init(smem_u32(&tmem_full[s]), 1);
      mbar_init(smem_u32(&tmem_empty[s]), kFcEpiWarps);
    }
    fence_barrier_init();
  }
  if (warp == 4) {
    tmem_alloc(smem_u32(&tmem_base_smem), 512u);
    tmem_relinquish();
  }
  const int wcount = p.oc * p.ic * 9;
  {
    uint32_t m = 0u;
    for (int i = threadIdx.x; i < wcount; i += kFcThreads) m = max(m, __float_as_uint(p.W[i]) & 0x7fffffffu);
    warp_amax_commit(m, &wmax_smem);                 // shared-memory atomic
  }
  for (int i = threadIdx.x; i < 256; i += kFcThreads) bias_s[i] = (p.bias && i < p.oc) ? p.bias[i] : 0.0f;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const int e_w = exp_of_amax(wmax_smem);
  {
    // weight images: [dy][chunk][oc row][8 halves]; chunk 0 = taps kw 0, 1, chunk 1 = tap kw 2
    const Pow2Scale sc(-e_w);
    const int rows = 6 * p.ocn;
    for (int i = threadIdx.x; i < rows; i += kFcThreads) {
      const int o = i % p.ocn;
      const int chunk = (i / p.ocn) & 1;
      const int dy = i / (2 * p.ocn);
      __align__(16) __half h[8];
      __align__(16) __half l[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int c = k % IC, kw = chunk * 2 + k / IC;
        float v = 0.0f;
        if (o < p.oc && k < 2 * IC && kw < 3) v = p.W[((o * IC + c) * 3 + dy) * 3 + kw];
        split_half(sc(v), h[k], l[k]);
      }
      *reinterpret_cast<uint4*>(gen_base + (size_t)i * 16) = *reinterpret_cast<const uint4*>(h);
      *reinterpret_cast<uint4*>(gen_base + p.w_bytes + (size_t)i * 16) = *reinterpret_cast<const uint4*>(l);
    }
    fence_proxy_async();
  }
  __syncthreads();
  const uint32_t tmem_base = tmem_base_smem;

  if (warp < 4) {
    // ---- producers ---------------------------------------------------------------------------
    const FastPow2 sc(-exp_of_amax(__ldg(p.amax_x)));
    const int64_t plane = (int64_t)p.ih * p.iw;
    const int slots = (kRows + 2) * p.pws;
    // thread t owns slots t, t + 128, ...: (row, column) advance without divisions
    const int r_first = threadIdx.x / p.pws, s_first = threadIdx.x - r_first * p.pws;
    const int r_step = kFcProducers / p.pws, s_step = kFcProducers - r_step * p.pws;
    uint32_t s = 0, ph = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      const int tw_i = tile % p.tiles_w;
      const int th_i = (tile / p.tiles_w) % p.tiles_h;
      const int img = tile / (p.tiles_w * p.tiles_h);
      const int row0 = th_i * kRows - p.padt, col0 = tw_i * 8 * p.nsub - p.padl;
      ok = mbar_wait(smem_u32(&patch_empty[s]), ph ^ 1u, abort_flag, p.status, 0, tile);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      uint8_t* const dst_hi = gen_base + 2 * p.w_bytes + (size_t)s * 2 * p.patch_bytes;
      uint8_t* const dst_lo = dst_hi + p.patch_bytes;
      const float* xin = p.X + (int64_t)img * p.ic * plane;
      // The input streams from HBM and a warp has nothing else to do while a load is in flight:
      // the loads of kBatch slots are issued before the first of them is converted.
      constexpr int kBatch = 5;
      int r = r_first, sidx = s_first;
      for (int i0 = threadIdx.x; i0 < (FC_DBG(p, 2) ? 0 : slots); i0 += kFcProducers * kBatch) {
        float v[kBatch][2 * IC];
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
          const int row = row0 + r, col = col0 + sidx;
          const bool live = i0 + b * kFcProducers < slots;
          const bool rok = live && row >= 0 && row < p.ih;
          const bool c0ok = rok && col >= 0 && col < p.iw, c1ok = rok && col + 1 >= 0 && col + 1 < p.iw;
          load_slot<IC>(v[b], xin + (int64_t)row * p.iw + col, plane, c0ok, c1ok);
          r += r_step; sidx += s_step;
          if (sidx >= p.pws) { sidx -= p.pws; ++r; }
        }
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
          const int i = i0 + b * kFcProducers;
          if (i < slots) store_slot<IC>(dst_hi + (size_t)i * 16, dst_lo + (size_t)i * 16, v[b], sc);
        }
      }
      fence_proxy_async();
      mbar_arrive(smem_u32(&patch_full[s]));
      if (++s == 2u) { s = 0; ph ^= 1u; }
    }
  } else if (warp == 4) {
    // ---- MMA issuer --------------------------------------------------------------------------
    if (lane == 0) {
      const uint32_t row_b = (uint32_t)p.pws * 16u;
      // A: pixels, SBO = one patch row, LBO = two slots; B: weights, SBO = 8 rows, LBO = one chunk image
      const uint64_t a_desc0 = make_smem_desc(0u, 32u, row_b, 0u);
      const uint64_t b_desc0 = make_smem_desc(0u, (uint32_t)p.ocn * 16u, 128u, 0u);
      const uint64_t a_lo16 = (uint64_t)(p.patch_bytes >> 4), b_lo16 = (uint64_t)(p.w_bytes >> 4);
      uint32_t s = 0, ph = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++it) {
        const int set = it & 1;
        const uint32_t set_ph = (uint32_t)(it >> 1) & 1u;
        if (!mbar_wait(smem_u32(&tmem_empty[set]), set_ph ^ 1u, abort_flag, p.status, 3, it)) { ok = false; break; }
        if (!mbar_wait(smem_u32(&patch_full[s]), ph, abort_flag, p.status, 1, it)) { ok = false; break; }
        tc_fence_after();
        const uint32_t pa = patch0 + s * 2u * (uint32_t)p.patch_bytes;
        for (int j = 0; j < (FC_DBG(p, 1) ? 0 : p.nsub); ++j) {
          const uint32_t d_tmem = tmem_base + (uint32_t)(set * set_cols + j * p.ocn);
#pragma unroll
          for (int dy = 0; dy < 3; ++dy) {
            const uint64_t ah = a_desc0 + (uint64_t)((pa + (uint32_t)(dy * p.pws + 8 * j) * 16u) >> 4);
            const uint64_t bh = b_desc0 + (uint64_t)((w_hi + (uint32_t)(dy * 2 * p.ocn) * 16u) >> 4);
            umma_f16(d_tmem, ah, bh, p.idesc, dy == 0 ? 0u : 1u);
            umma_f16(d_tmem, ah, bh + b_lo16, p.idesc, 1u);
            umma_f16(d_tmem, ah + a_lo16, bh, p.idesc, 1u);
          }
        }
        umma_commit(smem_u32(&patch_empty[s]));
        umma_commit(smem_u32(&tmem_full[set]));
        if (++s == 2u) { s = 0; ph ^= 1u; }
      }
    }
  } else {
    // ---- epilogue: lane = pixel (row 4*quarter + lane/8 of the tile, column lane%8), columns = channels
#ifdef FC_FIXED_EP
    const int ep_mode = FC_FIXED_EP;
#else
    const int ep_mode = p.ep_mode;
#endif
    const int quarter = warp & 3;
    const int jfirst = (warp - 5) >> 2;                         // the two warps of a quarter take alternate tiles
    const int prow = 4 * quarter + (lane >> 3), pcol = lane & 7;
    const FastPow2 sc(exp_of_amax(__ldg(p.amax_x)) + e_w);
    const FastPow2 so(p.ep_mode == 4 ? -exp_of_amax(__ldg(p.amax_out - 1)) : 0);
    const int ohp = p.oh >> 1, owp = p.ow >> 1;
    const int sub4 = (lane & 1) | ((lane >> 2) & 2);            // position inside the 2x2 window
    // Transposing stage of the fused pool: 32 pixels x 32 channels of fp32 per warp, a row = one
    // pixel = eight 16-byte chunks stored at chunk (j + rot(pixel)) mod 8.  rot makes both access
    // patterns conflict-free: the writes (a quarter-warp = eight consecutive pixels, one chunk
    // index) and the reads (a quarter-warp = four pixels two apart, two chunk indices two apart).
    uint8_t* const xpose = gen_base + 2 * p.w_bytes + 4 * (size_t)p.patch_bytes + (size_t)(warp - 5) * 4096;
    auto rot = [](int px) { return ((px >> 1) & 1) + 4 * ((px >> 2) & 1) + 2 * (px & 1); };
    const int wbase_px = lane & ~9;
    uint32_t amax_acc = 0u;
#ifdef LNN_TC_EXPERIMENTS
    long long dbg_wait = 0, dbg_work = 0, dbg_ph0 = 0, dbg_ph1 = 0;
#endif
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      const int tw_i = tile % p.tiles_w;
      const int th_i = (tile / p.tiles_w) % p.tiles_h;
      const int img = tile / (p.tiles_w * p.tiles_h);
      const int set = it & 1;
      const uint32_t set_ph = (uint32_t)(it >> 1) & 1u;
#ifdef LNN_TC_EXPERIMENTS
      const long long tw0 = clock64();
#endif
      bool have = mbar_wait(smem_u32(&tmem_full[set]), set_ph, abort_flag, p.status, 2, it);
      have = __all_sync(0xffffffffu, have);
      if (!have) break;
      tc_fence_after();
#ifdef LNN_TC_EXPERIMENTS
      const long long tw1 = clock64();
      dbg_wait += tw1 - tw0;
#endif
      const int orow = th_i * kRows + prow;
      // 32-column chunks of this warp's tiles, in order; the TMEM load of the next chunk is in
      // flight while the current one is processed
      const int chunks_per_tile = p.ocn >> 5;
      const int my_tiles = FC_DBG(p, 4) ? 0 : (p.nsub - jfirst + 1) >> 1;
      const int my_chunks = my_tiles * chunks_per_tile;
      const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(set * set_cols);
      uint32_t vnext[32];
      if (FC_DBG(p, 16)) {
#pragma unroll
        for (int k = 0; k < 32; ++k) vnext[k] = (uint32_t)(lane * 77 + k) << 20;
      }
      if (my_chunks > 0 && !FC_DBG(p, 16)) tmem_ld32(t_lane + (uint32_t)(jfirst * p.ocn), vnext);
      int j = jfirst, c0 = 0;
      for (int ci = 0; ci < my_chunks; ++ci) {
        const int ocol = (tw_i * p.nsub + j) * 8 + pcol;
        const bool inside = orow < p.oh && ocol < p.ow;
        {
          uint32_t v[32];
#ifdef LNN_TC_EXPERIMENTS
          const long long tp0 = clock64();
#endif
          if (!FC_DBG(p, 16)) tmem_ld_wait();
#pragma unroll
          for (int k = 0; k < 32; ++k) v[k] = vnext[k];
#ifdef LNN_TC_EXPERIMENTS
          dbg_ph0 += clock64() - tp0;
#endif
          int jn = j, cn = c0 + 32;
          if (cn >= p.ocn) { cn = 0; jn += 2; }
          if (ci + 1 < my_chunks && !FC_DBG(p, 16)) tmem_ld32(t_lane + (uint32_t)(jn * p.ocn + cn), vnext);
          // The arithmetic below is written stage by stage over all 32 (or 8) values: the chains
          // of the individual values are independent, and issuing them interleaved is what keeps a
          // warp that has a scheduler almost to itself busy.
          if (ep_mode == 0) {
            float t[32];
#pragma unroll
            for (int k = 0; k < 32; ++k) t[k] = sc(__uint_as_float(v[k]));
            if (p.bias) {
#pragma unroll
              for (int k = 0; k < 32; ++k) t[k] = __fadd_rn(t[k], bias_s[c0 + k]);
            }
            if (p.act) {
              float z[32];
#pragma unroll
              for (int k = 0; k < 32; ++k) z[k] = __fmul_rn(t[k], 0.0f);
#pragma unroll
              for (int k = 0; k < 32; ++k) t[k] = t[k] >= 0.0f ? t[k] : __fmul_rn(p.alpha, t[k]);
#pragma unroll
              for (int k = 0; k < 32; ++k) t[k] = __fadd_rn(t[k], z[k]);
            }
            if (inside) {
              float* dst = p.out + (((int64_t)img * p.oc + c0) * p.oh + orow) * p.ow + ocol;
              const int64_t cstride = (int64_t)p.oh * p.ow;
#pragma unroll
              for (int k = 0; k < 32; ++k) {
                if (FC_DBG(p, 8)) amax_acc = max(amax_acc, __float_as_uint(t[k]));
                else if (c0 + k < p.oc) dst[k * cstride] = t[k];
              }
            }
          } else {
            // 2x2 max pool: the four pixels of a window sit in four lanes (bits 0 and 3 of the lane
            // number).  Scaling by a power of two, adding the bias and leaky_relu with alpha >= 0 never
            // reverse the order of two values, so the maximum is taken on the raw accumulators and
            // only the winner goes through them: the same value as pooling the finished pixels
            // (op/pool2D.py:111-146), at a quarter of the arithmetic.  (An accumulator that
            // overflowed to infinity would win here and turn into the reference's NaN -> 0, where
            // the reference would have skipped it; alpha < 0 takes the literal order below.)
            // (the map of winning positions compares finished values: literal order as well)
            constexpr bool want_idx = WANT_IDX;
            const bool pool_first = !(p.act && p.alpha < 0.0f) && !want_idx;
            float y[32];
#pragma unroll
            for (int k = 0; k < 32; ++k) y[k] = __uint_as_float(v[k]);
            if (!pool_first) {
#pragma unroll
              for (int k = 0; k < 32; ++k) {
                float t = sc(y[k]);
                if (p.bias) t = __fadd_rn(t, bias_s[c0 + k]);
                y[k] = p.act ? lrelu_as_reference(t, p.alpha) : t;
              }
            }
            float q[8];
            uint8_t widx[8];
            const int cb = c0 + 8 * sub4;
            {
              // the four pixels of a window come together through shared memory: each lane leaves
              // with its quarter of the channels for all four, and the maximum is taken in-thread
              // (pooling by shuffles cost 64 shuffles and 24 selects per 32 accumulators)
              const int my_rot = rot(lane);
#pragma unroll
              for (int j = 0; j < 8; ++j)
                *reinterpret_cast<float4*>(xpose + lane * 128 + (((j + my_rot) & 7) << 4)) =
                    make_float4(y[4 * j], y[4 * j + 1], y[4 * j + 2], y[4 * j + 3]);
              __syncwarp();
              float w4[4][8];
#pragma unroll
              for (int pix = 0; pix < 4; ++pix) {
                const int px = wbase_px | (pix & 1) | ((pix >> 1) << 3);
                const int r = rot(px);
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                  const float4 t = *reinterpret_cast<const float4*>(xpose + px * 128 + (((2 * sub4 + i + r) & 7) << 4));
                  w4[pix][4 * i] = t.x; w4[pix][4 * i + 1] = t.y; w4[pix][4 * i + 2] = t.z; w4[pix][4 * i + 3] = t.w;
                }
              }
              __syncwarp();
#pragma unroll
              for (int k = 0; k < 8; ++k) q[k] = fmaxf(fmaxf(w4[0][k], w4[1][k]), fmaxf(w4[2][k], w4[3][k]));
              if (want_idx) {
                // Where the pooling gradient of each window goes: the first position, in row-major
                // order, whose (finished) value equals the stored one (op/pool2D.py:147-230); 4 = none.
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                  const float m = fmaxf(-CUDART_INF_F, q[k]);
                  const float st = (m == -CUDART_INF_F) ? 0.0f : m;
                  widx[k] = w4[0][k] == st ? 0 : w4[1][k] == st ? 1 : w4[2][k] == st ? 2 : w4[3][k] == st ? 3 : 4;
                }
              }
            }
#ifdef LNN_TC_EXPERIMENTS
            dbg_ph1 += clock64() - tp0;
#endif
            if (pool_first) {
#pragma unroll
              for (int k = 0; k < 8; ++k) q[k] = sc(q[k]);
              if (p.bias) {
#pragma unroll
                for (int k = 0; k < 8; ++k) q[k] = __fadd_rn(q[k], bias_s[cb + k]);
              }
              if (p.act) {
#pragma unroll
                for (int k = 0; k < 8; ++k) q[k] = lrelu_as_reference(q[k], p.alpha);
              }
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const float m = fmaxf(-CUDART_INF_F, q[k]);
              q[k] = (m == -CUDART_INF_F) ? 0.0f : m;          // a window of NaNs, as the pooling kernel
            }
            if (inside) {
              const int ph_ = orow >> 1, pw_ = ocol >> 1;
              if (ep_mode == 1) {
                float* dst = p.out + (((int64_t)img * p.oc + cb) * ohp + ph_) * owp + pw_;
                const int64_t cstride = (int64_t)ohp * owp;
#pragma unroll
                for (int k = 0; k < 8; ++k)
                  if (cb + k < p.oc) dst[k * cstride] = q[k];
                if (want_idx) {
                  uint8_t* di = p.idx_out + (((int64_t)img * p.oc + cb) * ohp + ph_) * owp + pw_;
#pragma unroll
                  for (int k = 0; k < 8; ++k) {
                    if (cb + k < p.oc) di[k * cstride] = widx[k];
                  }
                }
              } else if (ep_mode == 4 && cb < p.ocp) {
                // the next convolution's operand, written here: eight channels = 16 bytes of hi and of lo
                const int64_t off = (((int64_t)img * ohp + ph_) * owp + pw_) * p.ocp + cb;
                __align__(16) __half h[8];
                __align__(16) __half l[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) split_half(so(q[k]), h[k], l[k]);
                *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(p.out) + off) = *reinterpret_cast<const uint4*>(h);
                *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(p.out_lo) + off) = *reinterpret_cast<const uint4*>(l);
#pragma unroll
                for (int k = 0; k < 8; ++k) amax_acc = max(amax_acc, __float_as_uint(q[k]) & 0x7fffffffu);
              }
            }
          }
          __syncwarp();
        }
        c0 += 32;
        if (c0 >= p.ocn) { c0 = 0; j += 2; }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tmem_empty[set]));
#ifdef LNN_TC_EXPERIMENTS
      dbg_work += clock64() - tw1;
#endif
    }
    __syncwarp();
#ifdef LNN_TC_EXPERIMENTS
    if (FC_DBG(p, 32) && blockIdx.x == 0 && lane == 0)
      printf("epilogue warp %d: %d tiles, wait %lld work %lld clocks per tile; per tile: ld-wait %lld, through pooling %lld\n", warp, it,
             dbg_wait / max(it, 1), dbg_work / max(it, 1), dbg_ph0 / max(it, 1), dbg_ph1 / max(it, 1));
#endif
    if (ep_mode == 4 || (FC_DBG(p, 8) && p.amax_out)) warp_amax_commit(amax_acc, p.amax_out);
  }

  // ---- tear-down -----------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512u);
  }
}

}  // namespace

namespace lnn {

bool conv_fewch_applicable(const lnn_conv_geom* g) {
  if (g->ic > 4 || g->kh != 3 || g->kw != 3 || g->stride != 1 || g->dilation != 1) return false;
  if (g->oc > 256 || g->padl > 2 || g->padt > 2 || g->padl < 0 || g->padt < 0) return false;
  return true;
}

// ep_mode 0: Y = NCHW result; 1: pooled NCHW; 4: pooled channel-innermost split fp16 with channel
// pitch ocp (Y = hi, Y_lo = lo) scaled by the bound in amax_out[-1], the largest magnitude
// accumulated into *amax_out (which the caller zeroed).  amax_x
// holds the fp32 bit pattern of the input's largest magnitude.  idx (ep_mode 1, optional): one byte
// per pooled element, the window position that holds the pooled value.
int conv_fewch_fwd(Device* d, const lnn_conv_geom* g, float* Y, const float* X, const float* W,
                   const float* bias, int act, float alpha, int ep_mode, int ocp, const uint32_t* amax_x,
                   uint32_t* amax_out, float* Y_lo, uint8_t* idx) {
  FcParams p;
  memset(&p, 0, sizeof(p));
  p.X = X; p.W = W; p.bias = bias; p.out = Y; p.out_lo = Y_lo; p.idx_out = ep_mode == 1 ? idx : nullptr;
  p.n = g->n; p.ic = g->ic; p.ih = g->ih; p.iw = g->iw; p.oc = g->oc; p.oh = g->oh; p.ow = g->ow;
  p.padl = g->padl; p.padt = g->padt;
  p.ocn = (g->oc + 31) & ~31;
  p.nsub = std::max(1, std::min(std::min(8, 256 / p.ocn), (g->ow + 7) / 8));
  p.pws = 8 * p.nsub + 2;
  p.tiles_w = (g->ow + 8 * p.nsub - 1) / (8 * p.nsub);
  p.tiles_h = (g->oh + kRows - 1) / kRows;
  p.act = act; p.alpha = alpha; p.ep_mode = ep_mode; p.ocp = ocp;
  p.amax_x = amax_x; p.amax_out = amax_out;
  p.status = d->status_dev;
  // c_format F32, a/b format F16, both K-major, N = ocn, M = 128
  p.idesc = (1u << 4) | ((uint32_t)(p.ocn >> 3) << 17) | ((128u >> 4) << 24);
  p.patch_bytes = ((kRows + 2) * p.pws * 16 + 2 * 16 + 1023) & ~1023;   // + the slots chunk 1 of the last rows may touch
  p.w_bytes = 6 * p.ocn * 16;
#ifdef LNN_TC_EXPERIMENTS
  { const char* e = getenv("LNN_FC_DEBUG"); p.debug = e ? atoi(e) : 0; }
#endif
  const int64_t tiles = (int64_t)p.n * p.tiles_h * p.tiles_w;
  LNN_REQUIRE(tiles < (1ll << 31), "too many tiles");
  // operands, then 4 KB per epilogue warp for the transposing stage of the fused pool
  const int smem = 2 * p.w_bytes + 4 * p.patch_bytes + 1024 + kFcEpilogueWarps * 4096;
  LNN_REQUIRE(smem <= 227 * 1024 - 4096, "operands of %d bytes do not fit shared memory", smem);
  if (!(d->smem_attr_done & (1u << 9))) {
    const int lim = 227 * 1024 - 4096;
    LNN_CUDA(cudaFuncSetAttribute(fewch_conv_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
    LNN_CUDA(cudaFuncSetAttribute(fewch_conv_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
    LNN_CUDA(cudaFuncSetAttribute(fewch_conv_kernel<3, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
    LNN_CUDA(cudaFuncSetAttribute(fewch_conv_kernel<4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
    LNN_CUDA(cudaFuncSetAttribute(fewch_conv_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
    LNN_CUDA(cudaFuncSetAttribute(fewch_conv_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
    LNN_CUDA(cudaFuncSetAttribute(fewch_conv_kernel<3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
    LNN_CUDA(cudaFuncSetAttribute(fewch_conv_kernel<4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
    d->smem_attr_done |= 1u << 9;
  }
  const unsigned ctas = (unsigned)std::min<int64_t>(tiles, d->sm_count);
  {
    ProfScope prof(d, (int)LNN_PROF_FEWCH);
    if (p.idx_out) {
      switch (g->ic) {
        case 1: fewch_conv_kernel<1, true><<<ctas, kFcThreads, smem, d->stream>>>(p); break;
        case 2: fewch_conv_kernel<2, true><<<ctas, kFcThreads, smem, d->stream>>>(p); break;
        case 3: fewch_conv_kernel<3, true><<<ctas, kFcThreads, smem, d->stream>>>(p); break;
        default: fewch_conv_kernel<4, true><<<ctas, kFcThreads, smem, d->stream>>>(p); break;
      }
    } else {
      switch (g->ic) {
        case 1: fewch_conv_kernel<1, false><<<ctas, kFcThreads, smem, d->stream>>>(p); break;
        case 2: fewch_conv_kernel<2, false><<<ctas, kFcThreads, smem, d->stream>>>(p); break;
        case 3: fewch_conv_kernel<3, false><<<ctas, kFcThreads, smem, d->stream>>>(p); break;
        default: fewch_conv_kernel<4, false><<<ctas, kFcThreads, smem, d->stream>>>(p); break;
      }
    }
  }
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

}  // namespace lnn
