// tcgen05 tile engine: device kernel, operand pre-split passes, tensor-map construction
// and the planners behind lnn_gemm_f32 / lnn_conv2d_fwd / lnn_conv2d_dx / lnn_conv2d_dw.
#include "lnn_tc_dev.cuh"
#include <stdlib.h>
#include <math_constants.h>
#include <string.h>
#include <algorithm>

using namespace lnn_tc;

// Timing experiments (skip MMAs / loads / stores / tap shifts; the results are wrong by design)
// exist only in builds made with -DLNN_TC_EXPERIMENTS.
#ifdef LNN_TC_EXPERIMENTS
#define LNN_DBG(p, bit) (((p).debug & (bit)) != 0)
#else
#define LNN_DBG(p, bit) false
#endif

// =========================================================================================
// device helpers (inline PTX)
// =========================================================================================
namespace {
// Fused max_pool2D(2, 2) of a channels-on-M accumulator: v0 / v1 hold 32 consecutive pixels of
// two consecutive image rows for this lane's channel (row `a` even, first column `b0` even,
// `wvalid` of the 32 columns real).  The maximum is taken in the pooling kernel's order
// (t00, t01, t10, t11 on top of -inf; litenn/core/op/pool2D.py:111-146) after bias and
// activation, so the value equals the unfused chain bit for bit.
// ep_mode 4 collects the largest magnitude written by this thread in `amax`; the caller
// commits it once per warp when the kernel ends.
__device__ __forceinline__ void pooled_store(const TcParams& p, const Pow2Scale& sc, const uint32_t* v0,
                                             const uint32_t* v1, float bias_v, int oc, int64_t n, int a,
                                             int b0, int wvalid, uint32_t& amax) {
  const bool real = oc < p.OC;
  if (p.ep_mode == 1 && !real) return;
  if (p.ep_mode >= 2 && oc >= p.ocp) return;
  float m[16];
  // Scaling by a power of two, adding the bias and leaky_relu with alpha >= 0 never reverse the
  // order of two values, so the window's maximum is taken on the raw accumulators and only the
  // winner goes through them: a quarter of the arithmetic, the same value.  (An accumulator that
  // overflowed to +inf wins here and may become the NaN -> 0 of the pooling kernel where the
  // literal order would have skipped it.)  alpha < 0 takes the literal order.
  uint8_t widx[16];
  if (!(p.act && p.alpha < 0.0f) && p.idx_out == nullptr) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      float t = fmaxf(fmaxf(__uint_as_float(v0[2 * j]), __uint_as_float(v0[2 * j + 1])),
                      fmaxf(__uint_as_float(v1[2 * j]), __uint_as_float(v1[2 * j + 1])));
      if (p.esz == 2) t = sc(t);
      if (p.bias) t = __fadd_rn(t, bias_v);
      t = apply_act(t, p.act, p.alpha);
      const float mm = fmaxf(-CUDART_INF_F, t);
      m[j] = (mm == -CUDART_INF_F) ? 0.0f : mm;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      float t00 = __uint_as_float(v0[2 * j]), t01 = __uint_as_float(v0[2 * j + 1]);
      float t10 = __uint_as_float(v1[2 * j]), t11 = __uint_as_float(v1[2 * j + 1]);
      if (p.esz == 2) { t00 = sc(t00); t01 = sc(t01); t10 = sc(t10); t11 = sc(t11); }
      if (p.bias) {
        t00 = __fadd_rn(t00, bias_v); t01 = __fadd_rn(t01, bias_v);
        t10 = __fadd_rn(t10, bias_v); t11 = __fadd_rn(t11, bias_v);
      }
      t00 = apply_act(t00, p.act, p.alpha); t01 = apply_act(t01, p.act, p.alpha);
      t10 = apply_act(t10, p.act, p.alpha); t11 = apply_act(t11, p.act, p.alpha);
      const float mm = fmaxf(fmaxf(fmaxf(fmaxf(-CUDART_INF_F, t00), t01), t10), t11);
      m[j] = (mm == -CUDART_INF_F) ? 0.0f : mm;
      // where the pooling gradient goes: the first position equal to the stored value
      // (pool2D.py:147-230); none when the window held nothing comparable
      widx[j] = t00 == m[j] ? 0 : t01 == m[j] ? 1 : t10 == m[j] ? 2 : t11 == m[j] ? 3 : 4;
    }
  }
  const int npool = min(wvalid, p.AW - b0) >> 1;          // pooled pixels of this chunk that exist
  const int64_t base = n * p.out_sn + (int64_t)(a >> 1) * p.out_sa + (int64_t)(b0 >> 1) * p.out_sb +
                       (int64_t)oc * p.out_sc + p.out_base;
  if (p.ep_mode == 1) {
    float* dst = p.out + base;                               // 16 consecutive floats of one plane row
    if (npool == 16 && ((((uintptr_t)dst) & 15) == 0)) {
#pragma unroll
      for (int j = 0; j < 16; j += 4)
        *reinterpret_cast<float4*>(dst + j) = make_float4(m[j], m[j + 1], m[j + 2], m[j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (j < npool) dst[j] = m[j];
    }
    if (p.idx_out) {
      uint8_t* di = p.idx_out + base;
      if (npool == 16 && ((((uintptr_t)di) & 15) == 0)) {
        uint32_t w4[4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
          w4[q] = (uint32_t)widx[4 * q] | ((uint32_t)widx[4 * q + 1] << 8) | ((uint32_t)widx[4 * q + 2] << 16) |
                  ((uint32_t)widx[4 * q + 3] << 24);
        *reinterpret_cast<uint4*>(di) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (j < npool) di[j] = widx[j];
      }
    }
  } else if (p.ep_mode == 2) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      if (j < npool) {
        float hi = 0.0f, lo = 0.0f;
        if (real) split1(m[j], hi, lo);                      // pad channels are written as zeros
        p.out[base + (int64_t)j * p.out_sb] = hi;
        if (p.out_lo) p.out_lo[base + (int64_t)j * p.out_sb] = lo;
      }
    }
  } else {
    // fp16 split written directly: the scale comes from an upper bound of the result that was
    // known before the launch (word 0 of the output's trailer)
    const Pow2Scale so(-exp_of_amax(__ldg(p.amax_out - 1)));
    __half* const oh = reinterpret_cast<__half*>(p.out);
    __half* const ol = reinterpret_cast<__half*>(p.out_lo);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      if (j < npool) {
        const float v = real ? m[j] : 0.0f;
        __half h, l;
        split_half(so(v), h, l);
        oh[base + (int64_t)j * p.out_sb] = h;
        ol[base + (int64_t)j * p.out_sb] = l;
        amax = max(amax, __float_as_uint(v) & 0x7fffffffu);
      }
    }
  }
}

// =========================================================================================
// the tile kernel: persistent, one CTA per SM, two TMEM accumulators
// =========================================================================================
struct TileCoord {
  int m0, n0, bz;                 // GEMM
  int pb0, pa0, pn0;              // CONV pixel-tile origin (logical output coordinates)
  int split, oc_t, ic_t, tap, patch0;   // DW
  int nb0, nblk;                        // DW: first 32-wide column block and how many this tile owns
  int num_kb;
};

template <int MODE>
__device__ __forceinline__ TileCoord decode_tile(const TcParams& p, int tile) {
  TileCoord t;
  t.m0 = t.n0 = t.bz = t.pb0 = t.pa0 = t.pn0 = t.split = t.oc_t = t.ic_t = t.tap = t.patch0 = 0;
  t.nb0 = t.nblk = 0;
  t.num_kb = p.num_kb;
  const int x = tile % p.grid_x;
  const int r = tile / p.grid_x;
  const int y = r % p.grid_y;
  const int z = r / p.grid_y;
  if (MODE == MODE_GEMM) {
    t.m0 = x * 128; t.n0 = y * p.bn; t.bz = z;
  } else if (MODE == MODE_CONV || MODE == MODE_CONVT) {
    const int bt = x % p.tiles_b;
    const int at = (x / p.tiles_b) % p.tiles_a;
    const int nt = x / (p.tiles_b * p.tiles_a);
    t.pb0 = bt * p.tw; t.pa0 = at * p.th; t.pn0 = nt * p.tn;
    if (MODE == MODE_CONV) t.n0 = y * p.bn; else t.m0 = y * 128;
  } else {
    t.split = x;
    t.oc_t = y;
    t.nb0 = z * p.nb_group;                       // columns = (tap, 32-channel block) pairs
    t.nblk = min(p.nb_group, p.nb_total - t.nb0);
    t.patch0 = x * p.patches_per_split;
    t.num_kb = min(p.patches_per_split, p.patches_total - t.patch0);
    if (t.num_kb < 0) t.num_kb = 0;
  }
  return t;
}


template <int MODE>
__global__ void __launch_bounds__(kThreadsTc, 1)
tc_kernel(const __grid_constant__ CUtensorMap tmAh, const __grid_constant__ CUtensorMap tmAl,
          const __grid_constant__ CUtensorMap tmBh, const __grid_constant__ CUtensorMap tmBl,
          const __grid_constant__ TcParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[8];
  __shared__ uint64_t empty_bar[8];
  __shared__ uint64_t tmem_full_bar[2];
  __shared__ uint64_t tmem_empty_bar[2];
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag_smem;

  // an earlier CTA already gave up: leave as a whole CTA (the decision must be uniform)
  if (threadIdx.x == 0) abort_flag_smem = (*(volatile int*)p.status != 0) ? 2 : 0;
  __syncthreads();
  if (abort_flag_smem == 2) return;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &abort_flag_smem;

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;      // operand ring, 1024-byte aligned
  const int nbuf = p.passes == 1 ? 1 : 2;
  const uint32_t a_sz = (uint32_t)((p.a_tile_bytes + 1023) & ~1023);
  const uint32_t b_sz = (uint32_t)((p.b_tile_bytes + 1023) & ~1023);
  const uint32_t stage_sz = (uint32_t)p.kgroup * nbuf * (a_sz + b_sz);
  const int num_tiles = p.grid_x * p.grid_y * p.grid_z;

  // ---- set-up ---------------------------------------------------------------------------
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&tmem_full_bar[a]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[a]), kEpilogueWarps);     // one arrival per epilogue warp
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_smem), 2u * p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;

  // ---- roles ----------------------------------------------------------------------------
  // A stage of the ring holds `kgroup` units; a unit is one 32-wide K slab (GEMM), one
  // (tap, channel block) pair (CONV/CONVT) or one pixel patch (DW).  The two single-thread
  // roles below are scalar-issue bound, so their loops carry running counters instead of
  // recomputing positions with divisions.
  const uint32_t unit_sz = nbuf * (a_sz + b_sz);
  const uint32_t full0 = smem_u32(&full_bar[0]), empty0 = smem_u32(&empty_bar[0]);
  if (warp == 0) {
    if (lane == 0) {
      const uint32_t unit_tx =
          (uint32_t)nbuf * (uint32_t)(p.a_loads * p.a_load_bytes + p.b_loads * p.b_load_bytes);
      uint32_t s = 0, ph = 0;                           // ring position and its phase
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        const TileCoord t = decode_tile<MODE>(p, tile);
        int units_left = t.num_kb;
        int k0 = 0;                                     // GEMM: K offset
        int tp = 0, cbi = 0;                            // CONV: tap, channel block
        int pidx = t.patch0;                            // DW: patch
        const int cx = t.pb0 * p.es, cy = t.pa0 * p.es;
        while (units_left > 0) {
          const int nun = min(p.kgroup, units_left);
          if (!mbar_wait(empty0 + 8u * s, ph ^ 1u, abort_flag, p.status, 0, units_left)) { ok = false; break; }
          const uint32_t fb = full0 + 8u * s;
          if (LNN_DBG(p, 2)) { mbar_arrive(fb); }       // timing experiment: no loads
          else {
            // elements per 128/64/32-byte row of an MN-major box
            const int ea = p.swz_a / p.esz, eb = p.swz_b / p.esz;
            // DW: only the channel blocks of dY that hold real output channels are loaded; the
            // accumulator rows of the others are never read back
            const int a_valid = MODE == MODE_DW ? min(p.a_loads, (p.OC - t.oc_t * 128 + ea - 1) / ea) : p.a_loads;
            if (MODE == MODE_DW)
              mbar_expect_tx(fb, (uint32_t)nbuf * (uint32_t)(a_valid * p.a_load_bytes + t.nblk * p.b_load_bytes));
            else
              mbar_expect_tx(fb, unit_tx * (uint32_t)nun);
            uint32_t dst = tiles + s * stage_sz;
            for (int u = 0; u < nun; ++u, dst += unit_sz) {
              for (int half = 0; half < nbuf; ++half) {
                const CUtensorMap* ta = half ? &tmAl : &tmAh;
                const CUtensorMap* tb = half ? &tmBl : &tmBh;
                const uint32_t da = dst + half * a_sz;
                const uint32_t db = dst + nbuf * a_sz + half * b_sz;
                if (MODE == MODE_GEMM) {
                  if (p.a_major == 0) {
                    tma_load_3d(da, ta, fb, k0, t.m0, t.bz);
                  } else {
                    for (int i = 0; i < p.a_loads; ++i)
                      tma_load_3d(da + i * p.a_load_bytes, ta, fb, t.m0 + i * ea, k0, t.bz);
                  }
                  if (p.b_major == 0) {
                    tma_load_3d(db, tb, fb, k0, t.n0, t.bz);
                  } else {
                    for (int i = 0; i < p.b_loads; ++i)
                      tma_load_3d(db + i * p.b_load_bytes, tb, fb, t.n0 + i * eb, k0, t.bz);
                  }
                } else if (MODE == MODE_CONV) {
                  tma_load_4d(da, ta, fb, cbi * p.cb, cx + p.tap_dx[tp], cy + p.tap_dy[tp], t.pn0);
                  tma_load_3d(db, tb, fb, cbi * p.cb, t.n0, p.tap_w[tp]);
                } else if (MODE == MODE_CONVT) {
                  // channels on M: the kernel tile is operand A, the pixel patch operand B
                  tma_load_3d(da, ta, fb, cbi * p.cb, t.m0, p.tap_w[tp]);
                  tma_load_4d(db, tb, fb, cbi * p.cb, cx + p.tap_dx[tp], cy + p.tap_dy[tp], t.pn0);
                } else {
                  const int bt = pidx % p.tiles_b;
                  const int at = (pidx / p.tiles_b) % p.tiles_a;
                  const int nt = pidx / (p.tiles_b * p.tiles_a);
                  for (int i = 0; i < a_valid; ++i)
                    tma_load_4d(da + i * p.a_load_bytes, ta, fb, t.oc_t * 128 + i * ea, bt * p.tw,
                                at * p.th, nt * p.tn);
                  int tapi = t.nb0 / p.ic_tiles, icb = t.nb0 - tapi * p.ic_tiles;
                  for (int i = 0; i < t.nblk; ++i) {
                    tma_load_4d(db + i * p.b_load_bytes, tb, fb, icb * eb,
                                bt * p.tw * p.es + p.tap_dx[tapi], at * p.th * p.es + p.tap_dy[tapi],
                                nt * p.tn);
                    if (++icb == p.ic_tiles) { icb = 0; ++tapi; }
                  }
                }
              }
              k0 += p.kunit;
              if (++cbi == p.ncb) { cbi = 0; ++tp; }
              ++pidx;
            }
          }
          units_left -= nun;
          if (++s == (uint32_t)p.stages) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // K-major: 8-row swizzle atoms, SBO = 8 rows.  MN-major: rows of one swizzle span along
      // MN, k-rows stacked; fp16 uses the ordinary 128/64/32-byte swizzles (atoms of 8 k-rows,
      // SBO = 8 rows), tf32 only exists as the "128-byte swizzle with 32-byte atoms" layout
      // (4 k-rows per atom, SBO = 4 rows); the MN blocks are LBO apart.  One instruction
      // consumes 32 bytes of K: 8 (tf32) or 16 (fp16) k-rows of an MN-major tile.
      const bool f16 = p.esz == 2;
      const uint32_t la = (p.a_major && !f16) ? 1u : layout_of_swizzle(p.swz_a);
      const uint32_t lb = (p.b_major && !f16) ? 1u : layout_of_swizzle(p.swz_b);
      const uint32_t a_lbo = p.a_major ? (uint32_t)(p.a_krows * p.swz_a) : 16u;
      const uint32_t b_lbo = p.b_major ? (uint32_t)(p.b_krows * p.swz_b) : 16u;
      const uint32_t mn_atom = f16 ? 8u : 4u, mn_step = f16 ? 16u : 8u;
      const uint32_t a_sbo = (p.a_major ? mn_atom : 8u) * p.swz_a, b_sbo = (p.b_major ? mn_atom : 8u) * p.swz_b;
      // descriptors with a zero start address; the address field (bits 0-13, 16-byte units)
      // is added per use -- shared memory addresses stay below 2^18, so no carry leaves it
      const uint64_t a_desc0 = make_smem_desc(0u, a_lbo, a_sbo, la);
      const uint64_t b_desc0 = make_smem_desc(0u, b_lbo, b_sbo, lb);
      const uint64_t a_step16 = (p.a_major ? mn_step * p.swz_a : 32u) >> 4;
      const uint64_t b_step16 = (p.b_major ? mn_step * p.swz_b : 32u) >> 4;
      const uint64_t a_lo16 = a_sz >> 4, b_lo16 = b_sz >> 4;
      const int ksteps = LNN_DBG(p, 1) ? 0 : p.ksteps;     // experiment bit 0: no MMAs
      const uint32_t idesc = p.idesc;
      uint32_t s = 0, ph = 0;
      int it = 0;                                       // tiles processed by this CTA
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++it) {
        const TileCoord t = decode_tile<MODE>(p, tile);
        const int acc = it & 1;
        const uint32_t acc_ph = (uint32_t)(it >> 1) & 1u;
        // wait until the epilogue has drained this accumulator (passes at once the first time)
        if (!mbar_wait(smem_u32(&tmem_empty_bar[acc]), acc_ph ^ 1u, abort_flag, p.status, 3, it)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)acc * p.tmem_cols;
        int units_left = t.num_kb;
        uint32_t accum = 0u;                            // first MMA of a tile overwrites
        while (units_left > 0) {
          const int nun = min(p.kgroup, units_left);
          if (!mbar_wait(full0 + 8u * s, ph, abort_flag, p.status, 1, units_left)) { ok = false; break; }
          tc_fence_after();
          uint32_t ua = tiles + s * stage_sz;
          for (int u = 0; u < nun; ++u, ua += unit_sz) {
            const uint64_t ah = a_desc0 + (uint64_t)(ua >> 4);
            const uint64_t bh = b_desc0 + (uint64_t)((ua + nbuf * a_sz) >> 4);
            issue_unit(p.esz, nbuf, ksteps, d_tmem, ah, bh, a_step16, b_step16, a_lo16, b_lo16, idesc, accum);
            if (ksteps > 0) accum = 1u;
          }
          umma_commit(empty0 + 8u * s);                 // frees the stage when these MMAs retire
          units_left -= nun;
          if (++s == (uint32_t)p.stages) { s = 0; ph ^= 1u; }
        }
        if (ok) umma_commit(smem_u32(&tmem_full_bar[acc]));   // accumulator complete
      }
    }
  } else {
    // ---- epilogue warps: TMEM lane quarter = warp % 4; the two warps of a quarter take the
    // even and the odd 32-column chunks of the accumulator --------------------------------------
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    // fp16 split: the accumulator holds the product of the scaled operands
    const bool scaled = p.esz == 2;
    const Pow2Scale sc(scaled ? exp_of_amax(__ldg(p.amax_a)) + exp_of_amax(__ldg(p.amax_b)) : 0);
    uint32_t amax_acc = 0u;
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      const TileCoord t = decode_tile<MODE>(p, tile);
      const int acc = it & 1;
      const uint32_t acc_ph = (uint32_t)(it >> 1) & 1u;
      bool have_acc = mbar_wait(smem_u32(&tmem_full_bar[acc]), acc_ph, abort_flag, p.status, 2, it);
      have_acc = __all_sync(0xffffffffu, have_acc);   // tcgen05.ld below is warp-collective
      if (!have_acc) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + (uint32_t)acc * p.tmem_cols;

      if (MODE == MODE_CONVT) {
        // rows = output channels, columns = the pixels of the patch (tn x th x tw, W fastest)
        const int oc = t.m0 + r;
        const bool row_ok = oc < p.OC;
        const float bias_v = (row_ok && p.bias) ? __ldg(p.bias + oc) : 0.0f;
        if (p.ep_mode != 0) {
          // fused max pool: tw is a multiple of 32 and th even, so a 32-column chunk is a piece
          // of one image row and the chunk tw columns later is the row below it
          const int chunks_per_row = p.tw >> 5;
          int turn = 0;
          for (int tn_i = 0; tn_i < p.tn; ++tn_i) {
            for (int th_i = 0; th_i < p.th; th_i += 2) {
              for (int ch = 0; ch < chunks_per_row; ++ch) {
                if (((turn++) & 1) != half) continue;
                const int c_top = (tn_i * p.th + th_i) * p.tw + ch * 32;
                uint32_t v0[32], v1[32];
                tmem_ld32(d_tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c_top, v0);
                tmem_ld32(d_tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c_top + p.tw), v1);
                tmem_ld_wait();
                const int n = t.pn0 + tn_i, a = t.pa0 + th_i, b0 = t.pb0 + ch * 32;
                if (n < p.NL && a < p.AH && b0 < p.AW && !LNN_DBG(p, 4))
                  pooled_store(p, sc, v0, v1, bias_v, oc, n, a, b0, 32, amax_acc);
                __syncwarp();
              }
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
          continue;
        }
        float* const obase = p.out + p.out_base + (int64_t)oc * p.out_sc;
        for (int c0 = half * 32; c0 < p.bn; c0 += 64) {
          // (image, row, column) of the first pixel of the current group of four
          int tn_i = c0 / (p.th * p.tw);
          int th_i = (c0 - tn_i * p.th * p.tw) / p.tw;
          int tw_i = c0 - (tn_i * p.th + th_i) * p.tw;
          uint32_t v[32];
          tmem_ld32(d_tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
          tmem_ld_wait();
          if (row_ok && !LNN_DBG(p, 4)) {
            // Phase 1: where each group of four pixels goes, and (for "+=") its old values.  All
            // loads are issued before any store so that their latencies overlap.
            float* dsts[8];
            int pos[8];                                   // tw | th << 8 | tn << 16, or -1: nothing to store
            uint32_t four_mask = 0, vec_mask = 0;
            float4 old[8];
#pragma unroll
            for (int gi = 0; gi < 8; ++gi) {
              const int q = c0 + gi * 4;
              pos[gi] = -1;
              old[gi] = make_float4(0.f, 0.f, 0.f, 0.f);
              if (q < p.rows_valid) {
                pos[gi] = tw_i | (th_i << 8) | (tn_i << 16);
                const int n = t.pn0 + tn_i, a = t.pa0 + th_i, b = t.pb0 + tw_i;
                float* dst = obase + (int64_t)n * p.out_sn + (int64_t)a * p.out_sa + (int64_t)b * p.out_sb;
                dsts[gi] = dst;
                const bool four = (tw_i + 3 < p.tw) && (b + 3 < p.AW) && n < p.NL && a < p.AH;
                if (four) {
                  four_mask |= 1u << gi;
                  const bool vec = p.out_sb == 1 && ((((uintptr_t)dst) & 15) == 0);
                  if (vec) vec_mask |= 1u << gi;
                  if (p.accumulate) {
                    if (vec) old[gi] = *reinterpret_cast<const float4*>(dst);
                    else old[gi] = make_float4(dst[0], dst[p.out_sb], dst[2 * p.out_sb], dst[3 * p.out_sb]);
                  }
                }
              }
              tw_i += 4;
              while (tw_i >= p.tw) { tw_i -= p.tw; if (++th_i >= p.th) { th_i = 0; ++tn_i; } }
            }
            // Phase 2: bias, activation, add, store
#pragma unroll
            for (int gi = 0; gi < 8; ++gi) {
              if (pos[gi] < 0) continue;
              const int j = gi * 4;
              float x[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float tt = __uint_as_float(v[j + e]);
                if (scaled) tt = sc(tt);
                if (p.bias) tt = __fadd_rn(tt, bias_v);
                x[e] = apply_act(tt, p.act, p.alpha);
              }
              float* dst = dsts[gi];
              if (four_mask & (1u << gi)) {
                if (p.accumulate) {
                  x[0] = __fadd_rn(old[gi].x, x[0]); x[1] = __fadd_rn(old[gi].y, x[1]);
                  x[2] = __fadd_rn(old[gi].z, x[2]); x[3] = __fadd_rn(old[gi].w, x[3]);
                }
                if (vec_mask & (1u << gi)) *reinterpret_cast<float4*>(dst) = make_float4(x[0], x[1], x[2], x[3]);
                else { dst[0] = x[0]; dst[p.out_sb] = x[1]; dst[2 * p.out_sb] = x[2]; dst[3 * p.out_sb] = x[3]; }
              } else {
                // a group that crosses the end of a tile row or of the image: element by element
                int tw_e = pos[gi] & 0xff, th_e = (pos[gi] >> 8) & 0xff, tn_e = pos[gi] >> 16;
                const int q = c0 + j;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  if (q + e < p.rows_valid) {
                    const int ne = t.pn0 + tn_e, ae = t.pa0 + th_e, be = t.pb0 + tw_e;
                    if (ne < p.NL && ae < p.AH && be < p.AW) {
                      float* de = obase + (int64_t)ne * p.out_sn + (int64_t)ae * p.out_sa + (int64_t)be * p.out_sb;
                      *de = p.accumulate ? __fadd_rn(*de, x[e]) : x[e];
                    }
                  }
                  if (++tw_e >= p.tw) { tw_e = 0; if (++th_e >= p.th) { th_e = 0; ++tn_e; } }
                }
              }
            }
          }
          __syncwarp();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
        continue;
      }
      bool row_ok;
      int64_t row_off;
      int64_t col_stride = 1;
      int col0 = 0, col_limit = 0;
      if (MODE == MODE_GEMM) {
        const int64_t m = (int64_t)t.m0 + r;
        row_ok = m < p.M;
        row_off = (int64_t)t.bz * p.batch_stride_c + m * p.ldc;
        col0 = t.n0; col_limit = (int)min((int64_t)p.bn, p.N - t.n0);
      } else if (MODE == MODE_CONV) {
        const int hw = p.th * p.tw;
        const int tn_i = r / hw;
        const int rem = r - tn_i * hw;
        const int th_i = rem / p.tw;
        const int tw_i = rem - th_i * p.tw;
        const int n = t.pn0 + tn_i, a = t.pa0 + th_i, b = t.pb0 + tw_i;
        row_ok = r < p.rows_valid && n < p.NL && a < p.AH && b < p.AW;
        row_off = p.out_base + (int64_t)n * p.out_sn + (int64_t)a * p.out_sa + (int64_t)b * p.out_sb;
        col_stride = p.out_sc;
        col0 = t.n0; col_limit = min(p.bn, p.OC - t.n0);
      } else {
        row_ok = true;
        row_off = (int64_t)t.split * p.part_stride_split +
                  ((int64_t)t.oc_t * 128 + r) * p.part_ld + (int64_t)t.nb0 * (p.swz_b / p.esz);
        col0 = 0; col_limit = t.nblk * (p.swz_b / p.esz);
      }
      float* outp = p.out + row_off;
      const bool vec_ok = (MODE != MODE_CONV) && ((((uintptr_t)outp) & 15) == 0);
      for (int c0 = half * 32; c0 < p.bn; c0 += 64) {
        uint32_t v[32];
        if (t.num_kb > 0) {
          tmem_ld32(d_tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0u;
        }
        if (scaled) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(sc(__uint_as_float(v[j])));
        }
        if (!row_ok || LNN_DBG(p, 4)) {
          // nothing to store for this lane (experiment bit 2: no stores)
        } else if (MODE == MODE_DW) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            if (c0 + j < col_limit) {
              float4 q = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                     __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
              *reinterpret_cast<float4*>(outp + c0 + j) = q;
            }
          }
        } else if (MODE == MODE_GEMM && vec_ok && (c0 + 32) <= col_limit) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            float x[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float tt = __uint_as_float(v[j + e]);
              if (p.bias) tt = __fadd_rn(tt, __ldg(p.bias + col0 + c0 + j + e));
              x[e] = apply_act(tt, p.act, p.alpha);
            }
            float4* dst = reinterpret_cast<float4*>(outp + col0 + c0 + j);
            if (p.accumulate) {
              const float4 o = *dst;
              x[0] = __fadd_rn(o.x, x[0]); x[1] = __fadd_rn(o.y, x[1]);
              x[2] = __fadd_rn(o.z, x[2]); x[3] = __fadd_rn(o.w, x[3]);
            }
            *dst = make_float4(x[0], x[1], x[2], x[3]);
          }
        } else {
          // "+=": all old values are loaded before the first store (the compiler cannot reorder a
          // load past a store through the same pointer with a run-time stride)
          float oldv[32];
          if (p.accumulate) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              oldv[j] = (c0 + j < col_limit) ? outp[(int64_t)(col0 + c0 + j) * col_stride] : 0.0f;
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (c0 + j < col_limit) {
              float tt = __uint_as_float(v[j]);
              if (p.bias) tt = __fadd_rn(tt, __ldg(p.bias + col0 + c0 + j));
              tt = apply_act(tt, p.act, p.alpha);
              float* dst = outp + (int64_t)(col0 + c0 + j) * col_stride;
              if (p.accumulate) tt = __fadd_rn(oldv[j], tt);
              *dst = tt;
            }
          }
        }
        __syncwarp();   // reconverge before the next warp-collective TMEM load
      }
      // this warp no longer needs the accumulator: let the MMA warp reuse it
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
    }
    __syncwarp();
    if (p.ep_mode == 4) warp_amax_commit(amax_acc, p.amax_out);
  }

  // ---- tear-down ------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // copies issued before the abort may still be landing in this CTA's shared memory
    const long long t0 = clock64();
    while (clock64() - t0 < kAbortDelay) { }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2u * p.tmem_cols);
  }
}

// =========================================================================================
// unit-stride convolution with a halo-resident pixel patch
// =========================================================================================
// tc_kernel reloads the pixel patch for every tap, so a 3x3 convolution pulls nine copies of
// it from L2 into shared memory and the operand ring, not the tensor pipe, sets the pace.
// Here the patch of one 32-channel block is loaded ONCE per tile, halo included, as a flat
// array of pixels: (th + halo) rows of h_pw pixels, 128 bytes per pixel, 128-byte swizzle.
// Accumulator column n = h * h_pw + w stands for output pixel (h, w) of the tile; tap
// (dy, dx) needs patch pixel n + dy' * h_pw + dx', i.e. the SAME array read from a start
// address shifted by tap_shift rows, which a shared-memory descriptor can express.  Columns
// with w >= tw are computed and thrown away (they wrap into the next patch row).
// Channels sit on M (kernel tile = operand A, one unit per tap), pixels on N.
//   warp 0 : kernel-unit producer      warp 1 : MMA issuer, TMEM owner
//   warp 6 : patch producer            warps 2-5 : epilogue
constexpr int kThreadsHalo = 32 * (kEpilogueWarps + 3);   // two producers, the MMA warp, the epilogue warps

__global__ void __launch_bounds__(kThreadsHalo, 1)
tc_halo_kernel(const __grid_constant__ CUtensorMap tmAh, const __grid_constant__ CUtensorMap tmAl,
               const __grid_constant__ CUtensorMap tmBh, const __grid_constant__ CUtensorMap tmBl,
               const __grid_constant__ TcParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t a_full_bar[8];
  __shared__ uint64_t a_empty_bar[8];
  __shared__ uint64_t b_full_bar[4];
  __shared__ uint64_t b_empty_bar[4];
  __shared__ uint64_t tmem_full_bar[2];
  __shared__ uint64_t tmem_empty_bar[2];
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag_smem;

  if (threadIdx.x == 0) abort_flag_smem = (*(volatile int*)p.status != 0) ? 2 : 0;
  __syncthreads();
  if (abort_flag_smem == 2) return;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &abort_flag_smem;

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t ring = (raw + 1023u) & ~1023u;
  const int nbuf = p.passes == 1 ? 1 : 2;
  const uint32_t a_sz = (uint32_t)p.a_tile_bytes;            // 1024-byte multiples
  const uint32_t b_sz = (uint32_t)p.h_bbuf;
  const uint32_t a_unit = nbuf * a_sz, b_stage = nbuf * b_sz;
  const uint32_t a_ring = ring, b_ring = ring + (uint32_t)p.h_sa * a_unit;
  const int num_tiles = p.grid_x * p.grid_y;
  const int a_per_cb = p.cb / p.h_acb;                       // kernel units per (tap, channel block)
  const uint32_t row_bytes = (uint32_t)(p.cb * p.esz);        // one pixel of the patch

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.h_sa; ++s) {
      mbar_init(smem_u32(&a_full_bar[s]), 1);
      mbar_init(smem_u32(&a_empty_bar[s]), 1);
    }
    for (int s = 0; s < p.h_sb; ++s) {
      mbar_init(smem_u32(&b_full_bar[s]), 1);
      mbar_init(smem_u32(&b_empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&tmem_full_bar[a]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[a]), kEpilogueWarps);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_smem), 2u * p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;
  const uint32_t afull0 = smem_u32(&a_full_bar[0]), aempty0 = smem_u32(&a_empty_bar[0]);
  const uint32_t bfull0 = smem_u32(&b_full_bar[0]), bempty0 = smem_u32(&b_empty_bar[0]);

  if (warp == 2 + kEpilogueWarps) {
    // ---- patch producer -----------------------------------------------------------------
    if (lane == 0) {
      const uint32_t tx = (uint32_t)nbuf * (uint32_t)(p.h_pw * p.h_ph) * row_bytes;
      uint32_t s = 0, ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        const TileCoord t = decode_tile<MODE_CONVT>(p, tile);
        for (int cbi = 0; cbi < p.ncb; ++cbi) {
          if (!mbar_wait(bempty0 + 8u * s, ph ^ 1u, abort_flag, p.status, 4, cbi)) { ok = false; break; }
          const uint32_t fb = bfull0 + 8u * s;
          mbar_expect_tx(fb, tx);
          const uint32_t dst = b_ring + s * b_stage;
          tma_load_4d(dst, &tmBh, fb, cbi * p.cb, t.pb0 + p.h_x0, t.pa0 + p.h_y0, t.pn0);
          if (nbuf == 2) tma_load_4d(dst + b_sz, &tmBl, fb, cbi * p.cb, t.pb0 + p.h_x0, t.pa0 + p.h_y0, t.pn0);
          if (++s == (uint32_t)p.h_sb) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else if (warp == 0) {
    // ---- kernel-unit producer -----------------------------------------------------------
    if (lane == 0) {
      const uint32_t tx = (uint32_t)nbuf * (uint32_t)p.a_load_bytes;
      uint32_t s = 0, ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        const TileCoord t = decode_tile<MODE_CONVT>(p, tile);
        for (int cbi = 0; ok && cbi < p.ncb; ++cbi) {
          for (int tp = 0; ok && tp < p.ntaps; ++tp) {
            for (int h = 0; h < a_per_cb; ++h) {
              if (!mbar_wait(aempty0 + 8u * s, ph ^ 1u, abort_flag, p.status, 0, tp)) { ok = false; break; }
              const uint32_t fb = afull0 + 8u * s;
              if (LNN_DBG(p, 2)) { mbar_arrive(fb); }
              else {
                mbar_expect_tx(fb, tx);
                const uint32_t dst = a_ring + s * a_unit;
                const int c0 = cbi * p.cb + h * p.h_acb;
                tma_load_3d(dst, &tmAh, fb, c0, t.m0, p.tap_w[tp]);
                if (nbuf == 2) tma_load_3d(dst + a_sz, &tmAl, fb, c0, t.m0, p.tap_w[tp]);
              }
              if (++s == (uint32_t)p.h_sa) { s = 0; ph ^= 1u; }
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer -----------------------------------------------------------------------
    if (lane == 0) {
      const uint32_t a_swz = (uint32_t)(p.h_acb * p.esz);
      const uint64_t a_desc0 = make_smem_desc(0u, 16u, 8u * a_swz, layout_of_swizzle((int)a_swz));
      const uint64_t b_desc0 = make_smem_desc(0u, 16u, 8u * row_bytes, layout_of_swizzle((int)row_bytes));
      const uint64_t a_lo16 = a_sz >> 4, b_lo16 = b_sz >> 4;
      const int ksteps = LNN_DBG(p, 1) ? 0 : (int)(a_swz / 32u);   // one instruction = 32 bytes of K
      const uint32_t idesc = p.idesc;
      uint32_t sa = 0, pha = 0, sb = 0, phb = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_ph = (uint32_t)(it >> 1) & 1u;
        if (!mbar_wait(smem_u32(&tmem_empty_bar[acc]), acc_ph ^ 1u, abort_flag, p.status, 3, it)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)acc * p.tmem_cols;
        uint32_t accum = 0u;
        for (int cbi = 0; ok && cbi < p.ncb; ++cbi) {
          if (!mbar_wait(bfull0 + 8u * sb, phb, abort_flag, p.status, 5, cbi)) { ok = false; break; }
          tc_fence_after();
          const uint32_t b_base = b_ring + sb * b_stage;
          for (int tp = 0; ok && tp < p.ntaps; ++tp) {
            // the tap's window of the patch: same array, start address shifted by whole pixels
            const uint32_t b_addr = b_base + (LNN_DBG(p, 8) ? 0u : (uint32_t)p.tap_shift[tp] * row_bytes);
            // the swizzle is a function of the absolute shared-memory address, so a start address
            // that is not a multiple of the 1024-byte pattern needs no base-offset field
            const uint64_t bdesc = b_desc0 + (uint64_t)(b_addr >> 4);
            for (int h = 0; h < a_per_cb; ++h) {
              if (!mbar_wait(afull0 + 8u * sa, pha, abort_flag, p.status, 1, tp)) { ok = false; break; }
              tc_fence_after();
              const uint64_t ah = a_desc0 + (uint64_t)((a_ring + sa * a_unit) >> 4);
              const uint64_t bh = bdesc + (uint64_t)((h * p.h_acb * p.esz) >> 4);
              // one MMA step = 32 bytes of channels = 2 descriptor units
              issue_unit(p.esz, nbuf, ksteps, d_tmem, ah, bh, 2, 2, a_lo16, b_lo16, idesc, accum);
              if (ksteps > 0) accum = 1u;
              umma_commit(aempty0 + 8u * sa);
              if (++sa == (uint32_t)p.h_sa) { sa = 0; pha ^= 1u; }
            }
          }
          if (ok) umma_commit(bempty0 + 8u * sb);
          if (++sb == (uint32_t)p.h_sb) { sb = 0; phb ^= 1u; }
        }
        if (ok) umma_commit(smem_u32(&tmem_full_bar[acc]));
      }
    }
  } else {
    // ---- epilogue: lane = output channel, columns = flattened patch positions ---------------
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;                 // the two warps of a quarter alternate over the chunks
    const int r = quarter * 32 + lane;
    const int ncols = p.th * p.h_pw;                  // columns that can hold a real pixel
    const bool scaled = p.esz == 2;
    const Pow2Scale sc(scaled ? exp_of_amax(__ldg(p.amax_a)) + exp_of_amax(__ldg(p.amax_b)) : 0);
    uint32_t amax_acc = 0u;
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      const TileCoord t = decode_tile<MODE_CONVT>(p, tile);
      const int acc = it & 1;
      const uint32_t acc_ph = (uint32_t)(it >> 1) & 1u;
      bool have_acc = mbar_wait(smem_u32(&tmem_full_bar[acc]), acc_ph, abort_flag, p.status, 2, it);
      have_acc = __all_sync(0xffffffffu, have_acc);
      if (!have_acc) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + (uint32_t)acc * p.tmem_cols;
      const int oc = t.m0 + r;
      const bool row_ok = oc < p.OC;
      const float bias_v = (row_ok && p.bias) ? __ldg(p.bias + oc) : 0.0f;
      if (p.ep_mode != 0) {
        // fused max pool: th even, tw a multiple of 32; the row below column c is column c + h_pw
        int turn = 0;
        for (int h_i = 0; h_i < p.th; h_i += 2) {
          for (int w0 = 0; w0 < p.tw; w0 += 32) {
            if (((turn++) & 1) != half) continue;
            const int c_top = h_i * p.h_pw + w0;
            uint32_t v0[32], v1[32];
            tmem_ld32(d_tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c_top, v0);
            tmem_ld32(d_tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c_top + p.h_pw), v1);
            tmem_ld_wait();
            const int a = t.pa0 + h_i, b0 = t.pb0 + w0;
            if (a < p.AH && b0 < p.AW && !LNN_DBG(p, 4))
              pooled_store(p, sc, v0, v1, bias_v, oc, t.pn0, a, b0, 32, amax_acc);
            __syncwarp();
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
        continue;
      }
      float* const obase = p.out + p.out_base + (int64_t)oc * p.out_sc + (int64_t)t.pn0 * p.out_sn;
      for (int c0 = half * 32; c0 < ncols; c0 += 64) {
        int h_i = c0 / p.h_pw, w_i = c0 - h_i * p.h_pw;      // position of the current group of four
        uint32_t v[32];
        tmem_ld32(d_tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
        tmem_ld_wait();
        if (row_ok) {
          // Phase 1: destinations and (for "+=") old values of the eight groups, all loads first
          float* dsts[8];
          int wpos[8];                                  // column inside the tile, or -1: nothing to store
          uint32_t vec_mask = 0;
          float4 old[8];
#pragma unroll
          for (int gi = 0; gi < 8; ++gi) {
            const int a = t.pa0 + h_i, b = t.pb0 + w_i;
            wpos[gi] = -1;
            old[gi] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c0 + gi * 4 < ncols && w_i < p.tw && a < p.AH && b < p.AW && !LNN_DBG(p, 4)) {
              wpos[gi] = w_i;
              float* dst = obase + (int64_t)a * p.out_sa + (int64_t)b * p.out_sb;
              dsts[gi] = dst;
              const bool four = (w_i + 3 < p.tw) && (b + 3 < p.AW);
              const bool vec = four && p.out_sb == 1 && ((((uintptr_t)dst) & 15) == 0);
              if (vec) vec_mask |= 1u << gi;
              if (p.accumulate) {
                if (vec) old[gi] = *reinterpret_cast<const float4*>(dst);
                else {
                  old[gi].x = dst[0];
                  if (w_i + 1 < p.tw && b + 1 < p.AW) old[gi].y = dst[p.out_sb];
                  if (w_i + 2 < p.tw && b + 2 < p.AW) old[gi].z = dst[2 * p.out_sb];
                  if (w_i + 3 < p.tw && b + 3 < p.AW) old[gi].w = dst[3 * p.out_sb];
                }
              }
            }
            w_i += 4;
            if (w_i >= p.h_pw) { w_i = 0; ++h_i; }
          }
          // Phase 2: bias, activation, add, store
#pragma unroll
          for (int gi = 0; gi < 8; ++gi) {
            if (wpos[gi] < 0) continue;
            const int j = gi * 4;
            float x[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float tt = __uint_as_float(v[j + e]);
              if (scaled) tt = sc(tt);
              if (p.bias) tt = __fadd_rn(tt, bias_v);
              x[e] = apply_act(tt, p.act, p.alpha);
            }
            if (p.accumulate) {
              x[0] = __fadd_rn(old[gi].x, x[0]); x[1] = __fadd_rn(old[gi].y, x[1]);
              x[2] = __fadd_rn(old[gi].z, x[2]); x[3] = __fadd_rn(old[gi].w, x[3]);
            }
            float* dst = dsts[gi];
            if (vec_mask & (1u << gi)) {
              *reinterpret_cast<float4*>(dst) = make_float4(x[0], x[1], x[2], x[3]);
            } else {
              const int w0 = wpos[gi];
              const int b = t.pb0 + w0;
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (w0 + e < p.tw && b + e < p.AW) dst[(int64_t)e * p.out_sb] = x[e];
            }
          }
        }
        __syncwarp();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
    }
    __syncwarp();
    if (p.ep_mode == 4) warp_amax_commit(amax_acc, p.amax_out);
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < kAbortDelay) { }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2u * p.tmem_cols);
  }
}

// =========================================================================================
// operand preparation (HBM-bound)
// =========================================================================================
constexpr int kThreads = 256;

// Largest magnitude of a tensor as an fp32 bit pattern (*out must be zero before the launch).
__global__ void __launch_bounds__(kThreads)
absmax_kernel(const float* __restrict__ src, int64_t n, uint32_t* __restrict__ out) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  uint32_t m = 0u;
  if ((((uintptr_t)src) & 15) == 0) {
    const int64_t n4 = n >> 2;
    for (int64_t i = tid; i < n4; i += nthreads) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(src) + i);
      m = max(max(m, v.x & 0x7fffffffu), max(v.y & 0x7fffffffu, max(v.z & 0x7fffffffu, v.w & 0x7fffffffu)));
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += nthreads) m = max(m, __float_as_uint(src[i]) & 0x7fffffffu);
  } else {
    for (int64_t i = tid; i < n; i += nthreads) m = max(m, __float_as_uint(src[i]) & 0x7fffffffu);
  }
  warp_amax_commit(m, out);
}

// Upper bound of |act(conv2D(x, W) + bias)|: amax(x) * max over oc of sum |W[oc]| + max |bias|, times
// max(1, |alpha|) for leaky_relu, with a 2^-6 margin for the roundings on the way.  A result that is
// packed with the scale of this bound cannot overflow fp16, so the epilogue can write the split
// fp16 operand of the next layer itself instead of an fp32 tensor that a second pass would have to
// measure and split.  The bound exceeds the true maximum by a few bits, which only moves the
// 18-binade window of full relative precision; the absolute error floor of the format (2^-40 of
// the scale) stays far below an fp32 rounding of the tensor's large elements.
// out[0] = bound (bit pattern), out[1] = 0 (the epilogue accumulates the true maximum there).
__global__ void __launch_bounds__(1024)
conv_bound_kernel(uint32_t* __restrict__ out, const float* __restrict__ W, int oc, int per_oc,
                  const float* __restrict__ bias, const uint32_t* __restrict__ amax_x, int act, float alpha) {
  __shared__ float red_w[32], red_b[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  float best = 0.0f, bm = 0.0f;
  for (int o = warp; o < oc; o += nwarps) {          // one warp per output channel, coalesced
    const float* w = W + (int64_t)o * per_oc;
    float s = 0.0f;
    for (int k = lane; k < per_oc; k += 32) s += fabsf(__ldg(w + k));
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) s += __shfl_xor_sync(0xffffffffu, s, sh);
    best = fmaxf(best, s);
  }
  if (bias)
    for (int o = threadIdx.x; o < oc; o += blockDim.x) bm = fmaxf(bm, fabsf(__ldg(bias + o)));
#pragma unroll
  for (int sh = 16; sh > 0; sh >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, sh));
  if (lane == 0) { red_w[warp] = best; red_b[warp] = bm; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float wnorm = 0.0f, bmax = 0.0f;
    for (int i = 0; i < nwarps; ++i) { wnorm = fmaxf(wnorm, red_w[i]); bmax = fmaxf(bmax, red_b[i]); }
    const uint32_t ax_bits = amax_x[1] != 0u ? amax_x[1] : amax_x[0];
    float b = __uint_as_float(ax_bits) * wnorm + bmax;
    if (act) b *= fmaxf(1.0f, fabsf(alpha));
    b *= 1.015625f;       // covers the rounding of the sums above and of the accumulation itself
    // a non-finite bound (non-finite input, weights or bias) means "no scaling", like a measured one
    out[0] = __float_as_uint(b);
    out[1] = 0u;
  }
}

// Window position (0..3 in row-major order, 4 = none) of the first element equal to the pooled
// value, for max_pool2D(2, 2, 'same') of Y [planes][ih][iw] into P [planes][oh][ow]: where the
// pooling gradient goes (pool2D.py:147-230).  Used when the pool did not run in an epilogue.
__global__ void __launch_bounds__(kThreads)
pool2x2_argmax_kernel(uint8_t* __restrict__ idx, const float* __restrict__ Y, const float* __restrict__ P,
                      int64_t total, int ih, int iw, int oh, int ow) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t gid = tid; gid < total; gid += nthreads) {
    const int x = (int)(gid % ow);
    const int64_t t = gid / ow;
    const int y = (int)(t % oh);
    const int64_t plane = t / oh;
    const float o = P[gid];
    const float* src = Y + (plane * ih + 2 * y) * (int64_t)iw + 2 * x;
    const bool right = 2 * x + 1 < iw, below = 2 * y + 1 < ih;
    int w = 4;
    if (src[0] == o) w = 0;
    else if (right && src[1] == o) w = 1;
    else if (below && src[iw] == o) w = 2;
    else if (right && below && src[iw + 1] == o) w = 3;
    idx[gid] = (uint8_t)w;
  }
}

// What a split pass needs per thread: the tf32 split needs nothing, the fp16 split the two
// factors of 2^-e with e the scale exponent of the tensor.
template <bool F16> struct Splitter;
template <> struct Splitter<false> {
  typedef float T;
  __device__ __forceinline__ explicit Splitter(const uint32_t*) {}
  __device__ __forceinline__ void operator()(float x, float& h, float& l) const { split1(x, h, l); }
  static __device__ __forceinline__ float zero() { return 0.0f; }
};
template <> struct Splitter<true> {
  typedef __half T;
  Pow2Scale sc;
  __device__ __forceinline__ explicit Splitter(const uint32_t* amax) : sc(-exp_of_amax(__ldg(amax))) {}
  __device__ __forceinline__ void operator()(float x, __half& h, __half& l) const { split_half(sc(x), h, l); }
  static __device__ __forceinline__ __half zero() { return __float2half_rn(0.0f); }
};
// N consecutive elements as one vector store (N * sizeof(T) = 8 or 16 bytes)
template <class T, int N> __device__ __forceinline__ void store_vec(T* dst, const T* v, bool streaming) {
  if (sizeof(T) * N == 16) {
    const float4 q = *reinterpret_cast<const float4*>(v);
    if (streaming) __stcs(reinterpret_cast<float4*>(dst), q); else *reinterpret_cast<float4*>(dst) = q;
  } else {
    const float2 q = *reinterpret_cast<const float2*>(v);
    if (streaming) __stcs(reinterpret_cast<float2*>(dst), q); else *reinterpret_cast<float2*>(dst) = q;
  }
}

// NCHW -> channel-innermost hi/lo copies, 128-bit on both sides: a tile of 32 channels x 128
// pixels is read as float4 along the pixels and written as 16-byte vectors along the channels (the
// row pitch of 129 floats makes the transposed shared-memory reads conflict-free).  Needs
// hw % 4 == 0 and 16-byte aligned buffers; cp is a multiple of 8.
template <bool F16>
__global__ void __launch_bounds__(256)
nchw_to_nhwc_split_vec_kernel(typename Splitter<F16>::T* __restrict__ hi, typename Splitter<F16>::T* __restrict__ lo,
                              const float* __restrict__ src, int64_t n, int c, int64_t hw, int cp,
                              int want_lo, const uint32_t* __restrict__ amax) {
  typedef typename Splitter<F16>::T T;
  constexpr int CV = F16 ? 8 : 4;                    // channels per 16-byte store
  const Splitter<F16> split(amax);
  __shared__ float tile[32][129];
  const int64_t tiles_p = (hw + 127) / 128;
  const int tiles_c = (cp + 31) / 32;
  const int64_t total = n * tiles_p * tiles_c;
  for (int64_t t = blockIdx.x; t < total; t += gridDim.x) {
    const int tc = (int)(t % tiles_c);
    const int64_t t2 = t / tiles_c;
    const int64_t tp = t2 % tiles_p;
    const int64_t img = t2 / tiles_p;
    const float* sp = src + img * (int64_t)c * hw;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int idx = threadIdx.x + k * 256;
      const int chl = idx >> 5, p4 = idx & 31;
      const int ch = tc * 32 + chl;
      const int64_t px = tp * 128 + p4 * 4;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (ch < c && px < hw) v = __ldcs(reinterpret_cast<const float4*>(sp + (int64_t)ch * hw + px));
      tile[chl][p4 * 4 + 0] = v.x; tile[chl][p4 * 4 + 1] = v.y;
      tile[chl][p4 * 4 + 2] = v.z; tile[chl][p4 * 4 + 3] = v.w;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4 * 4 / CV; ++k) {
      const int item = threadIdx.x + k * 256;
      const int cq = item & (32 / CV - 1), pl = item / (32 / CV);
      const int64_t px = tp * 128 + pl;
      const int ch = tc * 32 + cq * CV;
      if (px < hw && ch < cp) {
        __align__(16) T h[CV];
        __align__(16) T l[CV];
#pragma unroll
        for (int e = 0; e < CV; ++e) split(tile[cq * CV + e][pl], h[e], l[e]);
        const int64_t o = (img * hw + px) * cp + ch;
        store_vec<T, CV>(hi + o, h, true);
        if (want_lo) store_vec<T, CV>(lo + o, l, true);
      }
    }
    __syncthreads();
  }
}

// hi/lo split of a dense [rows][cols] matrix into buffers of row pitch `pitch`
template <bool F16>
__global__ void __launch_bounds__(kThreads)
split_rows_kernel(typename Splitter<F16>::T* __restrict__ hi, typename Splitter<F16>::T* __restrict__ lo,
                  const float* __restrict__ src, int64_t rows, int64_t cols, int64_t pitch, int want_lo,
                  const uint32_t* __restrict__ amax) {
  typedef typename Splitter<F16>::T T;
  const Splitter<F16> split(amax);
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  if (pitch == cols && (cols & 3) == 0 && (((uintptr_t)src) & 15) == 0) {
    const int64_t n4 = rows * cols / 4;
    for (int64_t i = tid; i < n4; i += nthreads) {
      const float4 v = __ldcs(reinterpret_cast<const float4*>(src) + i);
      __align__(16) T h[4];
      __align__(16) T l[4];
      split(v.x, h[0], l[0]); split(v.y, h[1], l[1]); split(v.z, h[2], l[2]); split(v.w, h[3], l[3]);
      store_vec<T, 4>(hi + 4 * i, h, false);
      if (want_lo) store_vec<T, 4>(lo + 4 * i, l, false);
    }
  } else {
    const int64_t n = rows * pitch;
    for (int64_t i = tid; i < n; i += nthreads) {
      const int64_t r = i / pitch, c = i - r * pitch;
      T h = Splitter<F16>::zero(), l = Splitter<F16>::zero();
      if (c < cols) split(src[r * cols + c], h, l);
      hi[i] = h;
      if (want_lo) lo[i] = l;
    }
  }
}

// fp32 channel-innermost tensor -> its fp16 hi/lo copies (same layout), element by element
__global__ void __launch_bounds__(kThreads)
half_split_kernel(__half* __restrict__ hi, __half* __restrict__ lo, const float* __restrict__ src,
                  int64_t n8, const uint32_t* __restrict__ amax) {
  const Splitter<true> split(amax);
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = tid; i < n8; i += nthreads) {
    const float4 a = __ldcs(reinterpret_cast<const float4*>(src) + 2 * i);
    const float4 b = __ldcs(reinterpret_cast<const float4*>(src) + 2 * i + 1);
    __align__(16) __half h[8];
    __align__(16) __half l[8];
    split(a.x, h[0], l[0]); split(a.y, h[1], l[1]); split(a.z, h[2], l[2]); split(a.w, h[3], l[3]);
    split(b.x, h[4], l[4]); split(b.y, h[5], l[5]); split(b.z, h[6], l[6]); split(b.w, h[7], l[7]);
    store_vec<__half, 8>(hi + 8 * i, h, false);
    store_vec<__half, 8>(lo + 8 * i, l, false);
  }
}

// Gradient of max_pool2D(2, 2) + leaky_relu written straight into the packed fp16 operand format.
// Pass 1 (pooled size): T = the gradient that reaches the winner of each window,
// 0 + (0 + dP) then 0 + that * leaky_relu'(P) -- the roundings of the un-fused kernels
// (pool2D.py:147-230, element_wise_op.py:207-221) -- or 0 where no position matched, and its
// largest magnitude, which is the largest magnitude of the whole full-resolution gradient.
__device__ __forceinline__ float winner_grad_of(float g, float o, uint8_t w, float alpha, int act) {
  float u = __fadd_rn(0.0f, __fadd_rn(0.0f, g));
  if (act) {
    const float f = __fadd_rn(o >= 0.0f ? 1.0f : 0.0f, __fmul_rn(alpha, o < 0.0f ? 1.0f : 0.0f));
    u = __fadd_rn(0.0f, __fmul_rn(u, f));
  }
  return w > 3 ? 0.0f : u;
}

// VEC: four elements per thread with 128-bit loads (total % 4 == 0, 16-byte aligned buffers)
template <bool VEC>
__global__ void __launch_bounds__(kThreads)
pool_winner_grad_kernel(float* __restrict__ T, uint32_t* __restrict__ amax, const uint8_t* __restrict__ IDX,
                        const float* __restrict__ dP, const float* __restrict__ P, int64_t total, float alpha,
                        int act) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  uint32_t best = 0u;
  if (VEC) {
    for (int64_t i = tid; i < (total >> 2); i += nthreads) {
      const float4 g = __ldcs(reinterpret_cast<const float4*>(dP) + i);
      const float4 o = __ldg(reinterpret_cast<const float4*>(P) + i);
      const uchar4 w = __ldg(reinterpret_cast<const uchar4*>(IDX) + i);
      float4 u;
      u.x = winner_grad_of(g.x, o.x, w.x, alpha, act); u.y = winner_grad_of(g.y, o.y, w.y, alpha, act);
      u.z = winner_grad_of(g.z, o.z, w.z, alpha, act); u.w = winner_grad_of(g.w, o.w, w.w, alpha, act);
      reinterpret_cast<float4*>(T)[i] = u;
      best = max(max(best, __float_as_uint(u.x) & 0x7fffffffu), __float_as_uint(u.y) & 0x7fffffffu);
      best = max(max(best, __float_as_uint(u.z) & 0x7fffffffu), __float_as_uint(u.w) & 0x7fffffffu);
    }
  } else {
    for (int64_t i = tid; i < total; i += nthreads) {
      const float u = winner_grad_of(dP[i], P[i], IDX[i], alpha, act);
      T[i] = u;
      best = max(best, __float_as_uint(u) & 0x7fffffffu);
    }
  }
  if (amax) warp_amax_commit(best, amax);
}

// Pass 2: one thread = two adjacent windows x eight channels; consecutive threads take consecutive
// channel groups of the same pixels, so the 16-byte stores of a warp are contiguous.  hi / lo are
// [n][2*oh][2*ow][cp]; T and IDX are NCHW planes of [oh][ow].  Every element is written (zeros
// outside the winners and in the pad channels).
// (four blocks per SM: 64 registers and a few spilled bytes beat 78 registers at three blocks,
// 0.50 against 0.54 ms on 1024 x 64 x 64x64)
__global__ void __launch_bounds__(kThreads, 4)
unpool_packed_kernel(__half* __restrict__ hi, __half* __restrict__ lo, const float* __restrict__ T,
                     const uint8_t* __restrict__ IDX, const uint32_t* __restrict__ amax, int64_t n, int c, int cp,
                     int oh, int ow) {
  const Splitter<true> split(amax);
  const int cgs = cp >> 3, ow2 = ow >> 1;
  const int64_t total = n * oh * (int64_t)ow2 * cgs;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  const int64_t plane = (int64_t)oh * ow;
  for (int64_t gid = tid; gid < total; gid += nthreads) {
    const int cg = (int)(gid % cgs);
    int64_t r = gid / cgs;
    const int x2 = (int)(r % ow2); r /= ow2;
    const int y = (int)(r % oh);
    const int64_t img = r / oh;
    // the eight channels of both windows first (hi / lo of the winner's gradient and its position),
    // then one 16-byte vector per pixel: few values live at a time keeps four blocks on an SM
    __half th[8][2], tl[8][2];
    uint8_t wp[8][2];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int ch = cg * 8 + k;
      float2 t = make_float2(0.0f, 0.0f);
      uchar2 w = make_uchar2(4, 4);
      if (ch < c) {
        const int64_t off = (img * c + ch) * plane + (int64_t)y * ow + 2 * x2;
        t = *reinterpret_cast<const float2*>(T + off);
        w = *reinterpret_cast<const uchar2*>(IDX + off);
      }
      split(t.x, th[k][0], tl[k][0]);
      split(t.y, th[k][1], tl[k][1]);
      wp[k][0] = w.x; wp[k][1] = w.y;
    }
    const __half z = Splitter<true>::zero();
    const int64_t iw = 2 * (int64_t)ow;
#pragma unroll
    for (int row = 0; row < 2; ++row) {
#pragma unroll
      for (int col = 0; col < 4; ++col) {
        const int win = col >> 1, pos = row * 2 + (col & 1);
        __align__(16) __half hv[8];
        __align__(16) __half lv[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const bool hit = wp[k][win] == pos;
          hv[k] = hit ? th[k][win] : z;
          lv[k] = hit ? tl[k][win] : z;
        }
        const int64_t px = (img * 2 * oh + 2 * y + row) * iw + 4 * x2 + col;
        store_vec<__half, 8>(hi + px * cp + cg * 8, hv, true);
        store_vec<__half, 8>(lo + px * cp + cg * 8, lv, true);
      }
    }
  }
}

// NCHW -> NHWC with channel padding to cp, split into hi/lo.  One block transposes a
// [32 channels] x [32 pixels] tile of one image through shared memory.
template <bool F16>
__global__ void __launch_bounds__(256)
nchw_to_nhwc_split_kernel(typename Splitter<F16>::T* __restrict__ hi, typename Splitter<F16>::T* __restrict__ lo,
                          const float* __restrict__ src, int64_t n, int c, int64_t hw, int cp,
                          int want_lo, const uint32_t* __restrict__ amax) {
  typedef typename Splitter<F16>::T T;
  const Splitter<F16> split(amax);
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t tiles_p = (hw + 31) / 32;
  const int tiles_c = (cp + 31) / 32;
  const int64_t total = n * tiles_p * tiles_c;
  for (int64_t t = blockIdx.x; t < total; t += gridDim.x) {
    const int tc = (int)(t % tiles_c);
    const int64_t t2 = t / tiles_c;
    const int64_t tp = t2 % tiles_p;
    const int64_t img = t2 / tiles_p;
    const float* sp = src + img * (int64_t)c * hw;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int ch = tc * 32 + ty + k * 8;
      const int64_t px = tp * 32 + tx;
      tile[ty + k * 8][tx] = (ch < c && px < hw) ? sp[(int64_t)ch * hw + px] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int64_t px = tp * 32 + ty + k * 8;
      const int ch = tc * 32 + tx;
      if (px < hw && ch < cp) {
        T h, l;
        split(tile[tx][ty + k * 8], h, l);
        const int64_t o = (img * hw + px) * cp + ch;
        hi[o] = h;
        if (want_lo) lo[o] = l;
      }
    }
    __syncthreads();
  }
}

// NCHW -> NHWC for c <= 8 channels padded to exactly 8: thread = pixel.
template <bool F16>
__global__ void __launch_bounds__(kThreads)
nchw_to_nhwc8_split_kernel(typename Splitter<F16>::T* __restrict__ hi, typename Splitter<F16>::T* __restrict__ lo,
                           const float* __restrict__ src, int64_t n, int c, int64_t hw, int want_lo,
                           const uint32_t* __restrict__ amax) {
  typedef typename Splitter<F16>::T T;
  constexpr int CV = F16 ? 8 : 4;
  const Splitter<F16> split(amax);
  const int64_t total = n * hw;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = tid; i < total; i += nthreads) {
    const int64_t img = i / hw, px = i - img * hw;
    const float* sp = src + img * (int64_t)c * hw + px;
    __align__(16) T h[8];
    __align__(16) T l[8];
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) {
      h[ch] = Splitter<F16>::zero(); l[ch] = Splitter<F16>::zero();
      if (ch < c) split(__ldcs(sp + (int64_t)ch * hw), h[ch], l[ch]);
    }
#pragma unroll
    for (int q = 0; q < 8; q += CV) {
      store_vec<T, CV>(hi + i * 8 + q, h + q, false);
      if (want_lo) store_vec<T, CV>(lo + i * 8 + q, l + q, false);
    }
  }
}

// Kernel OIHW -> [tap][rows][kp] hi/lo.  transpose_io = 0: rows = oc, k = ic (forward);
// 1: rows = ic, k = oc (input gradient).  k is zero-padded to kp.
template <bool F16>
__global__ void __launch_bounds__(kThreads)
weight_split_kernel(typename Splitter<F16>::T* __restrict__ hi, typename Splitter<F16>::T* __restrict__ lo,
                    const float* __restrict__ w, int oc, int ic, int taps, int kp, int transpose_io,
                    int want_lo, const uint32_t* __restrict__ amax) {
  typedef typename Splitter<F16>::T T;
  const Splitter<F16> split(amax);
  const int rows = transpose_io ? ic : oc;
  const int64_t total = (int64_t)taps * rows * kp;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  const int kvalid = transpose_io ? oc : ic;
  for (int64_t i = tid; i < total; i += nthreads) {
    const int k = (int)(i % kp);
    const int64_t t2 = i / kp;
    const int row = (int)(t2 % rows);
    const int t = (int)(t2 / rows);
    T h = Splitter<F16>::zero(), l = Splitter<F16>::zero();
    if (k < kvalid) {
      const int o = transpose_io ? k : row;
      const int c = transpose_io ? row : k;
      split(w[((int64_t)o * ic + c) * taps + t], h, l);
    }
    hi[i] = h;
    if (want_lo) lo[i] = l;
  }
}

// dW[oc][ic][tap] += sum over splits of P[split][oc][(tap, ic block, eb)], splits added in order
__global__ void __launch_bounds__(kThreads)
dw_finalize_kernel(float* __restrict__ dW, const float* __restrict__ P, int oc, int ic, int taps,
                   int splits, int64_t stride_split, int icb, int64_t ld, int eb, int swapped) {
  const int64_t total = (int64_t)oc * ic * taps;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = tid; i < total; i += nthreads) {
    const int t = (int)(i % taps);
    const int64_t t2 = i / taps;
    const int c = (int)(t2 % ic);
    const int o = (int)(t2 / ic);
    const float* pp = P + (int64_t)o * ld + ((int64_t)t * icb + c / eb) * eb + c % eb;
    float s = 0.0f;
    for (int k = 0; k < splits; ++k) s = __fadd_rn(s, pp[(int64_t)k * stride_split]);
    const int64_t dst = swapped ? ((int64_t)c * oc + o) * taps + t : i;     // [ic][oc][tap] or [oc][ic][tap]
    dW[dst] = __fadd_rn(dW[dst], s);
  }
}

// =========================================================================================
// host side
// =========================================================================================
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int get_encode() {
  if (g_encode) return LNN_OK;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  LNN_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
  if (!fn || qres != cudaDriverEntryPointSuccess)
    return lnn::set_error(LNN_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  g_encode = (EncodeTiledFn)fn;
  return LNN_OK;
}

// dims/box/estr have `rank` entries, innermost first; strides_bytes has rank-1 entries.
// esz = 2: fp16 elements, 4: fp32 (tf32) elements
int encode_map(CUtensorMap* tm, const void* base, int esz, int rank, const uint64_t* dims,
               const uint64_t* strides_bytes, const uint32_t* box, const uint32_t* estr,
               int swz_bytes, bool mn_major = false) {
  int rc = get_encode();
  if (rc) return rc;
  cuuint64_t gd[5], gs[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) { gd[i] = dims[i]; bx[i] = box[i]; es[i] = estr[i]; }
  for (int i = 0; i + 1 < rank; ++i) gs[i] = strides_bytes[i];
  for (int i = 0; i < rank; ++i)
    if (bx[i] < 1 || bx[i] > 256)
      return lnn::set_error(LNN_E_UNSUPPORTED, "TMA box extent %u (dim %d) outside 1..256", bx[i], i);
  // MN-major tf32 operands use the 128-byte swizzle whose atom is 32 bytes; fp16 operands use
  // the ordinary swizzles in either orientation
  const CUtensorMapSwizzle sw = (mn_major && esz == 4) ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                              : swz_bytes == 128       ? CU_TENSOR_MAP_SWIZZLE_128B
                              : swz_bytes == 64        ? CU_TENSOR_MAP_SWIZZLE_64B
                                                       : CU_TENSOR_MAP_SWIZZLE_32B;
  CUresult r = g_encode(tm, esz == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                        (cuuint32_t)rank, (void*)base, gd, gs,
                        bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return lnn::set_error(LNN_E_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return LNN_OK;
}

inline int grid_for(const lnn::Device* d, int64_t work_items) {
  int64_t blocks = lnn_ceil_div(work_items, kThreads);
  int64_t cap = (int64_t)d->sm_count * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

inline int env_int(const char* name, int dflt) {
  const char* e = getenv(name);
  return (e && *e) ? atoi(e) : dflt;
}

// Planner overrides for A/B measurements, read from the environment once per process.
struct Knobs {
  int halo, orient, kgroup, stages, cb, bn, direct, fewch, debug;
  Knobs() {
    halo = env_int("LNN_TC_HALO", 1);          // 0 off, 1 planner's rule, 2 whenever a tiling fits
    orient = env_int("LNN_TC_ORIENT", 0);      // 1 pixels on M, 2 channels on M
    kgroup = env_int("LNN_TC_KGROUP", 0);
    stages = env_int("LNN_TC_STAGES", 0);
    cb = env_int("LNN_TC_CB", 0);
    bn = env_int("LNN_TC_BN", 0);
    direct = env_int("LNN_CONV_DIRECT", 1);
    fewch = env_int("LNN_CONV_FEWCH", 1);      // 0: layers with <= 4 input channels stay on the FP32 pipe
#ifdef LNN_TC_EXPERIMENTS
    debug = env_int("LNN_TC_DEBUG", 0);
#else
    debug = 0;
#endif
  }
};
inline const Knobs& knobs() {
  static const Knobs k;
  return k;
}

// precision (the `tf32_passes` argument of the entry points): 1 = plain TF32, 3 = split TF32,
// 2 = split FP16
inline int esz_of(int precision) { return precision == 2 ? 2 : 4; }

inline uint32_t make_idesc(int bn, int a_major, int b_major, int esz) {
  // c_format F32 (bits 4-5 = 1), a/b format (F16 = 0, TF32 = 2) at bits 7-9 / 10-12, majors at
  // 15 / 16, N >> 3 at bits 17-22, M >> 4 at bits 24-28.
  const uint32_t fmt = esz == 2 ? 0u : 2u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)a_major << 15) |
         ((uint32_t)b_major << 16) | ((uint32_t)(bn >> 3) << 17) | ((128u >> 4) << 24);
}

inline uint32_t tmem_cols_for(int bn) {
  uint32_t c = 32;
  while ((int)c < bn) c <<= 1;
  return c;
}

constexpr int kSmemLimit = 227 * 1024;
constexpr int kSmemSlack = 2048;   // alignment slack + static barriers

template <int MODE>
int launch_tc(lnn::Device* d, dim3 grid, const CUtensorMap& ah, const CUtensorMap& al,
              const CUtensorMap& bh, const CUtensorMap& bl, TcParams& p) {
  const int nbuf = p.passes == 1 ? 1 : 2;
  const int a_sz = (p.a_tile_bytes + 1023) & ~1023;
  const int b_sz = (p.b_tile_bytes + 1023) & ~1023;
  const int unit = nbuf * (a_sz + b_sz);
  // several small units share one stage so that a barrier round trip covers enough MMAs
  int kgroup = knobs().kgroup;
  if (kgroup <= 0) kgroup = std::max(1, std::min(p.num_kb, (72 * 1024) / unit));
  if (MODE == MODE_DW) kgroup = 1;
  const int stage = kgroup * unit;
  p.kgroup = kgroup;
  int stages = knobs().stages;
  if (stages <= 0) {
    stages = (kSmemLimit - kSmemSlack) / stage;
    if (stages > 6) stages = 6;
  }
  if (stages > 8) stages = 8;
  if (stages < 1 || stages * stage + kSmemSlack > kSmemLimit)
    return lnn::set_error(LNN_E_UNSUPPORTED, "operand stage of %d bytes does not fit shared memory", stage);
  p.stages = stages;
  p.debug = knobs().debug;
  p.status = d->status_dev;
  // persistent launch: the logical grid is walked by one CTA per SM
  p.grid_x = (int)grid.x; p.grid_y = (int)grid.y; p.grid_z = (int)grid.z;
  const int64_t num_tiles = (int64_t)grid.x * grid.y * grid.z;
  if (num_tiles >= (1ll << 31)) return lnn::set_error(LNN_E_UNSUPPORTED, "too many tiles");
  const unsigned ctas = (unsigned)std::min<int64_t>(num_tiles, d->sm_count);
  const int smem = stages * stage + 1024;
  // the opt-in to more than 48 KB of dynamic shared memory is a per-device property of the kernel
  if (!(d->smem_attr_done & (1u << MODE))) {
    LNN_CUDA(cudaFuncSetAttribute(tc_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  kSmemLimit - 1024));
    d->smem_attr_done |= 1u << MODE;
  }
  {
    lnn::ProfScope prof(d, MODE == MODE_CONVT ? (int)LNN_PROF_TC_CONV : MODE);   // slots follow the modes
    tc_kernel<MODE><<<ctas, kThreadsTc, smem, d->stream>>>(ah, al, bh, bl, p);
  }
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

int check_passes(int precision) {
  LNN_REQUIRE(precision >= 1 && precision <= 3,
              "precision must be 1 (TF32), 2 (split FP16) or 3 (split TF32)");
  return LNN_OK;
}

// Largest magnitude of `count` floats into *amax (zeroed first, on the stream).
int launch_absmax(lnn::Device* d, uint32_t* amax, const float* src, int64_t count) {
  // word 0: the magnitude that defines the scale; word 1: the measured largest magnitude when
  // word 0 is only an upper bound (0 = "the same as word 0")
  LNN_CUDA(cudaMemsetAsync(amax, 0, 2 * sizeof(uint32_t), d->stream));
  absmax_kernel<<<grid_for(d, count / 4 + 1), kThreads, 0, d->stream>>>(src, count, amax);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

// A packed fp16 operand keeps the fp32 bit pattern of its tensor's largest magnitude in a
// 16-byte trailer behind the hi copy.
inline uint64_t half_trailer_offset(uint64_t elems) { return (elems * 2 + 15) & ~15ull; }
inline uint64_t packed_hi_bytes(uint64_t elems, int precision) {
  return precision == 2 ? half_trailer_offset(elems) + 16 : elems * 4;
}
inline uint64_t packed_lo_bytes(uint64_t elems, int precision) {
  return precision == 1 ? 0 : elems * (uint64_t)esz_of(precision);
}
inline uint32_t* trailer_of(const void* hi, uint64_t elems) {
  return (uint32_t*)((uint8_t*)hi + half_trailer_offset(elems));
}

// One operand of a contraction: hi / lo copies and, for the fp16 split, the largest magnitude.
struct Operand {
  const void* hi = nullptr; const void* lo = nullptr; const uint32_t* amax = nullptr;
};

// Split a dense [rows][cols] matrix (per batch entry) into hi/lo scratch with padded pitch
// (in elements; rows start on 16-byte boundaries).
int split_matrix(lnn::Device* d, lnn::Scratch& hi, lnn::Scratch& lo, Operand* op, const float* src,
                 int64_t rows, int64_t cols, int64_t* pitch_out, int precision) {
  const int esz = esz_of(precision);
  const int want_lo = precision != 1;
  const int64_t align = 16 / esz;
  const int64_t pitch = (cols + align - 1) / align * align;
  const uint64_t elems = (uint64_t)rows * pitch;
  int rc = hi.get(packed_hi_bytes(elems, precision));
  if (rc) return rc;
  if (want_lo) { rc = lo.get(packed_lo_bytes(elems, precision)); if (rc) return rc; }
  lnn::ProfScope prof(d, LNN_PROF_PREP);
  if (esz == 2) {
    uint32_t* amax = trailer_of(hi.p, elems);
    rc = launch_absmax(d, amax, src, rows * cols);
    if (rc) return rc;
    split_rows_kernel<true><<<grid_for(d, rows * pitch / 4 + 1), kThreads, 0, d->stream>>>(
        hi.as<__half>(), lo.as<__half>(), src, rows, cols, pitch, 1, amax);
    op->amax = amax;
  } else {
    split_rows_kernel<false><<<grid_for(d, rows * pitch / 4 + 1), kThreads, 0, d->stream>>>(
        hi.as<float>(), want_lo ? lo.as<float>() : nullptr, src, rows, cols, pitch, want_lo, nullptr);
  }
  LNN_CHECK_LAUNCH(d);
  op->hi = hi.p; op->lo = want_lo ? lo.p : hi.p;
  *pitch_out = pitch;
  return LNN_OK;
}

// Geometry of the pixel tiling used by the convolution passes.
struct PixTile { int tw, th, tn, tiles_b, tiles_a, tiles_n; };

// rows of a CONV tile: up to 128 logical output pixels as tn x th x tw
PixTile plan_conv_tile(int NL, int AH, int AW, int es, int maxpix) {
  PixTile t;
  const int wcap = std::min(maxpix, 256 / es);
  if (AW >= wcap) { t.tw = wcap; t.th = 1; t.tn = 1; }
  else {
    t.tw = AW;
    int hmax = std::min(std::min(AH, maxpix / t.tw), 256 / es);
    if (hmax < 1) hmax = 1;
    // pick th <= hmax minimising padded rows over the image height
    int best = 1; double best_eff = 0;
    for (int th = 1; th <= hmax; ++th) {
      const int tiles = (AH + th - 1) / th;
      const double eff = (double)AH / (tiles * th) * (double)(th * t.tw) / (double)maxpix;
      if (eff > best_eff + 1e-9) { best_eff = eff; best = th; }
    }
    t.th = best;
    t.tn = 1;
    if (t.th == AH) t.tn = std::max(1, std::min(NL, maxpix / (t.tw * t.th)));
  }
  t.tiles_b = (AW + t.tw - 1) / t.tw;
  t.tiles_a = (AH + t.th - 1) / t.th;
  t.tiles_n = (NL + t.tn - 1) / t.tn;
  return t;
}

int gcd_int(int a, int b) { while (b) { int t = a % b; a = b; b = t; } return a; }
int chan_pad(int c) { return (c + 7) & ~7; }
// channels per unit: one swizzle row of 128, 64 or 32 bytes (a block wider than the padded
// channel count is zero-filled by the TMA unit)
int chan_block(int cp, int esz) {
  const int full = 128 / esz;
  return (cp % full == 0) ? full : ((cp % (full / 2) == 0) ? full / 2 : full / 4);
}

// 4-D map over an NHWC activation copy [N][H][W][cp]
int encode_nhwc(CUtensorMap* tm, const void* base, int esz, int n, int h, int w, int cp, int box_c,
                int box_w, int box_h, int box_n, int estride, bool mn_major = false) {
  uint64_t dims[4] = {(uint64_t)cp, (uint64_t)w, (uint64_t)h, (uint64_t)n};
  uint64_t str[3] = {(uint64_t)cp * esz, (uint64_t)w * cp * esz, (uint64_t)h * w * cp * esz};
  uint32_t box[4] = {(uint32_t)box_c, (uint32_t)(box_w * estride), (uint32_t)(box_h * estride),
                     (uint32_t)box_n};
  uint32_t es[4] = {1, (uint32_t)estride, (uint32_t)estride, 1};
  return encode_map(tm, base, esz, 4, dims, str, box, es, box_c * esz, mn_major);
}

// NCHW -> channel-innermost hi (and lo when lo_p is given) copies with channel pitch cp.  For the
// fp16 split `amax` receives the tensor's largest magnitude first (a second read of the source).
int nhwc_split_to(lnn::Device* d, void* hi_p, void* lo_p, uint32_t* amax, const float* src, int n, int c,
                  int h, int w, int cp, int precision) {
  const int want_lo = lo_p != nullptr;
  const bool f16 = precision == 2;
  const int64_t hw = (int64_t)h * w;
  lnn::ProfScope prof(d, LNN_PROF_PREP);
  if (f16) {
    LNN_REQUIRE(amax && lo_p, "the fp16 split needs a lo buffer and a word for the largest magnitude");
    const int rc = launch_absmax(d, amax, src, (int64_t)n * c * hw);
    if (rc) return rc;
  }
  if (cp == 8) {
    // few channels (the network's first layer): one thread per pixel, channel planes read
    // coalesced, one NHWC pixel written per thread
    if (f16)
      nchw_to_nhwc8_split_kernel<true><<<grid_for(d, (int64_t)n * hw), kThreads, 0, d->stream>>>(
          (__half*)hi_p, (__half*)lo_p, src, n, c, hw, want_lo, amax);
    else
      nchw_to_nhwc8_split_kernel<false><<<grid_for(d, (int64_t)n * hw), kThreads, 0, d->stream>>>(
          (float*)hi_p, (float*)lo_p, src, n, c, hw, want_lo, nullptr);
    LNN_CHECK_LAUNCH(d);
    return LNN_OK;
  }
  const bool vec = (hw % 4 == 0) && ((((uintptr_t)src | (uintptr_t)hi_p | (uintptr_t)lo_p) & 15) == 0);
  if (vec) {
    const int64_t tiles = (int64_t)n * ((hw + 127) / 128) * ((cp + 31) / 32);
    const int64_t grid = std::min<int64_t>(tiles, (int64_t)d->sm_count * 8);
    if (f16)
      nchw_to_nhwc_split_vec_kernel<true><<<(unsigned)grid, 256, 0, d->stream>>>(
          (__half*)hi_p, (__half*)lo_p, src, n, c, hw, cp, want_lo, amax);
    else
      nchw_to_nhwc_split_vec_kernel<false><<<(unsigned)grid, 256, 0, d->stream>>>(
          (float*)hi_p, (float*)lo_p, src, n, c, hw, cp, want_lo, nullptr);
    LNN_CHECK_LAUNCH(d);
    return LNN_OK;
  }
  const int64_t tiles = (int64_t)n * ((hw + 31) / 32) * ((cp + 31) / 32);
  int64_t grid = std::min<int64_t>(tiles, (int64_t)d->sm_count * 16);
  if (f16)
    nchw_to_nhwc_split_kernel<true><<<(unsigned)grid, 256, 0, d->stream>>>(
        (__half*)hi_p, (__half*)lo_p, src, n, c, hw, cp, want_lo, amax);
  else
    nchw_to_nhwc_split_kernel<false><<<(unsigned)grid, 256, 0, d->stream>>>(
        (float*)hi_p, (float*)lo_p, src, n, c, hw, cp, want_lo, nullptr);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

// Packed copies of an NCHW activation into scratch
int nhwc_split(lnn::Device* d, lnn::Scratch& hi, lnn::Scratch& lo, Operand* op, const float* src, int n,
               int c, int h, int w, int cp, int precision) {
  const uint64_t elems = (uint64_t)n * h * w * cp;
  const int want_lo = precision != 1;
  int rc = hi.get(packed_hi_bytes(elems, precision));
  if (rc) return rc;
  if (want_lo) { rc = lo.get(packed_lo_bytes(elems, precision)); if (rc) return rc; }
  uint32_t* amax = precision == 2 ? trailer_of(hi.p, elems) : nullptr;
  rc = nhwc_split_to(d, hi.p, want_lo ? lo.p : nullptr, amax, src, n, c, h, w, cp, precision);
  if (rc) return rc;
  op->hi = hi.p; op->lo = want_lo ? lo.p : hi.p; op->amax = amax;
  return LNN_OK;
}

// A caller-supplied packed activation (hi / lo copies [n][h][w][cp], see lnn_packed_bytes)
int packed_operand(Operand* op, uint64_t hi, uint64_t lo, uint64_t elems, int precision) {
  LNN_REQUIRE(hi, "null packed buffer");
  LNN_REQUIRE(precision == 1 || lo, "a packed operand needs its lo copy unless precision is 1");
  op->hi = (const void*)(uintptr_t)hi;
  op->lo = precision == 1 ? op->hi : (const void*)(uintptr_t)lo;
  op->amax = precision == 2 ? trailer_of(op->hi, elems) : nullptr;
  return LNN_OK;
}

int weights_split(lnn::Device* d, lnn::Scratch& hi, lnn::Scratch& lo, Operand* op, const float* w, int oc,
                  int ic, int taps, int kp, int transpose_io, int precision) {
  const int rows = transpose_io ? ic : oc;
  const int want_lo = precision != 1;
  const uint64_t elems = (uint64_t)taps * rows * kp;
  int rc = hi.get(packed_hi_bytes(elems, precision));
  if (rc) return rc;
  if (want_lo) { rc = lo.get(packed_lo_bytes(elems, precision)); if (rc) return rc; }
  lnn::ProfScope prof(d, LNN_PROF_PREP);
  if (precision == 2) {
    uint32_t* amax = trailer_of(hi.p, elems);
    rc = launch_absmax(d, amax, w, (int64_t)oc * ic * taps);
    if (rc) return rc;
    weight_split_kernel<true><<<grid_for(d, (int64_t)elems), kThreads, 0, d->stream>>>(
        hi.as<__half>(), lo.as<__half>(), w, oc, ic, taps, kp, transpose_io, 1, amax);
    op->amax = amax;
  } else {
    weight_split_kernel<false><<<grid_for(d, (int64_t)elems), kThreads, 0, d->stream>>>(
        hi.as<float>(), want_lo ? lo.as<float>() : nullptr, w, oc, ic, taps, kp, transpose_io, want_lo, nullptr);
  }
  LNN_CHECK_LAUNCH(d);
  op->hi = hi.p; op->lo = want_lo ? lo.p : hi.p;
  return LNN_OK;
}

int check_geom(const lnn_conv_geom* g) {
  LNN_REQUIRE(g, "geometry is null");
  LNN_REQUIRE(g->n > 0 && g->ic > 0 && g->ih > 0 && g->iw > 0 && g->oc > 0 && g->kh > 0 &&
              g->kw > 0 && g->oh > 0 && g->ow > 0, "bad convolution extents");
  LNN_REQUIRE(g->stride >= 1 && g->stride <= 8 && g->dilation >= 1, "stride must be 1..8, dilation >= 1");
  LNN_REQUIRE(g->kh * g->kw <= kMaxTaps, "kernels larger than %d taps are not supported", kMaxTaps);
  return LNN_OK;
}

// Tiling of the halo-resident kernel: tile = th rows x tw columns of one image, patch =
// (th + hy) x pw pixels with pw = tw + hx rounded up to 4 (so that groups of four columns never
// straddle a patch row).  Two patch stages (hi and lo each) plus at least three kernel units
// must fit shared memory; among the tilings that do, take the one with most real pixels per
// MMA clock under the measured cost of one tcgen05.mma in this kernel, about max(150, 0.7 * N) clocks.
// Optional fused pooling / packed output of the channels-on-M kernels (TcParams::ep_mode).
struct EpiExtra { int ep_mode; float* out_lo; int ocp; uint32_t* amax_out; uint8_t* idx_out = nullptr; };

struct HaloPlan { bool ok; int tw, th, pw, ph, bn, sa, bbuf, acb; double px_per_clk; };

HaloPlan plan_halo(int AH, int AW, int hx, int hy, int a_rows, int nbuf, int cb, int esz, bool pooled) {
  HaloPlan best;
  memset(&best, 0, sizeof(best));
  const int budget = kSmemLimit - kSmemSlack - 1024;
  const int divs[] = {1, 2, 3, 4, 6, 8};
  for (int acb = cb; acb * esz >= 64; acb >>= 1) {
    const int a_unit = nbuf * ((a_rows * acb * esz + 1023) & ~1023);
    const int min_sa = 3;
    for (int di = 0; di < 6; ++di) {
      int tw = (AW + divs[di] - 1) / divs[di];
      tw = pooled ? ((tw + 31) & ~31) : ((tw + 3) & ~3);     // the fused pool works on 32-column chunks
      const int pw = (tw + hx + 3) & ~3;
      if (pw > 256) continue;
      for (int th = 1; th <= AH && th * pw <= 256; ++th) {
        if (pooled && (th & 1)) continue;
        const int bn = std::max(16, (th * pw + 15) & ~15);
        const int ph = th + hy;
        if (bn > 256 || ph > 256) continue;
        const int bbuf = ((bn + hy * pw + hx) * cb * esz + 1023) & ~1023;
        int sa = (budget - 2 * nbuf * bbuf) / a_unit;
        if (sa < min_sa) continue;
        if (sa > 8) sa = 8;
        const double tiles = (double)((AW + tw - 1) / tw) * (double)((AH + th - 1) / th);
        const double cost = std::max(150.0, 0.7 * bn);
        const double ppc = (double)AH * AW / (tiles * cost);
        if (!best.ok || ppc > best.px_per_clk * 1.02) {
          best.ok = true; best.tw = tw; best.th = th; best.pw = pw; best.ph = ph; best.bn = bn;
          best.sa = sa; best.bbuf = bbuf; best.acb = acb; best.px_per_clk = ppc;
        }
      }
    }
  }
  return best;
}

// Everything a convolution-like launch needs besides the operands.
struct ConvLaunch {
  int NL, H, W, kp;                  // activation copy [NL][H][W][kp]
  int wrows, wtaps;                  // kernel copy [wtaps][wrows][kp]
  int AH, AW, es;                    // logical output grid per image, coordinate multiplier
  int ntaps; const int *dy, *dx, *widx;
  int OCv;
  float* out; int64_t out_base, out_sn, out_sa, out_sb, out_sc;
  const float* bias; int act; float alpha; int accumulate;
  int precision;
};

void fill_common(TcParams& p, const ConvLaunch& c, const Operand& act, const Operand& w, bool act_is_b) {
  p.passes = c.precision; p.esz = esz_of(c.precision);
  p.ntaps = c.ntaps;
  p.AW = c.AW; p.AH = c.AH; p.NL = c.NL; p.es = c.es;
  p.out_sn = c.out_sn; p.out_sa = c.out_sa; p.out_sb = c.out_sb; p.out_sc = c.out_sc; p.out_base = c.out_base;
  p.OC = c.OCv;
  p.accumulate = c.accumulate; p.act = c.act; p.alpha = c.alpha; p.bias = c.bias; p.out = c.out;
  p.amax_a = act_is_b ? w.amax : act.amax;
  p.amax_b = act_is_b ? act.amax : w.amax;
  for (int i = 0; i < c.ntaps; ++i) { p.tap_dy[i] = c.dy[i]; p.tap_dx[i] = c.dx[i]; p.tap_w[i] = c.widx[i]; }
}

int encode_weights(CUtensorMap* h, CUtensorMap* l, const Operand& w, const ConvLaunch& c, int box_k, int box_rows) {
  const int esz = esz_of(c.precision);
  uint64_t dims[3] = {(uint64_t)c.kp, (uint64_t)c.wrows, (uint64_t)c.wtaps};
  uint64_t str[2] = {(uint64_t)c.kp * esz, (uint64_t)c.wrows * c.kp * esz};
  uint32_t box[3] = {(uint32_t)box_k, (uint32_t)box_rows, 1};
  uint32_t es1[3] = {1, 1, 1};
  int rc = encode_map(h, w.hi, esz, 3, dims, str, box, es1, box_k * esz);
  if (rc) return rc;
  return encode_map(l, w.lo, esz, 3, dims, str, box, es1, box_k * esz);
}

// Unit-stride convolution through tc_halo_kernel.  Same operands as launch_conv_like with
// es == 1 and one swizzle row of channels per pixel; *taken = 0 (nothing launched, no error)
// when no tiling fits or the planner prefers the per-tap kernel.
int launch_conv_halo(lnn::Device* d, const Operand& act, const Operand& w, const ConvLaunch& c,
                     const EpiExtra* ex, int* taken) {
  *taken = 0;
  const int esz = esz_of(c.precision);
  const int cb = chan_block(c.kp, esz);
  const bool pooled = ex && ex->ep_mode != 0;
  if (pooled && ((c.AH | c.AW) & 1)) return LNN_OK;
  if (c.kp % cb != 0 || cb * esz < 64 || c.ntaps < 1) return LNN_OK;
  int x0 = c.dx[0], x1 = c.dx[0], y0 = c.dy[0], y1 = c.dy[0];
  for (int i = 1; i < c.ntaps; ++i) {
    x0 = std::min(x0, c.dx[i]); x1 = std::max(x1, c.dx[i]);
    y0 = std::min(y0, c.dy[i]); y1 = std::max(y1, c.dy[i]);
  }
  const int hx = x1 - x0, hy = y1 - y0;
  const int nbuf = c.precision == 1 ? 1 : 2;
  const int a_rows = std::min(128, (c.OCv + 7) & ~7);
  const HaloPlan hp = plan_halo(c.AH, c.AW, hx, hy, a_rows, nbuf, cb, esz, pooled);
  // Both kernels turn out to be bound by shared-memory bandwidth (operand reads of the MMAs plus
  // TMA writes, about 90 bytes per clock), so the resident patch only pays where the per-tap
  // kernel is at its worst: one tap per ring stage (a single channel block) or so few output
  // channels that it would put them on N; and only when few accumulator columns are wasted.
  // With the fused pool the tile must be whole rows of 32 pixels and the two halo columns of each
  // row cost accumulator columns (192 real pixels of 256 at best): measured slower than the
  // per-tap kernel on its full 256-pixel tiles (1.05 against 0.73 ms for 1024 x 32->64 @ 64x64).
  if (!hp.ok) return LNN_OK;
  if (pooled && knobs().halo != 2) return LNN_OK;
  // (with 2-byte elements the per-tap kernel in the channels-on-M orientation overtakes the
  // resident patch from 32 output channels up: 0.70 against 0.76 ms on the input gradient of a
  // 32 <- 64 channel layer at 64x64, 512 images)
  const int few_oc = esz == 2 ? 32 : 64;
  if (knobs().halo != 2 && !(hp.px_per_clk >= 1.15 && (c.OCv < few_oc || c.kp == cb))) return LNN_OK;

  TcParams p;
  memset(&p, 0, sizeof(p));
  fill_common(p, c, act, w, true);
  p.mode = MODE_CONVT; p.bn = hp.bn;
  p.swz_a = hp.acb * esz; p.swz_b = cb * esz;
  p.a_tile_bytes = (a_rows * hp.acb * esz + 1023) & ~1023;
  p.a_load_bytes = a_rows * hp.acb * esz;
  p.idesc = make_idesc(hp.bn, 0, 0, esz);
  p.tmem_cols = tmem_cols_for(hp.bn);
  p.ncb = c.kp / cb; p.cb = cb;
  p.tw = hp.tw; p.th = hp.th; p.tn = 1;
  p.tiles_b = (c.AW + hp.tw - 1) / hp.tw; p.tiles_a = (c.AH + hp.th - 1) / hp.th; p.tiles_n = c.NL;
  if (pooled) {
    p.ep_mode = ex->ep_mode; p.out_lo = ex->out_lo; p.ocp = ex->ocp; p.amax_out = ex->amax_out; p.idx_out = ex->idx_out;
  }
  p.h_pw = hp.pw; p.h_ph = hp.ph; p.h_x0 = x0; p.h_y0 = y0; p.h_arows = a_rows; p.h_acb = hp.acb;
  p.h_sa = hp.sa; p.h_sb = 2; p.h_bbuf = hp.bbuf;
  p.debug = knobs().debug;
  for (int i = 0; i < c.ntaps; ++i) p.tap_shift[i] = (c.dy[i] - y0) * hp.pw + (c.dx[i] - x0);
  p.status = d->status_dev;
  CUtensorMap act_h, act_l, w_h, w_l;
  int rc = encode_nhwc(&act_h, act.hi, esz, c.NL, c.H, c.W, c.kp, cb, hp.pw, hp.ph, 1, 1);
  if (rc) return rc;
  rc = encode_nhwc(&act_l, act.lo, esz, c.NL, c.H, c.W, c.kp, cb, hp.pw, hp.ph, 1, 1);
  if (rc) return rc;
  rc = encode_weights(&w_h, &w_l, w, c, hp.acb, a_rows);
  if (rc) return rc;
  const int64_t ptiles = (int64_t)p.tiles_b * p.tiles_a * p.tiles_n;
  const int64_t mtiles = (c.OCv + 127) / 128;
  LNN_REQUIRE(ptiles * mtiles < (1ll << 31), "too many tiles");
  p.grid_x = (int)ptiles; p.grid_y = (int)mtiles; p.grid_z = 1;
  const int smem = p.h_sa * nbuf * p.a_tile_bytes + p.h_sb * nbuf * p.h_bbuf + 1024;
  if (!(d->smem_attr_done & (1u << 8))) {
    LNN_CUDA(cudaFuncSetAttribute(tc_halo_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  kSmemLimit - 1024));
    d->smem_attr_done |= 1u << 8;
  }
  const unsigned ctas = (unsigned)std::min<int64_t>(ptiles * mtiles, d->sm_count);
  {
    lnn::ProfScope prof(d, (int)LNN_PROF_TC_CONV);
    tc_halo_kernel<<<ctas, kThreadsHalo, smem, d->stream>>>(w_h, w_l, act_h, act_l, p);
  }
  LNN_CHECK_LAUNCH(d);
  *taken = 1;
  return LNN_OK;
}

// Shared launcher of the implicit GEMM (forward and input gradient): tap t reads the
// activation at (a*es + dy[t], b*es + dx[t]) for output pixel (a, b) of the logical grid.
int launch_conv_like(lnn::Device* d, const Operand& act, const Operand& w, const ConvLaunch& c,
                     const EpiExtra* ex = nullptr, int* fused = nullptr) {
  // ex (fused pool / packed output) can only be honoured by the channels-on-M kernels with a
  // suitable tiling; *fused tells the caller whether it was (nothing is launched when not)
  const bool pooled = ex && ex->ep_mode != 0;
  const int esz = esz_of(c.precision);
  if (fused) *fused = 0;
  if (c.es == 1 && knobs().halo != 0) {
    int taken = 0;
    const int rc = launch_conv_halo(d, act, w, c, ex, &taken);
    if (rc) return rc;
    if (taken) { if (fused) *fused = 1; return LNN_OK; }
  }
  int cb = chan_block(c.kp, esz);
  {
    const int cb_env = knobs().cb;                       // tuning: channels per unit
    if (cb_env > 0 && cb_env < cb && (cb_env * esz == 32 || cb_env * esz == 64)) cb = cb_env;
  }
  const int swz = cb * esz;
  // Orientation.  A tcgen05.mma costs about max(90, 0.7 * N) clocks whatever M carries, so the
  // wide operand should sit on N: with more than a few output channels the pixel patch (up to
  // 256 pixels) goes on N and the channels on M ("channels on M", MODE_CONVT); with very few
  // output channels the pixels go on M and the channels on N.
  int orient = knobs().orient;
  // (measured: with 64 or more output channels the channels-on-M epilogue -- 128-bit stores along
  // W -- is the faster one whenever the output is unit-stride along W; the strided scatter of a
  // stride-2 input gradient is better served by pixels on M)
  // (a fused pool / packed output exists only in the channels-on-M epilogue)
  // (with 2-byte elements that holds from 32 output channels up, provided there are enough pixels
  // to give every SM a 256-pixel tile; a small problem gets more tiles with 128 pixels on M)
  const bool many_pixels = (int64_t)c.NL * c.AH * c.AW >= (int64_t)d->sm_count * 256;
  const int oc_for_chan_m = (esz == 2 && many_pixels) ? 32 : 64;
  if (orient == 0) orient = (pooled || (c.OCv >= oc_for_chan_m && c.out_sb == 1)) ? 2 : 1;
  const bool chan_m = orient == 2;
  PixTile t = plan_conv_tile(c.NL, c.AH, c.AW, c.es, chan_m ? 256 : 128);
  if (pooled) {
    // 32-column chunks must be pieces of one image row, rows must come in pairs
    if (!chan_m || c.es != 1 || (t.tw & 31) || (t.th & 1) || ((c.AH | c.AW) & 1)) return LNN_OK;
  }
  const int pix = t.tn * t.th * t.tw;
  int bn;
  if (chan_m) {
    bn = std::max(16, (pix + 15) & ~15);
  } else {
    bn = std::min(256, (c.OCv + 15) & ~15);
    const int bn_env = knobs().bn;
    if (bn_env >= 16 && bn_env <= 256 && bn_env % 16 == 0) bn = std::min(bn, bn_env);
  }
  TcParams p;
  memset(&p, 0, sizeof(p));
  fill_common(p, c, act, w, chan_m);
  p.mode = chan_m ? MODE_CONVT : MODE_CONV; p.bn = bn;
  p.a_major = 0; p.b_major = 0; p.swz_a = swz; p.swz_b = swz;
  p.ksteps = swz / 32;
  p.a_tile_bytes = 128 * swz; p.b_tile_bytes = bn * swz;
  p.a_loads = 1; p.b_loads = 1;
  if (chan_m) { p.a_load_bytes = 128 * swz; p.b_load_bytes = pix * swz; }
  else { p.a_load_bytes = pix * swz; p.b_load_bytes = bn * swz; }
  p.idesc = make_idesc(bn, 0, 0, esz);
  p.tmem_cols = tmem_cols_for(bn);
  p.ncb = (c.kp + cb - 1) / cb; p.cb = cb;
  p.num_kb = c.ntaps * p.ncb;
  p.tw = t.tw; p.th = t.th; p.tn = t.tn;
  p.tiles_b = t.tiles_b; p.tiles_a = t.tiles_a; p.tiles_n = t.tiles_n;
  p.rows_valid = pix;
  if (pooled) {
    p.ep_mode = ex->ep_mode; p.out_lo = ex->out_lo; p.ocp = ex->ocp; p.amax_out = ex->amax_out;
    p.idx_out = ex->idx_out;
    if (fused) *fused = 1;
  }
  CUtensorMap act_h, act_l, w_h, w_l;
  int rc = encode_nhwc(&act_h, act.hi, esz, c.NL, c.H, c.W, c.kp, cb, t.tw, t.th, t.tn, c.es);
  if (rc) return rc;
  rc = encode_nhwc(&act_l, act.lo, esz, c.NL, c.H, c.W, c.kp, cb, t.tw, t.th, t.tn, c.es);
  if (rc) return rc;
  rc = encode_weights(&w_h, &w_l, w, c, cb, chan_m ? 128 : bn);
  if (rc) return rc;
  const int64_t ptiles = (int64_t)t.tiles_b * t.tiles_a * t.tiles_n;
  LNN_REQUIRE(ptiles < (1ll << 31), "too many pixel tiles");
  if (chan_m) {
    dim3 grid((unsigned)ptiles, (unsigned)((c.OCv + 127) / 128), 1);
    return launch_tc<MODE_CONVT>(d, grid, w_h, w_l, act_h, act_l, p);
  }
  dim3 grid((unsigned)ptiles, (unsigned)((c.OCv + bn - 1) / bn), 1);
  return launch_tc<MODE_CONV>(d, grid, act_h, act_l, w_h, w_l, p);
}

}  // namespace

extern "C" {

int lnn_gemm_f32(int dev, uint64_t C, uint64_t A, uint64_t B, uint64_t bias, int64_t batch,
                 int64_t m, int64_t n, int64_t k, int trans_a, int trans_b, int accumulate,
                 int tf32_passes) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(C && A && B, "null buffer");
  LNN_REQUIRE(batch >= 1 && m >= 1 && n >= 1 && k >= 1, "bad GEMM extents");
  LNN_REQUIRE(batch < 65536, "batch too large");
  int rc = check_passes(tf32_passes);
  if (rc) return rc;
  const int esz = esz_of(tf32_passes);
  // A is stored [m][k] (K-major) or [k][m] (MN-major); same for B with n.
  const int64_t a_rows = trans_a ? k : m, a_cols = trans_a ? m : k;
  const int64_t b_rows = trans_b ? n : k, b_cols = trans_b ? k : n;
  lnn::Scratch ah(d), al(d), bh(d), bl(d);
  Operand oa, ob;
  int64_t a_pitch, b_pitch;
  rc = split_matrix(d, ah, al, &oa, (const float*)(uintptr_t)A, batch * a_rows, a_cols, &a_pitch, tf32_passes);
  if (rc) return rc;
  rc = split_matrix(d, bh, bl, &ob, (const float*)(uintptr_t)B, batch * b_rows, b_cols, &b_pitch, tf32_passes);
  if (rc) return rc;

  // one unit = one 128-byte swizzle row of K: 32 tf32 or 64 fp16 elements; an MN-major operand
  // is loaded as boxes of one such row along MN by `kunit` k-rows
  const int e128 = 128 / esz;
  int bn = (int)std::min<int64_t>(256, (n + e128 - 1) / e128 * e128);
  const int bn_env = knobs().bn;
  if (bn_env >= e128 && bn_env <= 256 && bn_env % e128 == 0) bn = std::min(bn, bn_env);
  TcParams p;
  memset(&p, 0, sizeof(p));
  p.mode = MODE_GEMM; p.passes = tf32_passes; p.esz = esz; p.bn = bn;
  p.amax_a = oa.amax; p.amax_b = ob.amax;
  p.a_major = trans_a ? 1 : 0;
  p.b_major = trans_b ? 0 : 1;
  p.swz_a = 128; p.swz_b = 128; p.ksteps = 4; p.kunit = e128;
  p.a_tile_bytes = 128 * 128; p.b_tile_bytes = bn * 128;
  if (p.a_major == 0) { p.a_loads = 1; p.a_load_bytes = 128 * 128; }
  else { p.a_loads = 128 / e128; p.a_load_bytes = e128 * 128; p.a_krows = e128; }
  if (p.b_major == 0) { p.b_loads = 1; p.b_load_bytes = bn * 128; }
  else { p.b_loads = bn / e128; p.b_load_bytes = e128 * 128; p.b_krows = e128; }
  p.idesc = make_idesc(bn, p.a_major, p.b_major, esz);
  p.tmem_cols = tmem_cols_for(bn);
  p.num_kb = (int)((k + e128 - 1) / e128);
  p.M = m; p.N = n; p.ldc = n; p.batch_stride_c = m * n;
  p.accumulate = accumulate; p.act = 0; p.alpha = 0.0f;
  p.bias = (const float*)(uintptr_t)bias;
  p.out = (float*)(uintptr_t)C;

  CUtensorMap mah, mal, mbh, mbl;
  {
    // innermost-first dims: (cols, rows, batch)
    uint64_t dims[3] = {(uint64_t)a_cols, (uint64_t)a_rows, (uint64_t)batch};
    uint64_t str[2] = {(uint64_t)a_pitch * esz, (uint64_t)a_rows * a_pitch * esz};
    uint32_t box[3] = {(uint32_t)e128, (uint32_t)(p.a_major ? e128 : 128), 1};
    uint32_t es[3] = {1, 1, 1};
    rc = encode_map(&mah, oa.hi, esz, 3, dims, str, box, es, 128, p.a_major != 0);
    if (rc) return rc;
    rc = encode_map(&mal, oa.lo, esz, 3, dims, str, box, es, 128, p.a_major != 0);
    if (rc) return rc;
  }
  {
    uint64_t dims[3] = {(uint64_t)b_cols, (uint64_t)b_rows, (uint64_t)batch};
    uint64_t str[2] = {(uint64_t)b_pitch * esz, (uint64_t)b_rows * b_pitch * esz};
    uint32_t box[3] = {(uint32_t)e128, (uint32_t)(p.b_major ? e128 : bn), 1};
    uint32_t es[3] = {1, 1, 1};
    rc = encode_map(&mbh, ob.hi, esz, 3, dims, str, box, es, 128, p.b_major != 0);
    if (rc) return rc;
    rc = encode_map(&mbl, ob.lo, esz, 3, dims, str, box, es, 128, p.b_major != 0);
    if (rc) return rc;
  }
  dim3 grid((unsigned)((m + 127) / 128), (unsigned)((n + bn - 1) / bn), (unsigned)batch);
  return launch_tc<MODE_GEMM>(d, grid, mah, mal, mbh, mbl, p);
}

int lnn_pool2d_fwd(int dev, int mode, uint64_t O, uint64_t I, int64_t n, int64_t c, int ih, int iw,
                   int oh, int ow, int pool, int stride, int padl, int padt);

int lnn_packed_bytes(int64_t n, int64_t c, int64_t h, int64_t w, int tf32_passes, uint64_t* hi_bytes,
                     uint64_t* lo_bytes) {
  int rc = check_passes(tf32_passes);
  if (rc) return rc;
  LNN_REQUIRE(n > 0 && c > 0 && h > 0 && w > 0 && hi_bytes && lo_bytes, "bad arguments");
  const uint64_t elems = (uint64_t)n * h * w * chan_pad((int)c);
  *hi_bytes = packed_hi_bytes(elems, tf32_passes);
  *lo_bytes = packed_lo_bytes(elems, tf32_passes);
  return LNN_OK;
}

}  // extern "C"

namespace {

struct FwdOpts {
  uint64_t y_lo = 0, x_lo = 0;
  int pool = 0;          // Y = max_pool2D(act(conv + bias), 2, 2, 'same')
  int in_packed = 0;     // X / x_lo are channel-innermost hi / lo copies [n][ih][iw][chan_pad(ic)]
  int out_packed = 0;    // Y / y_lo receive such copies of the result instead of the NCHW tensor
  int w_swapped = 0;     // W is stored [ic][oc][kh][kw] (the kernel of a transposed convolution)
};

void launch_winner_grad(lnn::Device* d, float* T, uint32_t* amax, const uint8_t* IDX, const float* dP, const float* P,
                        int64_t total, float alpha, int act) {
  const bool vec = (total & 3) == 0 && ((((uintptr_t)T | (uintptr_t)dP | (uintptr_t)P) & 15) == 0) &&
                   (((uintptr_t)IDX & 3) == 0);
  if (vec)
    pool_winner_grad_kernel<true><<<grid_for(d, total / 4), kThreads, 0, d->stream>>>(T, amax, IDX, dP, P, total, alpha, act);
  else
    pool_winner_grad_kernel<false><<<grid_for(d, total), kThreads, 0, d->stream>>>(T, amax, IDX, dP, P, total, alpha, act);
}

// fp32 channel-innermost tensor (its largest magnitude already in the trailer of `hi`) -> fp16 copies
int half_split_packed(lnn::Device* d, void* hi, void* lo, const float* src, uint64_t elems) {
  lnn::ProfScope prof(d, LNN_PROF_PREP);
  half_split_kernel<<<grid_for(d, (int64_t)(elems / 8)), kThreads, 0, d->stream>>>(
      (__half*)hi, (__half*)lo, src, (int64_t)(elems / 8), trailer_of(hi, elems));
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

// conv2D forward with the optional fusions.  Whatever cannot be fused into the convolution's
// epilogue (odd sizes, tilings that do not pair rows, the pixels-on-M orientation) runs as the
// separate pooling / repacking kernels, so every combination of options is always available.
int conv_fwd_impl(int dev, const lnn_conv_geom* g, uint64_t Y, uint64_t X, uint64_t W, uint64_t bias,
                  int act, float alpha, int accumulate, int precision, const FwdOpts& o) {
  LNN_DEV(d, dev);
  int rc = check_geom(g);
  if (rc) return rc;
  rc = check_passes(precision);
  if (rc) return rc;
  LNN_REQUIRE(Y && X && W, "null buffer");
  LNN_REQUIRE(act == 0 || act == 1, "unknown activation %d", act);
  LNN_REQUIRE(!(accumulate && (o.pool || o.out_packed)), "accumulate cannot be combined with pool / packed output");
  const int want_lo = precision != 1;
  const bool f16 = precision == 2;
  LNN_REQUIRE(!o.out_packed || !want_lo || o.y_lo, "packed output needs a lo buffer unless precision is 1");
  const float* biasp = (const float*)(uintptr_t)bias;
  const int oh_p = o.pool ? (g->oh + 1) / 2 : g->oh, ow_p = o.pool ? (g->ow + 1) / 2 : g->ow;
  const int ocp = chan_pad(g->oc);
  const uint64_t out_elems = (uint64_t)g->n * oh_p * ow_p * ocp;   // of a packed result
  float* const y_lo = want_lo ? (float*)(uintptr_t)o.y_lo : nullptr;
  // a pooled NCHW result may come with the map of winning window positions (one byte per element)
  uint8_t* const idx = (o.pool && !o.out_packed) ? (uint8_t*)(uintptr_t)o.y_lo : nullptr;
  auto argmax_of = [&](const float* full) -> int {
    const int64_t total = (int64_t)g->n * g->oc * oh_p * ow_p;
    pool2x2_argmax_kernel<<<grid_for(d, total), kThreads, 0, d->stream>>>(idx, full, (const float*)(uintptr_t)Y, total,
                                                                        g->oh, g->ow, oh_p, ow_p);
    LNN_CHECK_LAUNCH(d);
    return LNN_OK;
  };

  // fp16 packed output written by the epilogue itself: its scale comes from an upper bound of the
  // result (conv_bound_kernel) placed in word 0 of the output's trailer before the launch; the
  // epilogue accumulates the true largest magnitude in word 1 for the next layer's bound
  auto bound_target = [&](const uint32_t* amax_x, uint32_t** amax_true) -> int {
    uint32_t* tr = trailer_of((void*)(uintptr_t)Y, out_elems);
    lnn::ProfScope prof(d, LNN_PROF_PREP);
    conv_bound_kernel<<<1, 1024, 0, d->stream>>>(tr, (const float*)(uintptr_t)W, g->oc, g->ic * g->kh * g->kw, biasp,
                                                amax_x, act, alpha);
    LNN_CHECK_LAUNCH(d);
    *amax_true = tr + 1;
    return LNN_OK;
  };

  if (!o.in_packed && !o.w_swapped && f16 && !accumulate && knobs().fewch && lnn::conv_fewch_applicable(g)) {
    // few input channels, 3x3, unit stride: the tensor-core kernel that builds its own operand
    lnn::Scratch xmax(d), full(d), pooled(d);
    const float* xp = (const float*)(uintptr_t)X;
    const float* wp = (const float*)(uintptr_t)W;
    rc = xmax.get(16);
    if (rc) return rc;
    {
      lnn::ProfScope prof(d, LNN_PROF_PREP);
      rc = launch_absmax(d, xmax.as<uint32_t>(), xp, (int64_t)g->n * g->ic * g->ih * g->iw);
      if (rc) return rc;
    }
    const bool can_pool = o.pool && !((g->oh | g->ow) & 1);     // the fused pool pairs rows and columns
    if (can_pool && o.out_packed) {
      uint32_t* amax_true;
      rc = bound_target(xmax.as<uint32_t>(), &amax_true);
      if (rc) return rc;
      return lnn::conv_fewch_fwd(d, g, (float*)(uintptr_t)Y, xp, wp, biasp, act, alpha, 4, ocp, xmax.as<uint32_t>(),
                                 amax_true, y_lo);
    }
    if (can_pool || (!o.pool && !o.out_packed))
      return lnn::conv_fewch_fwd(d, g, (float*)(uintptr_t)Y, xp, wp, biasp, act, alpha, can_pool ? 1 : 0, ocp,
                                 xmax.as<uint32_t>(), nullptr, nullptr, idx);
    // what the epilogue cannot fuse (odd sizes, packed output without pooling) runs as separate kernels
    rc = full.get((uint64_t)g->n * g->oc * g->oh * g->ow * 4);
    if (rc) return rc;
    rc = lnn::conv_fewch_fwd(d, g, full.as<float>(), xp, wp, biasp, act, alpha, 0, ocp, xmax.as<uint32_t>(), nullptr);
    if (rc) return rc;
    const float* cur = full.as<float>();
    if (o.pool) {
      float* pdst = (float*)(uintptr_t)Y;
      if (o.out_packed) {
        rc = pooled.get((uint64_t)g->n * g->oc * oh_p * ow_p * 4);
        if (rc) return rc;
        pdst = pooled.as<float>();
      }
      rc = lnn_pool2d_fwd(dev, LNN_POOL_MAX, (uint64_t)(uintptr_t)pdst, (uint64_t)(uintptr_t)cur, g->n, g->oc, g->oh,
                          g->ow, oh_p, ow_p, 2, 2, 0, 0);
      if (rc) return rc;
      if (idx) { rc = argmax_of(cur); if (rc) return rc; }
      cur = pdst;
    }
    if (o.out_packed)
      return nhwc_split_to(d, (void*)(uintptr_t)Y, y_lo, trailer_of((void*)(uintptr_t)Y, out_elems), cur, g->n,
                           g->oc, oh_p, ow_p, ocp, precision);
    return LNN_OK;
  }
  if (!o.in_packed && !o.w_swapped && lnn::conv_direct_applicable(g) && knobs().direct &&
      (!o.out_packed || o.pool)) {
    if (idx) {
      // pooled result with the map of winning positions: this kernel's own values (the chain
      // conv2D -> max_pool2D takes it too), pooled and mapped by separate kernels
      lnn::Scratch full(d);
      rc = full.get((uint64_t)g->n * g->oc * g->oh * g->ow * 4);
      if (rc) return rc;
      rc = lnn::conv_direct_fwd(d, g, full.as<float>(), (const float*)(uintptr_t)X, (const float*)(uintptr_t)W,
                                biasp, act, alpha, 0, 0, 0, nullptr, ocp);
      if (rc) return rc;
      rc = lnn_pool2d_fwd(dev, LNN_POOL_MAX, Y, (uint64_t)(uintptr_t)full.as<float>(), g->n, g->oc, g->oh, g->ow,
                          oh_p, ow_p, 2, 2, 0, 0);
      if (rc) return rc;
      return argmax_of(full.as<float>());
    }
    if (o.out_packed && f16) {
      // this kernel writes fp32 and the largest magnitude; one element-wise pass splits it
      lnn::Scratch raw(d);
      rc = raw.get(out_elems * 4);
      if (rc) return rc;
      float* dst = raw.as<float>();
      uint32_t* amax = trailer_of((void*)(uintptr_t)Y, out_elems);
      LNN_CUDA(cudaMemsetAsync(amax, 0, 2 * sizeof(uint32_t), d->stream));
      rc = lnn::conv_direct_fwd(d, g, dst, (const float*)(uintptr_t)X, (const float*)(uintptr_t)W, biasp, act,
                                alpha, 0, o.pool, 2, (float*)amax, ocp);
      if (rc) return rc;
      return half_split_packed(d, (void*)(uintptr_t)Y, y_lo, dst, out_elems);
    }
    return lnn::conv_direct_fwd(d, g, (float*)(uintptr_t)Y, (const float*)(uintptr_t)X,
                                (const float*)(uintptr_t)W, biasp, act, alpha, accumulate, o.pool,
                                o.out_packed ? 1 : 0, y_lo, ocp);
  }

  const int cp = chan_pad(g->ic);
  const int taps = g->kh * g->kw;
  lnn::Scratch xh(d), xl(d), wh(d), wl(d);
  Operand ox, ow;
  if (o.in_packed)
    rc = packed_operand(&ox, X, o.x_lo, (uint64_t)g->n * g->ih * g->iw * cp, precision);
  else
    rc = nhwc_split(d, xh, xl, &ox, (const float*)(uintptr_t)X, g->n, g->ic, g->ih, g->iw, cp, precision);
  if (rc) return rc;
  // rows = output channels, k = input channels; a swapped kernel [ic][oc] is read transposed
  if (o.w_swapped)
    rc = weights_split(d, wh, wl, &ow, (const float*)(uintptr_t)W, g->ic, g->oc, taps, cp, 1, precision);
  else
    rc = weights_split(d, wh, wl, &ow, (const float*)(uintptr_t)W, g->oc, g->ic, taps, cp, 0, precision);
  if (rc) return rc;
  int dy[kMaxTaps], dx[kMaxTaps], wi[kMaxTaps];
  for (int kh = 0; kh < g->kh; ++kh)
    for (int kw = 0; kw < g->kw; ++kw) {
      const int t = kh * g->kw + kw;
      dy[t] = kh * g->dilation - g->padt;
      dx[t] = kw * g->dilation - g->padl;
      wi[t] = t;
    }
  const int64_t plane = (int64_t)g->oh * g->ow;
  ConvLaunch c;
  memset(&c, 0, sizeof(c));
  c.NL = g->n; c.H = g->ih; c.W = g->iw; c.kp = cp; c.wrows = g->oc; c.wtaps = taps;
  c.AH = g->oh; c.AW = g->ow; c.es = g->stride; c.ntaps = taps; c.dy = dy; c.dx = dx; c.widx = wi;
  c.OCv = g->oc; c.bias = biasp; c.act = act; c.alpha = alpha; c.precision = precision;
  if (o.pool && g->stride == 1) {
    // try the fused epilogue: pooled NCHW (ep_mode 1) or pooled, channel-innermost (2: tf32 hi/lo
    // written directly, 4: fp16 hi/lo written directly with the scale of a bound of the result)
    const int64_t pplane = (int64_t)oh_p * ow_p;
    EpiExtra ex{1, nullptr, ocp, nullptr};
    ConvLaunch cf = c;
    cf.es = 1; cf.accumulate = 0; cf.out_base = 0;
    if (o.out_packed) {
      cf.out = (float*)(uintptr_t)Y;
      if (f16) {
        ex.ep_mode = 4; ex.out_lo = y_lo;
        rc = bound_target(ox.amax, &ex.amax_out);
        if (rc) return rc;
      } else {
        ex.ep_mode = 2; ex.out_lo = y_lo;
      }
      cf.out_sn = pplane * ocp; cf.out_sa = (int64_t)ow_p * ocp; cf.out_sb = ocp; cf.out_sc = 1;
    } else {
      cf.out = (float*)(uintptr_t)Y;
      cf.out_sn = (int64_t)g->oc * pplane; cf.out_sa = ow_p; cf.out_sb = 1; cf.out_sc = pplane;
      ex.idx_out = idx;
    }
    int fused = 0;
    rc = launch_conv_like(d, ox, ow, cf, &ex, &fused);
    if (rc) return rc;
    if (fused) return LNN_OK;
  }
  // un-fused: convolution into its NCHW result (scratch when more steps follow)
  lnn::Scratch conv_out(d), pool_out(d);
  float* ydst = (float*)(uintptr_t)Y;
  if (o.pool || o.out_packed) {
    rc = conv_out.get((uint64_t)g->n * g->oc * plane * 4);
    if (rc) return rc;
    ydst = conv_out.as<float>();
  }
  c.out = ydst; c.out_base = 0; c.out_sn = (int64_t)g->oc * plane; c.out_sa = g->ow; c.out_sb = 1; c.out_sc = plane;
  c.accumulate = accumulate;
  rc = launch_conv_like(d, ox, ow, c);
  if (rc) return rc;
  const float* cur = ydst;
  if (o.pool) {
    float* pdst = (float*)(uintptr_t)Y;
    if (o.out_packed) {
      rc = pool_out.get((uint64_t)g->n * g->oc * oh_p * ow_p * 4);
      if (rc) return rc;
      pdst = pool_out.as<float>();
    }
    rc = lnn_pool2d_fwd(dev, LNN_POOL_MAX, (uint64_t)(uintptr_t)pdst, (uint64_t)(uintptr_t)cur, g->n, g->oc,
                        g->oh, g->ow, oh_p, ow_p, 2, 2, 0, 0);
    if (rc) return rc;
    if (idx) { rc = argmax_of(cur); if (rc) return rc; }
    cur = pdst;
  }
  if (o.out_packed)
    return nhwc_split_to(d, (void*)(uintptr_t)Y, y_lo, f16 ? trailer_of((void*)(uintptr_t)Y, out_elems) : nullptr,
                         cur, g->n, g->oc, oh_p, ow_p, ocp, precision);
  return LNN_OK;
}

}  // namespace

extern "C" {

int lnn_conv2d_fwd(int dev, const lnn_conv_geom* g, uint64_t Y, uint64_t X, uint64_t W,
                   uint64_t bias, int act, float alpha, int accumulate, int tf32_passes) {
  return conv_fwd_impl(dev, g, Y, X, W, bias, act, alpha, accumulate, tf32_passes, FwdOpts());
}

int lnn_conv2d_pool_fwd(int dev, const lnn_conv_geom* g, uint64_t Y, uint64_t X, uint64_t W,
                        uint64_t bias, int act, float alpha, int tf32_passes) {
  FwdOpts o;
  o.pool = 1;
  return conv_fwd_impl(dev, g, Y, X, W, bias, act, alpha, 0, tf32_passes, o);
}

int lnn_conv2d_fwd_packed(int dev, const lnn_conv_geom* g, uint64_t Y, uint64_t Y_lo, uint64_t X,
                          uint64_t X_lo, uint64_t W, uint64_t bias, int act, float alpha, int pool,
                          int in_packed, int out_packed, int tf32_passes) {
  FwdOpts o;
  o.y_lo = Y_lo; o.x_lo = X_lo; o.pool = pool; o.in_packed = in_packed; o.out_packed = out_packed;
  return conv_fwd_impl(dev, g, Y, X, W, bias, act, alpha, 0, tf32_passes, o);
}

int lnn_nhwc_split(int dev, uint64_t hi, uint64_t lo, uint64_t X, int n, int c, int h, int w, int tf32_passes) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(hi && X, "null buffer");
  LNN_REQUIRE(n > 0 && c > 0 && h > 0 && w > 0, "bad extents");
  int rc = check_passes(tf32_passes);
  if (rc) return rc;
  LNN_REQUIRE(tf32_passes == 1 || lo, "the lo buffer is required unless precision is 1");
  const int cp = chan_pad(c);
  void* hp = (void*)(uintptr_t)hi;
  return nhwc_split_to(d, hp, tf32_passes == 1 ? nullptr : (void*)(uintptr_t)lo,
                       tf32_passes == 2 ? trailer_of(hp, (uint64_t)n * h * w * cp) : nullptr,
                       (const float*)(uintptr_t)X, n, c, h, w, cp, tf32_passes);
}

int lnn_pool2x2_winner_grad(int dev, uint64_t T, uint64_t IDX, uint64_t P, uint64_t dP, int64_t n, int64_t c,
                            int oh, int ow, float alpha, int act) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(T && IDX && P && dP, "null buffer");
  LNN_REQUIRE(n > 0 && c > 0 && oh > 0 && ow > 0, "bad extents");
  LNN_REQUIRE(act == 0 || act == 1, "unknown activation %d", act);
  const int64_t pooled = n * c * oh * ow;
  launch_winner_grad(d, (float*)(uintptr_t)T, nullptr, (const uint8_t*)(uintptr_t)IDX, (const float*)(uintptr_t)dP,
                     (const float*)(uintptr_t)P, pooled, alpha, act);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

int lnn_conv2d_dw_winners(int dev, const lnn_conv_geom* g, uint64_t dW, uint64_t T, uint64_t IDX, uint64_t X) {
  LNN_DEV(d, dev);
  int rc = check_geom(g);
  if (rc) return rc;
  LNN_REQUIRE(dW && T && IDX && X, "null buffer");
  if (!lnn::conv_dw_winners_applicable(g) || ((T | X) & 15) || (IDX & 3))
    return lnn::set_error(LNN_E_UNSUPPORTED,
                          "the winners form of the kernel gradient needs at most 4 input channels, a 3x3 kernel, unit "
                          "stride, 'same' padding, an even height and a width that is a multiple of 64");
  return lnn::conv_dw_winners(d, g, (float*)(uintptr_t)dW, (const float*)(uintptr_t)T,
                              (const uint8_t*)(uintptr_t)IDX, (const float*)(uintptr_t)X);
}

int lnn_pool2x2_idx_lrelu_bwd_packed(int dev, uint64_t HI, uint64_t LO, uint64_t T, uint64_t IDX, uint64_t P,
                                     uint64_t dP, int64_t n, int64_t c, int ih, int iw, float alpha, int act) {
  LNN_DEV(d, dev);
  LNN_REQUIRE(HI && LO && T && IDX && P && dP, "null buffer");
  LNN_REQUIRE(n > 0 && c > 0 && ih > 0 && iw > 0, "bad extents");
  LNN_REQUIRE(act == 0 || act == 1, "unknown activation %d", act);
  if ((ih & 1) || (iw & 3) || ((HI | LO) & 15) || (T & 7) || (IDX & 1))
    return lnn::set_error(LNN_E_UNSUPPORTED,
                          "fused pooling gradient needs an even height, a width that is a multiple of 4 and aligned buffers");
  const int oh = ih / 2, ow = iw / 2, cp = chan_pad((int)c);
  const int64_t pooled = n * c * oh * ow;
  uint32_t* amax = trailer_of((void*)(uintptr_t)HI, (uint64_t)n * ih * iw * cp);
  lnn::ProfScope prof(d, LNN_PROF_PREP);
  LNN_CUDA(cudaMemsetAsync(amax, 0, 2 * sizeof(uint32_t), d->stream));
  launch_winner_grad(d, (float*)(uintptr_t)T, amax, (const uint8_t*)(uintptr_t)IDX, (const float*)(uintptr_t)dP,
                     (const float*)(uintptr_t)P, pooled, alpha, act);
  LNN_CHECK_LAUNCH(d);
  unpool_packed_kernel<<<grid_for(d, n * oh * (ow / 2) * (cp / 8)), kThreads, 0, d->stream>>>(
      (__half*)(uintptr_t)HI, (__half*)(uintptr_t)LO, (const float*)(uintptr_t)T, (const uint8_t*)(uintptr_t)IDX, amax,
      n, (int)c, cp, oh, ow);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

}  // extern "C"

namespace {

// dX += ...; dY is NCHW (dy_lo == 0, dy_packed == 0) or the packed hi / lo copies
// w_swapped: W is stored [ic][oc][kh][kw].  accumulate = 0: dX is overwritten (every input pixel
// belongs to exactly one residue class; classes no tap reaches are zero-filled).
int conv_dx_impl(int dev, const lnn_conv_geom* g, uint64_t dX, uint64_t dY, uint64_t dY_lo, int dy_packed,
                 uint64_t W, int precision, int w_swapped = 0, int accumulate = 1) {
  LNN_DEV(d, dev);
  int rc = check_geom(g);
  if (rc) return rc;
  rc = check_passes(precision);
  if (rc) return rc;
  LNN_REQUIRE(dX && dY && W, "null buffer");
  const int ocp = chan_pad(g->oc);
  const int taps = g->kh * g->kw;
  const int s = g->stride;
  lnn::Scratch yh(d), yl(d), wh(d), wl(d);
  Operand oy, ow;
  if (dy_packed)
    rc = packed_operand(&oy, dY, dY_lo, (uint64_t)g->n * g->oh * g->ow * ocp, precision);
  else
    rc = nhwc_split(d, yh, yl, &oy, (const float*)(uintptr_t)dY, g->n, g->oc, g->oh, g->ow, ocp, precision);
  if (rc) return rc;
  // rows = input channels, k = output channels
  if (w_swapped)
    rc = weights_split(d, wh, wl, &ow, (const float*)(uintptr_t)W, g->ic, g->oc, taps, ocp, 0, precision);
  else
    rc = weights_split(d, wh, wl, &ow, (const float*)(uintptr_t)W, g->oc, g->ic, taps, ocp, 1, precision);
  if (rc) return rc;
  const int64_t plane = (int64_t)g->ih * g->iw;
  if (!accumulate) {
    // a class without taps (kernel extent smaller than the stride) is never written by a launch
    bool all_reached = true;
    for (int ph = 0; ph < s && all_reached; ++ph)
      for (int pw = 0; pw < s; ++pw) {
        bool any_h = false, any_w = false;
        for (int kh = 0; kh < g->kh; ++kh) any_h |= (((ph + g->padt - kh * g->dilation) % s) + s) % s == 0;
        for (int kw = 0; kw < g->kw; ++kw) any_w |= (((pw + g->padl - kw * g->dilation) % s) + s) % s == 0;
        if (!(any_h && any_w)) { all_reached = false; break; }
      }
    if (!all_reached) {
      LNN_CUDA(cudaMemsetAsync((void*)(uintptr_t)dX, 0, (size_t)g->n * g->ic * plane * 4, d->stream));
      accumulate = 1;
    }
  }
  // One launch per residue class (ih % s, iw % s): within a class every tap that reaches an
  // input pixel does so from output row oh = a + dy with a = (ih - ph) / s.
  for (int ph = 0; ph < s; ++ph)
    for (int pw = 0; pw < s; ++pw) {
      const int AH = (g->ih - ph + s - 1) / s, AW = (g->iw - pw + s - 1) / s;
      if (AH <= 0 || AW <= 0) continue;
      int dy[kMaxTaps], dx[kMaxTaps], wi[kMaxTaps];
      int nt = 0;
      for (int kh = 0; kh < g->kh; ++kh) {
        const int ny = ph + g->padt - kh * g->dilation;
        if (((ny % s) + s) % s != 0) continue;
        for (int kw = 0; kw < g->kw; ++kw) {
          const int nx = pw + g->padl - kw * g->dilation;
          if (((nx % s) + s) % s != 0) continue;
          // exact division (ny, nx are multiples of s, possibly negative)
          dy[nt] = ny / s; dx[nt] = nx / s; wi[nt] = kh * g->kw + kw;
          ++nt;
        }
      }
      if (nt == 0) continue;
      ConvLaunch c;
      memset(&c, 0, sizeof(c));
      c.NL = g->n; c.H = g->oh; c.W = g->ow; c.kp = ocp; c.wrows = g->ic; c.wtaps = taps;
      c.AH = AH; c.AW = AW; c.es = 1; c.ntaps = nt; c.dy = dy; c.dx = dx; c.widx = wi;
      c.OCv = g->ic; c.out = (float*)(uintptr_t)dX; c.out_base = (int64_t)ph * g->iw + pw;
      c.out_sn = (int64_t)g->ic * plane; c.out_sa = (int64_t)s * g->iw; c.out_sb = s; c.out_sc = plane;
      c.accumulate = accumulate; c.precision = precision;
      rc = launch_conv_like(d, oy, ow, c);
      if (rc) return rc;
    }
  return LNN_OK;
}

// dW += ...; dY and X are each NCHW or the packed hi / lo copies
// out_swapped: dW is stored [ic][oc][kh][kw]
int conv_dw_impl(int dev, const lnn_conv_geom* g, uint64_t dW, uint64_t dY, uint64_t dY_lo, int dy_packed,
                 uint64_t X, uint64_t X_lo, int x_packed, int precision, int out_swapped = 0) {
  LNN_DEV(d, dev);
  int rc = check_geom(g);
  if (rc) return rc;
  rc = check_passes(precision);
  if (rc) return rc;
  LNN_REQUIRE(dW && dY && X, "null buffer");
  if (!dy_packed && !x_packed && !out_swapped && lnn::conv_direct_dw_applicable(g) && knobs().direct)
    return lnn::conv_direct_dw(d, g, (float*)(uintptr_t)dW, (const float*)(uintptr_t)dY,
                               (const float*)(uintptr_t)X);
  const int esz = esz_of(precision);
  const int s = g->stride;
  const int cp = chan_pad(g->ic), ocp = chan_pad(g->oc);
  const int taps = g->kh * g->kw;
  lnn::Scratch xh_s(d), xl_s(d), yh_s(d), yl_s(d), part(d);
  Operand ox, oy;
  if (x_packed)
    rc = packed_operand(&ox, X, X_lo, (uint64_t)g->n * g->ih * g->iw * cp, precision);
  else
    rc = nhwc_split(d, xh_s, xl_s, &ox, (const float*)(uintptr_t)X, g->n, g->ic, g->ih, g->iw, cp, precision);
  if (rc) return rc;
  if (dy_packed)
    rc = packed_operand(&oy, dY, dY_lo, (uint64_t)g->n * g->oh * g->ow * ocp, precision);
  else
    rc = nhwc_split(d, yh_s, yl_s, &oy, (const float*)(uintptr_t)dY, g->n, g->oc, g->oh, g->ow, ocp, precision);
  if (rc) return rc;

  // MN-major tiles: one swizzle row of channels wide.  tf32 rows are always 128 bytes (32
  // channels); fp16 rows are 128 or 64 bytes (64 or 32 channels) so that layers with 32
  // channels do not compute 32 columns of zeros.  Channels beyond the padded extent of the
  // NHWC copy are zero-filled by the TMA unit.
  const int ea = 128 / esz;
  const int eb = (esz == 2 && cp <= 32) ? 32 : 128 / esz;
  const int swa = ea * esz, swb = eb * esz;
  // Columns of the accumulator enumerate (tap, channel block) pairs, so one dY patch in
  // shared memory serves every tap; a tile owns up to 256 columns.
  const int icb = (cp + eb - 1) / eb;
  const int nb_total = taps * icb;
  const int nb_max = 256 / eb;
  const int ngroups = (nb_total + nb_max - 1) / nb_max;
  const int nb_group = (nb_total + ngroups - 1) / ngroups;
  int bn = nb_group * eb;
  const int oc_tiles = (g->oc + 127) / 128, ic_tiles = icb;
  // pixel patch = one k-block: tw x th output pixels of one image, a multiple of one
  // instruction's K (8 tf32 / 16 fp16 pixels), sized so that two stages of (128 + bn) x pix
  // elements (x2 for hi/lo) fit shared memory
  const int kq = 32 / esz;
  const int nbuf = precision == 1 ? 1 : 2;
  int pix_cap = ((kSmemLimit - kSmemSlack) / 2) / (nbuf * (128 + bn) * esz);
  pix_cap = std::min(pix_cap / kq * kq, 128);
  const int wcap = std::min(pix_cap, 256 / s);
  LNN_REQUIRE(wcap >= kq, "stride too large for the weight-gradient kernel");
  // Patch = th rows x tw columns of one image with tw*th a multiple of kq (the box may be wider than
  // the image: zero filled).  Among the shapes that fit, take the one that wastes the fewest of
  // its pixels over the whole image (the image width is cut into 1..8 equal pieces), larger first.
  int tw = kq, th = 1;
  {
    // real pixels per clock: a patch of P pixels costs about 480 clocks per instruction K of MMAs
    // (three passes) plus about 1500 clocks per ring hand-over (fitted to measurements)
    double best = -1.0;
    for (int h = 1; h <= 8 && h <= g->oh && h * s <= 256; ++h) {
      const int mult = kq / gcd_int(kq, h);
      for (int k = 1; k <= 8; ++k) {
        int w = (g->ow + k - 1) / k;
        w = ((w + mult - 1) / mult) * mult;
        if (w * h > pix_cap || w * s > 256 || w > wcap) continue;
        const double tiles = (double)((g->ow + w - 1) / w) * (double)((g->oh + h - 1) / h);
        const double score = (double)g->ow * g->oh / (tiles * (480.0 / kq * w * h + 1500.0));
        if (score > best * 1.001) { best = score; tw = w; th = h; }
      }
    }
    LNN_REQUIRE(best > 0, "no pixel patch fits the weight-gradient kernel");
  }
  const int pix = tw * th;
  const int tiles_b = (g->ow + tw - 1) / tw, tiles_a = (g->oh + th - 1) / th, tiles_n = g->n;
  const int64_t patches = (int64_t)tiles_b * tiles_a * tiles_n;
  LNN_REQUIRE(patches < (1ll << 30), "too many pixel patches");
  int64_t want_ctas = (int64_t)d->sm_count * 4;
  int64_t splits = want_ctas / ((int64_t)oc_tiles * ngroups);
  splits = std::max<int64_t>(1, std::min<int64_t>(splits, patches));
  const int pps = (int)((patches + splits - 1) / splits);
  splits = (patches + pps - 1) / pps;    // every split owns at least one patch

  const int64_t part_ld = (int64_t)nb_total * eb;
  const int64_t stride_split = (int64_t)oc_tiles * 128 * part_ld;
  rc = part.get((uint64_t)splits * stride_split * 4);
  if (rc) return rc;

  TcParams p;
  memset(&p, 0, sizeof(p));
  p.mode = MODE_DW; p.passes = precision; p.esz = esz; p.bn = bn;
  p.amax_a = oy.amax; p.amax_b = ox.amax;
  p.a_major = 1; p.b_major = 1; p.swz_a = swa; p.swz_b = swb;
  p.ksteps = pix / kq;
  p.a_loads = 128 / ea; p.b_loads = bn / eb;
  p.a_load_bytes = pix * swa; p.b_load_bytes = pix * swb;
  p.a_tile_bytes = p.a_loads * p.a_load_bytes; p.b_tile_bytes = p.b_loads * p.b_load_bytes;
  p.a_krows = pix; p.b_krows = pix;
  p.idesc = make_idesc(bn, 1, 1, esz);
  p.tmem_cols = tmem_cols_for(bn);
  p.tw = tw; p.th = th; p.tn = 1;
  p.tiles_b = tiles_b; p.tiles_a = tiles_a; p.tiles_n = tiles_n;
  p.es = s;
  p.patches_total = (int)patches; p.patches_per_split = pps; p.num_kb = pps;
  p.part_stride_split = stride_split; p.part_stride_tap = 0; p.part_ld = part_ld;
  p.oc_tiles = oc_tiles; p.ic_tiles = ic_tiles;
  p.nb_total = nb_total; p.nb_group = nb_group;
  p.OC = g->oc; p.ICv = g->ic;
  p.out = part.as<float>();
  for (int kh = 0; kh < g->kh; ++kh)
    for (int kw = 0; kw < g->kw; ++kw) {
      const int t = kh * g->kw + kw;
      p.tap_dy[t] = kh * g->dilation - g->padt;
      p.tap_dx[t] = kw * g->dilation - g->padl;
      p.tap_w[t] = t;
    }
  p.ntaps = taps;
  CUtensorMap mah, mal, mbh, mbl;
  rc = encode_nhwc(&mah, oy.hi, esz, g->n, g->oh, g->ow, ocp, ea, tw, th, 1, 1, true);
  if (rc) return rc;
  rc = encode_nhwc(&mal, oy.lo, esz, g->n, g->oh, g->ow, ocp, ea, tw, th, 1, 1, true);
  if (rc) return rc;
  rc = encode_nhwc(&mbh, ox.hi, esz, g->n, g->ih, g->iw, cp, eb, tw, th, 1, s, true);
  if (rc) return rc;
  rc = encode_nhwc(&mbl, ox.lo, esz, g->n, g->ih, g->iw, cp, eb, tw, th, 1, s, true);
  if (rc) return rc;
  dim3 grid((unsigned)splits, (unsigned)oc_tiles, (unsigned)ngroups);
  rc = launch_tc<MODE_DW>(d, grid, mah, mal, mbh, mbl, p);
  if (rc) return rc;
  dw_finalize_kernel<<<grid_for(d, (int64_t)g->oc * g->ic * taps), kThreads, 0, d->stream>>>(
      (float*)(uintptr_t)dW, part.as<float>(), g->oc, g->ic, taps, (int)splits, stride_split,
      icb, part_ld, eb, out_swapped);
  LNN_CHECK_LAUNCH(d);
  return LNN_OK;
}

}  // namespace

extern "C" {

int lnn_conv2d_dx(int dev, const lnn_conv_geom* g, uint64_t dX, uint64_t dY, uint64_t W,
                  int tf32_passes) {
  return conv_dx_impl(dev, g, dX, dY, 0, 0, W, tf32_passes);
}

int lnn_conv2d_dw(int dev, const lnn_conv_geom* g, uint64_t dW, uint64_t dY, uint64_t X,
                  int tf32_passes) {
  return conv_dw_impl(dev, g, dW, dY, 0, 0, X, 0, 0, tf32_passes);
}

int lnn_conv2d_dx_packed(int dev, const lnn_conv_geom* g, uint64_t dX, uint64_t dY_hi, uint64_t dY_lo,
                         uint64_t W, int tf32_passes) {
  return conv_dx_impl(dev, g, dX, dY_hi, dY_lo, 1, W, tf32_passes);
}

int lnn_conv2d_dw_packed(int dev, const lnn_conv_geom* g, uint64_t dW, uint64_t dY_hi, uint64_t dY_lo,
                         uint64_t X_hi, uint64_t X_lo, int tf32_passes) {
  return conv_dw_impl(dev, g, dW, dY_hi, dY_lo, 1, X_hi, X_lo, 1, tf32_passes);
}

// ---- transposed convolution ---------------------------------------------------------------
// Y[n, OC, OH, OW] = sum over (ic, kh, kw) of X[n, ic, ih, iw] * K[OC, ic, kh, kw] scattered to
// oh = ih*stride + kh*dilation - padt (conv2DTranspose.py:33-35, unfold2D.py:112-138): exactly the
// input gradient of the convolution that maps [n, OC, OH, OW] to [n, ic, ih, iw], with K stored
// [conv ic][conv oc] -- so the three GEMMs of the transposed convolution are the convolution's three
// with the roles swapped, and `g` is the geometry of THAT convolution: g->ic = OC, g->ih/iw = OH/OW,
// g->oc = the transposed convolution's input channels, g->oh/ow = its input size.
int lnn_conv2d_transpose_fwd(int dev, const lnn_conv_geom* g, uint64_t Y, uint64_t X, uint64_t K, int accumulate,
                             int precision) {
  return conv_dx_impl(dev, g, Y, X, 0, 0, K, precision, 1, accumulate);
}
// dX += conv2D(dY, K^T): the forward pass of the underlying convolution (conv2DTranspose.py:37-41)
int lnn_conv2d_transpose_dx(int dev, const lnn_conv_geom* g, uint64_t dX, uint64_t dY, uint64_t K, int precision) {
  FwdOpts o;
  o.w_swapped = 1;
  return conv_fwd_impl(dev, g, dX, dY, K, 0, 0, 0.0f, 1, precision, o);
}
// dK[OC][ic] += the underlying convolution's kernel gradient with dY in the role of its input and
// X in the role of its output gradient, written transposed (conv2DTranspose.py:43-46)
int lnn_conv2d_transpose_dk(int dev, const lnn_conv_geom* g, uint64_t dK, uint64_t dY, uint64_t X, int precision) {
  return conv_dw_impl(dev, g, dK, X, 0, 0, dY, 0, 0, precision, 1);
}

}  // extern "C"
