// tcgen05 / TMEM / TMA tile engine shared by matmul and the three convolution passes.
//
// One persistent CTA per SM (320 threads) walks the 128 x BN output tiles round-robin:
//   warp 0    : TMA producer  -- cp.async.bulk.tensor loads into a ring of smem stages,
//                                running ahead across tile boundaries
//   warp 1    : MMA issuer    -- one elected thread issues tcgen05.mma (kind::f16 or kind::tf32)
//                                into one of two TMEM accumulators, owns the TMEM allocation
//   warps 2-5 : epilogue      -- tcgen05.ld the finished accumulator, scale / bias / activation /
//                                "+=", store -- while the MMA warp fills the other one
// fp32 accuracy comes from a split of every operand into two 11-bit-significand halves by an
// HBM-bound pre-pass; the MMA warp issues hi*hi + hi*lo + lo*hi into the same fp32 accumulator.
//   precision 2 (default): hi = fp16(x / s), lo = fp16(x / s - hi) with s an exact power of two
//       taken from the tensor's largest magnitude (so that |x / s| < 2^15); kind::f16, K = 16 per
//       instruction, 2 bytes per element; the accumulator is multiplied by s_a * s_b on the way out
//   precision 3: hi = rna_tf32(x), lo = rna_tf32(x - hi); kind::tf32, K = 8, 4 bytes per element
//   precision 1: hi only (plain TF32)
// An fp16 and a tf32 value carry the same 11 significant bits, so 2 and 3 split x the same way;
// the fp16 form moves half the bytes and needs half the instructions for the same K.
// Operands may be K-major or MN-major in shared memory (both are native to tcgen05 for these
// types), so no transposes are materialised for the backward GEMMs, and the convolution
// A-tiles are gathered straight from an NHWC copy of the activations by 4-D tiled TMA (zero
// fill outside the image = padding).
//
// Unit-stride convolutions with few input channels per tap use a second kernel
// (tc_halo_kernel) that keeps the pixel patch with its halo resident in shared memory and
// reads every tap through a shifted descriptor.  The channels-on-M kernels can fold a 2x2
// max-pool into the epilogue and write the result in the next convolution's operand format.
//
// Every wait on an mbarrier is bounded: when the budget runs out the role records a
// status word, raises a CTA-wide abort flag and falls through to the common tear-down
// (bounded delay for TMA copies still in flight, TMEM dealloc), so a wrong descriptor
// shows up as LNN_E_TIMEOUT on the host instead of a hung GPU.
#pragma once
#include <cuda.h>
#include "lnn_common.cuh"

namespace lnn_tc {

constexpr int kEpilogueWarps = 8;                 // two per TMEM lane quarter
constexpr int kThreadsTc = 32 * (kEpilogueWarps + 2);   // producer warp, MMA warp, epilogue warps
constexpr int kMaxTaps = 64;
constexpr long long kWaitBudget = 1500000000ll;   // ~0.8 s of SM clocks
constexpr int kAbortDelay = 400000;               // cycles granted to in-flight TMA copies

enum { MODE_GEMM = 0, MODE_CONV = 1, MODE_DW = 2, MODE_CONVT = 3 };

struct TcParams {
  int mode, passes, stages, bn;
  int a_major, b_major;          // 0 = K-major, 1 = MN-major
  int swz_a, swz_b;              // bytes per smem row of the operand tiles (32/64/128)
  int esz;                       // bytes per operand element: 2 (fp16 split) or 4 (tf32)
  int kunit;                     // GEMM: K elements per unit (one 128-byte row)
  int ksteps;                    // MMA steps (32 bytes of K) per k-block
  int a_tile_bytes, b_tile_bytes;// bytes of one (hi or lo) operand tile
  int a_loads, b_loads;          // TMA boxes per operand tile
  int a_load_bytes, b_load_bytes;// bytes per box
  int a_krows, b_krows;          // MN-major: k rows per box (LBO = krows * swz)
  uint32_t idesc;
  uint32_t tmem_cols;
  int num_kb;                    // k-blocks per output tile (GEMM/CONV); patches per split (DW)
  int grid_x, grid_y, grid_z;    // logical tile grid walked by the persistent CTAs
  int debug;                     // timing experiments: 1 no MMA, 2 no TMA loads, 4 no stores, 8 no tap shift
  int kgroup;                    // units (K slabs / tap-channel blocks / patches) per ring stage
  // GEMM
  int64_t M, N;                  // logical output extents
  int64_t ldc, batch_stride_c;
  // CONV / DW tile geometry
  int tw, th, tn;                // logical pixels per tile along W, H, N
  int tiles_b, tiles_a, tiles_n;
  int AW, AH, NL;                // logical output grid (valid extents)
  int es;                        // coordinate multiplier of the activation tensor map
  int ncb, cb;                   // channel blocks per tap, channels per block
  int ntaps;
  int rows_valid;                // tn*th*tw
  int64_t out_sn, out_sa, out_sb, out_sc, out_base;   // output element strides (CONV)
  int OC;                        // valid output columns (CONV) / rows (DW)
  int ICv;                       // valid columns (DW)
  // DW
  int patches_total, patches_per_split;
  int64_t part_stride_split, part_stride_tap, part_ld;   // partial buffer [split][oc_pad128][(tap, block) x 32]
  int oc_tiles, ic_tiles;        // ic_tiles: 32-channel blocks of the input channels
  int nb_total, nb_group;        // DW: (tap, channel block) column blocks in total / per tile
  // epilogue
  int accumulate, act;
  float alpha;
  const float* bias;
  float* out;
  int* status;
  // fp16 split: largest magnitudes (fp32 bit patterns) of the two operand tensors; the
  // accumulator is scaled by the product of the powers of two derived from them
  const uint32_t* amax_a;
  const uint32_t* amax_b;
  uint32_t* amax_out;            // ep_mode 4: largest magnitude of what this launch wrote
  // fused 2x2/stride-2 max pool (channels-on-M kernels): ep_mode 1 writes the pooled NCHW
  // tensor, ep_mode 2 writes it channel-innermost and pre-split in tf32 (out = hi, out_lo = lo,
  // channel pitch ocp) as the next convolution's operand, ep_mode 4 writes the fp16 split (out = hi, out_lo = lo)
  // scaled by an upper bound that sits in the word before *amax_out, and records the true
  // largest magnitude in *amax_out; the out_s* strides then address pooled pixels
  int ep_mode;
  float* out_lo;
  uint8_t* idx_out;   // ep_mode 1 only, optional: window position (0..3 row-major, 4 = none) of each pooled value
  int ocp;
  int tap_dy[kMaxTaps], tap_dx[kMaxTaps], tap_w[kMaxTaps];
  // halo-resident pixel patch (tc_halo_kernel): the patch of one channel block, with its halo,
  // is loaded once per tile as a flat array of pixels (row pitch h_pw) and every tap reads it
  // through a descriptor shifted by tap_shift rows
  int h_pw, h_ph;                // patch width (multiple of 4) and height in pixels
  int h_x0, h_y0;                // smallest tap offsets: patch origin relative to the tile origin
  int h_arows;                   // kernel rows loaded per unit (the rest of the 128 is never stored)
  int h_acb;                     // channels per kernel unit (<= cb)
  int h_sa, h_sb;                // ring depths: kernel units, patch stages
  int h_bbuf;                    // bytes of one (hi or lo) patch buffer, 1024-byte multiple
  int tap_shift[kMaxTaps];
};

}  // namespace lnn_tc
