// Device-side building blocks of the tcgen05 kernels: mbarrier waits with a budget, TMA loads,
// TMEM allocation and loads, tcgen05.mma issue, shared-memory descriptors, and the arithmetic of
// the two operand splits.  Included by the translation units that define such kernels.
#pragma once
#include <cuda_fp16.h>
#include <math_constants.h>
#include "lnn_tc.cuh"

namespace lnn_tc {


__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Bounded wait.  Returns false when the budget ran out or another role aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int role, int step) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitBudget) {
      *abort_flag = 1;
      if (atomicCAS(status, 0, LNN_E_TIMEOUT) == 0) {
        status[1] = role;
        status[2] = (int)(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z));
        status[3] = step;
      }
      return false;
    }
  }
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* tm, uint32_t bar,
                                            int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"((uint64_t)tm), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* tm, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"((uint64_t)tm), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum)
      : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                         uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum)
      : "memory");
}
template <bool F16>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                     uint32_t accum) {
  if (F16) umma_f16(tmem_d, adesc, bdesc, idesc, accum);
  else umma_tf32(tmem_d, adesc, bdesc, idesc, accum);
}
// All MMAs of one k-block (KS steps of 32 bytes of K; hi*hi, hi*lo, lo*hi when NBUF == 2), fully
// unrolled with independent descriptor adds: the issuing thread is a single scalar stream and
// every dependent instruction between two tcgen05.mma shows up in the MMA rate.
template <int KS, int NBUF, bool F16>
__device__ __forceinline__ void issue_kblock(uint32_t d_tmem, uint64_t ah, uint64_t bh, uint64_t a_step,
                                             uint64_t b_step, uint64_t a_lo, uint64_t b_lo,
                                             uint32_t idesc, uint32_t accum_first) {
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    const uint64_t a = ah + (uint64_t)ks * a_step, b = bh + (uint64_t)ks * b_step;
    umma<F16>(d_tmem, a, b, idesc, ks == 0 ? accum_first : 1u);
    if (NBUF == 2) {
      umma<F16>(d_tmem, a, b + b_lo, idesc, 1u);
      umma<F16>(d_tmem, a + a_lo, b, idesc, 1u);
    }
  }
}
template <int NBUF, bool F16>
__device__ __forceinline__ void issue_kblock_n(int ksteps, uint32_t d_tmem, uint64_t ah, uint64_t bh,
                                               uint64_t a_step, uint64_t b_step, uint64_t a_lo,
                                               uint64_t b_lo, uint32_t idesc, uint32_t accum_first) {
  switch (ksteps) {
    case 4: issue_kblock<4, NBUF, F16>(d_tmem, ah, bh, a_step, b_step, a_lo, b_lo, idesc, accum_first); break;
    case 2: issue_kblock<2, NBUF, F16>(d_tmem, ah, bh, a_step, b_step, a_lo, b_lo, idesc, accum_first); break;
    case 1: issue_kblock<1, NBUF, F16>(d_tmem, ah, bh, a_step, b_step, a_lo, b_lo, idesc, accum_first); break;
    case 8: issue_kblock<8, NBUF, F16>(d_tmem, ah, bh, a_step, b_step, a_lo, b_lo, idesc, accum_first); break;
    default:
      for (int ks = 0; ks < ksteps; ++ks) {
        issue_kblock<1, NBUF, F16>(d_tmem, ah, bh, a_step, b_step, a_lo, b_lo, idesc, ks == 0 ? accum_first : 1u);
        ah += a_step; bh += b_step;
      }
  }
}
// precision dispatch: fp16 split always carries hi and lo; tf32 may be hi only
__device__ __forceinline__ void issue_unit(int esz, int nbuf, int ksteps, uint32_t d_tmem, uint64_t ah,
                                           uint64_t bh, uint64_t a_step, uint64_t b_step, uint64_t a_lo,
                                           uint64_t b_lo, uint32_t idesc, uint32_t accum_first) {
  if (esz == 2) issue_kblock_n<2, true>(ksteps, d_tmem, ah, bh, a_step, b_step, a_lo, b_lo, idesc, accum_first);
  else if (nbuf == 2) issue_kblock_n<2, false>(ksteps, d_tmem, ah, bh, a_step, b_step, a_lo, b_lo, idesc, accum_first);
  else issue_kblock_n<1, false>(ksteps, d_tmem, ah, bh, a_step, b_step, a_lo, b_lo, idesc, accum_first);
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of tcgen05.mma: start address, leading / stride byte
// offsets (all in 16-byte units), descriptor version 1, swizzle mode in bits 61-63.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes, uint32_t layout_type) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= (uint64_t)layout_type << 61;
  return d;
}
__device__ __forceinline__ uint32_t layout_of_swizzle(int swz_bytes) {
  return swz_bytes == 128 ? 2u : (swz_bytes == 64 ? 4u : 6u);
}

__device__ __forceinline__ float apply_act(float v, int act, float alpha) {
  if (act == 1) {
    // leaky_relu as the reference writes it: I*(I>=0) + alpha*I*(I<0)
    const float pos = __fmul_rn(v, v >= 0.0f ? 1.0f : 0.0f);
    const float neg = __fmul_rn(__fmul_rn(alpha, v), v < 0.0f ? 1.0f : 0.0f);
    return __fadd_rn(pos, neg);
  }
  return v;
}

__device__ __forceinline__ float to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}
__device__ __forceinline__ void split1(float x, float& hi, float& lo) {
  hi = to_tf32(x);
  lo = to_tf32(__fsub_rn(x, hi));
}

// ---- fp16 split: exact power-of-two scaling -----------------------------------------------
// The scale exponent of a tensor follows from the bit pattern of its largest magnitude:
// x * 2^-e lies in [2^14, 2^15) for that element, so no element overflows fp16 and every element
// within 2^17 of the largest keeps 22 significant bits in hi + lo (smaller ones keep an absolute
// error of 2^-25 on that scale).  Zero, infinite and NaN maxima give e = 0: the values then go
// through fp16 as they are and non-finite inputs stay non-finite.
__device__ __forceinline__ int exp_of_amax(uint32_t bits) {
  int E = (int)((bits >> 23) & 0xffu);
  if (bits == 0u || E == 255) return 0;
  if (E == 0) E = 1;
  return E - 127 - 14;
}
// 2^k as a float for -149 <= k <= 127
__device__ __forceinline__ float pow2f_int(int k) {
  return k >= -126 ? __int_as_float((k + 127) << 23) : __int_as_float(1 << (k + 149));
}
// multiplication by 2^k in two exact steps whose factors are always representable
struct Pow2Scale {
  float f1, f2;
  __device__ __forceinline__ explicit Pow2Scale(int k) {
    const int k1 = k / 2;
    f1 = pow2f_int(k1); f2 = pow2f_int(k - k1);
  }
  __device__ __forceinline__ float operator()(float v) const { return __fmul_rn(__fmul_rn(v, f1), f2); }
};
__device__ __forceinline__ void split_half(float xs, __half& hi, __half& lo) {
  hi = __float2half_rn(xs);
  lo = __float2half_rn(__fsub_rn(xs, __half2float(hi)));
}
// largest magnitude of a warp's values into *dst (bit patterns of non-negative floats order like
// unsigned integers; a NaN pattern is larger than infinity, which is what exp_of_amax expects)
__device__ __forceinline__ void warp_amax_commit(uint32_t bits, uint32_t* dst) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, o));
  if ((threadIdx.x & 31) == 0 && bits != 0u) atomicMax(dst, bits);
}

}  // namespace lnn_tc
