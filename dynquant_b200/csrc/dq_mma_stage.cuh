// Staging of the activation for the tensor-core GEMV kernels: one pass, one barrier.
//
// For every (activation row m, step s) the CTA needs
//   * the B fragments: x' = x * 2^e in the slot order of MmaPlan, as 16-bit pairs,
//   * sum(x) over the step            (multiplies the group's offset), and
//   * -MAGIC * sum(x') over all slots (removes the magic bias from the accumulator).
// Half a warp (a whole warp at 8-bit) builds one (m, s): each lane one uint4 of four
// slot pairs, then a fixed-order shuffle reduction of the two sums -- so the sums, and
// therefore the results, are bit-identical from run to run.
#pragma once

#include "dq_mma_plan.cuh"

namespace dq {

template <int BITS, bool XBF16>
__device__ __forceinline__ void stage_activation(const GemvArgs& a, int steps, int m_stride_u4, uint4* xb,
                                                 float* xsum, float* xneg, int tid, int nthreads,
                                                 const int* row_map = nullptr) {
  using Plan = MmaPlan<BITS>;
  constexpr int NA = Plan::kARegs;
  constexpr int QU = NA / 4;
  constexpr int LANES = QU * 4;  // lanes that build one (m, s): 16, or 32 at 8-bit
  constexpr float kMagicValue = XBF16 ? 128.0f : 0.0f;  // fp16 fragments are un-biased in registers
  const int lane = tid & (kWarp - 1);
  const int sub = lane / LANES;            // which (m, s) of this warp's batch
  const int l = lane - sub * LANES;        // lane within the builder group
  const int per_warp = kWarp / LANES;      // (m, s) items per warp iteration
  const int nitems = a.m * steps;
  const int q = l >> 2, tt = l & 3;
  for (int base = (tid >> 5) * per_warp; base < nitems; base += (nthreads >> 5) * per_warp) {
    const int idx = base + sub;
    const bool live = idx < nitems;
    const int m = live ? idx / steps : 0;
    const int s = live ? idx - m * steps : 0;
    const int64_t src_row = row_map != nullptr ? row_map[m] : m;  // gathered activation rows (MoE)
    const int kbase = s * 128 + 32 * tt;
    float sx = 0.0f, sb = 0.0f;
    uint32_t regs[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const Slot sl = Plan::slot(4 * q + r);
      const int k_lo = kbase + sl.v_lo;
      const int k_hi = kbase + sl.v_hi;
      float lo = 0.0f, hi = 0.0f;
      if (live && k_lo < a.in_features) lo = load_f32(a.x, src_row * a.in_features + k_lo, a.x_dtype);
      if (live && k_hi < a.in_features) hi = load_f32(a.x, src_row * a.in_features + k_hi, a.x_dtype);
      // every value of the unit appears in exactly one slot, except at 8-bit where the high
      // nibble's slot (e = 4) repeats it: count x once
      if (BITS != 8 || sl.e_lo == 0) sx += lo + hi;
      lo *= __uint_as_float(static_cast<uint32_t>(127 + sl.e_lo) << 23);  // exact: a power of two
      hi *= __uint_as_float(static_cast<uint32_t>(127 + sl.e_hi) << 23);
      uint32_t lo16, hi16;
      if constexpr (XBF16) {
        const __nv_bfloat16 l16 = __float2bfloat16_rn(lo), h16 = __float2bfloat16_rn(hi);
        lo16 = __bfloat16_as_ushort(l16), hi16 = __bfloat16_as_ushort(h16);
        sb += __bfloat162float(l16) + __bfloat162float(h16);
      } else {
        const __half l16 = __float2half_rn(lo), h16 = __float2half_rn(hi);
        lo16 = __half_as_ushort(l16), hi16 = __half_as_ushort(h16);
        sb += __half2float(l16) + __half2float(h16);
      }
      regs[r] = lo16 | (hi16 << 16);
    }
    if (live) {
      xb[m * m_stride_u4 + (s * QU + q) * 4 + tt] = make_uint4(regs[0], regs[1], regs[2], regs[3]);
    }
#pragma unroll
    for (int d = LANES / 2; d > 0; d >>= 1) {
      sx += __shfl_xor_sync(0xffffffffu, sx, d);
      sb += __shfl_xor_sync(0xffffffffu, sb, d);
    }
    if (live && l == 0) {
      xsum[s * 8 + m] = sx;
      xneg[s * 8 + m] = -kMagicValue * sb;
    }
  }
  // what lanes of absent activation rows read: a block of zero fragments, zero sums
  for (int idx = tid; idx < QU * 4; idx += nthreads) {
    xb[a.m * m_stride_u4 + idx] = make_uint4(0u, 0u, 0u, 0u);
  }
  if (a.m < 8) {
    for (int idx = tid; idx < steps * 8; idx += nthreads) {
      if ((idx & 7) >= a.m) {
        xsum[idx] = 0.0f;
        xneg[idx] = 0.0f;
      }
    }
  }
}

}  // namespace dq
