// The fp16-operand variant of the fragment plan (2-, 4- and 8-bit codes).
//
// dq_mma_plan.cuh keeps every code inside the 7 mantissa bits a bf16 operand offers, which costs
// shifts: a 2-bit word needs two of them, a 4-bit word three, and an 8-bit code has to be split
// into nibbles (twice the registers, twice the mma).  An fp16 operand has a 10-bit mantissa:
//
//   2-bit  five codes of each half sit inside the low 10 bits as they are (5 masks), one shift
//          brings the other three down (3 masks): 9 integer instructions per word instead of 10,
//   4-bit  two codes per half fit unshifted (2 masks), one shift, 2 masks: 5 instead of 7,
//   8-bit  a whole byte fits: 1 mask, 1 shift, 1 mask per word -- 16 registers and 8 mma per
//          step instead of 32 and 16.
//
// The magic exponent is 1024 (0x6400), too large a bias to cancel after the contraction, so it
// is removed in registers with one sub.f16x2 per register -- exact (integers below 2048), and
// issued on the FMA pipe, which the decode leaves idle, not on the half-rate integer pipe.
//
// The price is on the activation side: fp16 has 5 exponent bits.  Every (activation row, step)
// is therefore staged with its own power-of-two factor that brings the step's largest value to
// [2^14, 2^15) before the slot exponents (down to 2^-8) are applied; the factor is undone in the
// fp32 epilogue together with the group's scale.  A bf16 activation has 8 significant bits and an
// fp16 one 11, so nothing is rounded: only values more than 2^20 below their step's largest can
// lose bits (in fp16 subnormals), a contribution far inside the 1e-3 bar.
#pragma once

#include "dq_gemv.cuh"
#include "dq_mma_plan.cuh"
#include "dq_mma_stage.cuh"

namespace dq {

template <int BITS>
struct MmaPlan16 {
  static_assert(BITS == 2 || BITS == 4 || BITS == 8, "3-bit codes keep the bf16-safe plan");
  static constexpr int kARegs = 16;  // per row per step, at every width
  static constexpr int kMmas = 8;

  __host__ __device__ static constexpr Slot slot(int n) {
    if (BITS == 2) {
      const int wi = n / 8, i = n % 8;
      if (i < 5) return Slot{16 * wi + i, -2 * i, 16 * wi + 8 + i, -2 * i};
      return Slot{16 * wi + i, -2 * (i - 5), 16 * wi + 8 + i, -2 * (i - 5)};
    }
    if (BITS == 4) {
      const int wi = n / 4, r = n % 4;
      return Slot{8 * wi + r, (r & 1) ? -4 : 0, 8 * wi + 4 + r, (r & 1) ? -4 : 0};
    }
    const int wi = n / 2, r = n % 2;
    return Slot{4 * wi + r, 0, 4 * wi + 2 + r, 0};
  }
};

#ifdef __CUDACC__

__device__ __forceinline__ uint32_t sub_f16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// One unit (BITS words, 32 values) into 16 A registers of exact fp16 integers q << s.
// `magic` holds 0x6400 in both halves (a kernel parameter, so the lop3 keeps its immediate mask).
template <int BITS>
__device__ __forceinline__ void decode_unit16(const uint32_t* w, uint32_t magic, uint32_t* a) {
  if constexpr (BITS == 2) {
#pragma unroll
    for (int wi = 0; wi < 2; ++wi) {
      const uint32_t r0 = w[wi], r1 = r0 >> 10;
      a[8 * wi + 0] = magic_or<0x00030003u>(r0, magic);
      a[8 * wi + 1] = magic_or<0x000C000Cu>(r0, magic);
      a[8 * wi + 2] = magic_or<0x00300030u>(r0, magic);
      a[8 * wi + 3] = magic_or<0x00C000C0u>(r0, magic);
      a[8 * wi + 4] = magic_or<0x03000300u>(r0, magic);
      a[8 * wi + 5] = magic_or<0x00030003u>(r1, magic);
      a[8 * wi + 6] = magic_or<0x000C000Cu>(r1, magic);
      a[8 * wi + 7] = magic_or<0x00300030u>(r1, magic);
    }
  } else if constexpr (BITS == 4) {
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
      const uint32_t r0 = w[wi], r1 = r0 >> 8;
      a[4 * wi + 0] = magic_or<0x000F000Fu>(r0, magic);
      a[4 * wi + 1] = magic_or<0x00F000F0u>(r0, magic);
      a[4 * wi + 2] = magic_or<0x000F000Fu>(r1, magic);
      a[4 * wi + 3] = magic_or<0x00F000F0u>(r1, magic);
    }
  } else {
#pragma unroll
    for (int wi = 0; wi < 8; ++wi) {
      const uint32_t r0 = w[wi];
      a[2 * wi + 0] = magic_or<0x00FF00FFu>(r0, magic);
      a[2 * wi + 1] = magic_or<0x00FF00FFu>(r0 >> 8, magic);
    }
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) a[i] = sub_f16x2(a[i], magic);
}

// Staging for this plan: like stage_units (dq_mma_stage.cuh) -- a task is (activation row m, step j,
// quad lane tt), the lane loads the 32 values of that unit straight from global memory -- but the
// fragments are fp16, scaled by the step's own power of two, and the second array holds that
// factor's inverse instead of a bias sum:
//   xb      fragments  x * 2^(14 - E) * 2^e_slot         (E = exponent of the step's largest |x|)
//   xsum    [steps][8]  sum of x over the step            (multiplies the group's offset)
//   xscale  [steps][8]  2^(E - 14)                        (multiplies the accumulator, with the scale)
// Requires stage_units_ok(a).  The caller fills the absent rows (stage_zero_fill) and synchronises.
template <int BITS, bool XBF16>
__device__ __forceinline__ void stage_units16(const GemvArgs& a, int s_first, int nsteps, int m_stride_u4, uint4* xb,
                                              float* xsum, float* xscale, int tid, int nthreads, const int* row_map) {
  using Plan = MmaPlan16<BITS>;
  constexpr int NA = Plan::kARegs;
  constexpr int QU = NA / 4;
  const int total = a.m * nsteps * 4;
  const int rounds = (total + nthreads - 1) / nthreads;
#pragma unroll 1
  for (int r = 0; r < rounds; ++r) {
    const int id = tid + r * nthreads;
    const bool live = id < total;
    const int tt = id & 3;
    const int mj = live ? (id >> 2) : 0;
    const int m = mj / nsteps;
    const int j = mj - m * nsteps;
    const int64_t src_row = row_map != nullptr ? row_map[m] : m;
    const int k_step = (s_first + j) * 128;
    uint32_t w[16];  // the unit as 16 words of two 16-bit values: value v sits in word v / 2
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int k = k_step + 32 * tt + 8 * c;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (live && k < a.in_features) {
        v = __ldcg(reinterpret_cast<const uint4*>(static_cast<const unsigned short*>(a.x) + src_row * a.in_features + k));
      }
      w[4 * c] = v.x, w[4 * c + 1] = v.y, w[4 * c + 2] = v.z, w[4 * c + 3] = v.w;
    }
    auto value = [&](int v) -> float {
      const uint32_t word = w[v >> 1];
      if constexpr (XBF16) {
        return __uint_as_float((v & 1) ? (word & 0xFFFF0000u) : (word << 16));
      } else {
        const __half2 h = *reinterpret_cast<const __half2*>(&word);
        return (v & 1) ? __high2float(h) : __low2float(h);
      }
    };
    float sx = 0.0f, amax = 0.0f;
#pragma unroll
    for (int v = 0; v < 32; ++v) {
      const float f = value(v);
      sx += f;
      amax = fmaxf(amax, fabsf(f));
    }
    // over the four lanes of the quad: the step's sum and its largest magnitude
    sx += __shfl_xor_sync(0xffffffffu, sx, 1);
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    sx += __shfl_xor_sync(0xffffffffu, sx, 2);
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    // E = biased exponent of the largest value, kept where both factors are normal floats
    // (a step of zeros or of denormal-sized values is scaled as if its largest were 2^-112)
    const uint32_t ebits = min(max((__float_as_uint(amax) >> 23) & 0xFFu, 15u), 250u);
    const float up = __uint_as_float((268u - ebits) << 23);    // 2^(14 - E)
    const float down = __uint_as_float((ebits - 14u) << 23);   // 2^(E - 14)
    uint32_t regs[NA];
#pragma unroll
    for (int n = 0; n < NA; ++n) {
      const Slot sl = Plan::slot(n);
      const float lo = value(sl.v_lo) * (up * __uint_as_float(static_cast<uint32_t>(127 + sl.e_lo) << 23));
      const float hi = value(sl.v_hi) * (up * __uint_as_float(static_cast<uint32_t>(127 + sl.e_hi) << 23));
      const __half2 h2 = __floats2half2_rn(lo, hi);  // (exact: at most 11 significant bits, in range)
      regs[n] = *reinterpret_cast<const uint32_t*>(&h2);
    }
    if (live) {
#pragma unroll
      for (int q = 0; q < QU; ++q) {
        xb[m * m_stride_u4 + (j * QU + q) * 4 + tt] = make_uint4(regs[4 * q], regs[4 * q + 1], regs[4 * q + 2], regs[4 * q + 3]);
      }
      if (tt == 0) {
        xsum[j * 8 + m] = sx;
        xscale[j * 8 + m] = down;
      }
    }
  }
}

#endif  // __CUDACC__

}  // namespace dq
