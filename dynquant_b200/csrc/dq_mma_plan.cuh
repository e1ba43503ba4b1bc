// Decode of packed codes straight into tensor-core A fragments.
//
// Every thread of a warp owns, per step of 128 reduction values, a "unit" of 32
// consecutive values of each of its two weight rows: BITS consecutive words
// (2/3/4/8 words at 2/3/4/8-bit).  The unit is turned into kARegs 32-bit
// registers, each holding two 16-bit floats, by ONE logic instruction per
// register: mask two codes in place (one in each 16-bit half) and OR in the
// exponent of a magic constant, giving  MAGIC + (q << s)  in each half, where s
// is wherever the code happened to sit inside the low 7 mantissa bits.  A shift
// (or funnel shift across the 3-bit straddle) brings several codes into place at
// once.  Nothing is converted and nothing is un-biased in registers:
//
//   * the power of two 2^s is folded into the ACTIVATION, which is staged once
//     per CTA as x' = x * 2^(-s) (an exact exponent shift) in the matching
//     fragment order, and
//   * the MAGIC bias is removed after the tensor-core contraction by
//     subtracting MAGIC * sum(x') -- one fp32 number per (activation row, step),
//     also computed once per CTA.  With a 7-bit field the bias is only 2^7 times
//     the unit, so the cancellation costs about 2 decimal digits of the fp32
//     accumulator and leaves the result ~1e-5 from the exact sum.
//
// The reduction index inside one mma is arbitrary as long as A and B agree, so
// the fragment "k slots" are simply whatever values each thread decoded; no
// shuffle, no transposition, and the weights stay in the linear layout of the
// format (reference docs/format-spec.md:216-240).
//
// 8-bit codes do not fit a 7-bit mantissa field: they are split into nibbles,
// each its own slot, the high nibble's activation pre-multiplied by 16.
#pragma once

#include "dq_common.cuh"

namespace dq {

// Which value of the thread's 32-value unit sits in each half of A register n,
// and the power of two its activation must be multiplied by.
struct Slot {
  int v_lo, e_lo, v_hi, e_hi;
};

template <int BITS>
struct MmaPlan {
  static constexpr int kUnitWords = BITS;                 // 32 values * BITS bits
  static constexpr int kARegs = BITS == 8 ? 32 : 16;      // per row per step
  static constexpr int kMmas = kARegs / 2;                // m16n8k16 per step per 16-row tile

  __host__ __device__ static constexpr Slot slot(int n) {
    if (BITS == 2) {
      const int wi = n / 8, i = n % 8;
      return Slot{16 * wi + i, -2 * (i % 3), 16 * wi + i + 8, -2 * (i % 3)};
    }
    if (BITS == 4) {
      const int wi = n / 4, i = n % 4;
      return Slot{8 * wi + i, 0, 8 * wi + i + 4, 0};
    }
    if (BITS == 8) {
      const int wi = n / 4, c = n % 4;
      const int v = 4 * wi + (c >> 1);
      const int e = (c & 1) ? 4 : 0;
      return Slot{v, e, v + 2, e};
    }
    // 3-bit: values 0..9 and 10..19 pair up five apart, 20..31 six apart.
    if (n < 10) {
      const int base = 10 * (n / 5), r = n % 5;
      const bool second = (r == 1 || r == 3);  // the (j+1, j+6) pair of a window
      return Slot{base + r, second ? -4 : -1, base + r + 5, second ? -3 : 0};
    }
    const int a = 20 + (n - 10);
    return Slot{a, 0, a + 6, -2};
  }
};

#ifdef __CUDACC__

// Bits [SH, SH+32) of the 96-bit string (w0, w1, w2); bits outside are zero.
template <int SH>
__device__ __forceinline__ uint32_t window96(uint32_t w0, uint32_t w1, uint32_t w2) {
  if constexpr (SH < 0) {
    return w0 << (-SH);
  } else if constexpr (SH == 0) {
    return w0;
  } else if constexpr (SH < 32) {
    return __funnelshift_r(w0, w1, SH);
  } else if constexpr (SH == 32) {
    return w1;
  } else if constexpr (SH < 64) {
    return __funnelshift_r(w1, w2, SH - 32);
  } else if constexpr (SH == 64) {
    return w2;
  } else {
    return w2 >> (SH - 64);
  }
}

// (w & MASK) | magic as ONE three-input logic op: MASK is the instruction's immediate and
// magic must be a register whose value the compiler cannot see (a kernel parameter), or
// it folds both constants and has to split the operation in two.
template <uint32_t MASK>
__device__ __forceinline__ uint32_t magic_or(uint32_t w, uint32_t magic) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(w), "n"(MASK), "r"(magic));
  return r;
}

// Decode one unit (BITS words) into kARegs A registers.  `magic` holds the
// 16-bit magic constant in both halves (0x43004300 for bf16, 0x64006400 for fp16).
template <int BITS>
__device__ __forceinline__ void decode_unit(const uint32_t* w, uint32_t magic, uint32_t* a) {
  if constexpr (BITS == 2) {
#pragma unroll
    for (int wi = 0; wi < 2; ++wi) {
      const uint32_t r0 = w[wi], r1 = r0 >> 6, r2 = r0 >> 12;
      a[8 * wi + 0] = magic_or<0x00030003u>(r0, magic);
      a[8 * wi + 1] = magic_or<0x000C000Cu>(r0, magic);
      a[8 * wi + 2] = magic_or<0x00300030u>(r0, magic);
      a[8 * wi + 3] = magic_or<0x00030003u>(r1, magic);
      a[8 * wi + 4] = magic_or<0x000C000Cu>(r1, magic);
      a[8 * wi + 5] = magic_or<0x00300030u>(r1, magic);
      a[8 * wi + 6] = magic_or<0x00030003u>(r2, magic);
      a[8 * wi + 7] = magic_or<0x000C000Cu>(r2, magic);
    }
  } else if constexpr (BITS == 4) {
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
      const uint32_t r0 = w[wi];
      a[4 * wi + 0] = magic_or<0x000F000Fu>(r0, magic);
      a[4 * wi + 1] = magic_or<0x000F000Fu>(r0 >> 4, magic);
      a[4 * wi + 2] = magic_or<0x000F000Fu>(r0 >> 8, magic);
      a[4 * wi + 3] = magic_or<0x000F000Fu>(r0 >> 12, magic);
    }
  } else if constexpr (BITS == 8) {
#pragma unroll
    for (int wi = 0; wi < 8; ++wi) {
      const uint32_t r0 = w[wi];
      a[4 * wi + 0] = magic_or<0x000F000Fu>(r0, magic);        // low nibble of bytes 0, 2
      a[4 * wi + 1] = magic_or<0x000F000Fu>(r0 >> 4, magic);   // high nibble of bytes 0, 2
      a[4 * wi + 2] = magic_or<0x000F000Fu>(r0 >> 8, magic);   // low nibble of bytes 1, 3
      a[4 * wi + 3] = magic_or<0x000F000Fu>(r0 >> 12, magic);  // high nibble of bytes 1, 3
    }
  } else {
    static_assert(BITS == 3, "unsupported width");
    const uint32_t w0 = w[0], w1 = w[1], w2 = w[2];
    constexpr uint32_t kFirst = (7u << 1) | (7u << 16);   // values j, j+5 of a window at 3j-1
    constexpr uint32_t kSecond = (7u << 4) | (7u << 19);  // values j+1, j+6
    constexpr uint32_t kSix = 7u | (7u << 18);            // values a, a+6 of a window at 3a
    uint32_t r;
    r = window96<-1>(w0, w1, w2);
    a[0] = magic_or<kFirst>(r, magic);
    a[1] = magic_or<kSecond>(r, magic);
    r = window96<5>(w0, w1, w2);
    a[2] = magic_or<kFirst>(r, magic);
    a[3] = magic_or<kSecond>(r, magic);
    r = window96<11>(w0, w1, w2);
    a[4] = magic_or<kFirst>(r, magic);
    r = window96<29>(w0, w1, w2);
    a[5] = magic_or<kFirst>(r, magic);
    a[6] = magic_or<kSecond>(r, magic);
    r = window96<35>(w0, w1, w2);
    a[7] = magic_or<kFirst>(r, magic);
    a[8] = magic_or<kSecond>(r, magic);
    r = window96<41>(w0, w1, w2);
    a[9] = magic_or<kFirst>(r, magic);
    a[10] = magic_or<kSix>(window96<60>(w0, w1, w2), magic);
    a[11] = magic_or<kSix>(window96<63>(w0, w1, w2), magic);
    a[12] = magic_or<kSix>(window96<66>(w0, w1, w2), magic);
    a[13] = magic_or<kSix>(window96<69>(w0, w1, w2), magic);
    a[14] = magic_or<kSix>(window96<72>(w0, w1, w2), magic);
    a[15] = magic_or<kSix>(window96<75>(w0, w1, w2), magic);
  }
}

// fp16 operands only: remove the magic bias in registers (exact: both numbers are integers
// below 2048), because 1024 -- the smallest magic a 10-bit mantissa allows for fields in its
// low bits -- is too large a bias to cancel after the contraction at full fp32 accuracy.
// bf16 keeps the bias (128) and removes it afterwards.
template <bool BF16, int N>
__device__ __forceinline__ void unbias_fragments(uint32_t* a) {
  if constexpr (!BF16) {
    const __half2 magic = __half2half2(__ushort_as_half(static_cast<unsigned short>(0x6400)));
#pragma unroll
    for (int i = 0; i < N; ++i) {
      __half2 v = *reinterpret_cast<__half2*>(&a[i]);
      v = __hsub2(v, magic);
      a[i] = *reinterpret_cast<uint32_t*>(&v);
    }
  }
}

// D = A * B + C, m16n8k16, fp32 accumulate; bf16 or fp16 operands.  FIRST starts a fresh
// accumulator (C = 0 comes from the zero register, no moves).
template <bool BF16, bool FIRST>
__device__ __forceinline__ void mma_16816(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  if constexpr (FIRST) {
    if constexpr (BF16) {
      asm volatile(
          "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
          "{%10,%10,%10,%10};"
          : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
          : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
    } else {
      asm volatile(
          "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
          "{%10,%10,%10,%10};"
          : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
          : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
    }
  } else {
    if constexpr (BF16) {
      asm volatile(
          "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
          "{%0,%1,%2,%3};"
          : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
          : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
      asm volatile(
          "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
          "{%0,%1,%2,%3};"
          : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
          : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
  }
}

#endif  // __CUDACC__

}  // namespace dq
