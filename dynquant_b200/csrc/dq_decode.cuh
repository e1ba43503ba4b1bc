// Register-level decode of packed codes, specialised per bit width.
//
// Layout being decoded (reference docs/format-spec.md:216-240; device-side
// counterpart packages/dynquant-kernels/csrc/include/dynquant/nbit.cuh:106-121):
// value i of a group occupies bits [i*b, i*b+b) counted from the LSB of word
// floor(i*b/32); at 3-bit, values 10 and 21 of every 32 straddle two words.
//
// How a code becomes a float here
// -------------------------------
// No integer-to-float conversion instruction is issued.  A code q sitting at
// bits [s, s+b) of a word, with s+b <= 23, is turned into the fp32 number
// 2^(23-s) + q by ONE logic op: keep those bits as mantissa bits and OR in the
// exponent 150-s.  Two such numbers are then un-biased together by one packed
// fp32 add (add.rn.f32x2), which is exact because both operands are integers
// below 2^24.  The result is the exact integer q as fp32 -- unlike folding the
// 2^23 bias into the group offset, which the reference documents as losing
// half a scale of precision (csrc/gemv/gemv.cu:181-190).  Codes that sit too
// high in the word for s+b <= 23 are brought down by one shift (or funnel
// shift across the 3-bit straddle) shared by several codes.
//
// Per value this is one logic op, half a packed add and -- in the GEMV -- half
// a packed FMA per activation row.
#pragma once

#include "dq_common.cuh"

namespace dq {

template <int BITS>
struct Block;  // smallest run of whole words
template <>
struct Block<2> {
  static constexpr int kValues = 16, kWords = 1;
};
template <>
struct Block<3> {
  static constexpr int kValues = 32, kWords = 3;
};
template <>
struct Block<4> {
  static constexpr int kValues = 8, kWords = 1;
};
template <>
struct Block<8> {
  static constexpr int kValues = 4, kWords = 1;
};

// (2^(23-SA) + qa, 2^(23-SB) + qb) -> (qa, qb), exact.
template <int BITS, int SA, int SB>
__device__ __forceinline__ float2 code_pair(uint32_t w) {
  static_assert(SA + BITS <= 23 && SB + BITS <= 23, "code must sit inside the fp32 mantissa");
  constexpr uint32_t kField = (1u << BITS) - 1u;
  const float2 biased =
      make_float2(__uint_as_float((w & (kField << SA)) | (static_cast<uint32_t>(150 - SA) << 23)),
                  __uint_as_float((w & (kField << SB)) | (static_cast<uint32_t>(150 - SB) << 23)));
  const float2 bias = make_float2(-static_cast<float>(1u << (23 - SA)), -static_cast<float>(1u << (23 - SB)));
  return __fadd2_rn(biased, bias);
}

// pairsN(w, f) calls f(p, q2) for p = 0 .. kValues/2-1 with
// q2 = (code[2p], code[2p+1]) as exact fp32 integers.  `w` points at the
// block's kWords words (registers); p is a compile-time constant after inlining.

template <typename F>
__device__ __forceinline__ void pairs2(const uint32_t* w, F&& f) {
  const uint32_t lo = w[0];
  f(0, code_pair<2, 0, 2>(lo));
  f(1, code_pair<2, 4, 6>(lo));
  f(2, code_pair<2, 8, 10>(lo));
  f(3, code_pair<2, 12, 14>(lo));
  f(4, code_pair<2, 16, 18>(lo));
  const uint32_t hi = lo >> 12;  // values 6.. at bit 0
  f(5, code_pair<2, 8, 10>(hi));
  f(6, code_pair<2, 12, 14>(hi));
  f(7, code_pair<2, 16, 18>(hi));
}

template <typename F>
__device__ __forceinline__ void pairs4(const uint32_t* w, F&& f) {
  const uint32_t lo = w[0];
  f(0, code_pair<4, 0, 4>(lo));
  f(1, code_pair<4, 8, 12>(lo));
  const uint32_t hi = lo >> 16;
  f(2, code_pair<4, 0, 4>(hi));
  f(3, code_pair<4, 8, 12>(hi));
}

template <typename F>
__device__ __forceinline__ void pairs8(const uint32_t* w, F&& f) {
  // Byte i of the word dropped into the low mantissa byte of 2^23.
  const uint32_t v = w[0];
  const float2 bias = make_float2(-8388608.0f, -8388608.0f);
  f(0, __fadd2_rn(make_float2(__uint_as_float(__byte_perm(v, 0x4B000000u, 0x7440)),
                              __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7441))),
                  bias));
  f(1, __fadd2_rn(make_float2(__uint_as_float(__byte_perm(v, 0x4B000000u, 0x7442)),
                              __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7443))),
                  bias));
}

template <typename F>
__device__ __forceinline__ void pairs3(const uint32_t* w, F&& f) {
  // 96 bits = 32 values.  Six windows, each starting on a value boundary, so
  // every code is read at s in {0,3,...,15}; the two straddlers (values 10 and
  // 21) are covered by the funnel shifts.
  const uint32_t w0 = w[0], w1 = w[1], w2 = w[2];
  f(0, code_pair<3, 0, 3>(w0));
  f(1, code_pair<3, 6, 9>(w0));
  f(2, code_pair<3, 12, 15>(w0));
  const uint32_t a = w0 >> 18;  // value 6 at bit 0
  f(3, code_pair<3, 0, 3>(a));
  f(4, code_pair<3, 6, 9>(a));
  const uint32_t b = __funnelshift_r(w0, w1, 30);  // value 10 (bit 30) at bit 0
  f(5, code_pair<3, 0, 3>(b));
  f(6, code_pair<3, 6, 9>(b));
  f(7, code_pair<3, 12, 15>(b));
  const uint32_t c = __funnelshift_r(w1, w2, 16);  // value 16 (bit 48) at bit 0
  f(8, code_pair<3, 0, 3>(c));
  f(9, code_pair<3, 6, 9>(c));
  f(10, code_pair<3, 12, 15>(c));
  const uint32_t d = w2 >> 2;  // value 22 (bit 66) at bit 0
  f(11, code_pair<3, 0, 3>(d));
  f(12, code_pair<3, 6, 9>(d));
  f(13, code_pair<3, 12, 15>(d));
  const uint32_t e = w2 >> 20;  // value 28 (bit 84) at bit 0
  f(14, code_pair<3, 0, 3>(e));
  f(15, code_pair<3, 6, 9>(e));
}

template <int BITS, typename F>
__device__ __forceinline__ void for_each_pair(const uint32_t* w, F&& f) {
  if constexpr (BITS == 2) {
    pairs2(w, static_cast<F&&>(f));
  } else if constexpr (BITS == 3) {
    pairs3(w, static_cast<F&&>(f));
  } else if constexpr (BITS == 4) {
    pairs4(w, static_cast<F&&>(f));
  } else {
    static_assert(BITS == 8, "unsupported width");
    pairs8(w, static_cast<F&&>(f));
  }
}

// One code by run-time index out of a run of words (slow path: ragged tails,
// per-row tensors, groups smaller than a vector load).  `words_left` bounds the
// read of the straddled-into word.
template <int BITS>
__device__ __forceinline__ uint32_t code_at(const uint32_t* __restrict__ words, int i, int words_left) {
  const int bit = i * BITS;
  const int w = bit >> 5;
  const int s = bit & 31;
  uint32_t v = __ldg(words + w) >> s;
  if (BITS == 3 && 32 - s < BITS && w + 1 < words_left) {
    v |= __ldg(words + w + 1) << (32 - s);
  }
  return v & ((1u << BITS) - 1u);
}

}  // namespace dq
