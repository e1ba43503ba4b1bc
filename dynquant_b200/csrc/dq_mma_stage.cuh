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

// Position inside a 128-value step of value `v` (0..31) of quad lane `tt`'s unit.  Normally a
// unit is 32 consecutive values.  With 64-value groups (G64) a lane instead owns 16 values of
// EACH of the step's two groups -- [16 tt, 16 tt + 16) and [64 + 16 tt, 64 + 16 tt + 16) -- so
// that the first half of its fragment registers belongs to one group and the second half to
// the other, and the two halves can be accumulated (and scaled) separately.
//
// At 3 bits a 16-value half unit is 48 bits and does not start on a word, so there a lane keeps
// its whole 32-value unit: quad lanes 0,1 hold values of the first group, 2,3 of the second
// (SPLIT_QUAD), and the kernel separates the groups by giving the other pair of lanes a zero
// B fragment.
template <bool G64, int BITS>
__host__ __device__ constexpr int step_position(int tt, int v) {
  if (G64 && BITS != 3) return v < 16 ? 16 * tt + v : 64 + 16 * tt + (v - 16);
  return 32 * tt + v;
}

// Fixed-order reduction of a per-lane partial over the LANES lanes (lane index l = 4 q + tt)
// that build one (activation row, step).  MODE 0: one sum, in lane 0.  MODE 1 (groups are
// the two halves of the registers, i.e. of q): sums in lanes 0 and LANES/2.  MODE 2 (groups
// are the quad-lane pairs, bit 1 of l): sums in lanes 0 and 2.
template <int LANES, int MODE>
__device__ __forceinline__ void reduce_builder_group(float& sx, float& sb) {
#pragma unroll
  for (int d = LANES / 2; d > 0; d >>= 1) {
    if (MODE == 1 && d == LANES / 2) continue;
    if (MODE == 2 && d == 2) continue;
    sx += __shfl_xor_sync(0xffffffffu, sx, d);
    sb += __shfl_xor_sync(0xffffffffu, sb, d);
  }
}

// What lanes of absent activation rows read: a block of zero fragments after the last staged
// row, and zero sums in the columns of the rows that do not exist.  Nothing here depends on
// the activation, so a kernel may do it before its dependency wait (`prefilled` below).
template <int BITS, bool G64>
__device__ __forceinline__ void stage_zero_fill(int m, int nsteps, int m_stride_u4, uint4* xb, float* xsum,
                                                float* xneg, int tid, int nthreads) {
  constexpr int NA = MmaPlan<BITS>::kARegs;
  for (int idx = tid; idx < NA; idx += nthreads) {
    xb[m * m_stride_u4 + idx] = make_uint4(0u, 0u, 0u, 0u);
  }
  if (m < 8) {
    for (int idx = tid; idx < nsteps * (G64 ? 16 : 8); idx += nthreads) {
      if ((idx & 7) >= m) {
        xsum[idx] = 0.0f;
        xneg[idx] = 0.0f;
      }
    }
  }
}

// Unit-per-lane staging, the fast path of both variants below when the activation is 16-bit,
// 16-byte aligned and in_features is a multiple of 8.  A task is (activation row m, step j,
// quad lane tt): the lane loads the 32 values whose fragments quad lane tt of the compute
// warps will want -- four 128-bit L2-coherent loads straight from global memory, no bounce
// through shared memory -- builds ALL of that unit's fragment registers with compile-time
// slot positions, stores them, and reduces the two sums over the four lanes of its quad
// (two shuffle levels, fixed order).  Tasks tid, tid + nthreads, ... ; consecutive tasks of
// a quad are the four tt of one (m, j).  Steps are [s_first, s_first + nsteps) of the row and
// are indexed from 0 in xb / xsum / xneg.  The caller synchronises afterwards.
// PLAIN_LOADS: `a.x` points into shared memory (a raw block of the activation that was copied there
// asynchronously); ordinary loads instead of L2-coherent global ones.
template <int BITS, bool XBF16, bool G64, bool PLAIN_LOADS = false>
__device__ __forceinline__ void stage_units(const GemvArgs& a, int s_first, int nsteps, int m_stride_u4, uint4* xb,
                                            float* xsum, float* xneg, int tid, int nthreads,
                                            const int* row_map, bool prefilled = false) {
  using Plan = MmaPlan<BITS>;
  constexpr int NA = Plan::kARegs;
  constexpr int QU = NA / 4;
  constexpr float kMagicValue = XBF16 ? 128.0f : 0.0f;
  constexpr bool HALVES = G64 && BITS != 3;  // groups = halves of the registers
  constexpr bool QUADS = G64 && BITS == 3;   // groups = quad-lane pairs
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
    // the unit as 16 words of two 16-bit values: value v sits in word v / 2
    uint32_t w[16];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int k = k_step + step_position<G64, BITS>(tt, 8 * c);
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (live && k < a.in_features) {
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const unsigned short*>(a.x) + src_row * a.in_features + k);
        if constexpr (PLAIN_LOADS) {
          v = *src;
        } else {
          v = __ldcg(src);
        }
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
    float sx[2] = {0.0f, 0.0f}, sb[2] = {0.0f, 0.0f};  // per group of the step (one group: [0] only)
    uint32_t regs[NA];
#pragma unroll
    for (int n = 0; n < NA; ++n) {
      constexpr int kHalf = NA / 2;
      const Slot sl = Plan::slot(n);
      const int grp = HALVES ? (n >= kHalf) : 0;
      const float flo = value(sl.v_lo), fhi = value(sl.v_hi);
      // every value of the unit appears in exactly one slot, except at 8-bit where the high
      // nibble's slot (e = 4) repeats it: count x once
      if (BITS != 8 || sl.e_lo == 0) sx[grp] += flo + fhi;
      const float slo = flo * __uint_as_float(static_cast<uint32_t>(127 + sl.e_lo) << 23);  // exact powers of two
      const float shi = fhi * __uint_as_float(static_cast<uint32_t>(127 + sl.e_hi) << 23);
      if constexpr (XBF16) {
        sb[grp] += slo + shi;
        regs[n] = __byte_perm(__float_as_uint(slo), __float_as_uint(shi), 0x7632);  // high halves: nothing to round
      } else {
        const __half2 h2 = __floats2half2_rn(slo, shi);
        regs[n] = *reinterpret_cast<const uint32_t*>(&h2);
      }
    }
    if (live) {
#pragma unroll
      for (int q = 0; q < QU; ++q) {
        xb[m * m_stride_u4 + (j * QU + q) * 4 + tt] = make_uint4(regs[4 * q], regs[4 * q + 1], regs[4 * q + 2], regs[4 * q + 3]);
      }
    }
    // sums over the quad (QUADS: over the lane pair -- the pairs are the two groups)
#pragma unroll
    for (int g2 = 0; g2 < (HALVES ? 2 : 1); ++g2) {
      sx[g2] += __shfl_xor_sync(0xffffffffu, sx[g2], 1);
      sb[g2] += __shfl_xor_sync(0xffffffffu, sb[g2], 1);
      if (!QUADS) {
        sx[g2] += __shfl_xor_sync(0xffffffffu, sx[g2], 2);
        sb[g2] += __shfl_xor_sync(0xffffffffu, sb[g2], 2);
      }
    }
    if (live) {
      if (HALVES) {
        if (tt == 0) {
          xsum[(j * 2 + 0) * 8 + m] = sx[0], xneg[(j * 2 + 0) * 8 + m] = -kMagicValue * sb[0];
          xsum[(j * 2 + 1) * 8 + m] = sx[1], xneg[(j * 2 + 1) * 8 + m] = -kMagicValue * sb[1];
        }
      } else if (QUADS) {
        if ((tt & 1) == 0) {
          xsum[(j * 2 + (tt >> 1)) * 8 + m] = sx[0], xneg[(j * 2 + (tt >> 1)) * 8 + m] = -kMagicValue * sb[0];
        }
      } else if (tt == 0) {
        xsum[j * 8 + m] = sx[0], xneg[j * 8 + m] = -kMagicValue * sb[0];
      }
    }
  }
  if (!prefilled) stage_zero_fill<BITS, G64>(a.m, nsteps, m_stride_u4, xb, xsum, xneg, tid, nthreads);
}

__device__ __forceinline__ bool stage_units_ok(const GemvArgs& a) {
  return a.x_dtype != DQ_F32 && (a.in_features & 7) == 0 && (reinterpret_cast<uintptr_t>(a.x) & 15) == 0;
}

// The activation is read with L2-coherent loads (ld.global.cg): it was written by the previous
// kernel moments ago, is read once per CTA, and must not be served from a line this SM cached
// before the previous kernel finished.
//
// Aligned 16-bit activations take the unit-per-lane path (stage_units); anything else (fp32, odd
// alignment) is gathered value by value from global memory.
// With G64 the sums are per (step, group): xsum / xneg are [steps][2][8].
template <int BITS, bool XBF16, bool G64 = false>
__device__ __forceinline__ void stage_activation(const GemvArgs& a, int steps, int m_stride_u4, uint4* xb,
                                                 float* xsum, float* xneg, int tid, int nthreads,
                                                 const int* row_map = nullptr, bool prefilled = false) {
  if (stage_units_ok(a)) {  // (uniform over the CTA)
    stage_units<BITS, XBF16, G64>(a, 0, steps, m_stride_u4, xb, xsum, xneg, tid, nthreads, row_map, prefilled);
    return;
  }
  auto fetch = [&](int64_t src_row, int k) -> float { return load_f32(a.x, src_row * a.in_features + k, a.x_dtype); };
  using Plan = MmaPlan<BITS>;
  constexpr int NA = Plan::kARegs;
  constexpr int QU = NA / 4;
  constexpr int LANES = QU * 4;  // lanes that build one (m, s): 16, or 32 at 8-bit
  constexpr int kSplit = !G64 ? 0 : (BITS == 3 ? 2 : 1);       // how the two groups of a step map to lanes
  constexpr int kSecond = BITS == 3 ? 2 : LANES / 2;           // lane holding the second group's sums
  constexpr float kMagicValue = XBF16 ? 128.0f : 0.0f;  // fp16 fragments are un-biased in registers
  const int lane = tid & (kWarp - 1);
  const int sub = lane / LANES;            // which (m, s) of this warp's batch
  const int l = lane - sub * LANES;        // lane within the builder group
  const int per_warp = kWarp / LANES;      // (m, s) items per warp iteration
  const int nitems = a.m * steps;
  const int q = l >> 2, tt = l & 3;
  // this lane always builds the same four slots: resolve them once, not once per item
  int off_lo[4], off_hi[4];
  float mul_lo[4], mul_hi[4];
  bool count_x[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const Slot sl = Plan::slot(4 * q + r);
    off_lo[r] = step_position<G64, BITS>(tt, sl.v_lo);
    off_hi[r] = step_position<G64, BITS>(tt, sl.v_hi);
    mul_lo[r] = __uint_as_float(static_cast<uint32_t>(127 + sl.e_lo) << 23);  // exact powers of two
    mul_hi[r] = __uint_as_float(static_cast<uint32_t>(127 + sl.e_hi) << 23);
    // every value of the unit appears in exactly one slot, except at 8-bit where the high
    // nibble's slot (e = 4) repeats it: count x once
    count_x[r] = BITS != 8 || sl.e_lo == 0;
  }
  for (int base = (tid >> 5) * per_warp; base < nitems; base += (nthreads >> 5) * per_warp) {
    const int idx = base + sub;
    const bool live = idx < nitems;
    const int m = live ? idx / steps : 0;
    const int s = live ? idx - m * steps : 0;
    const int64_t src_row = row_map != nullptr ? row_map[m] : m;  // gathered activation rows (MoE)
    const int kbase = s * 128;
    float sx = 0.0f, sb = 0.0f;
    uint32_t regs[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int k_lo = kbase + off_lo[r];
      const int k_hi = kbase + off_hi[r];
      float lo = 0.0f, hi = 0.0f;
      if (live && k_lo < a.in_features) lo = fetch(src_row, k_lo);
      if (live && k_hi < a.in_features) hi = fetch(src_row, k_hi);
      if (count_x[r]) sx += lo + hi;
      lo *= mul_lo[r];
      hi *= mul_hi[r];
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
    reduce_builder_group<LANES, kSplit>(sx, sb);
    if (G64) {
      if (live && (l == 0 || l == kSecond)) {
        xsum[(s * 2 + (l != 0)) * 8 + m] = sx;
        xneg[(s * 2 + (l != 0)) * 8 + m] = -kMagicValue * sb;
      }
    } else if (live && l == 0) {
      xsum[s * 8 + m] = sx;
      xneg[s * 8 + m] = -kMagicValue * sb;
    }
  }
  // what lanes of absent activation rows read: a block of zero fragments, zero sums
  for (int idx = tid; idx < QU * 4; idx += nthreads) {
    xb[a.m * m_stride_u4 + idx] = make_uint4(0u, 0u, 0u, 0u);
  }
  if (a.m < 8) {
    for (int idx = tid; idx < steps * (G64 ? 16 : 8); idx += nthreads) {
      if ((idx & 7) >= a.m) {
        xsum[idx] = 0.0f;
        xneg[idx] = 0.0f;
      }
    }
  }
}

// Warp-local variant for the short-matrix kernel: a warp stages only the steps of its own
// slice of the reduction axis, into shared memory only it reads, with __syncwarp as the
// only synchronisation -- no CTA-wide barrier sits between the arrival of the activation and
// the first mma.  Layouts (all warp-private):
//   raw   [nsteps * 128] 16-bit scratch (one activation row at a time)
//   xb    [m][nsteps * QU*4 (+4 pad)] uint4, then a zero block of QU*4
//   xsum / xneg  [nsteps][8]   ([nsteps][2][8] with 64-value groups)
template <int BITS, bool XBF16, bool G64 = false>
__device__ __forceinline__ void stage_warp_slice(const GemvArgs& a, int s_begin, int nsteps, int m_stride_u4,
                                                 unsigned short* raw, uint4* xb, float* xsum, float* xneg,
                                                 int lane, bool prefilled = false) {
  using Plan = MmaPlan<BITS>;
  constexpr int NA = Plan::kARegs;
  constexpr int QU = NA / 4;
  constexpr int LANES = QU * 4;
  constexpr int kSplit = !G64 ? 0 : (BITS == 3 ? 2 : 1);
  constexpr int kSecond = BITS == 3 ? 2 : LANES / 2;
  constexpr int PER = kWarp / LANES;  // steps built per round
  constexpr float kMagicValue = XBF16 ? 128.0f : 0.0f;
  if (stage_units_ok(a)) {
    stage_units<BITS, XBF16, G64>(a, s_begin, nsteps, m_stride_u4, xb, xsum, xneg, lane, kWarp, nullptr, prefilled);
    __syncwarp();
    return;
  }
  const int sub = lane / LANES;
  const int l = lane - sub * LANES;
  const int q = l >> 2, tt = l & 3;
  int off_lo[4], off_hi[4];
  float mul_lo[4], mul_hi[4];
  bool count_x[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const Slot sl = Plan::slot(4 * q + r);
    off_lo[r] = step_position<G64, BITS>(tt, sl.v_lo);
    off_hi[r] = step_position<G64, BITS>(tt, sl.v_hi);
    mul_lo[r] = __uint_as_float(static_cast<uint32_t>(127 + sl.e_lo) << 23);
    mul_hi[r] = __uint_as_float(static_cast<uint32_t>(127 + sl.e_hi) << 23);
    count_x[r] = BITS != 8 || sl.e_lo == 0;
  }
  const int k0 = s_begin * 128;
  const bool vec_ok = a.x_dtype != DQ_F32 && (a.in_features & 7) == 0 && (reinterpret_cast<uintptr_t>(a.x) & 15) == 0;
  for (int m = 0; m < a.m; ++m) {
    // ---- this row's slice into the warp's scratch, as 16-bit values ----
    if (vec_ok) {
      const uint4* src = reinterpret_cast<const uint4*>(a.x) + (static_cast<int64_t>(m) * a.in_features + k0) / 8;
      for (int v = lane; v < nsteps * 16; v += kWarp) {
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (k0 + v * 8 < a.in_features) val = __ldcg(src + v);
        reinterpret_cast<uint4*>(raw)[v] = val;
      }
    } else {
      for (int v = lane; v < nsteps * 128; v += kWarp) {
        const int k = k0 + v;
        const float f = k < a.in_features ? load_f32(a.x, static_cast<int64_t>(m) * a.in_features + k, a.x_dtype) : 0.0f;
        raw[v] = XBF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(f)) : __half_as_ushort(__float2half_rn(f));
      }
    }
    __syncwarp();
    // ---- fragments and sums, PER steps per round ----
    for (int base = 0; base < nsteps; base += PER) {
      const int j = min(base + sub, nsteps - 1);
      const bool live = base + sub < nsteps;
      const unsigned short* row = raw + j * 128;
      float sx = 0.0f, sb = 0.0f;
      uint32_t regs[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const uint32_t lo = row[off_lo[r]], hi = row[off_hi[r]];
        float flo, fhi;
        if constexpr (XBF16) {
          flo = __uint_as_float(lo << 16), fhi = __uint_as_float(hi << 16);
        } else {
          flo = __half2float(__ushort_as_half(static_cast<unsigned short>(lo)));
          fhi = __half2float(__ushort_as_half(static_cast<unsigned short>(hi)));
        }
        if (count_x[r]) sx += flo + fhi;
        const float slo = flo * mul_lo[r], shi = fhi * mul_hi[r];  // exact: powers of two
        if constexpr (XBF16) {
          sb += slo + shi;
          regs[r] = __byte_perm(__float_as_uint(slo), __float_as_uint(shi), 0x7632);  // the high halves
        } else {
          regs[r] = static_cast<uint32_t>(__half_as_ushort(__float2half_rn(slo))) |
                    (static_cast<uint32_t>(__half_as_ushort(__float2half_rn(shi))) << 16);
        }
      }
      if (live) {
        xb[m * m_stride_u4 + (j * QU + q) * 4 + tt] = make_uint4(regs[0], regs[1], regs[2], regs[3]);
      }
      reduce_builder_group<LANES, kSplit>(sx, sb);
      if (G64) {
        if (live && (l == 0 || l == kSecond)) {
          xsum[(j * 2 + (l != 0)) * 8 + m] = sx;
          xneg[(j * 2 + (l != 0)) * 8 + m] = -kMagicValue * sb;
        }
      } else if (live && l == 0) {
        xsum[j * 8 + m] = sx;
        xneg[j * 8 + m] = -kMagicValue * sb;
      }
    }
    __syncwarp();  // everyone is done with raw before the next row overwrites it
  }
  for (int idx = lane; idx < QU * 4; idx += kWarp) {
    xb[a.m * m_stride_u4 + idx] = make_uint4(0u, 0u, 0u, 0u);
  }
  if (a.m < 8) {
    for (int idx = lane; idx < nsteps * (G64 ? 16 : 8); idx += kWarp) {
      if ((idx & 7) >= a.m) {
        xsum[idx] = 0.0f;
        xneg[idx] = 0.0f;
      }
    }
  }
  __syncwarp();
}

}  // namespace dq
