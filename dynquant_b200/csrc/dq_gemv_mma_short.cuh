// Tensor-core GEMV for SHORT matrices: the layers of a decoder block at decode time.
//
// A 2048 x 2048 projection at 3 bits is 1.7 MB -- a quarter of a microsecond of HBM time --
// so its cost is a chain of latencies, not a stream: launch, first weight bytes, activation
// staging, a few steps of math, the cross-warp sum, the store.  This kernel is built to
// shorten that chain and to let consecutive launches overlap:
//
//   * every warp's whole share of the weights (its row tile x its slice of the reduction
//     axis, at most kMaxSteps steps) is requested with cp.async in the first instructions of
//     the kernel, BEFORE griddepcontrol.wait: under programmatic dependent launch those bytes
//     travel while the previous layer is still computing;
//   * the copies land in shared memory, not registers, and the kernel stays at <= 64
//     registers per thread, so the CTAs of the next launch fit on the SM beside this one's;
//   * the grid is a single wave; the reduction axis is sliced over the warps of a CTA and
//     summed in a fixed order (bit-identical results run to run).
//
// Arithmetic is that of gemv_mma_kernel (dq_gemv_mma.cu).  The host checks the
// requirements: one group per 128-value step, an even number of steps per slice starting
// on an even step (so a slice's scales are whole 4-byte words), and the step count limit.
#pragma once

#include "dq_gemv.cuh"
#include "dq_gemv_mma_stream.cuh"
#include "dq_mma_plan.cuh"
#include "dq_mma_stage.cuh"

namespace dq {
namespace shortk {

constexpr int kMaxWarps = 16;  // a CTA is 8 or 16 warps (blockDim.x)
constexpr int kMaxThreads = kMaxWarps * kWarp;
constexpr int kMaxSteps = 8;  // per warp

struct Params {
  int steps;           // padded K / 128
  int tiles;           // ceil(rows / 16)
  int rw, kw;          // rw * kw == warps of the CTA
  int steps_per_warp;  // <= kMaxSteps
  int meta_words;      // 4-byte words of scales (= of offsets) a warp copies per row
  int m_stride_u4;     // uint4 per activation row of a WARP's staged fragments
  uint32_t magic;
};

template <int BITS>
__host__ __device__ constexpr int unit_bytes() {
  return 4 * BITS;
}

// Per-warp staging area: raw scratch, fragments (+ zero block), the two sums.
template <int BITS>
__host__ __device__ inline int warp_stage_bytes(int m, int steps_per_warp, int m_stride_u4) {
  const int aregs = BITS == 8 ? 32 : 16;
  return steps_per_warp * 256 + (m * m_stride_u4 + aregs) * 16 + steps_per_warp * 8 * 4 * 2;
}

// Shared memory: [weights: steps_per_warp][2 rows][threads][UNIT] [meta: meta_words][threads][4 B]
//                [red] [per-warp staging areas]
template <int BITS>
inline size_t smem_bytes(int m, const Params& p) {
  const int threads = p.rw * p.kw * kWarp;
  size_t bytes = static_cast<size_t>(p.steps_per_warp) * 2 * threads * unit_bytes<BITS>();
  bytes += static_cast<size_t>(p.meta_words) * threads * 4;
  bytes += static_cast<size_t>(p.kw) * p.rw * 16 * 8 * 4;
  bytes += static_cast<size_t>(p.rw * p.kw) * warp_stage_bytes<BITS>(m, p.steps_per_warp, p.m_stride_u4);
  return bytes;
}

template <int BITS, bool XBF16, bool MBF16>
__global__ void __launch_bounds__(kMaxThreads, 2) gemv_mma_short_kernel(const GemvArgs a, const Params p) {
  using Plan = MmaPlan<BITS>;
  constexpr int NA = Plan::kARegs;
  constexpr int QU = NA / 4;
  constexpr int UNIT = unit_bytes<BITS>();
  constexpr int STEP_WORDS = 4 * BITS;

  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int kThreads = blockDim.x;
  unsigned char* wbuf = smem_raw;
  unsigned char* mbuf = wbuf + p.steps_per_warp * 2 * kThreads * UNIT;
  float* red = reinterpret_cast<float*>(mbuf + p.meta_words * kThreads * 4);
  const int tid = threadIdx.x;
  const int lane = tid & (kWarp - 1);
  const int warp = tid >> 5;
  // this warp's private staging area
  unsigned char* area = reinterpret_cast<unsigned char*>(red + p.kw * p.rw * 16 * 8) +
                        warp * warp_stage_bytes<BITS>(a.m, p.steps_per_warp, p.m_stride_u4);
  unsigned short* raw = reinterpret_cast<unsigned short*>(area);
  uint4* xb = reinterpret_cast<uint4*>(area + p.steps_per_warp * 256);
  float* xsum = reinterpret_cast<float*>(xb + a.m * p.m_stride_u4 + QU * 4);
  float* xneg = xsum + p.steps_per_warp * 8;
  const int g = lane >> 2, t = lane & 3;
  const int rwi = warp / p.kw;
  const int kwi = warp - rwi * p.kw;
  const int tile = blockIdx.x * p.rw + rwi;
  const bool tile_live = tile < p.tiles;
  const int s_begin = kwi * p.steps_per_warp;
  const int nsteps = max(0, min(p.steps, s_begin + p.steps_per_warp) - s_begin);
  const bool has_off = a.offsets != nullptr;
  const int row_a = tile * 16 + g, row_b = row_a + 8;
  const int ld_a = min(row_a, a.rows - 1), ld_b = min(row_b, a.rows - 1);

  pdl_launch_dependents();

  // ---- every byte this warp will decode, requested now ----
  if (tile_live && nsteps > 0) {
    const uint32_t wdst = static_cast<uint32_t>(__cvta_generic_to_shared(wbuf)) + (tid - lane) * UNIT;
#pragma unroll 1
    for (int j = 0; j < nsteps; ++j) {
      const int word0 = (s_begin + j) * STEP_WORDS;
      stream::copy_block<BITS>(wdst + (j * 2 + 0) * (kThreads * UNIT), a.packed, a.words_per_row, tile * 16, a.rows - 1,
                       word0, lane);
      stream::copy_block<BITS>(wdst + (j * 2 + 1) * (kThreads * UNIT), a.packed, a.words_per_row, tile * 16 + 8,
                       a.rows - 1, word0, lane);
    }
    // lane t of a quad fetches array t: scale(row a), offset(row a), scale(row b), offset(row b)
    if (has_off || (t & 1) == 0) {
      const unsigned short* arr = reinterpret_cast<const unsigned short*>((t & 1) ? a.offsets : a.scales);
      // whole 4-byte words covering steps [s_begin, s_begin + nsteps): start at the even step below
      const int s_even = s_begin & ~1;
      const unsigned short* src = arr + static_cast<int64_t>((t & 2) ? ld_b : ld_a) * a.num_groups + s_even;
      const uint32_t mdst = static_cast<uint32_t>(__cvta_generic_to_shared(mbuf)) + tid * 4;
      const int words = (s_begin + nsteps - s_even + 1) >> 1;
#pragma unroll 1
      for (int w = 0; w < words; ++w) {
        stream::cp_async_n<4>(mdst + w * (kThreads * 4), src + 2 * w);
      }
    }
  }
  stream::cp_async_commit();

  // ---- the part that depends on the previous kernel ----
  pdl_wait_prior_grid();
  if (tile_live && nsteps > 0) {
    stage_warp_slice<BITS, XBF16>(a, s_begin, nsteps, p.m_stride_u4, raw, xb, xsum, xneg, lane);
  }
  stream::cp_async_wait<0>();
  __syncwarp();  // the quad's metadata copies are visible to each other; no CTA-wide barrier

  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  if (tile_live) {
    const bool b_live = g < a.m;
    const uint4* xb_lane = b_live ? xb + g * p.m_stride_u4 + t : xb + a.m * p.m_stride_u4;
    const int xb_step_u4 = b_live ? QU * 4 : 0;
    const unsigned char* wsrc = wbuf + tid * UNIT;
    const unsigned short* msrc = reinterpret_cast<const unsigned short*>(mbuf + (tid & ~3) * 4);
    const uint32_t magic = p.magic;
#pragma unroll 2
    for (int j = 0; j < nsteps; ++j) {
      uint32_t wa[BITS], wb[BITS];
      stream::read_unit<BITS>(wsrc + (j * 2 + 0) * (kThreads * UNIT), wa);
      stream::read_unit<BITS>(wsrc + (j * 2 + 1) * (kThreads * UNIT), wb);
      uint32_t aa[NA], ab[NA];
      decode_unit<BITS>(wa, magic, aa);
      decode_unit<BITS>(wb, magic, ab);
      unbias_fragments<XBF16, NA>(aa);
      unbias_fragments<XBF16, NA>(ab);
      const uint4* bsrc = xb_lane + j * xb_step_u4;  // fragments are indexed within the warp's slice
      // two accumulators: a short matrix has few warps per SM, so the latency of the
      // dependent mma chain (not its throughput) is what a step costs -- halve the chain
      float d[4], e[4];
#pragma unroll
      for (int q = 0; q < QU; ++q) {
        const uint4 b = bsrc[q * 4];
        if (q == 0) {
          mma_16816<XBF16, true>(d, aa[0], ab[0], aa[1], ab[1], b.x, b.y);
          mma_16816<XBF16, true>(e, aa[2], ab[2], aa[3], ab[3], b.z, b.w);
        } else {
          mma_16816<XBF16, false>(d, aa[4 * q], ab[4 * q], aa[4 * q + 1], ab[4 * q + 1], b.x, b.y);
          mma_16816<XBF16, false>(e, aa[4 * q + 2], ab[4 * q + 2], aa[4 * q + 3], ab[4 * q + 3], b.z, b.w);
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) d[i] += e[i];
      // metadata of step j: halfword jj & 1 of word jj / 2 of each of the quad's four arrays,
      // jj counted from the even step at or below s_begin
      const int jj = j + (s_begin & 1);
      const unsigned short* mrow = msrc + (jj / 2) * (kThreads * 2) + (jj & 1);
      auto meta = [&](int i) -> float {
        const unsigned short raw = mrow[i * 2];
        if constexpr (MBF16) {
          return __uint_as_float(static_cast<uint32_t>(raw) << 16);
        } else {
          return __half2float(__ushort_as_half(raw));
        }
      };
      const float2 xs2 = *reinterpret_cast<const float2*>(xsum + j * 8 + 2 * t);
      const float2 xn2 = *reinterpret_cast<const float2*>(xneg + j * 8 + 2 * t);
      const float sc_a = meta(0), sc_b = meta(2);
      acc[0] = fmaf(sc_a, d[0] + xn2.x, acc[0]);
      acc[1] = fmaf(sc_a, d[1] + xn2.y, acc[1]);
      acc[2] = fmaf(sc_b, d[2] + xn2.x, acc[2]);
      acc[3] = fmaf(sc_b, d[3] + xn2.y, acc[3]);
      if (has_off) {
        const float of_a = meta(1), of_b = meta(3);
        acc[0] = fmaf(of_a, xs2.x, acc[0]);
        acc[1] = fmaf(of_a, xs2.y, acc[1]);
        acc[2] = fmaf(of_b, xs2.x, acc[2]);
        acc[3] = fmaf(of_b, xs2.y, acc[3]);
      }
    }
  }

  // ---- sum the slices of the reduction axis in a fixed order, store ----
  if (p.kw > 1) {
    float* mine = red + ((kwi * p.rw + rwi) * 16) * 8;
    *reinterpret_cast<float2*>(mine + g * 8 + 2 * t) = make_float2(acc[0], acc[1]);
    *reinterpret_cast<float2*>(mine + (g + 8) * 8 + 2 * t) = make_float2(acc[2], acc[3]);
    __syncthreads();
    if (kwi == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i] = 0.0f;
      for (int k = 0; k < p.kw; ++k) {
        const float* part = red + ((k * p.rw + rwi) * 16) * 8;
        const float2 pa = *reinterpret_cast<const float2*>(part + g * 8 + 2 * t);
        const float2 pb = *reinterpret_cast<const float2*>(part + (g + 8) * 8 + 2 * t);
        acc[0] += pa.x, acc[1] += pa.y, acc[2] += pb.x, acc[3] += pb.y;
      }
    }
  }
  if (kwi == 0 && tile_live) {
    const int m0 = 2 * t;
    if (m0 < a.m) {
      if (row_a < a.rows) store_out(a, m0, row_a, acc[0]);
      if (row_b < a.rows) store_out(a, m0, row_b, acc[2]);
    }
    if (m0 + 1 < a.m) {
      if (row_a < a.rows) store_out(a, m0 + 1, row_a, acc[1]);
      if (row_b < a.rows) store_out(a, m0 + 1, row_b, acc[3]);
    }
  }
}

}  // namespace shortk
}  // namespace dq
