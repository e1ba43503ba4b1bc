// Tiled tensor-core GEMV: one launch for up to four packed matrices that share an activation.
//
// The decoder-block layers of a model at decode time are short (a 2048 x 2048 projection at
// 3 bits is 1.7 MB) or of middle size (a 14336 x 4096 one at 4 bits is 29 MB): too small to
// stream, large enough that more than one wave of one-shot CTAs costs as much as the bytes.
// This kernel covers both, and fuses the shards of a fused layer (q/k/v, gate/up), whatever
// their widths, into ONE launch -- at this size a launch costs more than the bytes do.
//
//   * A CTA is 8 warps laid out as rw row tiles x kw slices of the reduction axis.  A warp
//     keeps its slice for the whole kernel and walks over row tiles (items), CTAs striding
//     over the items of their matrix; partial sums of the kw slices meet in shared memory
//     once per item and are added in a fixed order (results are bit-identical run to run).
//   * Weights travel global -> shared with 16-byte cp.async into a per-warp ring of `nb`
//     stages of CH steps; all nb stages are requested BEFORE griddepcontrol.wait, so under
//     programmatic dependent launch they fly while the previous layer computes, and a slot
//     is refilled as soon as it has been consumed.  When a warp's whole share fits the ring
//     everything is requested up front (the one-shot regime of short matrices).
//   * The activation is staged once per CTA: warp-private slices when rw == 1 (no CTA
//     barrier between the arrival of x and the first mma), CTA-wide otherwise.
//   * Each CTA belongs to one matrix (a "job") and runs the body compiled for its width.
//
// Arithmetic is that of gemv_mma_kernel (dq_gemv_mma.cu).  Requirements, checked by the
// host: one group per 128-value step, or two (64-value groups), whose halves of a step are
// accumulated and scaled separately (see tile_body); 16-byte aligned rows, steps divisible
// by kw * CH, and scales/offsets rows aligned to a stage's worth of metadata.
#pragma once

#include "dq_gemv.cuh"
#include "dq_peer_push.cuh"
#include "dq_gemv_mma_stream.cuh"
#include "dq_mma_plan.cuh"
#include "dq_mma_stage.cuh"

namespace dq {
namespace tilek {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * kWarp;
constexpr int kMaxJobs = 4;
constexpr int kMaxRing = 8;
constexpr int kRedFloats = 2 * kWarps * 16 * 8;  // two buffers of one 16 x 8 partial per warp

struct Job {
  GemvArgs a;
  int bits;
  int tiles;      // ceil(rows / 16)
  int items;      // ceil(tiles / rw)
  int cta_begin;  // CTAs [cta_begin, cta_begin + cta_count) of the grid work on this job
  int cta_count;
};

struct Launch {
  Job job[kMaxJobs];
  int njobs;
  int steps;       // padded K / 128 (the jobs share the activation, hence K)
  int rw, kw;      // rw * kw == kWarps
  int spw;         // steps per slice = steps / kw, a multiple of CH
  int sb;          // per-warp staging (kw == kWarps): steps of the slice staged at a time (spw: the whole slice;
                   // less: the slice goes through the warp's staging area block by block, see tile_body)
  int nb;          // ring stages, 1..kMaxRing
  int wide_stage;  // 1: the CTA stages the whole activation; 0: every warp its own slice
  int meta_bf16;
  uint32_t magic;
  peerpush::Push push;  // enabled: the output rows also go to every rank's window (dq_peer_push.cuh)
};

template <int BITS, int CH, bool G64 = false>
struct Ring {
  static constexpr int UNIT = 4 * BITS;
  static constexpr int GPS = G64 ? 2 : 1;                    // groups per 128-value step
  static constexpr int META = CH * GPS * 2;                  // bytes of one metadata array of one stage
  static constexpr int STAGE_W = CH * 2 * UNIT * kThreads;  // weights of one stage, whole CTA
  static constexpr int STAGE_M = META * kThreads;            // one metadata array per lane
};

// Bytes of the staging area (after ring and reduction buffers).
// `gps`: groups per 128-value step (1, or 2 with 64-value groups): the sums are per group.
template <int BITS>
__host__ __device__ inline size_t stage_bytes(int m, int steps, int spw, int kw, bool wide, int in_features,
                                              int gps = 1, int sb = 0) {
  const int na = BITS == 8 ? 32 : 16;
  if (wide) {
    const size_t stride = static_cast<size_t>(steps) * na + 4;
    return (m * stride + na) * 16 + static_cast<size_t>(steps) * 64 * gps + 16;
  }
  if (sb <= 0) sb = spw;
  const size_t stride = static_cast<size_t>(sb) * na + 4;
  return static_cast<size_t>(kw) * (sb * 256 + (m * stride + na) * 16 + sb * 64 * gps);
}

__device__ __forceinline__ void wait_pending(int n) {
  switch (n) {
    case 0: stream::cp_async_wait<0>(); break;
    case 1: stream::cp_async_wait<1>(); break;
    case 2: stream::cp_async_wait<2>(); break;
    case 3: stream::cp_async_wait<3>(); break;
    case 4: stream::cp_async_wait<4>(); break;
    case 5: stream::cp_async_wait<5>(); break;
    case 6: stream::cp_async_wait<6>(); break;
    default: stream::cp_async_wait<7>(); break;
  }
}

// One lane's fragment source of one row of one step.  Normally its 32-value unit; with
// 64-value groups the two half units (16 values of each group), 2 * UNIT bytes apart.
template <int BITS, bool G64>
__device__ __forceinline__ void read_lane_words(const unsigned char* src, uint32_t* w) {
  if constexpr (!G64) {
    stream::read_unit<BITS>(src, w);
  } else {
    constexpr int UNIT = 4 * BITS;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const unsigned char* p = src + half * 2 * UNIT;
      if constexpr (BITS == 2) {
        w[half] = *reinterpret_cast<const uint32_t*>(p);
      } else if constexpr (BITS == 4) {
        const uint2 v = *reinterpret_cast<const uint2*>(p);
        w[2 * half] = v.x, w[2 * half + 1] = v.y;
      } else {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        w[4 * half] = v.x, w[4 * half + 1] = v.y, w[4 * half + 2] = v.z, w[4 * half + 3] = v.w;
      }
    }
  }
}

// KBLK: per-warp staging goes through the staging area block by block (L.sb < L.spw).  A template
// parameter, not a test of L.sb: the three-CTA build of the plain kernel sits at its register
// limit, and the extra state in its chunk loop cost it a few hundred bytes of spills.
template <int BITS, bool XBF16, int CH, bool G64, bool KBLK = false>
__device__ __forceinline__ void tile_body(const Launch& L, const Job& J, unsigned char* smem) {
  // 64-value groups: at 2, 4 and 8 bits a lane owns 16 values of each group (HALVES: the two
  // halves of its registers are the two groups).  3-bit half units do not start on words, so
  // there a lane keeps its whole unit -- quad lanes 0,1 are the first group, 2,3 the second --
  // and every step runs its mma twice, once per group, the lanes of the other group feeding
  // a zero B fragment (QUADS).
  constexpr bool HALVES = G64 && BITS != 3;
  constexpr bool QUADS = G64 && BITS == 3;
  using Plan = MmaPlan<BITS>;
  using R = Ring<BITS, CH, G64>;
  constexpr int GPS = R::GPS;
  constexpr int NA = Plan::kARegs;
  constexpr int QU = NA / 4;
  constexpr int UNIT = R::UNIT;
  constexpr int STEP_WORDS = 4 * BITS;
  const GemvArgs& a = J.a;

  const int tid = threadIdx.x;
  const int lane = tid & (kWarp - 1);
  const int warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int kw = L.kw, rw = L.rw, spw = L.spw, nb = L.nb;
  const int rwi = warp / kw;
  const int kwi = warp - rwi * kw;
  const int s_begin = kwi * spw;
  const int nchunks = spw / CH;
  const bool has_off = a.offsets != nullptr;
  const bool wide = L.wide_stage != 0;
  const int cta = blockIdx.x - J.cta_begin;

  unsigned char* ring_w = smem;
  unsigned char* ring_m = ring_w + nb * R::STAGE_W;
  float* red = reinterpret_cast<float*>(ring_m + nb * R::STAGE_M);
  unsigned char* area = reinterpret_cast<unsigned char*>(red + kRedFloats);

  // staging area: CTA-wide (indexed by global step) or this warp's own (indexed within its slice)
  const int sb = KBLK ? L.sb : spw;  // (per-warp staging only)
  const int span = wide ? L.steps : sb;
  const int m_stride_u4 = span * NA + 4;
  unsigned short* raw;
  uint4* xb;
  float *xsum, *xneg;
  if (wide) {
    xb = reinterpret_cast<uint4*>(area);
    xsum = reinterpret_cast<float*>(xb + a.m * m_stride_u4 + NA);
    xneg = xsum + span * 8 * GPS;
    raw = nullptr;  // CTA-wide staging reads the activation straight from global memory
  } else {
    unsigned char* mine = area + kwi * (sb * 256 + (a.m * m_stride_u4 + NA) * 16 + sb * 64 * GPS);
    raw = reinterpret_cast<unsigned short*>(mine);
    xb = reinterpret_cast<uint4*>(mine + sb * 256);
    xsum = reinterpret_cast<float*>(xb + a.m * m_stride_u4 + NA);
    xneg = xsum + span * 8 * GPS;
  }

  pdl_launch_dependents();

  // ---- prefetch cursor: walks (item, chunk) ahead of the compute loop ----
  // Kept as running pointers (integer instructions issue at half rate and the decode needs
  // that pipe): what depends on the lane or the row tile is resolved once per item, a stage
  // costs one pointer bump per source row and its copies use immediate offsets.
  constexpr int PIECES = 2 * UNIT;       // 16-byte pieces of one (step, row half) block
  constexpr int PER_ROW = UNIT / 4;      // pieces per row
  constexpr int NSRC = (PIECES + kWarp - 1) / kWarp;  // pieces of a block this lane copies
  constexpr int STEP_BYTES = STEP_WORDS * 4;
  const bool meta_lane = has_off || (t & 1) == 0;
  const unsigned short* meta_arr = reinterpret_cast<const unsigned short*>((t & 1) ? a.offsets : a.scales);
  bool pf_lane[NSRC];
#pragma unroll
  for (int i = 0; i < NSRC; ++i) pf_lane[i] = (PIECES % kWarp == 0) || (i * kWarp + lane < PIECES);
  const unsigned char* pf_src[2][NSRC];  // [row half][piece]: this lane's source at the stage's first step
  const unsigned short* pf_meta = nullptr;
  int pf_item = cta, pf_chunk = 0;
  bool pf_live = false;
  auto pf_point = [&]() {  // start of an item
    const int tile = pf_item * rw + rwi;
    pf_live = pf_item < J.items && tile < J.tiles;
    if (pf_live) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int i = 0; i < NSRC; ++i) {
          const int piece = i * kWarp + lane;
          const int pg = piece / PER_ROW;
          const int part = piece - pg * PER_ROW;
          const int row = min(tile * 16 + h * 8 + pg, a.rows - 1);
          pf_src[h][i] = reinterpret_cast<const unsigned char*>(a.packed + static_cast<int64_t>(row) * a.words_per_row +
                                                                 part * 4) + s_begin * STEP_BYTES;
        }
      }
      const int row = min(tile * 16 + g + ((t & 2) ? 8 : 0), a.rows - 1);
      pf_meta = meta_arr + static_cast<int64_t>(row) * a.num_groups + s_begin * GPS;
    }
  };
  pf_point();
  const uint32_t ring_w_s = static_cast<uint32_t>(__cvta_generic_to_shared(ring_w)) + (tid - lane) * UNIT + lane * 16;
  const uint32_t ring_m_s = static_cast<uint32_t>(__cvta_generic_to_shared(ring_m)) + tid * R::META;
  uint32_t pf_w = ring_w_s, pf_m = ring_m_s;
  const uint32_t pf_w_end = ring_w_s + nb * R::STAGE_W;
  auto prefetch_stage = [&]() {
    if (pf_item < J.items) {
      if (pf_live) {
#pragma unroll
        for (int j = 0; j < CH; ++j) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int i = 0; i < NSRC; ++i) {
              if (pf_lane[i]) {
                stream::cp_async_n<16>(pf_w + (j * 2 + h) * (UNIT * kThreads) + i * (kWarp * 16), pf_src[h][i] + j * STEP_BYTES);
              }
            }
          }
        }
        if (meta_lane) stream::cp_async_n<R::META>(pf_m, pf_meta);
      }
      if (++pf_chunk == nchunks) {
        pf_chunk = 0;
        pf_item += J.cta_count;
        pf_point();
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int i = 0; i < NSRC; ++i) pf_src[h][i] += CH * STEP_BYTES;
        }
        pf_meta += CH * GPS;
      }
    }
    pf_w += R::STAGE_W;
    pf_m += R::STAGE_M;
    if (pf_w == pf_w_end) {
      pf_w = ring_w_s;
      pf_m = ring_m_s;
    }
    stream::cp_async_commit();  // an empty group keeps the wait arithmetic uniform
  };
  for (int i = 0; i < nb; ++i) prefetch_stage();  // the whole ring is in flight before the wait

  const bool b_live = g < a.m;
  const int sl0 = wide ? s_begin : 0;  // first step of this warp's slice in the staged arrays
  const uint4* xb_lane = (b_live ? xb + g * m_stride_u4 + t : xb + a.m * m_stride_u4) + (b_live ? sl0 * QU * 4 : 0);
  const int xb_step_u4 = b_live ? QU * 4 : 0;
  const float* xsum_w = xsum + sl0 * 8 * GPS + 2 * t;
  const float* xneg_w = xneg + sl0 * 8 * GPS + 2 * t;
  const unsigned char* ring_w_mine = HALVES ? ring_w + (tid & ~3) * UNIT + t * (UNIT / 2) : ring_w + tid * UNIT;
  const unsigned char* ring_m_quad = ring_m + (tid & ~3) * R::META;
  const uint32_t magic = L.magic;
  const bool mbf = L.meta_bf16 != 0;

  // ---- the part that depends on the previous kernel: the activation ----
  int parity = 0;
  // the zero fragments and zero sums of absent activation rows do not depend on the
  // activation: written now, they are off the chain that starts when the wait releases
  const bool prefilled = stage_units_ok(a);
  if (prefilled) {
    if (wide) {
      stage_zero_fill<BITS, G64>(a.m, L.steps, m_stride_u4, xb, xsum, xneg, tid, kThreads);
    } else {
      stage_zero_fill<BITS, G64>(a.m, sb, m_stride_u4, xb, xsum, xneg, lane, kWarp);
    }
  }
  pdl_wait_prior_grid();
  if (wide) {
    stage_activation<BITS, XBF16, G64>(a, L.steps, m_stride_u4, xb, xsum, xneg, tid, kThreads, nullptr, prefilled);
    __syncthreads();
  } else {
    stage_warp_slice<BITS, XBF16, G64>(a, s_begin, sb, m_stride_u4, raw, xb, xsum, xneg, lane, prefilled);
  }
  // A slice longer than the staging area (many activation rows x a long reduction axis, which
  // staged whole would not fit shared memory) passes through it `sb` steps at a time: the warp
  // re-stages at every block boundary -- its own area, so a warp barrier is all it takes.
  const bool blocked = KBLK && !wide && sb < spw;

  const unsigned char* wslot = ring_w_mine;  // ring slot being consumed
  const unsigned char* mslot = ring_m_quad;
  const unsigned char* const wslot_end = ring_w_mine + nb * R::STAGE_W;
  const int xb_chunk_u4 = xb_step_u4 * CH;
  for (int item = cta; item < J.items; item += J.cta_count, parity ^= 1) {
    const int tile = item * rw + rwi;
    const bool live = tile < J.tiles;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const uint4* bchunk = xb_lane;
    const float* xs_chunk = xsum_w;
    const float* xn_chunk = xneg_w;
    for (int chunk = 0; chunk < nchunks; ++chunk) {
      if (KBLK && blocked && (chunk * CH) % sb == 0 && (chunk != 0 || item != cta)) {
        __syncwarp();  // every lane is done reading the block that is about to be replaced
        stage_warp_slice<BITS, XBF16, G64>(a, s_begin + chunk * CH, sb, m_stride_u4, raw, xb, xsum, xneg, lane, prefilled);
        bchunk = xb_lane;
        xs_chunk = xsum_w;
        xn_chunk = xneg_w;
      }
      wait_pending(nb - 1);  // groups are consumed in issue order: all but the nb-1 youngest are done
      __syncwarp();          // copies of other lanes (units, the quad's metadata) are visible
      if (live) {
        const unsigned char* wsrc = wslot;
        const unsigned char* msrc = mslot;
        constexpr int MW = R::META / 4;  // 32-bit words of one metadata array of this stage
        uint32_t mc[4][MW];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (has_off || (i & 1) == 0) {
            if constexpr (MW == 4) {
              const uint4 v = *reinterpret_cast<const uint4*>(msrc + i * R::META);
              mc[i][0] = v.x, mc[i][1] = v.y, mc[i][2] = v.z, mc[i][3] = v.w;
            } else if constexpr (MW == 2) {
              const uint2 v = *reinterpret_cast<const uint2*>(msrc + i * R::META);
              mc[i][0] = v.x, mc[i][1] = v.y;
            } else {
              mc[i][0] = *reinterpret_cast<const uint32_t*>(msrc + i * R::META);
            }
          }
        }
#pragma unroll
        for (int j = 0; j < CH; ++j) {
          uint32_t wa[BITS], wb[BITS];
          read_lane_words<BITS, HALVES>(wsrc + (j * 2 + 0) * (UNIT * kThreads), wa);
          read_lane_words<BITS, HALVES>(wsrc + (j * 2 + 1) * (UNIT * kThreads), wb);
          uint32_t aa[NA], ab[NA];
          decode_unit<BITS>(wa, magic, aa);
          decode_unit<BITS>(wb, magic, ab);
          unbias_fragments<XBF16, NA>(aa);
          unbias_fragments<XBF16, NA>(ab);
          const uint4* bsrc = bchunk + j * xb_step_u4;
          // two accumulators: the first half of the registers (d) and the second (e).  They
          // halve the chain of dependent mma; with 64-value groups they ARE the two groups.
          float d[4], e[4];
          if constexpr (QUADS) {
            // d: the first group (this lane's B is zero unless t < 2); e: the second
            const uint4* zsrc = xb + a.m * m_stride_u4;
            const uint4* bsrc_d = (t < 2) ? bsrc : zsrc;
            const uint4* bsrc_e = (t < 2) ? zsrc : bsrc;
            const int step_d = (t < 2) ? 4 : 0, step_e = (t < 2) ? 0 : 4;
#pragma unroll
            for (int q = 0; q < QU; ++q) {
              const uint4 b0 = bsrc_d[q * step_d];
              const uint4 b1 = bsrc_e[q * step_e];
              if (q == 0) {
                mma_16816<XBF16, true>(d, aa[0], ab[0], aa[1], ab[1], b0.x, b0.y);
                mma_16816<XBF16, true>(e, aa[0], ab[0], aa[1], ab[1], b1.x, b1.y);
              } else {
                mma_16816<XBF16, false>(d, aa[4 * q], ab[4 * q], aa[4 * q + 1], ab[4 * q + 1], b0.x, b0.y);
                mma_16816<XBF16, false>(e, aa[4 * q], ab[4 * q], aa[4 * q + 1], ab[4 * q + 1], b1.x, b1.y);
              }
              mma_16816<XBF16, false>(d, aa[4 * q + 2], ab[4 * q + 2], aa[4 * q + 3], ab[4 * q + 3], b0.z, b0.w);
              mma_16816<XBF16, false>(e, aa[4 * q + 2], ab[4 * q + 2], aa[4 * q + 3], ab[4 * q + 3], b1.z, b1.w);
            }
          } else {
#pragma unroll
            for (int q = 0; q < QU / 2; ++q) {
              const uint4 b0 = bsrc[q * 4];
              const uint4 b1 = bsrc[(q + QU / 2) * 4];
              if (q == 0) {
                mma_16816<XBF16, true>(d, aa[0], ab[0], aa[1], ab[1], b0.x, b0.y);
                mma_16816<XBF16, true>(e, aa[NA / 2], ab[NA / 2], aa[NA / 2 + 1], ab[NA / 2 + 1], b1.x, b1.y);
              } else {
                mma_16816<XBF16, false>(d, aa[4 * q], ab[4 * q], aa[4 * q + 1], ab[4 * q + 1], b0.x, b0.y);
                mma_16816<XBF16, false>(e, aa[NA / 2 + 4 * q], ab[NA / 2 + 4 * q], aa[NA / 2 + 4 * q + 1],
                                        ab[NA / 2 + 4 * q + 1], b1.x, b1.y);
              }
              mma_16816<XBF16, false>(d, aa[4 * q + 2], ab[4 * q + 2], aa[4 * q + 3], ab[4 * q + 3], b0.z, b0.w);
              mma_16816<XBF16, false>(e, aa[NA / 2 + 4 * q + 2], ab[NA / 2 + 4 * q + 2], aa[NA / 2 + 4 * q + 3],
                                      ab[NA / 2 + 4 * q + 3], b1.z, b1.w);
            }
          }
          // halfword `hw` of metadata array i of this stage
          auto meta_f32 = [&](int i, int hw) -> float {
            const uint32_t reg = mc[i][hw / 2];
            if (mbf) return __uint_as_float((hw & 1) ? (reg & 0xFFFF0000u) : (reg << 16));
            const __half2 h = *reinterpret_cast<const __half2*>(&reg);
            return (hw & 1) ? __high2float(h) : __low2float(h);
          };
          if constexpr (!G64) {
#pragma unroll
            for (int i = 0; i < 4; ++i) d[i] += e[i];
            const float2 xs2 = *reinterpret_cast<const float2*>(xs_chunk + j * 8);
            const float2 xn2 = *reinterpret_cast<const float2*>(xn_chunk + j * 8);
            const float sc_a = meta_f32(0, j), sc_b = meta_f32(2, j);
            acc[0] = fmaf(sc_a, d[0] + xn2.x, acc[0]);
            acc[1] = fmaf(sc_a, d[1] + xn2.y, acc[1]);
            acc[2] = fmaf(sc_b, d[2] + xn2.x, acc[2]);
            acc[3] = fmaf(sc_b, d[3] + xn2.y, acc[3]);
            if (has_off) {
              const float of_a = meta_f32(1, j), of_b = meta_f32(3, j);
              acc[0] = fmaf(of_a, xs2.x, acc[0]);
              acc[1] = fmaf(of_a, xs2.y, acc[1]);
              acc[2] = fmaf(of_b, xs2.x, acc[2]);
              acc[3] = fmaf(of_b, xs2.y, acc[3]);
            }
          } else {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              const float* dd = half == 0 ? d : e;
              const float2 xs2 = *reinterpret_cast<const float2*>(xs_chunk + (j * 2 + half) * 8);
              const float2 xn2 = *reinterpret_cast<const float2*>(xn_chunk + (j * 2 + half) * 8);
              const float sc_a = meta_f32(0, 2 * j + half), sc_b = meta_f32(2, 2 * j + half);
              acc[0] = fmaf(sc_a, dd[0] + xn2.x, acc[0]);
              acc[1] = fmaf(sc_a, dd[1] + xn2.y, acc[1]);
              acc[2] = fmaf(sc_b, dd[2] + xn2.x, acc[2]);
              acc[3] = fmaf(sc_b, dd[3] + xn2.y, acc[3]);
              if (has_off) {
                const float of_a = meta_f32(1, 2 * j + half), of_b = meta_f32(3, 2 * j + half);
                acc[0] = fmaf(of_a, xs2.x, acc[0]);
                acc[1] = fmaf(of_a, xs2.y, acc[1]);
                acc[2] = fmaf(of_b, xs2.x, acc[2]);
                acc[3] = fmaf(of_b, xs2.y, acc[3]);
              }
            }
          }
        }
      }
      bchunk += xb_chunk_u4;
      xs_chunk += CH * 8 * GPS;
      xn_chunk += CH * 8 * GPS;
      wslot += R::STAGE_W;
      mslot += R::STAGE_M;
      if (wslot == wslot_end) {
        wslot = ring_w_mine;
        mslot = ring_m_quad;
      }
      __syncwarp();      // every lane is done with the slot just consumed:
      prefetch_stage();  // refill it
    }

    // ---- sum the slices of the reduction axis in a fixed order, store ----
    if (kw > 1) {
      float* buf = red + parity * (kWarps * 128);
      float* mine = buf + (kwi * rw + rwi) * 128;
      *reinterpret_cast<float2*>(mine + g * 8 + 2 * t) = make_float2(acc[0], acc[1]);
      *reinterpret_cast<float2*>(mine + (g + 8) * 8 + 2 * t) = make_float2(acc[2], acc[3]);
      __syncthreads();  // the other buffer is free again once every warp has passed this point
      if (kwi == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i] = 0.0f;
        for (int k = 0; k < kw; ++k) {
          const float* part = buf + (k * rw + rwi) * 128;
          const float2 pa = *reinterpret_cast<const float2*>(part + g * 8 + 2 * t);
          const float2 pb = *reinterpret_cast<const float2*>(part + (g + 8) * 8 + 2 * t);
          acc[0] += pa.x, acc[1] += pa.y, acc[2] += pb.x, acc[3] += pb.y;
        }
      }
    }
    if (kwi == 0 && live) {
      const int row_a = tile * 16 + g, row_b = row_a + 8;
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
  stream::cp_async_wait<0>();
}

// CTAS: resident CTAs per SM the kernel is compiled for.  Two (128 registers, nothing spilled)
// is the faster build; three (80 registers, a few spills) exists for launches whose single
// wave needs the third CTA per SM -- the alternative there is a coarser slicing of the
// reduction axis, which costs more than the spills.
template <bool XBF16, int CH, bool G64, int CTAS, bool KBLK = false>
__global__ void __launch_bounds__(kThreads, CTAS) gemv_mma_tile_kernel(const __grid_constant__ Launch L) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int j = 0;
#pragma unroll
  for (int i = 1; i < kMaxJobs; ++i) {
    if (i < L.njobs && static_cast<int>(blockIdx.x) >= L.job[i].cta_begin) j = i;
  }
  const Job& J = L.job[j];
  switch (J.bits) {
    case 2:
      tile_body<2, XBF16, CH, G64, KBLK>(L, J, smem_raw);
      break;
    case 3:
      tile_body<3, XBF16, CH, G64, KBLK>(L, J, smem_raw);
      break;
    case 4:
      tile_body<4, XBF16, CH, G64, KBLK>(L, J, smem_raw);
      break;
    default:
      tile_body<8, XBF16, CH, G64, KBLK>(L, J, smem_raw);
      break;
  }
  if (L.push.enabled) {
    // This CTA's items are whole runs of rw row tiles: copy them, as stored, to every window.
    // (Every thread reads the epoch itself: no static shared memory beside the tuned dynamic layout.)
    const unsigned int epoch = peerpush::next_epoch(L.push);
    __syncthreads();  // the body's output stores are visible to the whole CTA
    const int rows_per_item = L.rw * 16;
    for (int item = static_cast<int>(blockIdx.x) - J.cta_begin; item < J.items; item += J.cta_count) {
      peerpush::push_rows(L.push, J.a, epoch, item * rows_per_item, min((item + 1) * rows_per_item, J.a.rows),
                          threadIdx.x, kThreads);
    }
    __syncthreads();
    if (threadIdx.x < kWarp) peerpush::arrive(L.push, epoch, gridDim.x, threadIdx.x);
  }
}

}  // namespace tilek
}  // namespace dq
