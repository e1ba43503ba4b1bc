// Many activation rows (9..64) against one packed matrix in one pass over the weights (two from 33
// rows on) -- and the kernel for matrices the tiled kernel is a poor fit for, at any row count.
//
// The GEMV kernels take at most eight activation rows: the eight columns of one m16n8k16
// accumulator.  More rows used to mean more passes (row chunks of eight, each decoding the
// weights again, the later ones from L2).  Here a warp decodes the fragments of a 16-row x
// 128-value step ONCE and feeds them to up to four column blocks of eight activation rows each
// -- the decode, which bounds the GEMV kernels, is amortised over the blocks, and the tensor
// pipe becomes the busy unit, as it should in a small-batch matrix product.
//
//   CTA       8 warps = 8 row tiles of 16 weight rows; warp w streams its tile's rows over the
//             CTA's part of the reduction axis through a private cp.async ring (the streaming
//             kernel's plumbing: blocks of P steps, no barrier for weights).
//   cluster   matrices with too few rows for a CTA per SM (down-projections): the grid's y axis
//             slices the reduction axis, the slices of one row group are a thread-block cluster
//             and their sums meet in the cluster's first CTA through distributed shared memory.
//   x         too large to stage whole (32 rows x 4096 values in fragment order: 256 KB), so it
//             passes through shared memory in blocks of P steps shared by the CTA's warps: the raw
//             rows of block b+2 travel by cp.async while block b is computed, all threads convert
//             raw block b+1 to fragment order (unit-per-lane staging, 16-bit aligned activations
//             only) between two CTA barriers.  Up to 32 rows per launch (four column blocks).
//   out       [m, rows] as the GEMV kernels write it; accumulation in fp32, scale and offset
//             applied per step, one rounding.
//
// Because the activation never has to fit shared memory whole and the reduction axis can be cut
// in any proportion, this is also the faster kernel at 1..8 rows where the tiled kernel is not
// at home (dq_gemv_mma.cu, rows_kernel_first): step counts with few factors of two (K = 8960,
// 11008, 18944) on matrices of few rows, and activations of six to eight rows x K >= 12288.
//
// Replaces, above eight rows, the reference's dequantize + dense matmul (runtime/ops.py:205-231):
// same result up to the summation order.  The hosts (dq_gemv.cu, dq_gemv_mma.cu) fall back to row
// chunks / the tiled kernel when a matrix does not qualify.
#include <algorithm>
#include <atomic>
#include <type_traits>

#include "dq_gemv.cuh"
#include "dq_gemv_mma_stream.cuh"
#include "dq_mma_plan.cuh"
#include "dq_mma_stage.cuh"

namespace dq {
namespace rowsk {

constexpr int kWarps = stream::kWarps;
constexpr int kThreads = stream::kThreads;
constexpr int kRingBlocks = 3;  // weight blocks in a warp's ring: requested two blocks ahead
constexpr int kRawBuffers = 2;  // raw blocks of x in flight: requested two blocks ahead
constexpr int kMaxRows = 32;    // activation rows per launch (four column blocks)

struct Params {
  int steps;        // K / 128, a multiple of P (no padded tail: in_features == steps * 128)
  int tiles;        // ceil(rows / 16)
  int m_stride_u4;  // uint4 per activation row of the staged block: P * NA + 4
  int meta_bf16;
  uint32_t magic;
};

// Steps per block PP: the streaming kernel's (four at 2 / 3 / 4 bits, two at 8), or two at the low
// widths too for reduction axes whose step count is even but not a multiple of four (K = 8960,
// 11008: 70 and 86 steps) -- a row's metadata is then copied four bytes at a time.
//
// G64: 64-value groups, two per step.  A row's metadata is twice as long, the activation's sums are
// per (step, group), and a lane's fragments belong half to one group and half to the other (at 3
// bits: the quad's lane pairs hold one group each) -- the layout of dq_mma_stage.cuh -- so a step's
// mma feed two accumulators per column block, scaled separately.
template <int BITS, int PP, bool G64 = false>
struct Cfg {
  static constexpr int P = PP;
  static constexpr int GPS = G64 ? 2 : 1;  // groups per step
  static constexpr int UNIT = 4 * BITS;
  static constexpr int BLOCK_BYTES = P * 2 * UNIT;
  static constexpr int META_BYTES = 2 * P * GPS;
};

// Bytes of one column block's fragment region for one x block: 8 rows of fragments, the zero
// block that lanes of absent rows read, and the two sums per (step, row).
template <int BITS, int PP, bool G64>
__host__ __device__ constexpr size_t region_bytes() {
  using C = Cfg<BITS, PP, G64>;
  constexpr int NA = BITS == 8 ? 32 : 16;
  return (static_cast<size_t>(8) * (C::P * NA + 4) + NA) * 16 + static_cast<size_t>(C::P) * C::GPS * 8 * 4 * 2;
}
// One column block of a raw x block: 8 rows x P steps x 128 values of 16 bits.
template <int PP>
__host__ __device__ constexpr size_t raw_bytes() {
  return static_cast<size_t>(8) * PP * 256;
}

template <int BITS, int PP, bool G64>
size_t smem_bytes(int mb) {
  using C = Cfg<BITS, PP, G64>;
  return static_cast<size_t>(kRingBlocks) * (C::BLOCK_BYTES + C::META_BYTES) * kThreads +
         static_cast<size_t>(mb) * (kRawBuffers * raw_bytes<PP>() + region_bytes<BITS, PP, G64>());
}

// Pipeline of one CTA, block b of P steps:
//   weights   cp.async into the warp's ring, two blocks ahead (the streaming kernel's plumbing);
//   x, raw    cp.async of the block's rows into one of two raw buffers, two blocks ahead -- the
//             global latency of the activation is off the critical path;
//   x, frags  after compute(b): all threads convert raw(b+1) into the (single) fragment buffer,
//             between two CTA barriers;
//   compute   every warp: decode a step once, feed it to the column blocks.
//
// KSPLIT: the grid's y axis slices the reduction axis and the CTAs of one row group form a
// thread-block cluster (1 x slices): every CTA runs the pipeline over its own range of blocks,
// then the slices' sums meet in the first CTA of the cluster through distributed shared memory,
// added in slice order (a fixed summation order: same bits on every run), and that CTA stores.
// For matrices with too few rows to fill the SMs with one CTA per eight row tiles -- a
// down-projection, 4096 x 14336.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t local_addr, uint32_t cta_rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(cta_rank));
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
  return v;
}

// One lane's fragment source of one row of one step with 64-value groups at 2 / 4 / 8 bits: the two
// half units (16 values of each group), 2 * UNIT bytes apart.
template <int BITS>
__device__ __forceinline__ void read_half_units(const unsigned char* src, uint32_t* w) {
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const unsigned char* q = src + half * 2 * (4 * BITS);
    if constexpr (BITS == 2) {
      w[half] = *reinterpret_cast<const uint32_t*>(q);
    } else if constexpr (BITS == 4) {
      const uint2 v = *reinterpret_cast<const uint2*>(q);
      w[2 * half] = v.x, w[2 * half + 1] = v.y;
    } else {
      const uint4 v = *reinterpret_cast<const uint4*>(q);
      w[4 * half] = v.x, w[4 * half + 1] = v.y, w[4 * half + 2] = v.z, w[4 * half + 3] = v.w;
    }
  }
}

template <int BITS, bool XBF16, int MB, bool KSPLIT, int PP, bool G64>
__global__ void __launch_bounds__(kThreads, 1) gemv_rows_kernel(const GemvArgs a, const Params p) {
  using Plan = MmaPlan<BITS>;
  using C = Cfg<BITS, PP, G64>;
  constexpr int GPS = C::GPS;
  constexpr bool HALVES = G64 && BITS != 3;  // groups = halves of a lane's registers
  [[maybe_unused]] constexpr bool QUADS = G64 && BITS == 3;  // groups = the quad's lane pairs
  constexpr int P = C::P;
  constexpr int NB = kRingBlocks;
  constexpr int NA = Plan::kARegs;
  constexpr int QU = NA / 4;
  constexpr int STEP_WORDS = 4 * BITS;
  constexpr int STEP_BYTES = STEP_WORDS * 4;
  constexpr size_t REGION = region_bytes<BITS, PP, G64>();
  constexpr size_t RAW = raw_bytes<PP>();

  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned char* ring_w = smem_raw;
  unsigned char* ring_m = ring_w + NB * C::BLOCK_BYTES * kThreads;
  unsigned char* raw = ring_m + NB * C::META_BYTES * kThreads;   // [kRawBuffers][MB][8 rows][P * 128] 16-bit
  unsigned char* frag = raw + kRawBuffers * MB * RAW;            // [MB] regions

  const int tid = threadIdx.x;
  const int lane = tid & (kWarp - 1);
  const int warp = tid >> 5;
  const int g = lane >> 2;
  const int t = lane & 3;
  const uint32_t magic = p.magic;
  const bool mbf = p.meta_bf16 != 0;
  const bool has_off = a.offsets != nullptr;
  const int nblocks = p.steps / P;
  const int tile = blockIdx.x * kWarps + warp;
  const bool live = tile < p.tiles;
  const int mbs = (a.m + 7) / 8;  // column blocks that have rows (the kernel is built for 2 or 4)
  // this CTA's range of blocks of the reduction axis (all of them without KSPLIT)
  const int slices = KSPLIT ? static_cast<int>(cluster_nctarank()) : 1;
  const int slice = KSPLIT ? static_cast<int>(cluster_ctarank()) : 0;
  const int blk_begin = KSPLIT ? (nblocks * slice) / slices : 0;
  const int blk_end = KSPLIT ? (nblocks * (slice + 1)) / slices : nblocks;

  const uint32_t ring_w_s = static_cast<uint32_t>(__cvta_generic_to_shared(ring_w)) + (tid - lane) * C::UNIT;
  const uint32_t ring_m_s = static_cast<uint32_t>(__cvta_generic_to_shared(ring_m)) + tid * C::META_BYTES;
  const uint32_t raw_s = static_cast<uint32_t>(__cvta_generic_to_shared(raw));
  const unsigned char* ring_w_mine = HALVES ? ring_w + (tid & ~3) * C::UNIT + t * (C::UNIT / 2) : ring_w + tid * C::UNIT;
  const unsigned char* ring_m_quad = ring_m + (tid & ~3) * C::META_BYTES;

  pdl_launch_dependents();

  // ---- weights: prefetch cursor over the blocks of this warp's tile ----
  constexpr int PIECES = 2 * C::UNIT;
  constexpr int PER_ROW = C::UNIT / 4;
  constexpr int NSRC = (PIECES + kWarp - 1) / kWarp;
  const unsigned char* pf_src[2][NSRC];
  bool pf_lane[NSRC];
#pragma unroll
  for (int i = 0; i < NSRC; ++i) pf_lane[i] = (PIECES % kWarp == 0) || (i * kWarp + lane < PIECES);
  const unsigned short* pf_meta = nullptr;
  if (live) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
      for (int i = 0; i < NSRC; ++i) {
        const int piece = i * kWarp + lane;
        const int pg = piece / PER_ROW;
        const int part = piece - pg * PER_ROW;
        const int row = min(tile * 16 + h * 8 + pg, a.rows - 1);
        pf_src[h][i] = reinterpret_cast<const unsigned char*>(a.packed + static_cast<int64_t>(row) * a.words_per_row + part * 4) +
                       static_cast<size_t>(blk_begin) * P * STEP_BYTES;
      }
    }
    const int ra = min(tile * 16 + g, a.rows - 1);
    const int rb = min(tile * 16 + g + 8, a.rows - 1);
    const unsigned short* arr = reinterpret_cast<const unsigned short*>((t & 1) ? a.offsets : a.scales);
    pf_meta = arr + static_cast<int64_t>((t & 2) ? rb : ra) * a.num_groups + blk_begin * P * GPS;
  }
  const bool meta_lane = has_off || (t & 1) == 0;
  uint32_t pf_w = ring_w_s + lane * 16, pf_m = ring_m_s;
  const uint32_t ring_w_end = ring_w_s + lane * 16 + NB * (C::BLOCK_BYTES * kThreads);
  int pf_blk = blk_begin;
  auto prefetch_weights = [&]() {  // (no commit: the caller commits weights and raw x together)
    if (live && pf_blk < blk_end) {
#pragma unroll
      for (int j = 0; j < P; ++j) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int i = 0; i < NSRC; ++i) {
            if (pf_lane[i]) {
              stream::cp_async_n<16>(pf_w + (j * 2 + h) * (C::UNIT * kThreads) + i * (kWarp * 16), pf_src[h][i] + j * STEP_BYTES);
            }
          }
        }
      }
      if (meta_lane) stream::cp_async_n<C::META_BYTES>(pf_m, pf_meta);
      ++pf_blk;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int i = 0; i < NSRC; ++i) pf_src[h][i] += P * STEP_BYTES;
      }
      pf_meta += P * GPS;
    }
    pf_w += C::BLOCK_BYTES * kThreads;
    pf_m += C::META_BYTES * kThreads;
    if (pf_w == ring_w_end) {
      pf_w -= NB * (C::BLOCK_BYTES * kThreads);
      pf_m -= NB * (C::META_BYTES * kThreads);
    }
  };

  // ---- x, raw: block `blk` of every existing row into raw buffer blk % kRawBuffers, 16 bytes a piece ----
  constexpr int kRowPieces = P * 16;  // 16-byte pieces of one row of one block
  auto request_raw = [&](int blk) {
    if (blk < blk_end) {
      const uint32_t dst0 = raw_s + static_cast<uint32_t>((blk % kRawBuffers) * MB * RAW);
      const unsigned char* src0 = static_cast<const unsigned char*>(a.x) + static_cast<size_t>(blk) * P * 256;
      const int pieces = a.m * kRowPieces;  // (raw rows are laid out 8 per column block, back to back: row r at r * P * 256)
      for (int i = tid; i < pieces; i += kThreads) {
        const int r = i / kRowPieces, c = i - r * kRowPieces;
        stream::cp_async_n<16>(dst0 + r * (P * 256) + c * 16, src0 + static_cast<size_t>(r) * a.in_features * 2 + c * 16);
      }
    }
  };

  // ---- x, fragments: raw buffer of block `blk` -> the fragment regions; thread groups of 32 * P
  // threads (one (row, step, quad lane) task per thread) take the column blocks in turn ----
  constexpr int kGroupThreads = 32 * P;
  constexpr int kGroups = kThreads / kGroupThreads;
  const int sg = tid / kGroupThreads, stid = tid - sg * kGroupThreads;
  auto convert = [&](int blk) {
    for (int cb = sg; cb < mbs; cb += kGroups) {
      unsigned char* region = frag + cb * REGION;
      uint4* xb = reinterpret_cast<uint4*>(region);
      float* xsum = reinterpret_cast<float*>(xb + 8 * p.m_stride_u4 + NA);
      float* xneg = xsum + P * GPS * 8;
      GemvArgs sub = {};
      sub.x = raw + (static_cast<size_t>(blk % kRawBuffers) * MB + cb) * RAW;
      sub.x_dtype = a.x_dtype;
      sub.in_features = P * 128;  // the raw block's row pitch
      sub.m = min(8, a.m - cb * 8);
      // (rows that do not exist: their fragments are the zero block, which sits after row `m`)
      stage_units<BITS, XBF16, G64, true>(sub, 0, P, p.m_stride_u4, xb, xsum, xneg, stid, kGroupThreads, nullptr, false);
    }
  };

  // prologue: weights do not depend on the previous kernel, x does
  prefetch_weights();
  stream::cp_async_commit();
  prefetch_weights();
  pdl_wait_prior_grid();
  request_raw(blk_begin);
  stream::cp_async_commit();
  request_raw(blk_begin + 1);
  stream::cp_async_commit();
  // groups so far: {w0}, {w1, raw0}, {raw1}; from here on one group per block: {w(b+2), raw(b+2)}
  stream::cp_async_wait<1>();  // raw0 (and w0, w1)
  __syncthreads();
  convert(blk_begin);
  __syncthreads();

  float acc[MB][4];
#pragma unroll
  for (int cb = 0; cb < MB; ++cb) {
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[cb][i] = 0.0f;
  }
  const unsigned char* wslot = ring_w_mine;
  const unsigned char* mslot = ring_m_quad;
  const unsigned char* const wslot_end = ring_w_mine + NB * (C::BLOCK_BYTES * kThreads);
  for (int blk = blk_begin; blk < blk_end; ++blk) {
    __syncwarp();  // every lane is done with the ring slot about to be refilled
    prefetch_weights();
    request_raw(blk + 2);  // into the buffer raw(blk) was converted from
    stream::cp_async_commit();
    stream::cp_async_wait<2>();  // all but the two youngest groups: w(blk) is in
    __syncwarp();
    if (live) {
      constexpr int MW = C::META_BYTES / 4;  // 32-bit words of one metadata array of a block
      uint32_t mc[4][MW];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (has_off || (i & 1) == 0) {
          if constexpr (MW == 4) {
            const uint4 v = *reinterpret_cast<const uint4*>(mslot + i * C::META_BYTES);
            mc[i][0] = v.x, mc[i][1] = v.y, mc[i][2] = v.z, mc[i][3] = v.w;
          } else if constexpr (MW == 2) {
            const uint2 v = *reinterpret_cast<const uint2*>(mslot + i * C::META_BYTES);
            mc[i][0] = v.x, mc[i][1] = v.y;
          } else {
            mc[i][0] = *reinterpret_cast<const uint32_t*>(mslot + i * C::META_BYTES);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < P; ++j) {
        uint32_t wa[BITS], wb[BITS];
        if constexpr (HALVES) {
          read_half_units<BITS>(wslot + (j * 2 + 0) * (C::UNIT * kThreads), wa);
          read_half_units<BITS>(wslot + (j * 2 + 1) * (C::UNIT * kThreads), wb);
        } else {
          stream::read_unit<BITS>(wslot + (j * 2 + 0) * (C::UNIT * kThreads), wa);
          stream::read_unit<BITS>(wslot + (j * 2 + 1) * (C::UNIT * kThreads), wb);
        }
        uint32_t aa[NA], ab[NA];
        decode_unit<BITS>(wa, magic, aa);
        decode_unit<BITS>(wb, magic, ab);
        unbias_fragments<XBF16, NA>(aa);
        unbias_fragments<XBF16, NA>(ab);
        // halfword `hw` of metadata array i of this block
        auto meta_f32 = [&](int i, int hw) -> float {
          const uint32_t reg = mc[i][hw / 2];
          if (mbf) return __uint_as_float((hw & 1) ? (reg & 0xFFFF0000u) : (reg << 16));
          const __half2 hh = *reinterpret_cast<const __half2*>(&reg);
          return (hw & 1) ? __high2float(hh) : __low2float(hh);
        };
        // The column blocks' accumulators are independent: their mma are interleaved, so that a
        // warp has MB chains in flight instead of one chain of 2 * QU dependent mma per block
        // (with eight warps on the SM nothing else would hide that latency).
        float d[MB][4];
        const uint4* bsrc[MB];
        int bstep[MB];
#pragma unroll
        for (int cb = 0; cb < MB; ++cb) {
          const uint4* xb = reinterpret_cast<const uint4*>(frag + cb * REGION);
          const int m_here = a.m - cb * 8;  // rows of this column block that exist (<= 0: none, the zero block)
          const bool mine = g < m_here;
          bsrc[cb] = mine ? xb + g * p.m_stride_u4 + t + j * (QU * 4) : xb + max(0, min(m_here, 8)) * p.m_stride_u4;
          bstep[cb] = mine ? 4 : 0;
        }
        if constexpr (!G64) {
#pragma unroll
          for (int q = 0; q < QU; ++q) {
            uint4 b[MB];
#pragma unroll
            for (int cb = 0; cb < MB; ++cb) b[cb] = bsrc[cb][q * bstep[cb]];
#pragma unroll
            for (int cb = 0; cb < MB; ++cb) {
              if (q == 0) {
                mma_16816<XBF16, true>(d[cb], aa[0], ab[0], aa[1], ab[1], b[cb].x, b[cb].y);
              } else {
                mma_16816<XBF16, false>(d[cb], aa[4 * q], ab[4 * q], aa[4 * q + 1], ab[4 * q + 1], b[cb].x, b[cb].y);
              }
            }
#pragma unroll
            for (int cb = 0; cb < MB; ++cb) {
              mma_16816<XBF16, false>(d[cb], aa[4 * q + 2], ab[4 * q + 2], aa[4 * q + 3], ab[4 * q + 3], b[cb].z, b[cb].w);
            }
          }
          const float sc_a = meta_f32(0, j), sc_b = meta_f32(2, j);
          const float of_a = has_off ? meta_f32(1, j) : 0.0f, of_b = has_off ? meta_f32(3, j) : 0.0f;
#pragma unroll
          for (int cb = 0; cb < MB; ++cb) {
            const uint4* xb = reinterpret_cast<const uint4*>(frag + cb * REGION);
            const float* xsum = reinterpret_cast<const float*>(xb + 8 * p.m_stride_u4 + NA);
            const float* xneg = xsum + P * 8;
            const float2 xs2 = *reinterpret_cast<const float2*>(xsum + j * 8 + 2 * t);
            const float2 xn2 = *reinterpret_cast<const float2*>(xneg + j * 8 + 2 * t);
            acc[cb][0] = fmaf(sc_a, d[cb][0] + xn2.x, acc[cb][0]);
            acc[cb][1] = fmaf(sc_a, d[cb][1] + xn2.y, acc[cb][1]);
            acc[cb][2] = fmaf(sc_b, d[cb][2] + xn2.x, acc[cb][2]);
            acc[cb][3] = fmaf(sc_b, d[cb][3] + xn2.y, acc[cb][3]);
            if (has_off) {
              acc[cb][0] = fmaf(of_a, xs2.x, acc[cb][0]);
              acc[cb][1] = fmaf(of_a, xs2.y, acc[cb][1]);
              acc[cb][2] = fmaf(of_b, xs2.x, acc[cb][2]);
              acc[cb][3] = fmaf(of_b, xs2.y, acc[cb][3]);
            }
          }
        } else {
          // two accumulators per column block: d the step's first group, e its second
          float e[MB][4];
          if constexpr (HALVES) {  // the first half of a lane's registers is the first group's
#pragma unroll
            for (int q = 0; q < QU / 2; ++q) {
              uint4 b0[MB], b1[MB];
#pragma unroll
              for (int cb = 0; cb < MB; ++cb) {
                b0[cb] = bsrc[cb][q * bstep[cb]];
                b1[cb] = bsrc[cb][(q + QU / 2) * bstep[cb]];
              }
#pragma unroll
              for (int cb = 0; cb < MB; ++cb) {
                if (q == 0) {
                  mma_16816<XBF16, true>(d[cb], aa[0], ab[0], aa[1], ab[1], b0[cb].x, b0[cb].y);
                  mma_16816<XBF16, true>(e[cb], aa[NA / 2], ab[NA / 2], aa[NA / 2 + 1], ab[NA / 2 + 1], b1[cb].x, b1[cb].y);
                } else {
                  mma_16816<XBF16, false>(d[cb], aa[4 * q], ab[4 * q], aa[4 * q + 1], ab[4 * q + 1], b0[cb].x, b0[cb].y);
                  mma_16816<XBF16, false>(e[cb], aa[NA / 2 + 4 * q], ab[NA / 2 + 4 * q], aa[NA / 2 + 4 * q + 1], ab[NA / 2 + 4 * q + 1],
                                          b1[cb].x, b1[cb].y);
                }
              }
#pragma unroll
              for (int cb = 0; cb < MB; ++cb) {
                mma_16816<XBF16, false>(d[cb], aa[4 * q + 2], ab[4 * q + 2], aa[4 * q + 3], ab[4 * q + 3], b0[cb].z, b0[cb].w);
                mma_16816<XBF16, false>(e[cb], aa[NA / 2 + 4 * q + 2], ab[NA / 2 + 4 * q + 2], aa[NA / 2 + 4 * q + 3],
                                        ab[NA / 2 + 4 * q + 3], b1[cb].z, b1[cb].w);
              }
            }
          } else {  // QUADS: lanes 0,1 of a quad hold the first group, 2,3 the second; the other pair feeds a zero B
#pragma unroll
            for (int q = 0; q < QU; ++q) {
              uint4 b0[MB], b1[MB];
#pragma unroll
              for (int cb = 0; cb < MB; ++cb) {
                const uint4 v = bsrc[cb][q * bstep[cb]];
                const uint4 z = make_uint4(0u, 0u, 0u, 0u);
                b0[cb] = (t < 2) ? v : z;
                b1[cb] = (t < 2) ? z : v;
              }
#pragma unroll
              for (int cb = 0; cb < MB; ++cb) {
                if (q == 0) {
                  mma_16816<XBF16, true>(d[cb], aa[0], ab[0], aa[1], ab[1], b0[cb].x, b0[cb].y);
                  mma_16816<XBF16, true>(e[cb], aa[0], ab[0], aa[1], ab[1], b1[cb].x, b1[cb].y);
                } else {
                  mma_16816<XBF16, false>(d[cb], aa[4 * q], ab[4 * q], aa[4 * q + 1], ab[4 * q + 1], b0[cb].x, b0[cb].y);
                  mma_16816<XBF16, false>(e[cb], aa[4 * q], ab[4 * q], aa[4 * q + 1], ab[4 * q + 1], b1[cb].x, b1[cb].y);
                }
              }
#pragma unroll
              for (int cb = 0; cb < MB; ++cb) {
                mma_16816<XBF16, false>(d[cb], aa[4 * q + 2], ab[4 * q + 2], aa[4 * q + 3], ab[4 * q + 3], b0[cb].z, b0[cb].w);
                mma_16816<XBF16, false>(e[cb], aa[4 * q + 2], ab[4 * q + 2], aa[4 * q + 3], ab[4 * q + 3], b1[cb].z, b1[cb].w);
              }
            }
          }
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const float sc_a = meta_f32(0, 2 * j + half), sc_b = meta_f32(2, 2 * j + half);
            const float of_a = has_off ? meta_f32(1, 2 * j + half) : 0.0f, of_b = has_off ? meta_f32(3, 2 * j + half) : 0.0f;
#pragma unroll
            for (int cb = 0; cb < MB; ++cb) {
              const float* dd = half == 0 ? d[cb] : e[cb];
              const uint4* xb = reinterpret_cast<const uint4*>(frag + cb * REGION);
              const float* xsum = reinterpret_cast<const float*>(xb + 8 * p.m_stride_u4 + NA);
              const float* xneg = xsum + P * GPS * 8;
              const float2 xs2 = *reinterpret_cast<const float2*>(xsum + (j * 2 + half) * 8 + 2 * t);
              const float2 xn2 = *reinterpret_cast<const float2*>(xneg + (j * 2 + half) * 8 + 2 * t);
              acc[cb][0] = fmaf(sc_a, dd[0] + xn2.x, acc[cb][0]);
              acc[cb][1] = fmaf(sc_a, dd[1] + xn2.y, acc[cb][1]);
              acc[cb][2] = fmaf(sc_b, dd[2] + xn2.x, acc[cb][2]);
              acc[cb][3] = fmaf(sc_b, dd[3] + xn2.y, acc[cb][3]);
              if (has_off) {
                acc[cb][0] = fmaf(of_a, xs2.x, acc[cb][0]);
                acc[cb][1] = fmaf(of_a, xs2.y, acc[cb][1]);
                acc[cb][2] = fmaf(of_b, xs2.x, acc[cb][2]);
                acc[cb][3] = fmaf(of_b, xs2.y, acc[cb][3]);
              }
            }
          }
        }
      }
    }
    wslot += C::BLOCK_BYTES * kThreads;
    mslot += C::META_BYTES * kThreads;
    if (wslot == wslot_end) {
      wslot = ring_w_mine;
      mslot = ring_m_quad;
    }
    if (blk + 1 < blk_end) {
      stream::cp_async_wait<1>();  // all but the youngest group: raw(blk + 1) is in
      __syncthreads();             // ... for every thread's pieces; and every warp is done with the fragments
      convert(blk + 1);
      __syncthreads();
    }
  }
  stream::cp_async_wait<0>();
  if constexpr (KSPLIT) {
    // Every CTA leaves its sums in its own shared memory ([MB][thread] float4, over the ring, which
    // nobody reads any more); the cluster's first CTA adds them to its own in slice order.  Both
    // cluster barriers are reached by every thread of every CTA: the second keeps a CTA's shared
    // memory alive until the first CTA has read it.
    __syncthreads();
    float4* mine = reinterpret_cast<float4*>(smem_raw);
#pragma unroll
    for (int cb = 0; cb < MB; ++cb) mine[cb * kThreads + tid] = make_float4(acc[cb][0], acc[cb][1], acc[cb][2], acc[cb][3]);
    cluster_sync_all();
    if (slice == 0 && live) {
      const uint32_t base = static_cast<uint32_t>(__cvta_generic_to_shared(smem_raw));
      for (int r = 1; r < slices; ++r) {
#pragma unroll
        for (int cb = 0; cb < MB; ++cb) {
          const float4 v = ld_cluster_f4(base + (cb * kThreads + tid) * 16, static_cast<uint32_t>(r));
          acc[cb][0] += v.x, acc[cb][1] += v.y, acc[cb][2] += v.z, acc[cb][3] += v.w;
        }
      }
    }
    cluster_sync_all();
    if (slice != 0) return;
  }
  if (live) {
    const int row_a = tile * 16 + g, row_b = row_a + 8;
#pragma unroll
    for (int cb = 0; cb < MB; ++cb) {
      const int m0 = cb * 8 + 2 * t;
      if (m0 < a.m) {
        if (row_a < a.rows) store_out(a, m0, row_a, acc[cb][0]);
        if (row_b < a.rows) store_out(a, m0, row_b, acc[cb][2]);
      }
      if (m0 + 1 < a.m) {
        if (row_a < a.rows) store_out(a, m0 + 1, row_a, acc[cb][1]);
        if (row_b < a.rows) store_out(a, m0 + 1, row_b, acc[cb][3]);
      }
    }
  }
}

// Clusters of `slices` CTAs of this kernel that the device holds at once (cached per kernel and
// size: the query costs microseconds on a path whose launches take as long).
// (TAG names the kernel build: every build has the same pointer type, so the type cannot.)
template <int TAG, typename Kernel>
int active_clusters(Kernel kernel, const cudaLaunchConfig_t& base, int slices) {
  static std::atomic<int> cache[9] = {{-1}, {-1}, {-1}, {-1}, {-1}, {-1}, {-1}, {-1}, {-1}};
  int n = cache[slices].load(std::memory_order_relaxed);
  if (n >= 0) return n;
  cudaLaunchConfig_t cfg = base;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = static_cast<unsigned>(slices);
  attr[0].val.clusterDim.z = 1;
  cfg.gridDim.y = static_cast<unsigned>(slices);
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
    (void)cudaGetLastError();
    n = 0;
  }
  cache[slices].store(n, std::memory_order_relaxed);
  return n;
}

// max_slices > 1: slice the reduction axis over a cluster.  The slice count is the largest one
// (<= max_slices) whose clusters are all resident at once -- a second wave costs more than fewer
// slices do (measured: 4096 x 14336, 32 row groups: 19 us with 4 slices, 36 with 8; clusters of
// eight one-CTA-per-SM blocks also pack badly into the GPCs) -- and that still gives a CTA to half
// of the SMs; `forced` takes max_slices as it is.
template <int BITS, int MB, int PP, bool G64>
int32_t launch_mb(const GemvArgs& a, const Params& p, int max_slices, bool forced, const DeviceInfo& dev, cudaStream_t stream_h, bool* taken) {
  const size_t smem = smem_bytes<BITS, PP, G64>(MB);
  if (smem > static_cast<size_t>(dev.max_smem_optin)) return DQ_OK;  // not taken
  const int row_ctas = static_cast<int>(ceil_div(p.tiles, kWarps));
  auto run = [&](auto kernel, auto tag) -> int32_t {
    constexpr int TAG = decltype(tag)::value;
    DQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(row_ctas));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream_h;
    int slices = 1;
    if (max_slices > 1) {
      if (forced) {
        if (active_clusters<TAG>(kernel, cfg, max_slices) < 1) return DQ_OK;
        slices = max_slices;
      } else {
        for (int s = max_slices; s >= 2 && slices == 1; --s) {
          if (active_clusters<TAG>(kernel, cfg, s) >= row_ctas) slices = s;
        }
        // ... and of the counts with the same longest slice, the smallest: same critical path, fewer CTAs
        const int nblocks = p.steps / PP;
        while (slices > 2 && ceil_div(nblocks, slices - 1) == ceil_div(nblocks, slices)) --slices;
        if (slices == 1 || row_ctas * slices * 2 < dev.sm_count) return DQ_OK;  // not taken: the row chunks are faster
      }
    }
    cfg.gridDim.y = static_cast<unsigned>(slices);
    cudaLaunchAttribute attr[2];
    int nattr = 0;
    if (slices > 1) {  // the slices of one row group: one cluster
      attr[nattr].id = cudaLaunchAttributeClusterDimension;
      attr[nattr].val.clusterDim.x = 1;
      attr[nattr].val.clusterDim.y = static_cast<unsigned>(slices);
      attr[nattr].val.clusterDim.z = 1;
      ++nattr;
    }
    if (pdl_enabled_for_rows()) {
      attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[nattr].val.programmaticStreamSerializationAllowed = 1;
      ++nattr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = nattr;
    DQ_CUDA(cudaLaunchKernelEx(&cfg, kernel, a, p));
    DQ_CHECK_LAUNCH("gemv rows");
    note_kernel("gemv_rows_kernel");
    *taken = true;
    return DQ_OK;
  };
  using Bf16 = std::integral_constant<int, BITS * 10000 + MB * 1000 + PP * 100 + (G64 ? 10 : 0) + 1>;
  using F16 = std::integral_constant<int, BITS * 10000 + MB * 1000 + PP * 100 + (G64 ? 10 : 0)>;
  if (max_slices > 1) {
    return a.x_dtype == DQ_BF16 ? run(gemv_rows_kernel<BITS, true, MB, true, PP, G64>, Bf16{})
                                : run(gemv_rows_kernel<BITS, false, MB, true, PP, G64>, F16{});
  }
  return a.x_dtype == DQ_BF16 ? run(gemv_rows_kernel<BITS, true, MB, false, PP, G64>, Bf16{})
                              : run(gemv_rows_kernel<BITS, false, MB, false, PP, G64>, F16{});
}

template <int BITS, int PP, bool G64>
int32_t launch_blocks(const GemvArgs& a, int want_slices, bool forced, const DeviceInfo& dev, cudaStream_t stream_h, bool* taken) {
  using C = Cfg<BITS, PP, G64>;
  const int steps = a.words_per_row / (4 * BITS);
  if (steps % C::P != 0 || a.num_groups != steps * C::GPS || a.in_features != steps * 128) return DQ_OK;
  const auto align = static_cast<uintptr_t>(C::META_BYTES);
  if (reinterpret_cast<uintptr_t>(a.scales) % align != 0 || reinterpret_cast<uintptr_t>(a.offsets) % align != 0 ||
      (static_cast<int64_t>(a.num_groups) * 2) % C::META_BYTES != 0) {
    return DQ_OK;
  }
  Params p = {};
  p.steps = steps;
  p.tiles = static_cast<int>(ceil_div(a.rows, 16));
  p.m_stride_u4 = C::P * (BITS == 8 ? 32 : 16) + 4;
  p.meta_bf16 = a.meta_dtype == DQ_BF16 ? 1 : 0;
  p.magic = a.x_dtype == DQ_BF16 ? 0x43004300u : 0x64006400u;
  // slices of the reduction axis: at least two blocks each (the pipeline's prologue requests two)
  const int slices = std::max(1, std::min(want_slices, (steps / C::P) / 2));
  if (want_slices > 1 && slices < 2) return DQ_OK;  // too short to slice, too few rows not to
  // at most kMaxRows rows per launch (four column blocks; two with 64-value groups, whose second
  // accumulator per column block would not fit the registers): more rows, more passes
  const size_t x_row = static_cast<size_t>(a.in_features) * 2, out_row = static_cast<size_t>(a.out_stride) * dtype_size(a.out_dtype);
  const int passes = static_cast<int>(ceil_div(a.m, G64 ? kMaxRows / 2 : kMaxRows));
  const int per = static_cast<int>(ceil_div(a.m, passes));
  for (int r0 = 0; r0 < a.m; r0 += per) {
    GemvArgs part = a;
    part.m = std::min(per, a.m - r0);
    part.x = static_cast<const unsigned char*>(a.x) + r0 * x_row;
    part.out = static_cast<unsigned char*>(a.out) + r0 * out_row;
    bool ok = false;
    int32_t rc;
    if (part.m <= 8) {
      rc = launch_mb<BITS, 1, PP, G64>(part, p, slices, forced, dev, stream_h, &ok);
    } else if (part.m <= 16) {
      rc = launch_mb<BITS, 2, PP, G64>(part, p, slices, forced, dev, stream_h, &ok);
    } else if constexpr (!G64) {
      rc = launch_mb<BITS, 4, PP, false>(part, p, slices, forced, dev, stream_h, &ok);
    } else {
      rc = DQ_OK;  // (not reached: passes of at most 16 rows)
    }
    if (rc != DQ_OK) return rc;
    if (!ok) return r0 == 0 ? DQ_OK : fail(DQ_ERR_UNSUPPORTED, "gemv rows: the second pass did not fit shared memory");
  }
  *taken = true;
  return DQ_OK;
}

// Blocks of the streaming kernel's size where the step count allows, of two steps otherwise.
template <int BITS>
int32_t launch_bits(const GemvArgs& a, int want_slices, bool forced, const DeviceInfo& dev, cudaStream_t stream_h, bool* taken) {
  constexpr int P = stream::Cfg<BITS>::P;
  const int steps = a.words_per_row / (4 * BITS);
  const bool g64 = a.group_values == 64;
  if constexpr (P > 2) {
    if (steps % P != 0) {
      return g64 ? launch_blocks<BITS, 2, true>(a, want_slices, forced, dev, stream_h, taken)
                 : launch_blocks<BITS, 2, false>(a, want_slices, forced, dev, stream_h, taken);
    }
  }
  return g64 ? launch_blocks<BITS, P, true>(a, want_slices, forced, dev, stream_h, taken)
             : launch_blocks<BITS, P, false>(a, want_slices, forced, dev, stream_h, taken);
}

}  // namespace rowsk

// min_rows..64 activation rows, one matrix, one pass.  *taken stays false (nothing launched) when
// the matrix or the activation does not qualify: the caller then runs row chunks (or, below nine
// rows, the tiled kernel).
int32_t launch_gemv_rows(const GemvArgs& a, int bits, cudaStream_t stream, bool* taken, int min_rows) {
  *taken = false;
  const DeviceInfo* dev = device_info();
  if (dev == nullptr) return DQ_ERR_CUDA;
  if (a.m < min_rows || a.m > 64) return DQ_OK;
  // Where this kernel wins (measured on B200 against row chunks, 2/4/8 bits): matrices with a CTA
  // for at least two thirds of the SMs -- 14336 x 4096: 19.5 / 19.9 / 37.9 us against 25.4 / 26.0 /
  // 41.7 at 16 rows, 31 / 32 / 55 against 50 / 51 / 82 at 32 rows, 61 / 63 / 110 against 100 / 102 /
  // 164 at 64 rows.  On 4096 x 4096 (32 CTAs of eight row tiles on 148 SMs) the chunks are faster
  // (10 against 19 us at 16 rows): every CTA converts the whole activation for its own tiles, so
  // smaller CTAs do not pay either.
  // Matrices with fewer rows than that and a long reduction axis (a down-projection, 4096 x 14336)
  // slice the reduction axis over a cluster of up to eight CTAs per row group instead.
  const int rows_switch = tuning_int("DQ_B200_ROWS_KERNEL", -1);
  if (rows_switch == 0) return DQ_OK;
  const int64_t row_ctas = ceil_div(a.rows, 16 * rowsk::kWarps);
  int slices = 1;
  if (row_ctas * 3 < static_cast<int64_t>(dev->sm_count) * 2) {
    slices = static_cast<int>(std::min<int64_t>(8, dev->sm_count / row_ctas));
  }
  const int forced_slices = tuning_int("DQ_B200_ROWS_SLICES", -1);  // 0: never slice; n: n slices
  if (forced_slices == 0 && slices > 1) {
    if (rows_switch != 1) return DQ_OK;
    slices = 1;
  }
  if (forced_slices > 0) slices = std::min(8, forced_slices);
  const bool forced = rows_switch == 1 || forced_slices > 0;
  if (a.x_dtype != DQ_BF16 && a.x_dtype != DQ_F16) return DQ_OK;
  if (a.meta_dtype != DQ_BF16 && a.meta_dtype != DQ_F16) return DQ_OK;
  if (a.group_values != 128 && a.group_values != 64) return DQ_OK;
  if ((a.in_features & 7) != 0 || (reinterpret_cast<uintptr_t>(a.x) & 15) != 0) return DQ_OK;  // unit-per-lane staging
  if (reinterpret_cast<uintptr_t>(a.packed) % 16 != 0 || (static_cast<int64_t>(a.words_per_row) * 4) % 16 != 0) return DQ_OK;
  switch (bits) {
    case 2:
      return rowsk::launch_bits<2>(a, slices, forced, *dev, stream, taken);
    case 3:
      return rowsk::launch_bits<3>(a, slices, forced, *dev, stream, taken);
    case 4:
      return rowsk::launch_bits<4>(a, slices, forced, *dev, stream, taken);
    default:
      return rowsk::launch_bits<8>(a, slices, forced, *dev, stream, taken);
  }
}

}  // namespace dq
