// Streaming variant of the tensor-core GEMV: the kernel every large matrix takes.
//
// Same arithmetic as gemv_mma_kernel (dq_gemv_mma.cu), different plumbing.  The
// weights do not wait in registers: each lane copies the words it will decode
// with cp.async into a slot of shared memory that only it reads back, two to
// three blocks of four steps ahead.  That keeps ~128 bytes per lane in flight
// at a cost of zero registers, so three CTAs of eight warps fit on an SM and
// the copies of one warp cover the load latency of the others.  No barrier is
// involved for the weights (a lane waits on its own cp.async groups only); the
// per-(row, group) scales and offsets are fetched the same way, one array per
// lane of a quad, and shared inside the warp after a __syncwarp.
//
// Requirements (the host checks them; anything else takes gemv_mma_kernel):
// one group per 128-value step, a whole number of blocks per row, block-aligned
// scale/offset rows, and the reduction axis not sliced over warps.
#pragma once

#include "dq_gemv.cuh"
#include "dq_peer_push.cuh"
#include "dq_mma_plan.cuh"
#include "dq_mma_stage.cuh"
#include "dq_mma_plan16.cuh"

namespace dq {
namespace stream {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * kWarp;

template <int BITS>
struct Cfg {
  static constexpr int P = BITS == 8 ? 2 : 4;                  // steps per block
  static constexpr int NB = BITS == 2 ? 3 : 2;                 // blocks in the ring
  static constexpr int UNIT = 4 * BITS;                        // bytes of one lane's unit of one row
  static constexpr int BLOCK_BYTES = P * 2 * UNIT;             // per lane per block
  static constexpr int META_BYTES = 2 * P;                     // per lane per block (one array, P groups)
  static constexpr int RING_BYTES = NB * (BLOCK_BYTES + META_BYTES) * kThreads;
};

template <int BYTES>
__device__ __forceinline__ void cp_async_n(uint32_t dst, const void* src) {
  if constexpr (BYTES == 16) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
  } else {
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(dst), "l"(src), "n"(BYTES) : "memory");
  }
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// One lane's unit of one row: UNIT bytes, global -> shared.
template <int BITS>
__device__ __forceinline__ void copy_unit(uint32_t dst, const uint32_t* src) {
  if constexpr (BITS == 2) {
    cp_async_n<8>(dst, src);
  } else if constexpr (BITS == 3) {
    cp_async_n<4>(dst, src);
    cp_async_n<4>(dst + 4, src + 1);
    cp_async_n<4>(dst + 8, src + 2);
  } else if constexpr (BITS == 4) {
    cp_async_n<16>(dst, src);
  } else {
    cp_async_n<16>(dst, src);
    cp_async_n<16>(dst + 16, src + 4);
  }
}

// One step of eight rows (8 rows x 4 units of `4*BITS` bytes) global -> shared, as 16-byte pieces.
//
// In shared memory a warp's block for (step, row half) is 32 consecutive units, lane l's
// unit at l * UNIT -- which is also the order of the bytes in global memory row by row:
// row g holds units 4g..4g+3.  So the block is copied as 2*UNIT pieces of 16 bytes, piece p
// coming from row p / (UNIT/4), whatever the unit size: at 3-bit one 16-byte copy per lane
// (24 lanes) replaces three 4-byte ones, at 2-bit 16 lanes replace 32.  A lane later reads a
// unit another lane copied, so a __syncwarp must follow the cp.async wait.
template <int BITS>
__device__ __forceinline__ void copy_block(uint32_t dst_block, const uint32_t* __restrict__ packed,
                                           int64_t words_per_row, int row0, int last_row, int word0, int lane) {
  constexpr int UNIT = 4 * BITS;
  constexpr int PIECES = 2 * UNIT;   // 16-byte pieces in the block
  constexpr int PER_ROW = UNIT / 4;  // pieces per row
#pragma unroll
  for (int p0 = 0; p0 < PIECES; p0 += kWarp) {
    const int p = p0 + lane;
    if (PIECES % kWarp == 0 || p < PIECES) {
      const int g = p / PER_ROW;
      const int part = p - g * PER_ROW;
      const int row = min(row0 + g, last_row);
      cp_async_n<16>(dst_block + p * 16, packed + row * words_per_row + word0 + part * 4);
    }
  }
}

template <int BITS>
__device__ __forceinline__ void read_unit(const unsigned char* src, uint32_t* w) {
  if constexpr (BITS == 2) {
    const uint2 v = *reinterpret_cast<const uint2*>(src);
    w[0] = v.x, w[1] = v.y;
  } else if constexpr (BITS == 3) {
    const uint32_t* s = reinterpret_cast<const uint32_t*>(src);
    w[0] = s[0], w[1] = s[1], w[2] = s[2];
  } else {
#pragma unroll
    for (int i = 0; i < BITS / 4; ++i) {
      const uint4 v = reinterpret_cast<const uint4*>(src)[i];
      w[4 * i] = v.x, w[4 * i + 1] = v.y, w[4 * i + 2] = v.z, w[4 * i + 3] = v.w;
    }
  }
}

struct Params {
  int steps;        // padded K / 128 (a multiple of P)
  int tiles;        // ceil(rows / 16)
  int m_stride_u4;  // uint4 per activation row of the staged B buffer
  uint32_t magic;   // a parameter so it stays a register operand of the decode
  int runs;         // 1: every CTA takes a contiguous run of tiles; 0: tiles strided over the grid
  peerpush::Push push;  // enabled: the output rows also go to every rank's window (dq_peer_push.cuh)
};

// P16: the fp16-operand plan (dq_mma_plan16.cuh; 2-, 4- and 8-bit codes, aligned 16-bit activations).
// PUSH: the launch also copies its output rows into every rank's window and ends with the bounded
// wait for the other ranks' rows (dq_peer_push.cuh).  A template parameter, not a flag: this
// kernel sits at its register limit and the plain build must stay exactly what it was.
//
// The body is a device function of (CTA index, CTA count) so that one launch can also run several
// matrices side by side, each on its own range of CTAs (gemv_mma_stream_multi_kernel,
// dq_gemv_stream_multi.cu); the single-matrix kernel below passes blockIdx.x / gridDim.x.
//
// SLICED (gemv_mma_stream_sliced_kernel below): `a` and `p` describe one slice of the reduction
// axis, every warp has at most one row tile, and the sums are not stored: they are left in acc_out
// for the caller, which adds the slices of a thread-block cluster.
template <int BITS, bool XBF16, bool MBF16, bool P16 = false, bool PUSH = false, bool SLICED = false>
__device__ __forceinline__ void stream_body(const GemvArgs& a, const Params& p, const unsigned int cta,
                                            const unsigned int ncta, unsigned char* smem_raw,
                                            float* acc_out = nullptr) {
  using Plan = MmaPlan<BITS>;
  using C = Cfg<BITS>;
  constexpr int P = C::P;
  constexpr int NB = C::NB;
  constexpr int NA = P16 ? 16 : Plan::kARegs;
  constexpr bool MMA_BF16 = P16 ? false : XBF16;  // operand type of the contraction
  constexpr int QU = NA / 4;
  constexpr int STEP_WORDS = 4 * BITS;
  constexpr int kTileRows = 16;
  constexpr float kMagicValue = XBF16 ? 128.0f : 1024.0f;

  // [ring weights: NB][P][2 rows][threads][UNIT] [ring meta: NB][threads][META_BYTES] [xb] [zero] [xsum] [xneg]
  unsigned char* ring_w = smem_raw;
  unsigned char* ring_m = ring_w + NB * C::BLOCK_BYTES * kThreads;
  uint4* xb = reinterpret_cast<uint4*>(ring_m + NB * C::META_BYTES * kThreads);
  float* xsum = reinterpret_cast<float*>(xb + a.m * p.m_stride_u4 + QU * 4);
  float* xneg = xsum + p.steps * 8;

  const int tid = threadIdx.x;
  const int lane = tid & (kWarp - 1);
  const int warp = tid >> 5;
  const int g = lane >> 2;
  const int t = lane & 3;
  const uint32_t magic = p.magic;
  const bool has_off = a.offsets != nullptr;
  const int nblocks = p.steps / P;
  // Two ways to deal the row tiles.  Strided (tile = CTA * warps + warp, + grid * warps, ...): the
  // whole grid moves through the matrix as one window, which the memory system likes best (4-bit
  // 262,144 rows: 80.1 % against 78.7 %), but a tile count that is not a multiple of the grid's
  // warps leaves some SMs a full round more than others (248,320 rows on 444 CTAs: 14 against 13
  // rounds, 7 % of the launch).  Runs (p.runs): a CTA takes a contiguous run of tiles, the runs
  // equal to within a tile, its warps interleaved over the run.  The host picks per launch.
  const bool runs = p.runs != 0;
  const int tile_lo = runs ? static_cast<int>(static_cast<int64_t>(p.tiles) * cta / ncta) : 0;
  const int tile_end = runs ? static_cast<int>(static_cast<int64_t>(p.tiles) * (cta + 1) / ncta) : p.tiles;
  const int tile_stride = runs ? kWarps : static_cast<int>(ncta) * kWarps;
  const int first_tile = runs ? tile_lo + warp : static_cast<int>(cta) * kWarps + warp;

  const uint32_t ring_w_s = static_cast<uint32_t>(__cvta_generic_to_shared(ring_w)) + (tid - lane) * C::UNIT;
  const uint32_t ring_m_s = static_cast<uint32_t>(__cvta_generic_to_shared(ring_m)) + tid * C::META_BYTES;
  const unsigned char* ring_w_mine = ring_w + tid * C::UNIT;
  // metadata of this lane's quad: arrays 0..3 = scale(row g), offset(row g), scale(row g+8), offset(row g+8)
  const unsigned char* ring_m_quad = ring_m + (tid & ~3) * C::META_BYTES;

  pdl_launch_dependents();

  // ---- prefetch cursor: walks (tile, block) ahead of the compute loop ----
  // Integer instructions issue at half rate on this GPU and the decode needs that pipe, so
  // the cursor is kept as running pointers: everything that depends on the lane or the tile
  // is resolved once per tile, a block costs a pointer bump per source row and its copies
  // use immediate offsets.
  constexpr int PIECES = 2 * C::UNIT;        // 16-byte pieces of one (step, row half) block
  constexpr int PER_ROW = C::UNIT / 4;       // pieces per row
  constexpr int NSRC = (PIECES + kWarp - 1) / kWarp;  // pieces of a block this lane copies
  constexpr int STEP_BYTES = STEP_WORDS * 4;
  int pf_tile = first_tile;
  int pf_blk = 0;
  const unsigned char* pf_src[2][NSRC];  // [row half][piece]: this lane's source at the block's first step
  const unsigned short* pf_meta = nullptr;  // this lane's array (scales or offsets) at its row, at the block's first group
  bool pf_lane[NSRC];
#pragma unroll
  for (int i = 0; i < NSRC; ++i) pf_lane[i] = (PIECES % kWarp == 0) || (i * kWarp + lane < PIECES);
  auto pf_point = [&]() {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
      for (int i = 0; i < NSRC; ++i) {
        const int piece = i * kWarp + lane;
        const int pg = piece / PER_ROW;
        const int part = piece - pg * PER_ROW;
        const int row = min(pf_tile * kTileRows + h * 8 + pg, a.rows - 1);
        pf_src[h][i] = reinterpret_cast<const unsigned char*>(a.packed + static_cast<int64_t>(row) * a.words_per_row + part * 4);
      }
    }
    const int ra = min(pf_tile * kTileRows + g, a.rows - 1);
    const int rb = min(pf_tile * kTileRows + g + 8, a.rows - 1);
    const unsigned short* arr = reinterpret_cast<const unsigned short*>((t & 1) ? a.offsets : a.scales);
    pf_meta = arr + static_cast<int64_t>((t & 2) ? rb : ra) * a.num_groups;
  };
  if (pf_tile < tile_end) pf_point();
  const bool meta_lane = has_off || (t & 1) == 0;
  // ring slot of the block being requested, as byte offsets into the two rings
  uint32_t pf_w = ring_w_s + lane * 16, pf_m = ring_m_s;
  const uint32_t ring_w_end = ring_w_s + lane * 16 + NB * (C::BLOCK_BYTES * kThreads);
  const uint32_t ring_m_end = ring_m_s + NB * (C::META_BYTES * kThreads);
  auto prefetch_block = [&]() {
    if (pf_tile < tile_end) {
#pragma unroll
      for (int j = 0; j < P; ++j) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int i = 0; i < NSRC; ++i) {
            if (pf_lane[i]) {
              cp_async_n<16>(pf_w + (j * 2 + h) * (C::UNIT * kThreads) + i * (kWarp * 16), pf_src[h][i] + j * STEP_BYTES);
            }
          }
        }
      }
      if (meta_lane) cp_async_n<C::META_BYTES>(pf_m, pf_meta);
      if (++pf_blk == nblocks) {
        pf_blk = 0;
        pf_tile += tile_stride;
        if (pf_tile < tile_end) pf_point();
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int i = 0; i < NSRC; ++i) pf_src[h][i] += P * STEP_BYTES;
        }
        pf_meta += P;
      }
    }
    pf_w += C::BLOCK_BYTES * kThreads;
    pf_m += C::META_BYTES * kThreads;
    if (pf_w == ring_w_end) {
      pf_w -= NB * (C::BLOCK_BYTES * kThreads);
      pf_m = ring_m_end - NB * (C::META_BYTES * kThreads);
    }
    cp_async_commit();  // an empty group keeps the wait arithmetic uniform
  };
#pragma unroll
  for (int i = 0; i < NB - 1; ++i) {
    prefetch_block();
  }

  // ---- stage the activation (the only part that depends on the previous kernel) ----
  pdl_wait_prior_grid();
  if constexpr (P16) {
    if constexpr (BITS != 3) {
      // (xneg holds the steps' inverse power-of-two factors in this plan, not a bias sum)
      stage_zero_fill<4, false>(a.m, p.steps, p.m_stride_u4, xb, xsum, xneg, tid, kThreads);
      stage_units16<BITS, XBF16>(a, 0, p.steps, p.m_stride_u4, xb, xsum, xneg, tid, kThreads, nullptr);
    }
  } else {
    stage_activation<BITS, XBF16>(a, p.steps, p.m_stride_u4, xb, xsum, xneg, tid, kThreads);
  }
  __syncthreads();

  // ---- compute loop: one block of P steps per iteration ----
  const bool b_live = g < a.m;
  const uint4* xb_lane = b_live ? xb + g * p.m_stride_u4 + t : xb + a.m * p.m_stride_u4;
  const int xb_blk_u4 = b_live ? QU * 4 * P : 0;  // uint4 per block of steps (0: the zero block, re-read)
  const int xb_step_u4 = b_live ? QU * 4 : 0;
  const float* xsum_t = xsum + 2 * t;
  const float* xneg_t = xneg + 2 * t;
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  // ring slot being consumed
  const unsigned char* wslot = ring_w_mine;
  const unsigned char* mslot = ring_m_quad;
  const unsigned char* const wslot_end = ring_w_mine + NB * (C::BLOCK_BYTES * kThreads);
  for (int tile = first_tile; tile < tile_end; tile += tile_stride) {
    const uint4* bblk = xb_lane;
    const float* xs_blk = xsum_t;
    const float* xn_blk = xneg_t;
    for (int blk = 0; blk < nblocks; ++blk) {
      __syncwarp();      // every lane is done with the slot about to be refilled
      prefetch_block();  // refills the slot consumed one iteration ago
      cp_async_wait<NB - 1>();
      __syncwarp();      // the quad's metadata copies are visible to each other
      const unsigned char* wsrc = wslot;
      const unsigned char* msrc = mslot;
      uint32_t mc[4][P / 2];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (has_off || (i & 1) == 0) {
          if constexpr (P == 4) {
            const uint2 v = *reinterpret_cast<const uint2*>(msrc + i * C::META_BYTES);
            mc[i][0] = v.x, mc[i][1] = v.y;
          } else {
            mc[i][0] = *reinterpret_cast<const uint32_t*>(msrc + i * C::META_BYTES);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < P; ++j) {
        uint32_t wa[BITS], wb[BITS];
        read_unit<BITS>(wsrc + (j * 2 + 0) * (C::UNIT * kThreads), wa);
        read_unit<BITS>(wsrc + (j * 2 + 1) * (C::UNIT * kThreads), wb);
        uint32_t aa[NA], ab[NA];
        if constexpr (P16 && BITS != 3) {
          decode_unit16<BITS>(wa, magic, aa);
          decode_unit16<BITS>(wb, magic, ab);
        } else {
          decode_unit<BITS>(wa, magic, aa);
          decode_unit<BITS>(wb, magic, ab);
          unbias_fragments<XBF16, NA>(aa);
          unbias_fragments<XBF16, NA>(ab);
        }
        const uint4* bsrc = bblk + j * xb_step_u4;
        float d[4];
#pragma unroll
        for (int q = 0; q < QU; ++q) {
          const uint4 b = bsrc[q * 4];
          if (q == 0) {
            mma_16816<MMA_BF16, true>(d, aa[0], ab[0], aa[1], ab[1], b.x, b.y);
          } else {
            mma_16816<MMA_BF16, false>(d, aa[4 * q], ab[4 * q], aa[4 * q + 1], ab[4 * q + 1], b.x, b.y);
          }
          mma_16816<MMA_BF16, false>(d, aa[4 * q + 2], ab[4 * q + 2], aa[4 * q + 3], ab[4 * q + 3], b.z, b.w);
        }
        auto meta_f32 = [&](int i) -> float {
          const uint32_t reg = mc[i][j / 2];
          if constexpr (MBF16) {
            return __uint_as_float((j & 1) ? (reg & 0xFFFF0000u) : (reg << 16));
          } else {
            const __half2 h = *reinterpret_cast<const __half2*>(&reg);
            return (j & 1) ? __high2float(h) : __low2float(h);
          }
        };
        const float2 xs2 = *reinterpret_cast<const float2*>(xs_blk + j * 8);
        const float2 xn2 = *reinterpret_cast<const float2*>(xn_blk + j * 8);
        const float sc_a = meta_f32(0), sc_b = meta_f32(2);
        if constexpr (P16) {
          // xn2: the step's inverse power-of-two factor per activation row
          acc[0] = fmaf(sc_a * xn2.x, d[0], acc[0]);
          acc[1] = fmaf(sc_a * xn2.y, d[1], acc[1]);
          acc[2] = fmaf(sc_b * xn2.x, d[2], acc[2]);
          acc[3] = fmaf(sc_b * xn2.y, d[3], acc[3]);
        } else {
          acc[0] = fmaf(sc_a, d[0] + xn2.x, acc[0]);
          acc[1] = fmaf(sc_a, d[1] + xn2.y, acc[1]);
          acc[2] = fmaf(sc_b, d[2] + xn2.x, acc[2]);
          acc[3] = fmaf(sc_b, d[3] + xn2.y, acc[3]);
        }
        if (has_off) {
          const float of_a = meta_f32(1), of_b = meta_f32(3);
          acc[0] = fmaf(of_a, xs2.x, acc[0]);
          acc[1] = fmaf(of_a, xs2.y, acc[1]);
          acc[2] = fmaf(of_b, xs2.x, acc[2]);
          acc[3] = fmaf(of_b, xs2.y, acc[3]);
        }
      }
      bblk += xb_blk_u4;
      xs_blk += P * 8;
      xn_blk += P * 8;
      wslot += C::BLOCK_BYTES * kThreads;
      mslot += C::META_BYTES * kThreads;
      if (wslot == wslot_end) {
        wslot = ring_w_mine;
        mslot = ring_m_quad;
      }
    }
    if constexpr (SLICED) {
#pragma unroll
      for (int i = 0; i < 4; ++i) acc_out[i] = acc[i];
    } else {
      const int row_a = tile * kTileRows + g, row_b = row_a + 8;
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
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[i] = 0.0f;
    }
  }
  cp_async_wait<0>();
  if constexpr (PUSH) {
    // Copy this CTA's rows, as stored, to every window: one run of tiles, or runs of kWarps tiles
    // at the grid's stride.
    // (Every thread reads the epoch itself: no static shared memory, which would cost the third CTA per SM.)
    const unsigned int epoch = peerpush::next_epoch(p.push);
    __syncthreads();  // the output stores above are visible to the whole CTA
    if (runs) {
      peerpush::push_rows(p.push, a, epoch, tile_lo * kTileRows, min(tile_end * kTileRows, a.rows), tid, kThreads);
    } else {
      constexpr int kRun = kWarps * kTileRows;
      for (int row = static_cast<int>(cta) * kRun; row < a.rows; row += static_cast<int>(ncta) * kRun) {
        peerpush::push_rows(p.push, a, epoch, row, min(row + kRun, a.rows), tid, kThreads);
      }
    }
    __syncthreads();
    if (tid < kWarp) peerpush::arrive(p.push, epoch, ncta, tid);
  }
}

template <int BITS, bool XBF16, bool MBF16, bool P16 = false, bool PUSH = false>
__global__ void __launch_bounds__(kThreads, 3) gemv_mma_stream_kernel(const GemvArgs a, const Params p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  stream_body<BITS, XBF16, MBF16, P16, PUSH>(a, p, blockIdx.x, gridDim.x, smem_raw);
}

// Matrices of too few rows to be a stream for the kernel above (a warp there owns whole rows): the
// grid's y axis slices the reduction axis, the CTAs of one group of eight row tiles form a
// thread-block cluster (1 x slices), each runs the streaming body over its own range of blocks
// -- staging only its part of the activation -- and the sums meet in the cluster's first CTA
// through distributed shared memory, added in slice order (a fixed summation order), which stores.
// p.steps is the whole row's step count here; the slices are whole blocks, equal to within one.
template <int BITS, bool XBF16, bool MBF16, bool P16 = false>
__global__ void __launch_bounds__(kThreads, 3) gemv_mma_stream_sliced_kernel(const GemvArgs a, const Params p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int P = Cfg<BITS>::P;
  constexpr int NA = P16 ? 16 : MmaPlan<BITS>::kARegs;
  uint32_t slice, slices;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(slice));
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(slices));
  const int nblocks = p.steps / P;
  const int blk_begin = static_cast<int>(static_cast<unsigned>(nblocks) * slice / slices);
  const int blk_end = static_cast<int>(static_cast<unsigned>(nblocks) * (slice + 1) / slices);
  GemvArgs sa = a;
  Params sp = p;
  sp.steps = (blk_end - blk_begin) * P;
  sp.m_stride_u4 = sp.steps * NA + 4;
  sp.runs = 0;
  const int s0 = blk_begin * P;  // first step of the slice
  sa.packed = a.packed + s0 * (4 * BITS);
  sa.scales = static_cast<const unsigned short*>(a.scales) + s0;
  sa.offsets = a.offsets != nullptr ? static_cast<const unsigned short*>(a.offsets) + s0 : nullptr;
  sa.x = static_cast<const unsigned short*>(a.x) + s0 * 128;  // (the row pitch stays a.in_features)
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  stream_body<BITS, XBF16, MBF16, P16, false, true>(sa, sp, blockIdx.x, gridDim.x, smem_raw, acc);

  // Both cluster barriers are reached by every thread of every CTA; the second keeps a CTA's shared
  // memory alive until the first CTA has read it.
  const int tid = threadIdx.x;
  __syncthreads();  // every warp is done with the ring and the staged activation
  reinterpret_cast<float4*>(smem_raw)[tid] = make_float4(acc[0], acc[1], acc[2], acc[3]);
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (slice == 0) {
    const uint32_t mine = static_cast<uint32_t>(__cvta_generic_to_shared(smem_raw)) + tid * 16;
    for (uint32_t r = 1; r < slices; ++r) {
      uint32_t remote;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(mine), "r"(r));
      float4 v;
      asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
      acc[0] += v.x, acc[1] += v.y, acc[2] += v.z, acc[3] += v.w;
    }
  }
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (slice != 0) return;
  const int lane = tid & (kWarp - 1), warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int tile = static_cast<int>(blockIdx.x) * kWarps + warp;
  if (tile >= p.tiles) return;
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

}  // namespace stream
}  // namespace dq
