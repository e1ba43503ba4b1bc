// Packed decode GEMV on the tensor cores, M = 1..8 activation rows at one price.
//
// Same operator as dq_gemv.cu (reference: gemv_cuda,
// packages/dynquant-kernels/csrc/gemv/gemv.cu:695-756) for 16-bit activations
// and groups that are a multiple of 128 values.  The SIMT kernel spends about
// two instructions per weight VALUE (one logic op, half a packed add, half a
// packed FMA per activation row), which at 2 and 3 bits per value is more
// instruction issue than the memory system needs time to deliver the bytes
// (measured: 17-55 % of the HBM peak depending on width).  Here a weight value costs 0.6-0.9
// integer instructions and 1/8 of an mma, whatever M is:
//
//   * out tile = 16 weight rows x 8 activation rows = one m16n8k16 accumulator.
//     The 8 columns are exactly the operator's row limit (DQ_GEMV_MAX_ROWS).
//   * a thread streams two weight rows (g and g+8 of the tile) and, per step of
//     128 reduction values (one quantization group, or a 128-value slice of a
//     larger one), decodes its 32-value unit of each row straight into A
//     fragments (dq_mma_plan.cuh).  B fragments -- the activation, pre-scaled
//     and pre-permuted to match -- come from shared memory, staged once per CTA.
//   * one accumulator covers one step, so the per-(row, group) scale and offset
//     are applied to it in fp32 right after the step's mmas:
//         acc += s * (D - MAGIC * sum x')  +  o * sum x
//   * rows are split over warps, and for short matrices the reduction axis is
//     split over the warps of a CTA too (summed in a fixed order through shared
//     memory: results are bit-identical run to run).
//   * weight words and raw scale/offset bits are loaded a block of steps ahead and
//     only converted when used, so a warp never stalls on a load it just issued.
//     The first loads go out BEFORE griddepcontrol.wait: under programmatic
//     dependent launch the next layer's weights start streaming while the
//     previous layer is still finishing, and only the activation staging waits.
//
// A zero pad past in_features needs no special case: the staged activation is
// zero there (reference docs/format-spec.md:205-214).
#include <algorithm>
#include <cstdlib>
#include <type_traits>

#include "dq_gemv.cuh"
#include "dq_gemv_mma_tile.cuh"
#include "dq_gemv_mma_stream.cuh"
#include "dq_mma_plan.cuh"
#include "dq_mma_stage.cuh"

namespace dq {
namespace {

constexpr int kStepValues = 128;
constexpr int kTileRows = 16;
constexpr int kMaxWarps = 16;

struct MmaParams {
  int steps;            // padded K / 128
  int steps_per_group;  // group_values / 128
  int tiles;            // ceil(rows / 16)
  int rw, kw;           // warps of a CTA: rw row tiles x kw slices of the reduction axis
  int steps_per_warp;   // steps of one slice
  int m_stride_u4;      // uint4 per activation row in the staged B buffer
  int vec_meta;         // scales/offsets of a whole block of steps may be read with one vector load
  uint32_t magic;       // 16-bit magic constant in both halves; a parameter so it stays a register operand
};

template <int BITS>
struct Depth {
  static constexpr int value = BITS == 8 ? 2 : 4;  // steps kept in flight per warp
};

template <int BITS>
__device__ __forceinline__ void load_unit(const uint32_t* __restrict__ src, uint32_t* w) {
  if constexpr (BITS == 2) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(src));
    w[0] = v.x;
    w[1] = v.y;
  } else if constexpr (BITS == 3) {
    // 12 bytes at a 12-byte stride: three 32-bit loads, kept in L1 so the sector a
    // neighbouring step shares is fetched from L2 once.
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(w[i]) : "l"(src + i));
    }
  } else {
#pragma unroll
    for (int i = 0; i < BITS / 4; ++i) {
      const uint4 v = ldg_stream_128(src + 4 * i);
      w[4 * i + 0] = v.x;
      w[4 * i + 1] = v.y;
      w[4 * i + 2] = v.z;
      w[4 * i + 3] = v.w;
    }
  }
}

__device__ __forceinline__ uint32_t ld_u16(const unsigned short* p) {
  unsigned short v;
  asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ld_u32(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ld_u64(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

// Element j (0 or 1) of a register holding two 16-bit floats, widened to fp32.
template <bool BF16>
__device__ __forceinline__ float half_of(uint32_t reg, int j) {
  if constexpr (BF16) {
    return __uint_as_float(j ? (reg & 0xFFFF0000u) : (reg << 16));
  } else {
    const __half2 h = *reinterpret_cast<const __half2*>(&reg);
    return j ? __high2float(h) : __low2float(h);
  }
}

template <bool BF16>
__device__ __forceinline__ uint32_t to_raw16(float v) {
  if constexpr (BF16) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(v));
  } else {
    return __half_as_ushort(__float2half_rn(v));
  }
}

// Where one 16-row tile's data starts for this lane.
struct TilePtr {
  const uint32_t* wa;  // row g   : words of this lane's unit at step 0
  const uint32_t* wb;  // row g+8
  int64_t ma, mb;      // element index of (row, group 0) in scales / offsets
};

// FAST: whole, aligned blocks only (the register ring runs without predicates and with
// vector metadata loads).  !FAST: any step count.
template <int BITS, bool XBF16, bool MBF16, bool FAST>
__global__ void __launch_bounds__(kMaxWarps* kWarp)
    gemv_mma_kernel(const GemvArgs a, const MmaParams p) {
  using Plan = MmaPlan<BITS>;
  constexpr int P = Depth<BITS>::value;
  constexpr int NA = Plan::kARegs;
  constexpr int QU = NA / 4;          // uint4 of B fragments per (step, lane)
  constexpr int STEP_WORDS = 4 * BITS;  // words one step occupies in a row

  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint4* xb = reinterpret_cast<uint4*>(smem_raw);
  float* xsum = reinterpret_cast<float*>(xb + a.m * p.m_stride_u4 + QU * 4);  // [steps][8]  sum of x
  float* xneg = xsum + p.steps * 8;                                  // [steps][8]  -MAGIC * sum of x'
  float* red = xneg + p.steps * 8;                                   // [kw][rw][16][8]

  const int lane = threadIdx.x & (kWarp - 1);
  const int warp = threadIdx.x >> 5;
  const int nthreads = blockDim.x;
  const int g = lane >> 2;  // row of the tile; also the activation row this lane feeds into B
  const int t = lane & 3;   // which 32-value unit of a step
  const int rwi = warp / p.kw;
  const int kwi = warp - rwi * p.kw;
  constexpr float kMagicValue = XBF16 ? 128.0f : 1024.0f;
  const uint32_t magic = p.magic;

  const int s_begin = kwi * p.steps_per_warp;
  const int s_end = min(p.steps, s_begin + p.steps_per_warp);
  const int nsteps = max(0, s_end - s_begin);
  const int tile_stride = gridDim.x * p.rw;
  const bool has_off = a.offsets != nullptr;
  const unsigned short* scales16 = reinterpret_cast<const unsigned short*>(a.scales);
  const unsigned short* offsets16 = reinterpret_cast<const unsigned short*>(a.offsets);

  auto tile_ptr = [&](int tile) {
    TilePtr tp;
    const int ra = min(tile * kTileRows + g, a.rows - 1);
    const int rb = min(tile * kTileRows + g + 8, a.rows - 1);
    tp.wa = a.packed + static_cast<int64_t>(ra) * a.words_per_row + s_begin * STEP_WORDS + t * BITS;
    tp.wb = a.packed + static_cast<int64_t>(rb) * a.words_per_row + s_begin * STEP_WORDS + t * BITS;
    tp.ma = static_cast<int64_t>(ra) * a.num_groups;
    tp.mb = static_cast<int64_t>(rb) * a.num_groups;
    return tp;
  };

  pdl_launch_dependents();

  // ---- prefetch state ----
  uint32_t raw[P][2][BITS];      // weight words, one slot per step of a block
  uint32_t mcur[4][P / 2];       // scale_a, offset_a, scale_b, offset_b of the current block (2 x 16 bit / reg)
  uint32_t mnext[4][P / 2];      // ... of the block after it

  // Weight words of relative step `rs` (counted from s_begin) of a tile into a slot.
  auto load_weights = [&](const TilePtr& tp, int slot, int rs) {
    load_unit<BITS>(tp.wa + rs * STEP_WORDS, raw[slot][0]);
    load_unit<BITS>(tp.wb + rs * STEP_WORDS, raw[slot][1]);
  };
  // Scales/offsets of the P steps starting at relative step rs0 (`valid` of them exist).
  auto load_meta = [&](const TilePtr& tp, int rs0, int valid, uint32_t (&dst)[4][P / 2]) {
    const int s0 = s_begin + rs0;
    if (p.vec_meta && valid == P) {
      // one group per step, block-aligned: P consecutive 16-bit values per array
      const int64_t ia = tp.ma + s0, ib = tp.mb + s0;
      if constexpr (P == 4) {
        const uint2 sa = ld_u64(scales16 + ia), sb = ld_u64(scales16 + ib);
        dst[0][0] = sa.x, dst[0][1] = sa.y, dst[2][0] = sb.x, dst[2][1] = sb.y;
        if (has_off) {
          const uint2 oa = ld_u64(offsets16 + ia), ob = ld_u64(offsets16 + ib);
          dst[1][0] = oa.x, dst[1][1] = oa.y, dst[3][0] = ob.x, dst[3][1] = ob.y;
        }
      } else {
        dst[0][0] = ld_u32(scales16 + ia), dst[2][0] = ld_u32(scales16 + ib);
        if (has_off) {
          dst[1][0] = ld_u32(offsets16 + ia), dst[3][0] = ld_u32(offsets16 + ib);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < P; ++j) {
        if (j < valid) {
          const int grp = (s0 + j) / p.steps_per_group;
          const uint32_t sa = ld_u16(scales16 + tp.ma + grp), sb = ld_u16(scales16 + tp.mb + grp);
          const uint32_t oa = has_off ? ld_u16(offsets16 + tp.ma + grp) : 0u;
          const uint32_t ob = has_off ? ld_u16(offsets16 + tp.mb + grp) : 0u;
          if (j & 1) {
            dst[0][j / 2] |= sa << 16, dst[1][j / 2] |= oa << 16;
            dst[2][j / 2] |= sb << 16, dst[3][j / 2] |= ob << 16;
          } else {
            dst[0][j / 2] = sa, dst[1][j / 2] = oa, dst[2][j / 2] = sb, dst[3][j / 2] = ob;
          }
        }
      }
    }
  };

  int tile = blockIdx.x * p.rw + rwi;
  TilePtr cur = tile_ptr(min(tile, p.tiles - 1));
  const bool any_work = tile < p.tiles && nsteps > 0;
  if (any_work) {
#pragma unroll
    for (int i = 0; i < P; ++i) {
      if (i < nsteps) load_weights(cur, i, i);
    }
    load_meta(cur, 0, min(P, nsteps), mcur);
  }

  // ---- stage the activation: the only part that depends on the previous kernel ----
  pdl_wait_prior_grid();
  stage_activation<BITS, XBF16>(a, p.steps, p.m_stride_u4, xb, xsum, xneg, threadIdx.x, nthreads);
  __syncthreads();

  // ---- main loop: persistent over row tiles when the reduction axis is not sliced ----
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // (row g; m=2t, 2t+1), (row g+8; m=2t, 2t+1)
  const bool b_live = g < a.m;
  // Lanes whose activation row does not exist read a block of zeros, with a zero step stride.
  const uint4* xb_lane = b_live ? xb + g * p.m_stride_u4 + t : xb + a.m * p.m_stride_u4;
  const int xb_step_u4 = b_live ? QU * 4 : 0;
  const int nblocks = (nsteps + P - 1) / P;

  auto store_tile = [&](int tl, const float* v) {
    const int row_a = tl * kTileRows + g, row_b = row_a + 8;
    const int m0 = 2 * t;
    if (m0 < a.m) {
      if (row_a < a.rows) store_out(a, m0, row_a, v[0]);
      if (row_b < a.rows) store_out(a, m0, row_b, v[2]);
    }
    if (m0 + 1 < a.m) {
      if (row_a < a.rows) store_out(a, m0 + 1, row_a, v[1]);
      if (row_b < a.rows) store_out(a, m0 + 1, row_b, v[3]);
    }
  };

  // The mmas of one step and the affine map of its group:
  //   acc += scale * (D - MAGIC * sum x') + offset * sum x      (scalar FMAs: that pipe is idle)
  auto finish_step = [&](const uint32_t* aa, const uint32_t* ab, int s, int slot,
                         const uint32_t (&mc)[4][P / 2]) {
    const uint4* bsrc = xb_lane + s * xb_step_u4;
    float d[4];
#pragma unroll
    for (int q = 0; q < QU; ++q) {
      const uint4 b = bsrc[q * 4];
      if (q == 0) {
        mma_16816<XBF16, true>(d, aa[0], ab[0], aa[1], ab[1], b.x, b.y);
      } else {
        mma_16816<XBF16, false>(d, aa[4 * q], ab[4 * q], aa[4 * q + 1], ab[4 * q + 1], b.x, b.y);
      }
      mma_16816<XBF16, false>(d, aa[4 * q + 2], ab[4 * q + 2], aa[4 * q + 3], ab[4 * q + 3], b.z, b.w);
    }
    const float2 xs2 = *reinterpret_cast<const float2*>(xsum + s * 8 + 2 * t);
    const float2 xn2 = *reinterpret_cast<const float2*>(xneg + s * 8 + 2 * t);
    const float sc_a = half_of<MBF16>(mc[0][slot / 2], slot & 1);
    const float sc_b = half_of<MBF16>(mc[2][slot / 2], slot & 1);
    acc[0] = fmaf(sc_a, d[0] + xn2.x, acc[0]);
    acc[1] = fmaf(sc_a, d[1] + xn2.y, acc[1]);
    acc[2] = fmaf(sc_b, d[2] + xn2.x, acc[2]);
    acc[3] = fmaf(sc_b, d[3] + xn2.y, acc[3]);
    if (has_off) {
      const float of_a = half_of<MBF16>(mc[1][slot / 2], slot & 1);
      const float of_b = half_of<MBF16>(mc[3][slot / 2], slot & 1);
      acc[0] = fmaf(of_a, xs2.x, acc[0]);
      acc[1] = fmaf(of_a, xs2.y, acc[1]);
      acc[2] = fmaf(of_b, xs2.x, acc[2]);
      acc[3] = fmaf(of_b, xs2.y, acc[3]);
    }
  };

  if (any_work) {
    while (true) {
      const int next_tile = tile + tile_stride;
      const bool has_next = p.kw == 1 && next_tile < p.tiles;
      const TilePtr nxt = tile_ptr(has_next ? next_tile : tile);

      if constexpr (FAST) {
        // Every block is full and block-aligned: no predicates, vector metadata loads, and the
        // refill of a slot is always a real load (of this tile's next block, the next tile's
        // first block, or -- at the very end -- a harmless re-read of this tile's first block).
        for (int blk = 0; blk < nblocks; ++blk) {
          const int rs0 = blk * P;
          const bool last_blk = blk + 1 == nblocks;
          const uint32_t* wa_n = last_blk ? nxt.wa : cur.wa + (rs0 + P) * STEP_WORDS;
          const uint32_t* wb_n = last_blk ? nxt.wb : cur.wb + (rs0 + P) * STEP_WORDS;
          TilePtr mp = last_blk ? nxt : cur;
          load_meta(mp, last_blk ? 0 : rs0 + P, P, mnext);
#pragma unroll
          for (int slot = 0; slot < P; ++slot) {
            uint32_t aa[NA], ab[NA];
            decode_unit<BITS>(raw[slot][0], magic, aa);
            decode_unit<BITS>(raw[slot][1], magic, ab);
            unbias_fragments<XBF16, NA>(aa);
            unbias_fragments<XBF16, NA>(ab);
            load_unit<BITS>(wa_n + slot * STEP_WORDS, raw[slot][0]);
            load_unit<BITS>(wb_n + slot * STEP_WORDS, raw[slot][1]);
            finish_step(aa, ab, s_begin + rs0 + slot, slot, mcur);
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int j = 0; j < P / 2; ++j) {
              mcur[i][j] = mnext[i][j];
            }
          }
        }
      } else {
        for (int blk = 0; blk < nblocks; ++blk) {
          const int rs0 = blk * P;
          const int valid = min(P, nsteps - rs0);
          const bool last_blk = blk + 1 == nblocks;
          if (!last_blk) {
            load_meta(cur, rs0 + P, min(P, nsteps - rs0 - P), mnext);
          } else if (has_next) {
            load_meta(nxt, 0, min(P, nsteps), mnext);
          }
#pragma unroll
          for (int slot = 0; slot < P; ++slot) {
            if (slot < valid) {
              uint32_t aa[NA], ab[NA];
              decode_unit<BITS>(raw[slot][0], magic, aa);
              decode_unit<BITS>(raw[slot][1], magic, ab);
              unbias_fragments<XBF16, NA>(aa);
              unbias_fragments<XBF16, NA>(ab);
              // Refill this slot: P steps ahead in this tile, or the next tile's first block.
              const int rs_next = rs0 + slot + P;
              if (rs_next < nsteps) {
                load_weights(cur, slot, rs_next);
              } else if (last_blk && has_next) {
                load_weights(nxt, slot, slot);
              }
              finish_step(aa, ab, s_begin + rs0 + slot, slot, mcur);
            } else if (last_blk && has_next && slot < nsteps) {
              load_weights(nxt, slot, slot);
            }
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int j = 0; j < P / 2; ++j) {
              mcur[i][j] = mnext[i][j];
            }
          }
        }
      }

      if (p.kw > 1) {
        break;  // one tile per warp group; the slices are summed below
      }
      store_tile(tile, acc);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[i] = 0.0f;
      }
      if (!has_next) {
        break;
      }
      tile = next_tile;
      cur = nxt;
    }
  }

  // ---- sliced reduction axis: sum the slices in a fixed order and store ----
  if (p.kw > 1) {
    float* mine = red + ((kwi * p.rw + rwi) * kTileRows) * 8;
    *reinterpret_cast<float2*>(mine + g * 8 + 2 * t) = make_float2(acc[0], acc[1]);
    *reinterpret_cast<float2*>(mine + (g + 8) * 8 + 2 * t) = make_float2(acc[2], acc[3]);
    __syncthreads();
    if (kwi == 0 && tile < p.tiles) {
      float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      for (int k = 0; k < p.kw; ++k) {
        const float* part = red + ((k * p.rw + rwi) * kTileRows) * 8;
        const float2 pa = *reinterpret_cast<const float2*>(part + g * 8 + 2 * t);
        const float2 pb = *reinterpret_cast<const float2*>(part + (g + 8) * 8 + 2 * t);
        v[0] += pa.x, v[1] += pa.y, v[2] += pb.x, v[3] += pb.y;
      }
      store_tile(tile, v);
    }
  }
}

int floor_pow2(int v) {
  int p = 1;
  while (2 * p <= v) p *= 2;
  return p;
}

bool mma_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("DQ_B200_GEMV_PATH");
    return !(v != nullptr && v[0] == 's');  // "simt" forces the SIMT kernels
  }();
  return on;
}

bool pdl_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("DQ_B200_NO_PDL");
    return !(v != nullptr && v[0] != '\0' && v[0] != '0');
  }();
  return on;
}

size_t mma_smem_bytes(int m, int steps, int aregs, int rw, int kw, int* m_stride_u4) {
  const int stride = steps * aregs + 4;  // +4 uint4: consecutive activation rows land 64 B apart mod 128
  *m_stride_u4 = stride;
  size_t bytes = (static_cast<size_t>(m) * stride + aregs) * 16;  // + the zero block
  bytes += static_cast<size_t>(steps) * 8 * 4 * 2;
  if (kw > 1) bytes += static_cast<size_t>(kw) * rw * kTileRows * 8 * 4;
  return bytes;
}

template <typename Kernel>
int32_t launch_mma_kernel(Kernel kernel, const GemvArgs& a, MmaParams p, int threads, size_t smem,
                          const DeviceInfo& dev, cudaStream_t stream) {
  if (smem > 48 * 1024) {
    DQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  }
  int grid = static_cast<int>(ceil_div(p.tiles, p.rw));
  if (p.kw == 1) {
    // persistent: no more CTAs than the device holds at once; warps stride over the tiles
    int per_sm = 0;
    DQ_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem));
    grid = std::min(grid, std::max(1, per_sm) * dev.sm_count);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(static_cast<unsigned>(threads));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  DQ_CUDA(cudaLaunchKernelEx(&cfg, kernel, a, p));
  DQ_CHECK_LAUNCH("gemv");
  note_kernel("gemv_mma_kernel");
  return DQ_OK;
}

template <int BITS>
int32_t launch_mma_bits(const GemvArgs& a, const MmaParams& p, int threads, size_t smem,
                        const DeviceInfo& dev, cudaStream_t stream) {
  const bool xbf = a.x_dtype == DQ_BF16;
  const bool mbf = a.meta_dtype == DQ_BF16;
  constexpr int P = Depth<BITS>::value;
  const bool fast = p.vec_meta && p.steps_per_warp % P == 0 && (p.kw == 1 || p.steps % p.kw == 0);
  if (fast) {
    if (xbf && mbf) return launch_mma_kernel(gemv_mma_kernel<BITS, true, true, true>, a, p, threads, smem, dev, stream);
    if (xbf) return launch_mma_kernel(gemv_mma_kernel<BITS, true, false, true>, a, p, threads, smem, dev, stream);
    if (mbf) return launch_mma_kernel(gemv_mma_kernel<BITS, false, true, true>, a, p, threads, smem, dev, stream);
    return launch_mma_kernel(gemv_mma_kernel<BITS, false, false, true>, a, p, threads, smem, dev, stream);
  }
  if (xbf && mbf) return launch_mma_kernel(gemv_mma_kernel<BITS, true, true, false>, a, p, threads, smem, dev, stream);
  if (xbf) return launch_mma_kernel(gemv_mma_kernel<BITS, true, false, false>, a, p, threads, smem, dev, stream);
  if (mbf) return launch_mma_kernel(gemv_mma_kernel<BITS, false, true, false>, a, p, threads, smem, dev, stream);
  return launch_mma_kernel(gemv_mma_kernel<BITS, false, false, false>, a, p, threads, smem, dev, stream);
}

// ---- streaming kernel (dq_gemv_mma_stream.cuh) ----

template <int BITS>
bool stream_ok(const GemvArgs& a, const DeviceInfo& dev, int tiles, int steps) {
  using C = stream::Cfg<BITS>;
  if (tuning_int("DQ_B200_NO_STREAM") != 0) return false;
  // Measured on B200: with 16-byte block copies and running source pointers the cp.async ring is
  // as fast or faster than the register ring of gemv_mma_kernel<FAST> at every width (it fits
  // three CTAs per SM).
  if (BITS == 2 && tuning_int("DQ_B200_RING_2BIT") == 1) return false;
  if (reinterpret_cast<uintptr_t>(a.packed) % 16 != 0 || (static_cast<int64_t>(a.words_per_row) * 4) % 16 != 0) {
    return false;  // whole steps are copied in 16-byte pieces
  }
  if (a.group_values != kStepValues || steps % C::P != 0 || a.num_groups % C::P != 0) return false;
  // From eight row tiles per SM on; 8-bit matrices from six (measured with the threshold lowered:
  // 14336 x 4096 at 8 bits 14.3 us here against 19.7 in the tiled kernel, at 4 bits 10.7 against
  // 11.7 but 17408 x 5120 20.2 against 15.2, at 2 bits 12.0 against 10.2 and 24.7 against 12.8).
  if (tiles < dev.sm_count * tuning_int("DQ_B200_STREAM_MIN_TILES_PER_SM", BITS == 8 ? 6 : stream::kWarps)) return false;
  const auto align = static_cast<uintptr_t>(C::META_BYTES);
  if (reinterpret_cast<uintptr_t>(a.scales) % align != 0 || reinterpret_cast<uintptr_t>(a.offsets) % align != 0) {
    return false;
  }
  return true;
}

template <int BITS>
int32_t launch_stream(const GemvArgs& a, const DeviceInfo& dev, int tiles, int steps, cudaStream_t stream_h,
                      const peerpush::Push* push) {
  using C = stream::Cfg<BITS>;
  // The fp16-operand plan at 8 bits, where a code no longer has to be split into nibbles: half
  // the fragment registers, half the mma and half the staged activation per step.  (At 2 and 4
  // bits it saves one or two integer instructions per word but adds a sub.f16x2 per register;
  // measured on 262144 x 2048 it is slower there -- 43 vs 49 % and 72 vs 80 % of the copy
  // bandwidth -- so those widths keep the bf16-safe plan.)  Needs the unit-per-lane staging:
  // a 16-byte aligned 16-bit activation.
  const bool plan16 = (BITS == 8 || (BITS != 3 && tuning_int("DQ_B200_PLAN16_ALL") != 0)) &&
                      (a.in_features & 7) == 0 && (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 &&
                      tuning_int("DQ_B200_NO_PLAN16") == 0;
  stream::Params p = {};
  p.steps = steps;
  p.tiles = tiles;
  p.magic = (plan16 || a.x_dtype != DQ_BF16) ? 0x64006400u : 0x43004300u;
  if (push != nullptr) p.push = *push;
  const int aregs = plan16 ? 16 : (BITS == 8 ? 32 : 16);
  p.m_stride_u4 = steps * aregs + 4;
  const size_t smem = C::RING_BYTES + (static_cast<size_t>(a.m) * p.m_stride_u4 + aregs) * 16 +
                      static_cast<size_t>(steps) * 8 * 4 * 2;
  if (smem > static_cast<size_t>(dev.max_smem_optin)) {
    return DQ_ERR_UNSUPPORTED;
  }
  auto run = [&](auto kernel) -> int32_t {
    DQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    int per_sm = 0;
    DQ_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, stream::kThreads, smem));
    const int resident = std::max(1, per_sm) * dev.sm_count;
    int grid = std::min(static_cast<int>(ceil_div(tiles, stream::kWarps)), resident);
    // Strided tiles unless that leaves the busiest SM well above the average.  Several rounds:
    // with f = the fraction of CTAs that get one round more, an SM holds per_sm * f of them on
    // average and ceil(per_sm * f) at worst, each worth a round of kWarps tiles -- runs when that
    // excess is more than 3 % of an SM's share.  A single round that does not fill the machine
    // (fewer CTAs than fit): whole CTAs of kWarps tiles land unevenly on the SMs (20,480 rows:
    // 160 CTAs on 148 SMs, 16 tiles on some against 8.6 on average) -- then every resident CTA
    // slot gets a run of a few tiles instead.
    stream::Params q = p;
    {
      const int64_t per_round = static_cast<int64_t>(grid) * stream::kWarps;
      const int64_t rounds = ceil_div(tiles, per_round);
      const double average = static_cast<double>(tiles) / dev.sm_count;
      if (rounds > 1) {
        const double f = static_cast<double>(ceil_div(tiles - (rounds - 1) * per_round, stream::kWarps)) / grid;
        const double held = std::max(1, per_sm);
        const double excess = (std::ceil(held * f - 1e-9) - held * f) * stream::kWarps;
        q.runs = excess > 0.03 * average ? 1 : 0;
      } else if (grid < resident && ceil_div(grid, dev.sm_count) * stream::kWarps > 1.10 * average) {
        q.runs = 1;
        grid = std::min(tiles, resident);
      }
      const int forced = tuning_int("DQ_B200_STREAM_RUNS", -1);
      if (forced == 0) q.runs = 0, grid = std::min(static_cast<int>(ceil_div(tiles, stream::kWarps)), resident);
      if (forced == 1) q.runs = 1;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(stream::kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream_h;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    DQ_CUDA(cudaLaunchKernelEx(&cfg, kernel, a, q));
    DQ_CHECK_LAUNCH("gemv");
    note_kernel("gemv_mma_stream_kernel");
    return DQ_OK;
  };
  const bool xbf = a.x_dtype == DQ_BF16;
  const bool mbf = a.meta_dtype == DQ_BF16;
#ifdef DQ_TUNING
  constexpr bool kHasPlan16 = BITS != 3;
#else
  constexpr bool kHasPlan16 = BITS == 8;
#endif
  auto pick = [&](auto p16, auto pushing) -> int32_t {
    constexpr bool P = decltype(p16)::value, Q = decltype(pushing)::value;
    if (xbf && mbf) return run(stream::gemv_mma_stream_kernel<BITS, true, true, P, Q>);
    if (xbf) return run(stream::gemv_mma_stream_kernel<BITS, true, false, P, Q>);
    if (mbf) return run(stream::gemv_mma_stream_kernel<BITS, false, true, P, Q>);
    return run(stream::gemv_mma_stream_kernel<BITS, false, false, P, Q>);
  };
  if constexpr (kHasPlan16) {
    if (plan16) return push != nullptr ? pick(std::true_type{}, std::true_type{}) : pick(std::true_type{}, std::false_type{});
  }
  return push != nullptr ? pick(std::false_type{}, std::true_type{}) : pick(std::false_type{}, std::false_type{});
}

template <int BITS>
int32_t try_stream(const GemvArgs& a, const DeviceInfo& dev, int tiles, int steps, cudaStream_t stream_h,
                   bool* taken, const peerpush::Push* push) {
  *taken = false;
  if (!stream_ok<BITS>(a, dev, tiles, steps)) return DQ_OK;
  const int32_t rc = launch_stream<BITS>(a, dev, tiles, steps, stream_h, push);
  if (rc == DQ_ERR_UNSUPPORTED) return DQ_OK;  // does not fit: the generic kernel takes it
  *taken = true;
  return rc;
}

// ---- tiled kernel (dq_gemv_mma_tile.cuh): short and middle-sized matrices, fused shards ----

// One launch for `n` matrices sharing the activation.  *taken stays false (and nothing is
// launched) when the jobs do not meet the kernel's requirements.
int32_t try_tile(const GemvArgs* jobs, const int* bits, int n, const DeviceInfo& dev, cudaStream_t stream_h,
                 bool* taken, const peerpush::Push* push = nullptr) {
  *taken = false;
  const bool off = tuning_int("DQ_B200_NO_TILE") != 0;
  const int force_kw = tuning_int("DQ_B200_TILE_KW"), force_nb = tuning_int("DQ_B200_TILE_NB"),
            force_per_sm = tuning_int("DQ_B200_TILE_PER_SM");
  if (off || n < 1 || n > tilek::kMaxJobs) return DQ_OK;
  const GemvArgs& a0 = jobs[0];
  const int steps = a0.words_per_row / (4 * bits[0]);
  int max_bits = 0, max_tiles_total = 0;
  const bool g64_jobs = a0.group_values == kStepValues / 2;
  for (int i = 0; i < n; ++i) {
    const GemvArgs& a = jobs[i];
    // (The activations may differ -- row chunks of one activation over the same matrix -- as long
    // as they have the same shape: every CTA stages the activation of its own job.)
    if (a.m != a0.m || a.x_dtype != a0.x_dtype || a.meta_dtype != a0.meta_dtype ||
        a.in_features != a0.in_features || a.out_dtype != a0.out_dtype) {
      return DQ_OK;
    }
    if (a.group_values != a0.group_values || a.words_per_row / (4 * bits[i]) != steps) return DQ_OK;
    if (a.group_values == kStepValues / 2) {
      if (a.num_groups != 2 * steps) return DQ_OK;
    } else if (a.group_values != kStepValues || a.num_groups != steps) {
      return DQ_OK;
    }
    if (reinterpret_cast<uintptr_t>(a.packed) % 16 != 0 || (static_cast<int64_t>(a.words_per_row) * 4) % 16 != 0) {
      return DQ_OK;
    }
    max_bits = std::max(max_bits, bits[i]);
    max_tiles_total += static_cast<int>(ceil_div(a.rows, kTileRows));
  }
  // Long matrices with one group per step have leaner kernels of their own (the streaming
  // kernel, or the register ring at 2 bits): this one is for what does not fill the machine
  // eight tiles per SM deep, for fused shards and for 64-value groups.
  const bool tile_all = tuning_int("DQ_B200_TILE_ALL") != 0;
  if (n == 1 && !g64_jobs && !tile_all && max_tiles_total >= dev.sm_count * tilek::kWarps) return DQ_OK;
  // Shape of the CTAs.  First choice: ONE wave in which every warp's whole share of the
  // weights is in flight before the activation arrives -- the finest slicing of the reduction
  // axis whose grid is resident at once.  Otherwise CTAs persist over several items with a
  // ring of a few stages, sliced as finely as leaves four steps between two reductions.
  constexpr size_t kSmemPerSm = 228 * 1024, kCtaReserve = 1024;
  int ctas_by_registers = 3;  // which build of the kernel: see gemv_mma_tile_kernel
  struct Shape {
    int kw = 0, ch = 0, nb = 0, per_sm = 0, ipc = 0, sb = 0;
    size_t smem = 0;
  };
  const bool g64 = a0.group_values == kStepValues / 2;
  const int gps = g64 ? 2 : 1;  // groups per step
  auto meta_aligned = [&](int c) {
    for (int i = 0; i < n; ++i) {
      const auto al = static_cast<uintptr_t>(2 * c * gps);  // a stage's metadata of one row, copied whole
      if (jobs[i].num_groups % (c * gps) != 0 || reinterpret_cast<uintptr_t>(jobs[i].scales) % al != 0 ||
          reinterpret_cast<uintptr_t>(jobs[i].offsets) % al != 0) {
        return false;
      }
    }
    return true;
  };
  auto items_at = [&](int kw) {
    const int rw = tilek::kWarps / kw;
    int64_t items = 0;
    for (int i = 0; i < n; ++i) items += ceil_div(ceil_div(jobs[i].rows, kTileRows), rw);
    return items;
  };
  auto shape_with = [&](int kw, bool one_shot, int ch) {
    Shape sh;
    const int spw = steps / kw;
    const bool wide = kw < tilek::kWarps;
    const size_t stage = static_cast<size_t>(ch) * 2 * (4 * max_bits) * tilek::kThreads + ch * gps * 2 * tilek::kThreads;
    auto fixed_with = [&](int sb) {
      return tilek::kRedFloats * 4 +
             (max_bits == 8 ? tilek::stage_bytes<8>(a0.m, steps, spw, kw, wide, a0.in_features, gps, sb)
                            : tilek::stage_bytes<4>(a0.m, steps, spw, kw, wide, a0.in_features, gps, sb));
    };
    size_t fixed = fixed_with(spw);
    int sb = spw;
    // Per-warp staging whose whole slices do not fit beside a two-stage ring (many activation rows
    // x a long reduction axis): the slices go through the staging area block by block -- the
    // longest block with which two CTAs still fit on an SM, else the longest that fits at all.
    if (!wide && 2 * stage + fixed > static_cast<size_t>(dev.max_smem_optin)) {
      if (ch != 2) return sh;  // (the block-by-block kernel is built for stages of two steps only)
      const size_t rooms[2] = {kSmemPerSm / 2 - kCtaReserve, static_cast<size_t>(dev.max_smem_optin)};
      for (int r = 0; r < 2 && sb == spw; ++r) {
        for (int cand = spw - ch; cand >= ch; cand -= ch) {
          if (spw % cand == 0 && 2 * stage + fixed_with(cand) <= rooms[r]) {
            sb = cand;
            break;
          }
        }
      }
      if (sb == spw) return sh;
      fixed = fixed_with(sb);
    }
    const int stages = spw / ch;
    int nb = one_shot ? stages : std::min(stages * 2, ch == 4 ? 2 : 4);
    if (force_nb > 0 && !one_shot) nb = force_nb;
    nb = std::min(nb, tilek::kMaxRing);
    if (one_shot && nb < stages) return sh;
    if (!one_shot) {  // a persistent CTA takes whatever ring still fits, two stages at least
      while (nb > 2 && nb * stage + fixed > static_cast<size_t>(dev.max_smem_optin)) --nb;
    }
    const size_t smem = nb * stage + fixed;
    if (smem > static_cast<size_t>(dev.max_smem_optin)) return sh;
    sh.kw = kw;
    sh.ch = ch;
    sh.nb = nb;
    sh.sb = sb;
    sh.smem = smem;
    sh.per_sm = std::min<int>(ctas_by_registers, static_cast<int>(kSmemPerSm / (smem + kCtaReserve)));
    if (force_per_sm > 0) sh.per_sm = std::min(sh.per_sm, force_per_sm);
    const int64_t cap = static_cast<int64_t>(sh.per_sm) * dev.sm_count;
    sh.ipc = static_cast<int>(ceil_div(items_at(kw), cap));
    return sh;
  };
  // stages of four steps where they fit, of two otherwise (long rows x many activation rows
  // leave little shared memory beside the staged activation)
  auto shape_at = [&](int kw, bool one_shot) {
    Shape sh;
    if (steps % kw != 0) return sh;
    const int spw = steps / kw;
    if (spw % 4 == 0 && meta_aligned(4)) sh = shape_with(kw, one_shot, 4);
    if (sh.kw == 0 && spw % 2 == 0 && meta_aligned(2)) sh = shape_with(kw, one_shot, 2);
    return sh;
  };
  auto choose = [&]() {
    Shape best;
    // Several activation rows: staging them is the larger part of a CTA's prologue, so whole
    // rows per warp (the activation staged once per eight row tiles) win over the finest
    // slicing as soon as that still gives every other SM a CTA (measured, 12288 x 2048 at
    // eight rows: 8.4-8.8 us against 9.1-11.1).
    if (a0.m >= 6 && force_kw == 0) {
      const Shape sh = shape_at(1, true);
      if (sh.kw != 0 && sh.per_sm >= 1 && sh.ipc == 1 && items_at(1) * 2 >= dev.sm_count) best = sh;
    }
    for (int kw = tilek::kWarps; kw >= 1 && best.kw == 0; kw /= 2) {
      if (force_kw > 0 && kw != force_kw) continue;
      const Shape sh = shape_at(kw, true);
      if (sh.kw != 0 && sh.per_sm >= 1 && sh.ipc == 1) best = sh;
    }
    for (int kw = tilek::kWarps; kw >= 1 && best.kw == 0; kw /= 2) {
      if (force_kw > 0 && kw != force_kw) continue;
      if (force_kw == 0 && kw > 1 && (steps % kw != 0 || steps / kw < 4)) continue;
      const Shape sh = shape_at(kw, false);
      if (sh.kw != 0 && sh.per_sm >= 1) best = sh;
    }
    return best;
  };
  // The three-CTA build only where its third CTA per SM buys a finer one-wave slicing.
  const int force_ctas = tuning_int("DQ_B200_TILE_CTAS");
  ctas_by_registers = 3;
  Shape pick = choose();
  const bool needs_three = pick.kw != 0 && pick.ipc == 1 && pick.nb == (steps / pick.kw) / pick.ch &&
                           items_at(pick.kw) > 2LL * dev.sm_count;
  if ((!needs_three && force_ctas != 3) || force_ctas == 2) {
    ctas_by_registers = 2;
    pick = choose();
  }
  if (pick.kw == 0) return DQ_OK;
  const int kw = pick.kw, rw = tilek::kWarps / kw, spw = steps / kw, ch = pick.ch;
  const bool wide = kw < tilek::kWarps;
  const size_t smem = pick.smem;

  tilek::Launch L = {};
  L.njobs = n;
  L.steps = steps;
  L.rw = rw;
  L.kw = kw;
  L.spw = spw;
  L.sb = pick.sb;
  L.nb = pick.nb;
  L.wide_stage = wide ? 1 : 0;
  L.meta_bf16 = a0.meta_dtype == DQ_BF16 ? 1 : 0;
  L.magic = a0.x_dtype == DQ_BF16 ? 0x43004300u : 0x64006400u;
  if (push != nullptr) L.push = *push;
  for (int i = 0; i < n; ++i) {
    L.job[i].a = jobs[i];
    L.job[i].bits = bits[i];
    L.job[i].tiles = static_cast<int>(ceil_div(jobs[i].rows, kTileRows));
    L.job[i].items = static_cast<int>(ceil_div(L.job[i].tiles, rw));
  }
  // every CTA of a job takes the same number of items (ipc), the jobs' CTAs side by side
  const int64_t cap = static_cast<int64_t>(pick.per_sm) * dev.sm_count;
  int grid = 0;
  for (int ipc = pick.ipc;; ++ipc) {
    grid = 0;
    for (int i = 0; i < n; ++i) {
      L.job[i].cta_begin = grid;
      L.job[i].cta_count = static_cast<int>(ceil_div(L.job[i].items, ipc));
      grid += L.job[i].cta_count;
    }
    if (grid <= cap || ipc > pick.ipc + 4) break;
  }

  auto run = [&](auto kernel) -> int32_t {
    if (smem > 48 * 1024) {
      DQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(tilek::kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream_h;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    DQ_CUDA(cudaLaunchKernelEx(&cfg, kernel, L));
    DQ_CHECK_LAUNCH("gemv");
    note_kernel("gemv_mma_tile_kernel");
    *taken = true;
    return DQ_OK;
  };
  const bool xbf = a0.x_dtype == DQ_BF16;
  auto dispatch = [&](auto ctas) -> int32_t {
    constexpr int N = decltype(ctas)::value;
    if (g64) {
      if (ch == 4) return xbf ? run(tilek::gemv_mma_tile_kernel<true, 4, true, N>) : run(tilek::gemv_mma_tile_kernel<false, 4, true, N>);
      return xbf ? run(tilek::gemv_mma_tile_kernel<true, 2, true, N>) : run(tilek::gemv_mma_tile_kernel<false, 2, true, N>);
    }
    if (ch == 4) return xbf ? run(tilek::gemv_mma_tile_kernel<true, 4, false, N>) : run(tilek::gemv_mma_tile_kernel<false, 4, false, N>);
    return xbf ? run(tilek::gemv_mma_tile_kernel<true, 2, false, N>) : run(tilek::gemv_mma_tile_kernel<false, 2, false, N>);
  };
  if (pick.sb < spw) {  // slices staged block by block: its own build (two CTAs per SM, stages of two steps)
    if (g64) return xbf ? run(tilek::gemv_mma_tile_kernel<true, 2, true, 2, true>) : run(tilek::gemv_mma_tile_kernel<false, 2, true, 2, true>);
    return xbf ? run(tilek::gemv_mma_tile_kernel<true, 2, false, 2, true>) : run(tilek::gemv_mma_tile_kernel<false, 2, false, 2, true>);
  }
  if (ctas_by_registers == 3) return dispatch(std::integral_constant<int, 3>{});
  return dispatch(std::integral_constant<int, 2>{});
}

}  // namespace

bool mma_enabled_for_rows() { return mma_enabled(); }
bool pdl_enabled_for_rows() { return pdl_enabled(); }

bool mma_path_supports(const GemvArgs& a, int bits) {
  if (!mma_enabled()) return false;
  if (a.x_dtype != DQ_BF16 && a.x_dtype != DQ_F16) return false;
  if (a.meta_dtype != DQ_BF16 && a.meta_dtype != DQ_F16) return false;
  if (a.group_values != kStepValues / 2 && a.group_values % kStepValues != 0) {
    return false;  // (64-value groups: the tiled kernel only)
  }
  const auto addr = reinterpret_cast<uintptr_t>(a.packed);
  const int align = bits == 2 ? 8 : (bits == 3 ? 4 : 16);
  if (addr % align != 0 || (static_cast<int64_t>(a.words_per_row) * 4) % align != 0) return false;
  // (Whether the staged activation fits shared memory is each kernel's own question: the tiled
  // kernel passes long slices through its staging area block by block, the others refuse.)
  return device_info() != nullptr;
}

int32_t launch_gemv_mma_fused(const GemvArgs* jobs, const int* bits, int n, cudaStream_t stream, bool* taken,
                              const peerpush::Push* push) {
  *taken = false;
  const DeviceInfo* dev = device_info();
  if (dev == nullptr) return DQ_ERR_CUDA;
  for (int i = 0; i < n; ++i) {
    if (!mma_path_supports(jobs[i], bits[i])) return DQ_OK;
  }
  if (push == nullptr && tuning_int("DQ_B200_NO_STREAM_MULTI") == 0) {
    // matrices long enough to be streamed: the streaming body, a range of CTAs per matrix
    if (const int32_t rc = launch_gemv_stream_fused(jobs, bits, n, stream, taken)) return rc;
    if (*taken) return DQ_OK;
  }
  return try_tile(jobs, bits, n, *dev, stream, taken, push);
}

// The tiled kernel slices the reduction axis 8, 4 or 2 ways over the warps of a CTA, in slices of
// an even number of 128-value steps.  A step count with few such factors (K = 8960, 11008, 18944:
// 70, 86 and 148 steps) on a matrix of few rows leaves it with CTAs for a fraction of the SMs; the
// many-rows kernel, which slices the reduction axis over a cluster in any proportion, is then the
// faster kernel at every number of activation rows (measured at 2 / 4 / 8 bits, one row: 3584 x
// 18944 21 / 19 / 37 us against 25 / 26 / 52; 4096 x 11008 19 / 21 / 23 against 28 / 38 / 51;
// 1536 x 8960 10 / 11 / 12 against 23 / 31 / 41).
bool rows_kernel_first(const GemvArgs& a, int bits) {
  const DeviceInfo* dev = device_info();
  if (dev == nullptr || (a.group_values != 128 && a.group_values != 64) || a.words_per_row % (4 * bits) != 0) return false;
  const int steps = a.words_per_row / (4 * bits);
  int kw = 8;
  while (kw > 1 && (steps % kw != 0 || (steps / kw) % 2 != 0)) kw /= 2;
  const int64_t ctas = ceil_div(ceil_div(a.rows, 16) * kw, 8);
  // (... and a long chain per warp: with 28 steps, K = 3584, two slices of 14 are over soon enough --
  // 3584 x 3584 and 4608 x 3584 at 2 / 3 bits run 6.4-7.8 us there against 7.9-10.3 here)
  if (ctas * 2 < dev->sm_count && steps / kw >= 24) return true;
  // The tiled kernel stages the whole activation in fragment order (16 bytes per register of the
  // plan, step and row).  Where that leaves little room for a ring (six rows x K = 14336; at 8 bits
  // four rows) it passes the slices through shared memory block by block, every CTA again; the
  // many-rows kernel does that once per eight row tiles and reads ahead meanwhile (4096 x 14336,
  // eight rows, 2 / 3 / 4 / 8 bits: 21 / 28 / 16 / 30 us against 27 / 30 / 37 / 53).
  const int64_t frag_bytes = static_cast<int64_t>(a.m) * steps * (bits == 8 ? 32 : 16) * 16;
  return frag_bytes > (144 << 10);
}

// Where the streaming body with the reduction axis sliced over a cluster (dq_gemv_stream_sliced.cu)
// goes first, all measured against the tiled (or many-rows) kernel on matrices of 16 MB and more:
//  * the many-rows kernel would be handed the matrix anyway (3584 x 18944 at one row, 2 / 3 / 4 / 8
//    bits: 13 / 18 / 15 / 18 us against 21 / 30 / 19 / 34; 4096 x 14336 at eight rows 13 / 17 / 17 / 19
//    against 21 / 28 / 16 / 28);
//  * the tiled kernel has about a CTA of eight warps per SM or fewer and 24 steps or more per warp
//    -- the decode wants more resident warps (5120 x 17408 at one row 14 / 20 / 17 / 21 against 21 /
//    29 / 26 / 46);
//  * it cannot slice the reduction axis eight ways (K = 5120: 40 steps) and has fewer than 2.5 CTAs
//    per SM, from 20 MB on (10240 x 5120 at one row, 4 / 8 bits: 12.0 / 15.5 against 14.7 / 22.5;
//    but 7168 x 5120 at 4 bits, 18 MB, 10.8 against 9.0, and 17408 x 5120, 544 CTAs, 14.0 / 19.5 /
//    17.0 at 2 / 3 / 4 bits against 13.0 / 17.0 / 15.7);
//  * seven or eight activation rows (8192 x 8192 13.7 / 16.9 / 16.8 / 22.9 against 18.5 / 20.7 / 20.6
//    / 32; 11008 x 4096 11.1 / 13.7 / 11.7 / 14.1 against 13.9 / 14.5 / 13.7 / 21.1);
//  * up to 8192 weight rows: four and more activation rows from 20 MB on (4096 x 14336 at 3 / 4 bits
//    15.4 / 13.7 against 18.5 / 17.3; 8192 x 8192 15.8 / 13.9 against 18.2 / 16.5; but 12288 x 8192 26.7
//    / 25.5 against 25.0 / 22.5), any number from 56 MB on (8192 x 28672 at one row, 2 / 3 / 4 bits: 28
//    / 42 / 34 against 33 / 45 / 39; 4096 x 14336 and 8192 x 8192 at 8 bits 17 against 22);
//  * 8-bit codes with two or more rows from 24 MB on, with one row from 96 MB on (8192 x 8192 at
//    four rows 18 against 44; 8192 x 28672 at one row 49 against 102; 4096 x 4096, 17 MB, at two rows
//    9.6 against 8.6).
// Elsewhere -- one to three rows on matrices the tiled kernel fills the SMs with twice over (4096 x
// 14336, 8192 x 8192 below 56 MB, 12288 x 8192 at any row count), small matrices (4096 x 4096, 2048 x
// 6144, 7168 x 5120 at 2-4 bits) -- the tiled kernel is level or faster, by up to 50 % on the small
// ones: its eight slices share one CTA's staged activation.
bool stream_sliced_first(const GemvArgs& a, int bits, bool rows_first) {
  const DeviceInfo* dev = device_info();
  if (dev == nullptr || a.group_values != kStepValues || a.words_per_row % (4 * bits) != 0) return false;
  const int64_t bytes = static_cast<int64_t>(a.rows) * a.words_per_row * 4;
  if (bytes < (16 << 20)) return false;
  if (rows_first || a.m >= 7) return true;
  const int steps = a.words_per_row / (4 * bits);
  int kw = 8;
  while (kw > 1 && (steps % kw != 0 || (steps / kw) % 2 != 0)) kw /= 2;
  const int64_t ctas = ceil_div(ceil_div(a.rows, 16) * kw, 8);
  // (a CTA per SM AND a long chain per warp: 2048 x 16384 has 128 CTAs there but slices of 16 steps,
  // and runs 9.0 us at 4 bits against 14.1 here, whose 16 row groups x 8 slices cannot fill the SMs)
  if (ctas * 4 < static_cast<int64_t>(dev->sm_count) * 5 && steps / kw >= 24) return true;
  if (kw < 8 && bytes >= (20 << 20) && ctas * 2 < static_cast<int64_t>(dev->sm_count) * 5) return true;
  if (a.rows <= 8192 && ((a.m >= 4 && bytes >= (20 << 20)) || bytes >= (56 << 20))) return true;
  return bits == 8 && ((a.m >= 2 && bytes >= (24 << 20)) || bytes >= (96 << 20));
}

int32_t launch_gemv_mma(const GemvArgs& a, int bits, cudaStream_t stream, const peerpush::Push* push) {
  const DeviceInfo* dev = device_info();
  if (dev == nullptr) return DQ_ERR_CUDA;
  // the many-rows kernel where the tiled kernel is known to be the slower one (rows_kernel_first)
  const int rows_switch = tuning_int("DQ_B200_ROWS_SMALL_M", -1);  // 0: never below nine rows; 1: wherever it qualifies
  const bool rows_first = push == nullptr && (rows_switch == 1 || (rows_switch != 0 && rows_kernel_first(a, bits)));
  if (a.group_values == kStepValues / 2) {  // two groups per step: the tiled and the many-rows kernel do that
    bool taken = false;
    if (rows_first) {
      const int32_t rc = launch_gemv_rows(a, bits, stream, &taken, 1);
      if (taken || rc != DQ_OK) return rc;
    }
    const int32_t rc = try_tile(&a, &bits, 1, *dev, stream, &taken, push);
    return (rc == DQ_OK && !taken) ? DQ_ERR_UNSUPPORTED : rc;
  }
  MmaParams p = {};
  p.steps = a.words_per_row / (4 * bits);  // a step is 4 units of `bits` words
  p.steps_per_group = a.group_values / kStepValues;
  p.tiles = static_cast<int>(ceil_div(a.rows, kTileRows));
  {
    bool taken = false;
    int32_t rc = DQ_OK;
    switch (bits) {
      case 2:
        rc = try_stream<2>(a, *dev, p.tiles, p.steps, stream, &taken, push);
        break;
      case 3:
        rc = try_stream<3>(a, *dev, p.tiles, p.steps, stream, &taken, push);
        break;
      case 4:
        rc = try_stream<4>(a, *dev, p.tiles, p.steps, stream, &taken, push);
        break;
      default:
        rc = try_stream<8>(a, *dev, p.tiles, p.steps, stream, &taken, push);
        break;
    }
    if (taken || rc != DQ_OK) return rc;
    // (not a stream of bytes for the streaming kernel)
    const int sliced_switch = tuning_int("DQ_B200_STREAM_SLICED", -1);  // 0: never; 1: wherever it qualifies
    if (push == nullptr && (sliced_switch == 1 || (sliced_switch != 0 && stream_sliced_first(a, bits, rows_first)))) {
      rc = launch_gemv_stream_sliced(a, bits, stream, &taken);
      if (taken || rc != DQ_OK) return rc;
    }
    if (rows_first) {
      rc = launch_gemv_rows(a, bits, stream, &taken, 1);
      if (taken || rc != DQ_OK) return rc;
    }
    rc = try_tile(&a, &bits, 1, *dev, stream, &taken, push);
    if (taken || rc != DQ_OK) return rc;
  }
  if (push != nullptr) return DQ_ERR_UNSUPPORTED;  // the register-ring kernel below does not push
  // Shape of a CTA: rw row tiles x kw slices of the reduction axis, 8 or 16 warps.  A short
  // matrix is over in one dependent chain of latencies (launch, activation staging, a few
  // steps, reduction), so what matters is that EVERY CTA is resident at once -- a second
  // wave doubles the chain -- and, within that, that as many warps as possible share the
  // work.  Long matrices take kw = 1 and let the warps persist over the tiles.
  {
    const int kw_max = std::min(kMaxWarps, floor_pow2(p.steps));
    // CTAs of 8 warps fit twice on an SM at this kernel's register count, 16 warps once.
    const int cap8 = 2 * dev->sm_count, cap16 = dev->sm_count;
    int best_rw = 8, best_kw = 1;
    int64_t best_warps = -1;
    for (int warps = 8; warps <= kMaxWarps; warps *= 2) {
      for (int kw = 1; kw <= std::min(warps, kw_max); kw *= 2) {
        const int rw = warps / kw;
        const int grid = static_cast<int>(ceil_div(p.tiles, rw));
        if (grid > (warps == 8 ? cap8 : cap16)) continue;  // would need a second wave
        const int64_t busy = static_cast<int64_t>(std::min(p.tiles, grid * rw)) * kw;
        // more busy warps first; then smaller CTAs (they spread over more SMs)
        if (busy > best_warps || (busy == best_warps && warps < best_rw * best_kw)) {
          best_warps = busy;
          best_rw = rw;
          best_kw = kw;
        }
      }
    }
    p.rw = best_rw;  // nothing fits in one wave: 8 persistent warps per CTA, kw = 1
    p.kw = best_kw;
  }
  {
    const int force_kw = tuning_int("DQ_B200_MMA_KW"), force_rw = tuning_int("DQ_B200_MMA_RW");
    if (force_kw > 0) p.kw = std::min(force_kw, floor_pow2(p.steps));
    if (force_rw > 0) p.rw = std::min(force_rw, kMaxWarps / p.kw);
  }
  p.steps_per_warp = static_cast<int>(ceil_div(p.steps, p.kw));
  const int depth = bits == 8 ? 2 : 4;
  const auto meta_align = static_cast<uintptr_t>(2 * depth);
  p.vec_meta = p.steps_per_group == 1 && a.num_groups % depth == 0 && p.steps_per_warp % depth == 0 &&
               reinterpret_cast<uintptr_t>(a.scales) % meta_align == 0 &&
               reinterpret_cast<uintptr_t>(a.offsets) % meta_align == 0;
  p.magic = a.x_dtype == DQ_BF16 ? 0x43004300u : 0x64006400u;
  const int aregs = bits == 8 ? 32 : 16;
  const size_t smem = mma_smem_bytes(a.m, p.steps, aregs, p.rw, p.kw, &p.m_stride_u4);
  if (smem > static_cast<size_t>(dev->max_smem_optin)) return DQ_ERR_UNSUPPORTED;  // the caller halves the rows
  const int threads = p.rw * p.kw * kWarp;
  switch (bits) {
    case 2:
      return launch_mma_bits<2>(a, p, threads, smem, *dev, stream);
    case 3:
      return launch_mma_bits<3>(a, p, threads, smem, *dev, stream);
    case 4:
      return launch_mma_bits<4>(a, p, threads, smem, *dev, stream);
    default:
      return launch_mma_bits<8>(a, p, threads, smem, *dev, stream);
  }
}

}  // namespace dq

