// Packed words -> dense [rows, in_features] matrix, bit-exact against the
// reference's QuantTensor.dequantize.
//
// Replaces dequant_kernel / dequant_cuda
// (packages/dynquant-kernels/csrc/quant/dequant.cu:47-93, :130-165).  It is the
// prefill (M > 8) feed for a dense GEMM, the embedding-row decoder, and the
// anchor of the parity suite: a wrong bit anywhere in the decode shows here as
// a wrong number, with no accumulation to hide behind.
//
// Arithmetic: w = float(q) * scale, then + offset, both rounded to fp32
// (packages/dynquant-core/src/dynquant/quant/tensor.py:417-426 multiplies and
// then adds), then one rounding to the output dtype.  With fp16/bf16 scales the
// product is exact in fp32, so this equals the reference CUDA kernel's single
// fmaf as well; with fp32 scales it follows the torch definition.  An absent
// offsets tensor means "no add", not "+0".
//
// Two kernels.  dequant_octet_kernel is the one nearly every tensor takes (in_features and
// the group size multiples of 8): a thread produces 8 consecutive values -- one 16-byte
// store for a 16-bit output, so a warp writes 512 contiguous bytes per store instruction --
// from the 8 * BITS bits at bit 8 * BITS * octet of its row (the packed row is one
// contiguous LSB-first bit string: groups are whole numbers of 32-value blocks).  Rows run
// over blockIdx.y and octets over blockIdx.x, so no thread divides anything.  dequant_kernel
// is the general one: one thread per block of 16/32/8/4 values at 2/3/4/8-bit, any tail.
#include <algorithm>

#include "dq_decode.cuh"

namespace dq {
namespace {

constexpr int kDequantThreads = 256;

struct DequantArgs {
  const uint32_t* packed;
  const void* scales;
  const void* offsets;
  void* out;
  int meta_dtype, out_dtype;
  int rows;
  int words_per_row, num_groups, words_per_group, group_values, in_features;
  int blocks_per_group, blocks_per_row;
};

// 8 consecutive values of one row per thread.  `group_shift` >= 0: the group size is 2^shift.
template <int BITS>
__global__ void __launch_bounds__(kDequantThreads) dequant_octet_kernel(const DequantArgs a, int octets_per_row,
                                                                        int group_shift) {
  const bool has_offsets = a.offsets != nullptr;
  constexpr uint32_t kMask = (1u << BITS) - 1u;
  for (int row = blockIdx.y; row < a.rows; row += gridDim.y) {
    const uint32_t* src = a.packed + static_cast<int64_t>(row) * a.words_per_row;
    for (int o = blockIdx.x * kDequantThreads + threadIdx.x; o < octets_per_row; o += gridDim.x * kDequantThreads) {
      const int bit = o * 8 * BITS;
      const int word = bit >> 5;
      // the octet's 8 * BITS bits (64 at 8-bit: two whole words)
      uint32_t lo, hi = 0u;
      if constexpr (BITS == 8) {
        const uint2 v = __ldg(reinterpret_cast<const uint2*>(src) + o);
        lo = v.x, hi = v.y;
      } else if constexpr (BITS == 4) {
        lo = __ldg(src + word);
      } else if constexpr (BITS == 2) {
        lo = __ldg(src + word) >> (bit & 31);
      } else {
        const uint32_t w0 = __ldg(src + word);
        const uint32_t w1 = (bit & 31) > 8 ? __ldg(src + word + 1) : 0u;  // 24 bits from bit (bit & 31)
        lo = __funnelshift_r(w0, w1, bit & 31);
      }
      const int value0 = o * 8;
      const int g = group_shift >= 0 ? (value0 >> group_shift) : value0 / a.group_values;
      const int64_t meta = static_cast<int64_t>(row) * a.num_groups + g;
      const float scale = load_f32(a.scales, meta, a.meta_dtype);
      const float offset = has_offsets ? load_f32(a.offsets, meta, a.meta_dtype) : 0.0f;
      float vals[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        uint32_t q;
        if constexpr (BITS == 8) {
          q = ((i < 4 ? lo : hi) >> (8 * (i & 3))) & 0xFFu;
        } else {
          q = (lo >> (BITS * i)) & kMask;
        }
        // float(q) without the conversion unit (a quarter-rate pipe): 2^23 + q is exactly
        // representable, so OR-ing q into the mantissa of 2^23 and subtracting 2^23 is exact
        const float qf = __uint_as_float(0x4B000000u | q) - 8388608.0f;
        float v = __fmul_rn(qf, scale);
        if (has_offsets) v = __fadd_rn(v, offset);
        vals[i] = v;
      }
      const int64_t out_base = static_cast<int64_t>(row) * a.in_features + value0;
      if (a.out_dtype == DQ_F32) {
        float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.out) + out_base);
        dst[0] = make_float4(vals[0], vals[1], vals[2], vals[3]);
        dst[1] = make_float4(vals[4], vals[5], vals[6], vals[7]);
      } else {
        uint32_t p16[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          p16[j] = round_pair_to_16(vals[2 * j], vals[2 * j + 1], a.out_dtype);
        }
        *reinterpret_cast<uint4*>(reinterpret_cast<unsigned short*>(a.out) + out_base) =
            make_uint4(p16[0], p16[1], p16[2], p16[3]);
      }
    }
  }
}

template <int BITS>
__global__ void __launch_bounds__(kDequantThreads) dequant_kernel(const DequantArgs a) {
  constexpr int VB = Block<BITS>::kValues;
  constexpr int WB = Block<BITS>::kWords;
  const int64_t total = static_cast<int64_t>(a.rows) * a.blocks_per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const bool has_offsets = a.offsets != nullptr;

  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += stride) {
    const int row = static_cast<int>(idx / a.blocks_per_row);
    const int blk = static_cast<int>(idx - static_cast<int64_t>(row) * a.blocks_per_row);
    const int g = blk / a.blocks_per_group;
    const int bg = blk - g * a.blocks_per_group;
    const int word_base = g * a.words_per_group + (bg * VB * BITS) / 32;
    const int words_left = a.words_per_row - word_base;
    const int value_base = g * a.group_values + bg * VB;
    // Values of this block that exist: bounded by the group (per-row tail) and
    // by in_features (zero pad of the last group).
    const int live = min(min(VB, a.group_values - bg * VB), a.in_features - value_base);
    if (live <= 0) {
      continue;
    }
    const uint32_t* src = a.packed + static_cast<int64_t>(row) * a.words_per_row + word_base;
    const int64_t meta = static_cast<int64_t>(row) * a.num_groups + g;
    const float scale = load_f32(a.scales, meta, a.meta_dtype);
    const float offset = has_offsets ? load_f32(a.offsets, meta, a.meta_dtype) : 0.0f;
    const int64_t out_base = static_cast<int64_t>(row) * a.in_features + value_base;

    if (live == VB && words_left >= WB) {
      uint32_t w[WB];
#pragma unroll
      for (int i = 0; i < WB; ++i) {
        w[i] = __ldg(src + i);
      }
      float vals[VB];
      for_each_pair<BITS>(w, [&](int p, float2 q2) {
        float lo = __fmul_rn(q2.x, scale);
        float hi = __fmul_rn(q2.y, scale);
        if (has_offsets) {
          lo = __fadd_rn(lo, offset);
          hi = __fadd_rn(hi, offset);
        }
        vals[2 * p] = lo;
        vals[2 * p + 1] = hi;
      });
      if (a.out_dtype == DQ_F32) {
        float* dst = reinterpret_cast<float*>(a.out) + out_base;
        if ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
          for (int j = 0; j < VB / 4; ++j) {
            reinterpret_cast<float4*>(dst)[j] =
                make_float4(vals[4 * j], vals[4 * j + 1], vals[4 * j + 2], vals[4 * j + 3]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < VB; ++j) {
            dst[j] = vals[j];
          }
        }
      } else {
        unsigned short* dst = reinterpret_cast<unsigned short*>(a.out) + out_base;
        uint32_t packed16[VB / 2];
#pragma unroll
        for (int j = 0; j < VB / 2; ++j) {
          packed16[j] = round_to_16(vals[2 * j], a.out_dtype) |
                        (round_to_16(vals[2 * j + 1], a.out_dtype) << 16);
        }
        const uintptr_t addr = reinterpret_cast<uintptr_t>(dst);
        if (VB % 8 == 0 && (addr & 15) == 0) {
#pragma unroll
          for (int j = 0; j < VB / 8; ++j) {
            reinterpret_cast<uint4*>(dst)[j] = make_uint4(packed16[4 * j], packed16[4 * j + 1],
                                                          packed16[4 * j + 2], packed16[4 * j + 3]);
          }
        } else if ((addr & 3) == 0) {
#pragma unroll
          for (int j = 0; j < VB / 2; ++j) {
            reinterpret_cast<uint32_t*>(dst)[j] = packed16[j];
          }
        } else {
#pragma unroll
          for (int j = 0; j < VB / 2; ++j) {
            dst[2 * j] = static_cast<unsigned short>(packed16[j] & 0xFFFFu);
            dst[2 * j + 1] = static_cast<unsigned short>(packed16[j] >> 16);
          }
        }
      }
    } else {
      for (int j = 0; j < live; ++j) {
        const float q = static_cast<float>(code_at<BITS>(src, j, words_left));
        float v = __fmul_rn(q, scale);
        if (has_offsets) {
          v = __fadd_rn(v, offset);
        }
        store_f32(a.out, out_base + j, a.out_dtype, v);
      }
    }
  }
}

}  // namespace
}  // namespace dq

extern "C" int32_t dq_dequant(const dq_weight* w, void* out, int32_t out_dtype, void* stream) {
  dq_geometry g;
  if (const int32_t rc = dq_resolve_geometry("dequant", w, &g)) return rc;
  DQ_REQUIRE(dq::dtype_ok(out_dtype), "dequant: unsupported output dtype tag %d", out_dtype);
  if (w->rows == 0) return DQ_OK;
  DQ_REQUIRE(out != nullptr, "dequant: null output pointer");

  dq::DequantArgs a = {};
  a.packed = static_cast<const uint32_t*>(w->packed);
  a.scales = w->scales;
  a.offsets = w->offsets;
  a.out = out;
  a.meta_dtype = w->meta_dtype;
  a.out_dtype = out_dtype;
  a.rows = static_cast<int>(w->rows);
  a.words_per_row = g.words_per_row;
  a.num_groups = g.num_groups;
  a.words_per_group = g.words_per_group;
  a.group_values = g.group_values;
  a.in_features = g.in_features;
  a.blocks_per_group = g.blocks_per_group;
  a.blocks_per_row = g.blocks_per_row;

  const dq::DeviceInfo* dev = dq::device_info();
  if (dev == nullptr) return DQ_ERR_CUDA;
  auto s = static_cast<cudaStream_t>(stream);
  // The octet kernel: whole octets per row and per group, 16-byte aligned output rows, and
  // (8-bit) 8-byte aligned packed rows.
  const size_t out_elem = static_cast<size_t>(dq::dtype_size(out_dtype));
  const bool octets = a.in_features % 8 == 0 && a.group_values % 8 == 0 &&
                      reinterpret_cast<uintptr_t>(out) % 16 == 0 && (a.in_features * out_elem) % 16 == 0 &&
                      (w->bits != 8 || (reinterpret_cast<uintptr_t>(a.packed) % 8 == 0 && a.words_per_row % 2 == 0));
  if (octets) {
    const int octets_per_row = a.in_features / 8;
    int shift = -1;
    if ((a.group_values & (a.group_values - 1)) == 0) {
      shift = 0;
      while ((1 << shift) < a.group_values) ++shift;
    }
    const int gx = static_cast<int>(std::min<int64_t>(dq::ceil_div(octets_per_row, dq::kDequantThreads), 64));
    const int gy = static_cast<int>(std::min<int64_t>(a.rows, std::max<int64_t>(1, (static_cast<int64_t>(dev->sm_count) * 64) / gx)));
    const dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy));
    switch (w->bits) {
      case 2:
        dq::dequant_octet_kernel<2><<<grid, dq::kDequantThreads, 0, s>>>(a, octets_per_row, shift);
        break;
      case 3:
        dq::dequant_octet_kernel<3><<<grid, dq::kDequantThreads, 0, s>>>(a, octets_per_row, shift);
        break;
      case 4:
        dq::dequant_octet_kernel<4><<<grid, dq::kDequantThreads, 0, s>>>(a, octets_per_row, shift);
        break;
      default:
        dq::dequant_octet_kernel<8><<<grid, dq::kDequantThreads, 0, s>>>(a, octets_per_row, shift);
        break;
    }
    DQ_CHECK_LAUNCH("dequant");
    return DQ_OK;
  }
  const int64_t total = static_cast<int64_t>(a.rows) * a.blocks_per_row;
  const int64_t want = dq::ceil_div(total, dq::kDequantThreads);
  const int grid = static_cast<int>(std::min<int64_t>(want, static_cast<int64_t>(dev->sm_count) * 32));
  switch (w->bits) {
    case 2:
      dq::dequant_kernel<2><<<grid, dq::kDequantThreads, 0, s>>>(a);
      break;
    case 3:
      dq::dequant_kernel<3><<<grid, dq::kDequantThreads, 0, s>>>(a);
      break;
    case 4:
      dq::dequant_kernel<4><<<grid, dq::kDequantThreads, 0, s>>>(a);
      break;
    default:
      dq::dequant_kernel<8><<<grid, dq::kDequantThreads, 0, s>>>(a);
      break;
  }
  DQ_CHECK_LAUNCH("dequant");
  return DQ_OK;
}
