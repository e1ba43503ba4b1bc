// Packed decode GEMV for sm_100a:  out[m, n] = sum_k x[m, k] * (q[n, k] * s[n, g] + o[n, g]).
//
// Replaces the reference's gemv_vec_kernel / gemv_kernel / gemv_cuda
// (packages/dynquant-kernels/csrc/gemv/gemv.cu:275-432, :444-555, :695-756).
// Same contract -- fp32 accumulation, a fixed summation order so a result is
// bit-identical run to run, one rounding at the store -- but a different
// machine in mind:
//
//  * The activation is staged ONCE per CTA into shared memory as fp32 (so the
//    inner loop never converts an activation), in a layout padded by 16 bytes
//    per lane-chunk so that 32 lanes reading 32 different chunks hit 32
//    different bank groups.  Per-chunk activation sums are precomputed there
//    too, which is what lets the affine map be applied once per chunk:
//        sum_i (q_i*s + o) x_i  =  s * sum_i q_i x_i  +  o * sum_i x_i.
//  * Weights stream through 128-bit no-allocate loads, software-pipelined one
//    iteration ahead across row tiles, so every lane always has its next
//    16..48 bytes in flight while it decodes the current ones.  The first
//    prefetch is issued BEFORE griddepcontrol.wait: under programmatic
//    dependent launch the weight stream of layer i+1 starts while layer i is
//    still draining, and only the activation staging waits for layer i.
//  * Codes are decoded without conversion instructions and multiplied with
//    packed fp32 FMAs (dq_decode.cuh).
//  * CTAs are persistent: the grid is capped at what the device can hold and
//    warps stride over row tiles, so the staging cost is paid once per CTA.
//
// A second kernel covers every geometry the format allows and the fast path
// refuses (pad tails, per-row tensors, groups smaller than a chunk, unaligned
// views), like the reference's general kernel.
#include <algorithm>
#include <cstdlib>

#include "dq_decode.cuh"
#include "dq_gemv.cuh"
#include "dq_peer_push.cuh"

namespace dq {
namespace {

constexpr int kWarpsPerCta = 8;
constexpr int kThreads = kWarpsPerCta * kWarp;

template <int BITS, int CW>
struct ChunkCfg {
  static constexpr int kWords = CW;
  static constexpr int kValues = CW * 32 / BITS;
  static constexpr int kBlocks = CW / Block<BITS>::kWords;
  static constexpr int kPad = 4;  // floats of padding per chunk in shared memory
  static constexpr int kStride = kValues + kPad;
};

// CW words of one row's chunk into registers.
template <int CW>
__device__ __forceinline__ void load_chunk(const uint32_t* __restrict__ src, uint32_t* w) {
  if constexpr (CW % 4 == 0) {
#pragma unroll
    for (int i = 0; i < CW / 4; ++i) {
      const uint4 v = ldg_stream_128(src + 4 * i);
      w[4 * i + 0] = v.x;
      w[4 * i + 1] = v.y;
      w[4 * i + 2] = v.z;
      w[4 * i + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < CW; ++i) {
      w[i] = ldg_stream_32(src + i);
    }
  }
}

// ---------------------------------------------------------------------------
// Fast path
// ---------------------------------------------------------------------------
//
// MT activation rows are kept in shared memory (rows >= a.m are zero), a warp
// owns R consecutive output rows per tile and its lanes stride over the row's
// chunks.
template <int BITS, int CW, int MT, int R>
__global__ void __launch_bounds__(kThreads) gemv_fast_kernel(const GemvArgs a) {
  using Cfg = ChunkCfg<BITS, CW>;
  constexpr int V = Cfg::kValues;
  constexpr int VB = Block<BITS>::kValues;
  constexpr int WB = Block<BITS>::kWords;

  extern __shared__ __align__(16) float smem[];
  const int C = a.chunks_per_row;
  const int xs_stride = C * Cfg::kStride;  // floats per activation row
  float* xs = smem;
  float* xsum = smem + MT * xs_stride;

  const int lane = threadIdx.x & (kWarp - 1);
  const int warp = threadIdx.x >> 5;
  const int total_warps = gridDim.x * kWarpsPerCta;
  const int first_tile = blockIdx.x * kWarpsPerCta + warp;
  const int num_tiles = (a.rows + R - 1) / R;
  const int iters_per_tile = (C + kWarp - 1) / kWarp;

  pdl_launch_dependents();

  // ---- software pipeline state: one (tile, chunk) step ahead ----
  uint32_t wnext[R][CW];
  int tile = first_tile;
  int ci = 0;  // iteration within the tile
  auto issue_loads = [&](int t, int i) {
    const int c = i * kWarp + lane;
    if (t < num_tiles && c < C) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int row = min(t * R + r, a.rows - 1);
        load_chunk<CW>(a.packed + static_cast<int64_t>(row) * a.words_per_row + c * CW, wnext[r]);
      }
    }
  };
  issue_loads(tile, ci);

  // ---- stage the activation (this is what depends on the previous kernel) ----
  pdl_wait_prior_grid();
  for (int i = threadIdx.x; i < MT * a.in_features; i += kThreads) {
    const int m = i / a.in_features;
    const int k = i - m * a.in_features;
    const float v = m < a.m ? load_f32(a.x, static_cast<int64_t>(m) * a.in_features + k, a.x_dtype) : 0.0f;
    xs[m * xs_stride + k + Cfg::kPad * (k / V)] = v;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < MT * C; i += kThreads) {
    const int m = i / C;
    const int c = i - m * C;
    const float* p = xs + m * xs_stride + c * Cfg::kStride;
    float s = 0.0f;
#pragma unroll 8
    for (int j = 0; j < V; ++j) {
      s += p[j];
    }
    xsum[i] = s;
  }
  __syncthreads();

  float acc[R][MT];
#pragma unroll
  for (int r = 0; r < R; ++r) {
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      acc[r][m] = 0.0f;
    }
  }

  while (tile < num_tiles) {
    // Take ownership of the prefetched words, then put the next step in flight.
    uint32_t w[R][CW];
#pragma unroll
    for (int r = 0; r < R; ++r) {
#pragma unroll
      for (int i = 0; i < CW; ++i) {
        w[r][i] = wnext[r][i];
      }
    }
    const int cur_tile = tile;
    const int c = ci * kWarp + lane;
    const bool last_iter = (ci + 1 == iters_per_tile);
    if (last_iter) {
      tile += total_warps;
      ci = 0;
    } else {
      ++ci;
    }
    issue_loads(tile, ci);

    if (c < C) {
      const int g = c / a.chunks_per_group;
      float scale[R], offset[R];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int row = min(cur_tile * R + r, a.rows - 1);
        const int64_t meta = static_cast<int64_t>(row) * a.num_groups + g;
        scale[r] = load_f32(a.scales, meta, a.meta_dtype);
        offset[r] = a.offsets != nullptr ? load_f32(a.offsets, meta, a.meta_dtype) : 0.0f;
      }

      float2 qacc[R][MT];
#pragma unroll
      for (int r = 0; r < R; ++r) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          qacc[r][m] = make_float2(0.0f, 0.0f);
        }
      }

      const float* xc = xs + c * Cfg::kStride;
#pragma unroll
      for (int b = 0; b < Cfg::kBlocks; ++b) {
        if constexpr (MT == 1) {
          // Activations of this block in registers, shared by the R rows.
          float2 xv[VB / 2];
#pragma unroll
          for (int j = 0; j < VB / 4; ++j) {
            const float4 t = *reinterpret_cast<const float4*>(xc + b * VB + 4 * j);
            xv[2 * j] = make_float2(t.x, t.y);
            xv[2 * j + 1] = make_float2(t.z, t.w);
          }
#pragma unroll
          for (int r = 0; r < R; ++r) {
            for_each_pair<BITS>(&w[r][b * WB], [&](int p, float2 q2) {
              qacc[r][0] = __ffma2_rn(q2, xv[p], qacc[r][0]);
            });
          }
        } else {
#pragma unroll
          for (int r = 0; r < R; ++r) {
            for_each_pair<BITS>(&w[r][b * WB], [&](int p, float2 q2) {
#pragma unroll
              for (int m = 0; m < MT; ++m) {
                const float2 x2 =
                    *reinterpret_cast<const float2*>(xc + m * xs_stride + b * VB + 2 * p);
                qacc[r][m] = __ffma2_rn(q2, x2, qacc[r][m]);
              }
            });
          }
        }
      }

#pragma unroll
      for (int r = 0; r < R; ++r) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const float dot = qacc[r][m].x + qacc[r][m].y;
          acc[r][m] = fmaf(scale[r], dot, fmaf(offset[r], xsum[m * C + c], acc[r][m]));
        }
      }
    }

    if (last_iter) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          float v = acc[r][m];
#pragma unroll
          for (int d = kWarp / 2; d > 0; d >>= 1) {
            v += __shfl_xor_sync(0xffffffffu, v, d);
          }
          acc[r][m] = 0.0f;
          const int row = cur_tile * R + r;
          if (lane == 0 && row < a.rows && m < a.m) {
            store_out(a, m, row, v);
          }
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// General path: any legal geometry.  One warp per output row; a lane takes one
// block (the smallest run of whole words) at a time, word by word, with the
// pad tail (v >= in_features) skipped as in the reference (gemv.cu:513).
// ---------------------------------------------------------------------------
template <int BITS, int MT>
__global__ void __launch_bounds__(kThreads) gemv_general_kernel(const GemvArgs a) {
  constexpr int VB = Block<BITS>::kValues;
  const int lane = threadIdx.x & (kWarp - 1);
  const int warp = threadIdx.x >> 5;
  const int total_warps = gridDim.x * kWarpsPerCta;
  const int blocks_per_group = (a.group_values + VB - 1) / VB;
  const int blocks_per_row = blocks_per_group * a.num_groups;
  const uint32_t* packed = a.packed;

  pdl_launch_dependents();
  pdl_wait_prior_grid();

  for (int row = blockIdx.x * kWarpsPerCta + warp; row < a.rows; row += total_warps) {
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      acc[m] = 0.0f;
    }
    const uint32_t* row_words = packed + static_cast<int64_t>(row) * a.words_per_row;
    for (int blk = lane; blk < blocks_per_row; blk += kWarp) {
      const int g = blk / blocks_per_group;
      const int bg = blk - g * blocks_per_group;
      const int word_base = g * a.words_per_group + (bg * VB * BITS) / 32;
      const int words_left = a.words_per_row - word_base;
      const int value_base = g * a.group_values + bg * VB;
      const int in_group = min(VB, a.group_values - bg * VB);
      const int64_t meta = static_cast<int64_t>(row) * a.num_groups + g;
      const float scale = load_f32(a.scales, meta, a.meta_dtype);
      const float offset = a.offsets != nullptr ? load_f32(a.offsets, meta, a.meta_dtype) : 0.0f;
      for (int j = 0; j < in_group; ++j) {
        const int v = value_base + j;
        if (v >= a.in_features) {
          break;
        }
        const float q = static_cast<float>(code_at<BITS>(row_words + word_base, j, words_left));
        const float wv = fmaf(q, scale, offset);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          if (m < a.m) {
            acc[m] = fmaf(wv, load_f32(a.x, static_cast<int64_t>(m) * a.in_features + v, a.x_dtype),
                          acc[m]);
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      float v = acc[m];
#pragma unroll
      for (int d = kWarp / 2; d > 0; d >>= 1) {
        v += __shfl_xor_sync(0xffffffffu, v, d);
      }
      if (lane == 0 && m < a.m) {
        store_out(a, m, row, v);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Host dispatch
// ---------------------------------------------------------------------------

bool force_general() {
  // Same switch the reference reads (DYNQUANT_GEMV_SCALAR, gemv.cu:604-610): an
  // A/B control that sends every call down the general kernel.  Read once.
  static const bool forced = [] {
    const char* v = std::getenv("DYNQUANT_GEMV_SCALAR");
    return v != nullptr && v[0] != '\0' && v[0] != '0';
  }();
  return forced;
}

bool use_pdl() {
  static const bool on = [] {
    const char* v = std::getenv("DQ_B200_NO_PDL");
    return !(v != nullptr && v[0] != '\0' && v[0] != '0');
  }();
  return on;
}

// Chunk width (words) of the fast path for this tensor, or 0 if it must take
// the general kernel.  Host-side twin of the reference's vec_geometry_ok
// (gemv.cu:566-598).
int fast_chunk_words(const dq_weight& w, const dq_geometry& g, const void* x, int x_dtype) {
  if (force_general()) return 0;
  if (static_cast<int64_t>(g.num_groups) * g.group_values != g.in_features) return 0;  // pad tail
  (void)x;
  (void)x_dtype;
  const auto addr = reinterpret_cast<uintptr_t>(w.packed);
  if (w.bits == 3) {
    if (g.words_per_group % 12 == 0 && addr % 16 == 0 && g.words_per_row % 4 == 0) return 12;
    if (g.words_per_group % 3 == 0 && addr % 4 == 0) return 3;
    return 0;
  }
  if (g.words_per_group % 4 != 0 || addr % 16 != 0) return 0;
  return 4;
}

template <typename Kernel>
int32_t launch(Kernel kernel, const GemvArgs& args, int grid, size_t smem, cudaStream_t stream,
               const char* what /* kernel name, for dq_last_kernel */) {
  if (smem > 48 * 1024) {
    DQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem)));
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = use_pdl() ? 1 : 0;
  DQ_CUDA(cudaLaunchKernelEx(&cfg, kernel, args));
  DQ_CHECK_LAUNCH("gemv");
  note_kernel(what);
  return DQ_OK;
}

template <int BITS>
int32_t launch_general(const GemvArgs& args, cudaStream_t stream);

template <int BITS, int CW, int MT, int R>
int32_t launch_fast(const GemvArgs& args, cudaStream_t stream) {
  using Cfg = ChunkCfg<BITS, CW>;
  const DeviceInfo* dev = device_info();
  if (dev == nullptr) return DQ_ERR_CUDA;
  const size_t smem =
      sizeof(float) * static_cast<size_t>(MT) * (static_cast<size_t>(args.chunks_per_row) * Cfg::kStride + args.chunks_per_row);
  if (smem > static_cast<size_t>(dev->max_smem_optin)) {
    return launch_general<BITS>(args, stream);  // M x K too large to stage: slower, still correct
  }
  auto kernel = gemv_fast_kernel<BITS, CW, MT, R>;
  const int tiles = static_cast<int>(ceil_div(args.rows, R));
  const int ctas = static_cast<int>(ceil_div(tiles, kWarpsPerCta));
  // Persistent cap: what fits on the device at once (register / smem limited).
  const size_t per_sm_smem = 220 * 1024;
  int per_sm = static_cast<int>(std::min<size_t>(2048 / kThreads, smem ? per_sm_smem / (smem + 1024) : 8));
  per_sm = std::max(per_sm, 1);
  const int grid = std::min(ctas, dev->sm_count * per_sm);
  return launch(kernel, args, grid, smem, stream, "gemv_fast_kernel");
}

template <int BITS, int CW>
int32_t launch_fast_m(const GemvArgs& args, int rows_per_warp, cudaStream_t stream) {
  const int m = args.m;
  if (m == 1) {
    if (CW <= 4 && rows_per_warp >= 4) return launch_fast<BITS, CW, 1, 4>(args, stream);
    if (rows_per_warp >= 2) return launch_fast<BITS, CW, 1, 2>(args, stream);
    return launch_fast<BITS, CW, 1, 1>(args, stream);
  }
  if (m == 2) {
    if (rows_per_warp >= 2) return launch_fast<BITS, CW, 2, 2>(args, stream);
    return launch_fast<BITS, CW, 2, 1>(args, stream);
  }
  if (m <= 4) {
    if (CW <= 4 && rows_per_warp >= 2) return launch_fast<BITS, CW, 4, 2>(args, stream);
    return launch_fast<BITS, CW, 4, 1>(args, stream);
  }
  return launch_fast<BITS, CW, 8, 1>(args, stream);
}

template <int BITS>
int32_t launch_general(const GemvArgs& args, cudaStream_t stream) {
  const DeviceInfo* dev = device_info();
  if (dev == nullptr) return DQ_ERR_CUDA;
  const int ctas = static_cast<int>(ceil_div(args.rows, kWarpsPerCta));
  const int grid = std::min(ctas, dev->sm_count * 8);
  const int m = args.m;
  if (m == 1) return launch(gemv_general_kernel<BITS, 1>, args, grid, 0, stream, "gemv_general_kernel");
  if (m == 2) return launch(gemv_general_kernel<BITS, 2>, args, grid, 0, stream, "gemv_general_kernel");
  if (m <= 4) return launch(gemv_general_kernel<BITS, 4>, args, grid, 0, stream, "gemv_general_kernel");
  return launch(gemv_general_kernel<BITS, 8>, args, grid, 0, stream, "gemv_general_kernel");
}

// Rows per warp: as many as still leave every resident warp a tile.
int pick_rows_per_warp(int rows, const DeviceInfo& dev) {
  const int64_t resident_warps = static_cast<int64_t>(dev.sm_count) * (2048 / kWarp) / 2;
  if (rows >= 4 * resident_warps) return 4;
  if (rows >= 2 * resident_warps) return 2;
  return 1;
}

GemvArgs make_args(const void* x, int32_t x_dtype, int64_t m, const dq_weight& w, const dq_geometry& g,
                   const void* bias, void* out, int64_t out_stride, int64_t out_col0, int32_t out_dtype) {
  GemvArgs a = {};
  a.x = x;
  a.packed = static_cast<const uint32_t*>(w.packed);
  a.scales = w.scales;
  a.offsets = w.offsets;
  a.bias = bias;
  a.out = out;
  a.out_stride = out_stride;
  a.out_col0 = out_col0;
  a.x_dtype = x_dtype;
  a.meta_dtype = w.meta_dtype;
  a.out_dtype = out_dtype;
  a.m = static_cast<int>(m);
  a.rows = static_cast<int>(w.rows);
  a.words_per_row = g.words_per_row;
  a.num_groups = g.num_groups;
  a.words_per_group = g.words_per_group;
  a.group_values = g.group_values;
  a.in_features = g.in_features;
  return a;
}

// The first `count` activation rows from row `first` on: same weight, shifted x and out.
GemvArgs activation_rows(const GemvArgs& a, int first, int count) {
  GemvArgs b = a;
  b.x = static_cast<const char*>(a.x) + static_cast<int64_t>(first) * a.in_features * dtype_size(a.x_dtype);
  b.out = static_cast<char*>(a.out) + static_cast<int64_t>(first) * a.out_stride * dtype_size(a.out_dtype);
  b.m = count;
  return b;
}

// Row chunks over one matrix share a launch only where the tiled kernel is the right kernel for
// the matrix anyway; a matrix long enough for the streaming kernel goes chunk by chunk.
bool fusable_rows(const GemvArgs& a) {
  const DeviceInfo* dev = device_info();
  return dev != nullptr && ceil_div(a.rows, 16) < static_cast<int64_t>(dev->sm_count) * 8;
}

int32_t gemv_args(GemvArgs a, const dq_weight& w, const dq_geometry& g, cudaStream_t stream) {
  if (!force_general()) {
    const int rows_switch = tuning_int("DQ_B200_ROWS_SMALL_M", -1);  // 0: the many-rows kernel never below nine rows
    if (mma_path_supports(a, w.bits)) {
      const int32_t rc = launch_gemv_mma(a, w.bits, stream);
      if (rc != DQ_ERR_UNSUPPORTED) return rc;  // (unsupported: silently on to the SIMT kernels)
    }
    // The staged activation of all rows may be what does not fit (eight rows x a long reduction
    // axis).  The many-rows kernel passes the activation through shared memory block by block and
    // reads the weights once (5120 x 17408 at 8 bits, eight rows: 47 us against 179 in passes) ...
    if (a.m > 1 && rows_switch != 0 && mma_enabled_for_rows() && mma_path_supports(activation_rows(a, 0, 1), w.bits)) {
      bool taken = false;
      if (const int32_t rc = launch_gemv_rows(a, w.bits, stream, &taken, 1)) return rc;
      if (taken) return DQ_OK;
    }
    // ... else passes over half the rows each (halved again if need be) re-read the weights,
    // mostly from L2, but stay on the tensor-core path.
    if (a.m > 1 && mma_path_supports(activation_rows(a, 0, 1), w.bits)) {
      const int half = (a.m + 1) / 2;
      if (const int32_t rc = gemv_args(activation_rows(a, 0, half), w, g, stream)) return rc;
      return gemv_args(activation_rows(a, half, a.m - half), w, g, stream);
    }
  }
  const int cw = fast_chunk_words(w, g, a.x, a.x_dtype);
  if (cw == 0) {
    switch (w.bits) {
      case 2:
        return launch_general<2>(a, stream);
      case 3:
        return launch_general<3>(a, stream);
      case 4:
        return launch_general<4>(a, stream);
      default:
        return launch_general<8>(a, stream);
    }
  }
  a.chunks_per_group = g.words_per_group / cw;
  a.chunks_per_row = g.words_per_row / cw;
  const DeviceInfo* dev = device_info();
  if (dev == nullptr) return DQ_ERR_CUDA;
  const int rpw = pick_rows_per_warp(a.rows, *dev);
  switch (w.bits) {
    case 2:
      return launch_fast_m<2, 4>(a, rpw, stream);
    case 3:
      return cw == 12 ? launch_fast_m<3, 12>(a, rpw, stream) : launch_fast_m<3, 3>(a, rpw, stream);
    case 4:
      return launch_fast_m<4, 4>(a, rpw, stream);
    default:
      return launch_fast_m<8, 4>(a, rpw, stream);
  }
}

int32_t gemv_one(const void* x, int32_t x_dtype, int64_t m, const dq_weight& w, const dq_geometry& g,
                 const void* bias, void* out, int64_t out_stride, int64_t out_col0,
                 int32_t out_dtype, cudaStream_t stream) {
  return gemv_args(make_args(x, x_dtype, m, w, g, bias, out, out_stride, out_col0, out_dtype), w, g, stream);
}

int32_t check_activation(const void* x, int32_t x_dtype, int64_t m, void* out, int32_t out_dtype) {
  DQ_REQUIRE(dtype_ok(x_dtype), "gemv: unsupported activation dtype tag %d", x_dtype);
  DQ_REQUIRE(dtype_ok(out_dtype), "gemv: unsupported output dtype tag %d", out_dtype);
  DQ_REQUIRE(m >= 0, "gemv: x must be 2-D [rows, in_features], got %lld rows", static_cast<long long>(m));
  DQ_REQUIRE(m <= DQ_GEMV_MAX_ROWS,
             "gemv: %lld activation rows exceeds the kernel's limit of %d. Above this a quantized "
             "matmul is compute-bound and the dequant + dense GEMM path is faster; dispatch there "
             "instead.",
             static_cast<long long>(m), DQ_GEMV_MAX_ROWS);
  DQ_REQUIRE(m == 0 || (x != nullptr && out != nullptr), "gemv: null activation or output pointer");
  return DQ_OK;
}

}  // namespace
}  // namespace dq

extern "C" {

int32_t dq_gemv(const void* x, int32_t x_dtype, int64_t m, const dq_weight* w, void* out,
                int32_t out_dtype, void* stream) {
  dq_geometry g;
  if (const int32_t rc = dq_resolve_geometry("gemv", w, &g)) return rc;
  if (const int32_t rc = dq::check_activation(x, x_dtype, m, out, out_dtype)) return rc;
  if (m == 0 || w->rows == 0) return DQ_OK;
  return dq::gemv_one(x, x_dtype, m, *w, g, nullptr, out, w->rows, 0, out_dtype,
                      static_cast<cudaStream_t>(stream));
}

int32_t dq_gemv_shards(const void* x, int32_t x_dtype, int64_t m, const dq_weight* shards,
                       int32_t num_shards, const void* bias, void* out, int64_t out_stride,
                       int32_t out_dtype, void* stream) {
  DQ_REQUIRE(shards != nullptr && num_shards > 0, "gemv_shards: need at least one shard");
  int64_t total = 0;
  for (int i = 0; i < num_shards; ++i) {
    dq_geometry g;
    if (const int32_t rc = dq_resolve_geometry("gemv_shards", &shards[i], &g)) return rc;
    DQ_REQUIRE(shards[i].in_features == shards[0].in_features,
               "gemv_shards: shard %d has in_features=%lld but shard 0 has %lld", i,
               static_cast<long long>(shards[i].in_features),
               static_cast<long long>(shards[0].in_features));
    total += shards[i].rows;
  }
  DQ_REQUIRE(out_stride >= total, "gemv_shards: out_stride=%lld is smaller than the %lld rows of the shards",
             static_cast<long long>(out_stride), static_cast<long long>(total));
  if (const int32_t rc = dq::check_activation(x, x_dtype, m, out, out_dtype)) return rc;
  if (m == 0) return DQ_OK;
  // Shards share the activation: up to four at a time go out as ONE launch when the tiled
  // tensor-core kernel takes them, one launch each otherwise.
  constexpr int kBatch = 4;
  int64_t col0 = 0;
  for (int first = 0; first < num_shards; first += kBatch) {
    const int count = std::min(kBatch, num_shards - first);
    dq::GemvArgs args[kBatch];
    dq_geometry geo[kBatch];
    int bits[kBatch];
    int64_t cols[kBatch];
    int live = 0;
    for (int i = first; i < first + count; ++i) {
      if (shards[i].rows > 0) {
        dq_resolve_geometry("gemv_shards", &shards[i], &geo[live]);
        args[live] = dq::make_args(x, x_dtype, m, shards[i], geo[live], bias, out, out_stride, col0, out_dtype);
        bits[live] = shards[i].bits;
        cols[live] = i;
        ++live;
      }
      col0 += shards[i].rows;
    }
    bool taken = false;
    if (live > 1 && !dq::force_general()) {
      const int32_t rc = dq::launch_gemv_mma_fused(args, bits, live, static_cast<cudaStream_t>(stream), &taken);
      if (rc) return rc;
    }
    if (!taken) {
      for (int k = 0; k < live; ++k) {
        const int32_t rc = dq::gemv_args(args[k], shards[cols[k]], geo[k], static_cast<cudaStream_t>(stream));
        if (rc) return rc;
      }
    }
  }
  return DQ_OK;
}

int32_t dq_gemv_shards_rows(const void* x, int32_t x_dtype, int64_t m, const dq_weight* shards, int32_t num_shards,
                            const void* bias, void* out, int64_t out_stride, int32_t out_dtype, void* stream) {
  constexpr int64_t kMaxRows = DQ_GEMV_CHUNKED_MAX_ROWS;
  DQ_REQUIRE(shards != nullptr && num_shards > 0, "gemv_shards_rows: need at least one shard");
  DQ_REQUIRE(m >= 0 && m <= kMaxRows,
             "gemv_shards_rows: %lld activation rows exceeds the limit of %lld; above it a quantized matmul is "
             "compute-bound and the dequant + dense GEMM path is faster",
             static_cast<long long>(m), static_cast<long long>(kMaxRows));
  if (m <= DQ_GEMV_MAX_ROWS) {
    return dq_gemv_shards(x, x_dtype, m, shards, num_shards, bias, out, out_stride, out_dtype, stream);
  }
  DQ_REQUIRE(dq::dtype_ok(x_dtype) && dq::dtype_ok(out_dtype) && x != nullptr && out != nullptr,
             "gemv_shards_rows: bad dtype tag or null pointer");
  int64_t total = 0;
  for (int i = 0; i < num_shards; ++i) {
    dq_geometry g;
    if (const int32_t rc = dq_resolve_geometry("gemv_shards_rows", &shards[i], &g)) return rc;
    DQ_REQUIRE(shards[i].in_features == shards[0].in_features, "gemv_shards_rows: shard %d has in_features=%lld but shard 0 has %lld",
               i, static_cast<long long>(shards[i].in_features), static_cast<long long>(shards[0].in_features));
    total += shards[i].rows;
  }
  DQ_REQUIRE(out_stride >= total, "gemv_shards_rows: out_stride=%lld is smaller than the %lld rows of the shards",
             static_cast<long long>(out_stride), static_cast<long long>(total));
  // Row chunks of at most eight rows, as equal as possible (the members of one launch must have
  // the same number of rows); chunk after chunk, shard after shard, up to four jobs per launch.
  const int64_t chunks = dq::ceil_div(m, DQ_GEMV_MAX_ROWS);
  const int64_t base = m / chunks, longer = m % chunks;  // the first `longer` chunks take base + 1 rows
  const size_t x_row = static_cast<size_t>(shards[0].in_features) * dq::dtype_size(x_dtype);
  const size_t out_row = static_cast<size_t>(out_stride) * dq::dtype_size(out_dtype);
  auto s = static_cast<cudaStream_t>(stream);
  constexpr int kBatch = 4;
  dq::GemvArgs args[kBatch];
  dq_geometry geo[kBatch];
  int bits[kBatch];
  const dq_weight* which[kBatch];
  int live = 0;
  auto flush = [&]() -> int32_t {
    if (live == 0) return DQ_OK;
    bool taken = false;
    // (matrices long enough for the streaming kernel go out one by one: it is the faster kernel there)
    bool fusable = live > 1 && !dq::force_general();
    for (int k = 0; k < live && fusable; ++k) fusable = dq::fusable_rows(args[k]);
    if (fusable) {
      if (const int32_t rc = dq::launch_gemv_mma_fused(args, bits, live, s, &taken)) return rc;
    }
    if (!taken) {
      for (int k = 0; k < live; ++k) {
        if (const int32_t rc = dq::gemv_args(args[k], *which[k], geo[k], s)) return rc;
      }
    }
    live = 0;
    return DQ_OK;
  };
  // A shard whose geometry the many-rows kernel takes goes through it whole: one pass over its
  // weights for all the rows.  The others run as row chunks.
  constexpr int kMaxShards = 64;
  bool whole[kMaxShards] = {};
  if (!dq::force_general() && dq::mma_enabled_for_rows()) {
    int64_t col0 = 0;
    for (int i = 0; i < num_shards; ++i) {
      if (i < kMaxShards && shards[i].rows > 0) {
        dq_geometry g;
        dq_resolve_geometry("gemv_shards_rows", &shards[i], &g);
        const dq::GemvArgs all = dq::make_args(x, x_dtype, m, shards[i], g, bias, out, out_stride, col0, out_dtype);
        if (const int32_t rc = dq::launch_gemv_rows(all, shards[i].bits, s, &whole[i])) return rc;
      }
      col0 += shards[i].rows;
    }
  }
  int64_t row0 = 0;
  for (int64_t c = 0; c < chunks; ++c) {
    const int64_t rows_here = base + (c < longer ? 1 : 0);
    int64_t col0 = 0;
    for (int i = 0; i < num_shards; ++i) {
      if (shards[i].rows > 0 && !(i < kMaxShards && whole[i])) {
        if (live == kBatch || (live > 0 && args[0].m != rows_here)) {
          if (const int32_t rc = flush()) return rc;
        }
        dq_resolve_geometry("gemv_shards_rows", &shards[i], &geo[live]);
        args[live] = dq::make_args(static_cast<const unsigned char*>(x) + row0 * x_row, x_dtype, rows_here, shards[i], geo[live],
                                   bias, static_cast<unsigned char*>(out) + row0 * out_row, out_stride, col0, out_dtype);
        bits[live] = shards[i].bits;
        which[live] = &shards[i];
        ++live;
      }
      col0 += shards[i].rows;
    }
    row0 += rows_here;
  }
  return flush();
}

int32_t dq_gemv_sequence(const dq_gemv_job* jobs, int32_t num_jobs, void* stream) {
  DQ_REQUIRE(num_jobs >= 0 && (jobs != nullptr || num_jobs == 0), "gemv_sequence: null job list");
  for (int i = 0; i < num_jobs; ++i) {
    const dq_gemv_job& j = jobs[i];
    dq_geometry g;
    if (const int32_t rc = dq_resolve_geometry("gemv_sequence", &j.weight, &g)) return rc;
    if (const int32_t rc = dq::check_activation(j.x, j.x_dtype, j.m, j.out, j.out_dtype)) return rc;
    DQ_REQUIRE(j.out_col0 >= 0 && j.out_stride >= j.out_col0 + j.weight.rows,
               "gemv_sequence: job %d writes columns [%lld, %lld) of a row of %lld", i,
               static_cast<long long>(j.out_col0), static_cast<long long>(j.out_col0 + j.weight.rows),
               static_cast<long long>(j.out_stride));
  }
  // Consecutive jobs that read the SAME activation (q/k/v, gate/up) cannot depend on one
  // another, so up to four of them go out as one launch when the tiled kernel takes them.
  constexpr int kBatch = 4;
  auto s = static_cast<cudaStream_t>(stream);
  int i = 0;
  while (i < num_jobs) {
    const dq_gemv_job& head = jobs[i];
    if (head.m == 0 || head.weight.rows == 0) {
      ++i;
      continue;
    }
    int end = i + 1;
    while (end < num_jobs && end - i < kBatch && jobs[end].x == head.x && jobs[end].m == head.m &&
           jobs[end].x_dtype == head.x_dtype && jobs[end].out_dtype == head.out_dtype &&
           jobs[end].weight.rows > 0 && jobs[end].weight.in_features == head.weight.in_features) {
      ++end;
    }
    dq::GemvArgs args[kBatch];
    dq_geometry geo[kBatch];
    int bits[kBatch];
    for (int k = i; k < end; ++k) {
      const dq_gemv_job& j = jobs[k];
      dq_resolve_geometry("gemv_sequence", &j.weight, &geo[k - i]);
      args[k - i] = dq::make_args(j.x, j.x_dtype, j.m, j.weight, geo[k - i], j.bias, j.out, j.out_stride,
                                  j.out_col0, j.out_dtype);
      bits[k - i] = j.weight.bits;
    }
    bool taken = false;
    if (end - i > 1 && !dq::force_general()) {
      if (const int32_t rc = dq::launch_gemv_mma_fused(args, bits, end - i, s, &taken)) return rc;
    }
    if (!taken) {
      for (int k = i; k < end; ++k) {
        if (const int32_t rc = dq::gemv_args(args[k - i], jobs[k].weight, geo[k - i], s)) return rc;
      }
    }
    i = end;
  }
  return DQ_OK;
}

int32_t dq_gemv_stage_push(const dq_gemv_job* jobs, int32_t num_jobs, const dq_peer_push* push, void* stream) {
  using dq::peerpush::Push;
  constexpr int kBatch = 4;
  DQ_REQUIRE(jobs != nullptr && num_jobs >= 1 && num_jobs <= kBatch, "gemv_stage_push: 1..%d jobs, got %d", kBatch, num_jobs);
  DQ_REQUIRE(push != nullptr && push->windows != nullptr, "gemv_stage_push: null push descriptor");
  DQ_REQUIRE(push->world >= 1 && push->world <= dq::peerpush::kMaxWorld && push->rank >= 0 && push->rank < push->world,
             "gemv_stage_push: rank %d of %d (at most %d ranks)", push->rank, push->world, dq::peerpush::kMaxWorld);
  const dq_gemv_job& head = jobs[0];
  dq::GemvArgs args[kBatch];
  dq_geometry geo[kBatch];
  int bits[kBatch];
  for (int i = 0; i < num_jobs; ++i) {
    const dq_gemv_job& j = jobs[i];
    if (const int32_t rc = dq_resolve_geometry("gemv_stage_push", &j.weight, &geo[i])) return rc;
    if (const int32_t rc = dq::check_activation(j.x, j.x_dtype, j.m, j.out, j.out_dtype)) return rc;
    DQ_REQUIRE(j.m >= 1 && j.weight.rows >= 1, "gemv_stage_push: job %d is empty", i);
    DQ_REQUIRE(j.out_col0 >= 0 && j.out_stride >= j.out_col0 + j.weight.rows,
               "gemv_stage_push: job %d writes columns [%lld, %lld) of a row of %lld", i,
               static_cast<long long>(j.out_col0), static_cast<long long>(j.out_col0 + j.weight.rows),
               static_cast<long long>(j.out_stride));
    DQ_REQUIRE(j.x == head.x && j.m == head.m && j.x_dtype == head.x_dtype && j.out_dtype == head.out_dtype &&
                   j.out == head.out && j.out_stride == head.out_stride,
               "gemv_stage_push: job %d does not share the activation and the output buffer of job 0", i);
    args[i] = dq::make_args(j.x, j.x_dtype, j.m, j.weight, geo[i], j.bias, j.out, j.out_stride, j.out_col0, j.out_dtype);
    bits[i] = j.weight.bits;
  }
  const int64_t need = head.m * head.out_stride * static_cast<int64_t>(dq::dtype_size(head.out_dtype));
  DQ_REQUIRE(push->piece_bytes >= need && push->piece_bytes % 16 == 0 && push->data_offset % 16 == 0 &&
                 reinterpret_cast<uintptr_t>(head.out) % 16 == 0,
             "gemv_stage_push: the piece is %lld bytes (a multiple of 16, 16-byte aligned), the output buffer needs %lld",
             static_cast<long long>(push->piece_bytes), static_cast<long long>(need));
  DQ_REQUIRE(push->flags_offset % 4 == 0 && push->state_offset % 8 == 0 && push->status_offset % 4 == 0 &&
                 push->flags_offset >= 0 && push->state_offset >= 0 && push->status_offset >= 0 && push->data_offset >= 0 &&
                 push->flags_offset < (1LL << 31) && push->state_offset < (1LL << 31) && push->status_offset < (1LL << 31),
             "gemv_stage_push: misaligned or out-of-range flag / state / status offsets");
  Push P = {};
  for (int r = 0; r < push->world; ++r) {
    DQ_REQUIRE(push->windows[r] != nullptr && reinterpret_cast<uintptr_t>(push->windows[r]) % 16 == 0,
               "gemv_stage_push: window %d is null or not 16-byte aligned", r);
    P.window[r] = static_cast<unsigned char*>(push->windows[r]);
  }
  P.data_off = push->data_offset;
  P.piece_bytes = push->piece_bytes;
  P.flags_off = static_cast<int>(push->flags_offset);
  P.state_off = static_cast<int>(push->state_offset);
  P.status_off = static_cast<int>(push->status_offset);
  P.world = push->world;
  P.rank = push->rank;
  P.spin_limit = push->spin_limit > 0 ? push->spin_limit : (1 << 21);
  P.enabled = 1;
  auto s = static_cast<cudaStream_t>(stream);
  if (dq::force_general()) return dq::fail(DQ_ERR_UNSUPPORTED, "gemv_stage_push: the general SIMT kernel is forced; it does not push");
  int32_t rc = DQ_OK;
  bool taken = false;
  if (num_jobs == 1) {
    rc = dq::mma_path_supports(args[0], bits[0]) ? dq::launch_gemv_mma(args[0], bits[0], s, &P) : DQ_ERR_UNSUPPORTED;
    taken = rc == DQ_OK;
  } else {
    rc = dq::launch_gemv_mma_fused(args, bits, num_jobs, s, &taken, &P);
  }
  if (rc != DQ_OK && rc != DQ_ERR_UNSUPPORTED) return rc;
  if (!taken) {
    return dq::fail(DQ_ERR_UNSUPPORTED,
                    "gemv_stage_push: these jobs do not leave as one launch of the tiled or the streaming kernel");
  }
  return DQ_OK;
}

int32_t dq_peer_push_status(const dq_peer_push* push, void* stream) {
  DQ_REQUIRE(push != nullptr && push->windows != nullptr && push->rank >= 0 && push->rank < push->world,
             "peer_push_status: null or inconsistent descriptor");
  auto s = static_cast<cudaStream_t>(stream);
  unsigned int word = 0;
  DQ_CUDA(cudaMemcpyAsync(&word, static_cast<const unsigned char*>(push->windows[push->rank]) + push->status_offset,
                          sizeof(word), cudaMemcpyDeviceToHost, s));
  DQ_CUDA(cudaStreamSynchronize(s));
  if (word != 0u) {
    return dq::fail(DQ_ERR_DEVICE, "stage push: rank %d gave up waiting for the rows of rank %u", push->rank, word >> 8);
  }
  return DQ_OK;
}

int32_t dq_gemv_host(const void* x_host, int32_t x_dtype, int64_t m, const dq_weight* w,
                     void* out_host, int32_t out_dtype, void* x_dev, void* out_dev, void* stream) {
  dq_geometry g;
  if (const int32_t rc = dq_resolve_geometry("gemv", w, &g)) return rc;
  if (const int32_t rc = dq::check_activation(x_host, x_dtype, m, out_host, out_dtype)) return rc;
  if (m == 0 || w->rows == 0) return DQ_OK;
  DQ_REQUIRE(x_dev != nullptr && out_dev != nullptr, "gemv_host: device staging buffers are required");
  auto s = static_cast<cudaStream_t>(stream);
  const size_t x_bytes = static_cast<size_t>(m) * g.in_features * dq::dtype_size(x_dtype);
  const size_t out_bytes = static_cast<size_t>(m) * w->rows * dq::dtype_size(out_dtype);
  DQ_CUDA(cudaMemcpyAsync(x_dev, x_host, x_bytes, cudaMemcpyHostToDevice, s));
  if (const int32_t rc = dq::gemv_one(x_dev, x_dtype, m, *w, g, nullptr, out_dev, w->rows, 0, out_dtype, s)) {
    return rc;
  }
  DQ_CUDA(cudaMemcpyAsync(out_host, out_dev, out_bytes, cudaMemcpyDeviceToHost, s));
  DQ_CUDA(cudaStreamSynchronize(s));
  return DQ_OK;
}

}  // extern "C"
