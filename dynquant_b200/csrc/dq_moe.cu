// MoE grouped GEMV: y[t] = sum_k p[t,k] * W_down[e] ( silu(W_gate[e] x[t]) * (W_up[e] x[t]) ),  e = ids[t,k].
//
// The reference has no such kernel: its serving plugins refuse fused-MoE layers
// (integration/vllm_plugin/config.py:107-112) and pack_model refuses expert banks
// (runtime/linear.py:442-456).  What it does define is the weight format of a bank --
// a stacked tensor [E, out, in] folds to rows, expert e owning rows [e*out, (e+1)*out)
// (quant/tensor.py:253-255; shapes from graph/experts.py:35-43: gate_up [E, 2I, H] with
// the gate rows first, down [E, H, I]) -- and this file computes on exactly that.
//
// Four launches, all on the caller's stream, no host round trip:
//   1. route    one CTA: per-expert token counts, offsets, and the (token, slot)
//               assignments sorted by expert (stable: ascending assignment id).
//   2. gate_up  grid (row-tile pairs, experts).  An expert's packed rows are streamed ONCE
//               per step for up to 8 of its tokens at a time -- the tokens are the 8
//               columns of the m16n8k16 accumulator, exactly like the activation rows of
//               the dense GEMV (dq_gemv_mma.cu), gathered by index while staging.  A warp
//               computes 16 gate rows and the matching 16 up rows and writes
//               h = silu(g) * u, rounded to the activation dtype, to scratch.
//   3. down     same machinery over the down bank with h as the activation; the fp32
//               result of every assignment goes to scratch.
//   4. combine  y[t] = sum_k p[t,k] * d[t,k] in slot order -- a fixed order, so the layer is
//               bit-identical run to run (no atomics anywhere).
// Experts with no token exit at once; ids outside [0, num_experts) are skipped, which is how
// an expert-parallel rank passes "not mine".
#include <algorithm>
#include <cstdlib>

#include "dq_gemv.cuh"
#include "dq_mma_plan.cuh"
#include "dq_mma_stage.cuh"

namespace dq {
namespace {

constexpr int kMoeWarps = 8;
constexpr int kMoeThreads = kMoeWarps * kWarp;
constexpr int kMaxAssign = DQ_MOE_MAX_TOKENS * 16;

struct Routing {
  int* counts;   // [E]
  int* offsets;  // [E + 1]
  int* sorted;   // [A] assignment ids (t * topk + k), grouped by expert
};

__global__ void __launch_bounds__(512) moe_route_kernel(const int32_t* __restrict__ ids, int assignments,
                                                        int num_experts, Routing r) {
  extern __shared__ int sm[];  // [E] counts, [E + 1] offsets
  int* cnt = sm;
  int* off = sm + num_experts;
  pdl_launch_dependents();
  pdl_wait_prior_grid();
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int a = threadIdx.x; a < assignments; a += blockDim.x) {
    const int e = ids[a];
    if (e >= 0 && e < num_experts) atomicAdd(&cnt[e], 1);  // integer count: order-independent
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < num_experts; ++e) {
      off[e] = run;
      run += cnt[e];
    }
    off[num_experts] = run;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    r.counts[e] = cnt[e];
    r.offsets[e] = off[e];
  }
  if (threadIdx.x == 0) r.offsets[num_experts] = off[num_experts];
  // stable placement: rank of a among the assignments of the same expert with a smaller id
  for (int a = threadIdx.x; a < assignments; a += blockDim.x) {
    const int e = ids[a];
    if (e < 0 || e >= num_experts) continue;
    int rank = 0;
    for (int b = 0; b < a; ++b) rank += (ids[b] == e);
    r.sorted[off[e] + rank] = a;
  }
}

struct MoeArgs {
  const void* act;          // gate_up: x [tokens, K]; down: h [assignments, K]
  const uint32_t* packed;   // the bank, [E * rows_per_expert(*2), words_per_row]
  const void* scales;
  const void* offsets;      // may be null
  void* out;                // gate_up: h [assignments, inter] act dtype; down: d [assignments, hidden] fp32
  Routing route;
  int act_dtype, meta_dtype;
  int topk;
  int rows;                 // output rows per expert of this launch (inter, or hidden)
  int words_per_row, num_groups, in_features;
  int steps;                // padded K / 128
  int kw, rw;               // warps: rw row tiles x kw slices of the reduction axis
  int steps_per_warp;
  int m_stride_u4;
  uint32_t magic;
};

template <bool BF16>
__device__ __forceinline__ float meta_to_f32(uint32_t raw) {
  if constexpr (BF16) {
    return __uint_as_float(raw << 16);
  } else {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(raw)));
  }
}

// One 16-row tile over this warp's slice of the reduction axis: acc[4] as in the dense kernel.
template <int BITS, bool XBF16, bool MBF16>
__device__ __forceinline__ void moe_tile(const MoeArgs& a, int64_t row_a, int64_t row_b, int s_begin, int s_end,
                                         const uint4* xb_lane, int xb_step_u4, const float* xsum,
                                         const float* xneg, int t, float* acc) {
  using Plan = MmaPlan<BITS>;
  constexpr int NA = Plan::kARegs;
  constexpr int QU = NA / 4;
  constexpr int STEP_WORDS = 4 * BITS;
  const uint32_t* wa = a.packed + row_a * a.words_per_row + t * BITS;
  const uint32_t* wb = a.packed + row_b * a.words_per_row + t * BITS;
  const unsigned short* sc = reinterpret_cast<const unsigned short*>(a.scales);
  const unsigned short* of = reinterpret_cast<const unsigned short*>(a.offsets);
#pragma unroll 1
  for (int s0 = s_begin; s0 < s_end; s0 += 4) {
    // a block of up to four steps: all loads first, then the math
    uint32_t raw[4][2][BITS];
    uint32_t meta[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (s0 + j < s_end) {
#pragma unroll
        for (int i = 0; i < BITS; ++i) {
          raw[j][0][i] = __ldg(wa + (s0 + j) * STEP_WORDS + i);
          raw[j][1][i] = __ldg(wb + (s0 + j) * STEP_WORDS + i);
        }
        const int64_t ia = row_a * a.num_groups + (s0 + j), ib = row_b * a.num_groups + (s0 + j);
        meta[j][0] = __ldg(sc + ia);
        meta[j][2] = __ldg(sc + ib);
        meta[j][1] = of != nullptr ? __ldg(of + ia) : 0u;
        meta[j][3] = of != nullptr ? __ldg(of + ib) : 0u;
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (s0 + j < s_end) {
        const int s = s0 + j;
        uint32_t aa[NA], ab[NA];
        decode_unit<BITS>(raw[j][0], a.magic, aa);
        decode_unit<BITS>(raw[j][1], a.magic, ab);
        unbias_fragments<XBF16, NA>(aa);
        unbias_fragments<XBF16, NA>(ab);
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
        const float sc_a = meta_to_f32<MBF16>(meta[j][0]), of_a = meta_to_f32<MBF16>(meta[j][1]);
        const float sc_b = meta_to_f32<MBF16>(meta[j][2]), of_b = meta_to_f32<MBF16>(meta[j][3]);
        acc[0] = fmaf(sc_a, d[0] + xn2.x, fmaf(of_a, xs2.x, acc[0]));
        acc[1] = fmaf(sc_a, d[1] + xn2.y, fmaf(of_a, xs2.y, acc[1]));
        acc[2] = fmaf(sc_b, d[2] + xn2.x, fmaf(of_b, xs2.x, acc[2]));
        acc[3] = fmaf(sc_b, d[3] + xn2.y, fmaf(of_b, xs2.y, acc[3]));
      }
    }
  }
}

// GATE_UP: a tile is 16 gate rows plus the matching 16 up rows, output silu(g)*u.
template <int BITS, bool XBF16, bool MBF16, bool GATE_UP>
__global__ void __launch_bounds__(kMoeThreads) moe_grouped_kernel(const MoeArgs a) {
  using Plan = MmaPlan<BITS>;
  constexpr int QU = Plan::kARegs / 4;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint4* xb = reinterpret_cast<uint4*>(smem_raw);
  float* xsum = reinterpret_cast<float*>(xb + 8 * a.m_stride_u4 + QU * 4);
  float* xneg = xsum + a.steps * 8;
  float* red = xneg + a.steps * 8;                       // [halves][kw][rw][16][8]
  int* row_map = reinterpret_cast<int*>(red + (GATE_UP ? 2 : 1) * a.kw * a.rw * 16 * 8);  // [8]

  const int e = blockIdx.y;
  pdl_launch_dependents();
  pdl_wait_prior_grid();  // routing (and for the down pass, h) come from the previous kernels
  const int count = a.route.counts[e];
  if (count == 0) return;
  const int first = a.route.offsets[e];

  const int tid = threadIdx.x;
  const int lane = tid & (kWarp - 1);
  const int warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int rwi = warp / a.kw;
  const int kwi = warp - rwi * a.kw;
  const int tile = blockIdx.x * a.rw + rwi;
  const int tiles = (a.rows + 15) / 16;
  const bool tile_live = tile < tiles;
  const int s_begin = kwi * a.steps_per_warp;
  const int s_end = min(a.steps, s_begin + a.steps_per_warp);
  const int64_t expert_row0 = static_cast<int64_t>(e) * a.rows * (GATE_UP ? 2 : 1);
  const int r_a = min(tile * 16 + g, a.rows - 1), r_b = min(tile * 16 + g + 8, a.rows - 1);

  GemvArgs stage = {};
  stage.x = a.act;
  stage.x_dtype = a.act_dtype;
  stage.in_features = a.in_features;

  for (int c0 = 0; c0 < count; c0 += 8) {  // up to 8 of this expert's tokens per pass
    const int m = min(8, count - c0);
    __syncthreads();  // the previous pass is done with row_map / xb / red
    if (tid < 8) {
      const int aid = a.route.sorted[first + min(c0 + tid, count - 1)];
      row_map[tid] = GATE_UP ? aid / a.topk : aid;  // x is per token, h per assignment
    }
    __syncthreads();
    stage.m = m;
    stage_activation<BITS, XBF16>(stage, a.steps, a.m_stride_u4, xb, xsum, xneg, tid, kMoeThreads, row_map);
    __syncthreads();

    const bool b_live = g < m;
    const uint4* xb_lane = b_live ? xb + g * a.m_stride_u4 + t : xb + m * a.m_stride_u4;
    const int xb_step_u4 = b_live ? QU * 4 : 0;
    float acc[GATE_UP ? 2 : 1][4];
#pragma unroll
    for (int h = 0; h < (GATE_UP ? 2 : 1); ++h) {
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[h][i] = 0.0f;
      if (tile_live) {
        const int64_t base = expert_row0 + static_cast<int64_t>(h) * a.rows;  // gate rows, then up rows
        moe_tile<BITS, XBF16, MBF16>(a, base + r_a, base + r_b, s_begin, s_end, xb_lane, xb_step_u4, xsum, xneg,
                                     t, acc[h]);
      }
    }
    // sum the slices of the reduction axis in a fixed order
    if (a.kw > 1) {
#pragma unroll
      for (int h = 0; h < (GATE_UP ? 2 : 1); ++h) {
        float* mine = red + (((h * a.kw + kwi) * a.rw + rwi) * 16) * 8;
        *reinterpret_cast<float2*>(mine + g * 8 + 2 * t) = make_float2(acc[h][0], acc[h][1]);
        *reinterpret_cast<float2*>(mine + (g + 8) * 8 + 2 * t) = make_float2(acc[h][2], acc[h][3]);
      }
      __syncthreads();
      if (kwi == 0) {
#pragma unroll
        for (int h = 0; h < (GATE_UP ? 2 : 1); ++h) {
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[h][i] = 0.0f;
          for (int k = 0; k < a.kw; ++k) {
            const float* part = red + (((h * a.kw + k) * a.rw + rwi) * 16) * 8;
            const float2 pa = *reinterpret_cast<const float2*>(part + g * 8 + 2 * t);
            const float2 pb = *reinterpret_cast<const float2*>(part + (g + 8) * 8 + 2 * t);
            acc[h][0] += pa.x, acc[h][1] += pa.y, acc[h][2] += pb.x, acc[h][3] += pb.y;
          }
        }
      }
    }
    if (kwi == 0 && tile_live) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int mm = 2 * t + (i & 1);
        const int row = tile * 16 + g + ((i & 2) ? 8 : 0);
        if (mm < m && row < a.rows) {
          const int aid = a.route.sorted[first + c0 + mm];
          if constexpr (GATE_UP) {
            const float gate = acc[0][i], up = acc[1][i];
            const float h = (gate / (1.0f + __expf(-gate))) * up;
            store_f32(a.out, static_cast<int64_t>(aid) * a.rows + row, a.act_dtype, h);
          } else {
            reinterpret_cast<float*>(a.out)[static_cast<int64_t>(aid) * a.rows + row] = acc[0][i];
          }
        }
      }
    }
  }
}

__global__ void moe_combine_kernel(const float* __restrict__ d, const float* __restrict__ w,
                                   const int32_t* __restrict__ ids, int tokens, int topk, int hidden,
                                   int num_experts, void* y, int y_dtype) {
  pdl_launch_dependents();
  pdl_wait_prior_grid();
  const int64_t total = static_cast<int64_t>(tokens) * hidden;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int tkn = static_cast<int>(i / hidden);
    const int col = static_cast<int>(i - static_cast<int64_t>(tkn) * hidden);
    float acc = 0.0f;
    for (int k = 0; k < topk; ++k) {
      const int aid = tkn * topk + k;
      const int e = ids[aid];
      if (e >= 0 && e < num_experts) {
        acc = fmaf(w[aid], d[static_cast<int64_t>(aid) * hidden + col], acc);
      }
    }
    store_f32(y, i, y_dtype, acc);
  }
}

struct ScratchLayout {
  size_t counts, offsets, sorted, h, d, total;
};

ScratchLayout scratch_layout(int64_t tokens, int64_t topk, int64_t hidden, int64_t inter, int64_t experts,
                             int act_bytes) {
  auto up = [](size_t v) { return (v + 255) / 256 * 256; };
  ScratchLayout l = {};
  const size_t assignments = static_cast<size_t>(tokens * topk);
  size_t at = 0;
  l.counts = at, at = up(at + static_cast<size_t>(experts) * 4);
  l.offsets = at, at = up(at + static_cast<size_t>(experts + 1) * 4);
  l.sorted = at, at = up(at + assignments * 4);
  l.h = at, at = up(at + assignments * static_cast<size_t>(inter) * act_bytes);
  l.d = at, at = up(at + assignments * static_cast<size_t>(hidden) * 4);
  l.total = at;
  return l;
}

// Scratch for dq_moe_gemv_static: lives in the library image, one copy per GPU that loads
// it, for as long as the process runs.  Host code must never pass this NAME to a kernel --
// on the host it is only a stand-in for the symbol; the device address comes from
// cudaGetSymbolAddress (see static_scratch_address below).
static __device__ __align__(256) unsigned char g_moe_static_scratch[DQ_MOE_STATIC_SCRATCH_BYTES];

// Device address of g_moe_static_scratch on the CURRENT device, looked up once per device.
int32_t static_scratch_address(void** out) {
  constexpr int kMaxDevices = 64;
  static void* address[kMaxDevices] = {nullptr};
  int device = 0;
  DQ_CUDA(cudaGetDevice(&device));
  DQ_REQUIRE(device >= 0 && device < kMaxDevices, "moe_gemv_static: device ordinal %d out of range", device);
  if (address[device] == nullptr) {
    void* ptr = nullptr;
    DQ_CUDA(cudaGetSymbolAddress(&ptr, g_moe_static_scratch));
    DQ_REQUIRE(ptr != nullptr, "moe_gemv_static: cudaGetSymbolAddress returned a null address");
    address[device] = ptr;  // same value from every thread that races here
  }
  *out = address[device];
  return DQ_OK;
}

template <typename Kernel>
int32_t launch_pdl(Kernel kernel, dim3 grid, int threads, size_t smem, cudaStream_t stream, const MoeArgs& args,
                   const char* what) {
  if (smem > 48 * 1024) {
    DQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(static_cast<unsigned>(threads));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  DQ_CUDA(cudaLaunchKernelEx(&cfg, kernel, args));
  DQ_CHECK_LAUNCH(what);
  return DQ_OK;
}

template <int BITS, bool GATE_UP>
int32_t launch_grouped(const MoeArgs& a, int experts, size_t smem, cudaStream_t stream) {
  const int tiles = (a.rows + 15) / 16;
  const dim3 grid(static_cast<unsigned>(ceil_div(tiles, a.rw)), static_cast<unsigned>(experts));
  const bool xbf = a.act_dtype == DQ_BF16, mbf = a.meta_dtype == DQ_BF16;
  const char* what = GATE_UP ? "moe_gemv(gate_up)" : "moe_gemv(down)";
  if (xbf && mbf) return launch_pdl(moe_grouped_kernel<BITS, true, true, GATE_UP>, grid, kMoeThreads, smem, stream, a, what);
  if (xbf) return launch_pdl(moe_grouped_kernel<BITS, true, false, GATE_UP>, grid, kMoeThreads, smem, stream, a, what);
  if (mbf) return launch_pdl(moe_grouped_kernel<BITS, false, true, GATE_UP>, grid, kMoeThreads, smem, stream, a, what);
  return launch_pdl(moe_grouped_kernel<BITS, false, false, GATE_UP>, grid, kMoeThreads, smem, stream, a, what);
}

template <bool GATE_UP>
int32_t launch_bank(const dq_weight& w, const dq_geometry& g, MoeArgs a, int experts, cudaStream_t stream) {
  a.packed = static_cast<const uint32_t*>(w.packed);
  a.scales = w.scales;
  a.offsets = w.offsets;
  a.meta_dtype = w.meta_dtype;
  a.words_per_row = g.words_per_row;
  a.num_groups = g.num_groups;
  a.in_features = g.in_features;
  a.steps = g.words_per_row / (4 * w.bits);
  // 8 warps: slice the reduction axis as far as the steps allow (at most 4 ways), the rest
  // of the warps take neighbouring row tiles
  int kw = 1;
  while (kw < 4 && a.steps / (kw * 2) >= 2) kw *= 2;
  a.kw = kw;
  a.rw = kMoeWarps / kw;
  a.steps_per_warp = static_cast<int>(ceil_div(a.steps, a.kw));
  const int aregs = w.bits == 8 ? 32 : 16;
  a.m_stride_u4 = a.steps * aregs + 4;
  a.magic = a.act_dtype == DQ_BF16 ? 0x43004300u : 0x64006400u;
  const size_t smem = (static_cast<size_t>(8) * a.m_stride_u4 + aregs) * 16 + static_cast<size_t>(a.steps) * 8 * 4 * 2 +
                      static_cast<size_t>(GATE_UP ? 2 : 1) * a.kw * a.rw * 16 * 8 * 4 + 8 * 4;
  const DeviceInfo* dev = device_info();
  if (dev == nullptr) return DQ_ERR_CUDA;
  if (smem > static_cast<size_t>(dev->max_smem_optin)) {
    return fail(DQ_ERR_UNSUPPORTED, "moe_gemv: in_features=%d needs %zu bytes of shared memory", a.in_features, smem);
  }
  switch (w.bits) {
    case 2:
      return launch_grouped<2, GATE_UP>(a, experts, smem, stream);
    case 3:
      return launch_grouped<3, GATE_UP>(a, experts, smem, stream);
    case 4:
      return launch_grouped<4, GATE_UP>(a, experts, smem, stream);
    default:
      return launch_grouped<8, GATE_UP>(a, experts, smem, stream);
  }
}

}  // namespace
}  // namespace dq

extern "C" {

int32_t dq_moe_scratch_bytes(int64_t tokens, int64_t topk, int64_t hidden, int64_t inter, int64_t num_experts,
                             int32_t act_dtype, int64_t* bytes) {
  DQ_REQUIRE(bytes != nullptr, "moe_scratch_bytes: null result pointer");
  DQ_REQUIRE(tokens >= 0 && tokens <= DQ_MOE_MAX_TOKENS, "moe_gemv: %lld tokens exceeds the limit of %d per call",
             static_cast<long long>(tokens), DQ_MOE_MAX_TOKENS);
  DQ_REQUIRE(topk > 0 && topk <= 16 && hidden > 0 && inter > 0 && num_experts > 0 && dq::dtype_ok(act_dtype),
             "moe_gemv: bad sizes (topk=%lld hidden=%lld inter=%lld experts=%lld)", static_cast<long long>(topk),
             static_cast<long long>(hidden), static_cast<long long>(inter), static_cast<long long>(num_experts));
  *bytes = static_cast<int64_t>(
      dq::scratch_layout(tokens, topk, hidden, inter, num_experts, dq::dtype_size(act_dtype)).total);
  return DQ_OK;
}

int32_t dq_moe_gemv(const void* x, int32_t x_dtype, int64_t tokens, const int32_t* topk_ids, const float* topk_w,
                    int64_t topk, int64_t num_experts, const dq_weight* gate_up, const dq_weight* down,
                    int64_t hidden, int64_t inter, void* y, int32_t y_dtype, void* scratch, int64_t scratch_bytes,
                    void* stream) {
  int64_t need = 0;
  if (const int32_t rc = dq_moe_scratch_bytes(tokens, topk, hidden, inter, num_experts, x_dtype, &need)) return rc;
  DQ_REQUIRE(gate_up != nullptr && down != nullptr, "moe_gemv: null bank descriptor");
  dq_geometry g_gu, g_dn;
  if (const int32_t rc = dq_resolve_geometry("moe_gemv(gate_up)", gate_up, &g_gu)) return rc;
  if (const int32_t rc = dq_resolve_geometry("moe_gemv(down)", down, &g_dn)) return rc;
  DQ_REQUIRE(gate_up->rows == num_experts * 2 * inter && gate_up->in_features == hidden,
             "moe_gemv: gate_up bank must be [%lld * 2 * %lld, %lld] folded to rows, got [%lld, %lld]",
             static_cast<long long>(num_experts), static_cast<long long>(inter), static_cast<long long>(hidden),
             static_cast<long long>(gate_up->rows), static_cast<long long>(gate_up->in_features));
  DQ_REQUIRE(down->rows == num_experts * hidden && down->in_features == inter,
             "moe_gemv: down bank must be [%lld * %lld, %lld] folded to rows, got [%lld, %lld]",
             static_cast<long long>(num_experts), static_cast<long long>(hidden), static_cast<long long>(inter),
             static_cast<long long>(down->rows), static_cast<long long>(down->in_features));
  DQ_REQUIRE(dq::dtype_ok(y_dtype), "moe_gemv: unsupported output dtype tag %d", y_dtype);
  if (tokens == 0) return DQ_OK;
  DQ_REQUIRE(x != nullptr && topk_ids != nullptr && topk_w != nullptr && y != nullptr, "moe_gemv: null pointer");
  DQ_REQUIRE(scratch != nullptr && scratch_bytes >= need && reinterpret_cast<uintptr_t>(scratch) % 256 == 0,
             "moe_gemv: scratch must be 256-byte aligned and at least %lld bytes (dq_moe_scratch_bytes), got %lld",
             static_cast<long long>(need), static_cast<long long>(scratch_bytes));
  const bool act16 = x_dtype == DQ_BF16 || x_dtype == DQ_F16;
  const auto meta16 = [](const dq_weight* w) { return w->meta_dtype == DQ_BF16 || w->meta_dtype == DQ_F16; };
  if (!act16 || !meta16(gate_up) || !meta16(down) || gate_up->group_values != 128 || down->group_values != 128 ||
      reinterpret_cast<uintptr_t>(gate_up->packed) % 4 != 0) {
    return dq::fail(DQ_ERR_UNSUPPORTED,
                    "moe_gemv: this build handles fp16/bf16 activations and metadata with 128-value groups");
  }

  auto s = static_cast<cudaStream_t>(stream);
  const dq::ScratchLayout lay = dq::scratch_layout(tokens, topk, hidden, inter, num_experts, dq::dtype_size(x_dtype));
  auto* base = static_cast<unsigned char*>(scratch);
  dq::Routing route = {reinterpret_cast<int*>(base + lay.counts), reinterpret_cast<int*>(base + lay.offsets),
                       reinterpret_cast<int*>(base + lay.sorted)};
  const int assignments = static_cast<int>(tokens * topk);
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(512);
    cfg.dynamicSmemBytes = static_cast<size_t>(2 * num_experts + 1) * 4;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    DQ_CUDA(cudaLaunchKernelEx(&cfg, dq::moe_route_kernel, topk_ids, assignments, static_cast<int>(num_experts), route));
    DQ_CHECK_LAUNCH("moe_gemv(route)");
  }
  dq::MoeArgs a = {};
  a.route = route;
  a.topk = static_cast<int>(topk);
  a.act_dtype = x_dtype;
  // gate_up: x -> h
  a.act = x;
  a.out = base + lay.h;
  a.rows = static_cast<int>(inter);
  if (const int32_t rc = dq::launch_bank<true>(*gate_up, g_gu, a, static_cast<int>(num_experts), s)) return rc;
  // down: h -> d
  a.act = base + lay.h;
  a.out = base + lay.d;
  a.rows = static_cast<int>(hidden);
  if (const int32_t rc = dq::launch_bank<false>(*down, g_dn, a, static_cast<int>(num_experts), s)) return rc;
  {
    const int64_t total = tokens * hidden;
    const int threads = 256;
    const int grid = static_cast<int>(std::min<int64_t>(dq::ceil_div(total, threads), 1184));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(threads);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    DQ_CUDA(cudaLaunchKernelEx(&cfg, dq::moe_combine_kernel, reinterpret_cast<const float*>(base + lay.d), topk_w,
                               topk_ids, static_cast<int>(tokens), static_cast<int>(topk), static_cast<int>(hidden),
                               static_cast<int>(num_experts), y, y_dtype));
    DQ_CHECK_LAUNCH("moe_gemv(combine)");
  }
  return DQ_OK;
}

int32_t dq_moe_gemv_static(const void* x, int32_t x_dtype, int64_t tokens, const int32_t* topk_ids,
                           const float* topk_w, int64_t topk, int64_t num_experts, const dq_weight* gate_up,
                           const dq_weight* down, int64_t hidden, int64_t inter, void* y, int32_t y_dtype,
                           void* stream) {
  int64_t need = 0;
  if (const int32_t rc = dq_moe_scratch_bytes(tokens, topk, hidden, inter, num_experts, x_dtype, &need)) return rc;
  DQ_REQUIRE(need <= DQ_MOE_STATIC_SCRATCH_BYTES,
             "moe_gemv_static: this problem needs %lld bytes of scratch but the built-in buffer holds %d "
             "(tokens=%lld topk=%lld hidden=%lld inter=%lld experts=%lld); use dq_moe_gemv with your own scratch",
             static_cast<long long>(need), DQ_MOE_STATIC_SCRATCH_BYTES, static_cast<long long>(tokens),
             static_cast<long long>(topk), static_cast<long long>(hidden), static_cast<long long>(inter),
             static_cast<long long>(num_experts));
  void* scratch = nullptr;
  if (const int32_t rc = dq::static_scratch_address(&scratch)) return rc;
  return dq_moe_gemv(x, x_dtype, tokens, topk_ids, topk_w, topk, num_experts, gate_up, down, hidden, inter, y,
                     y_dtype, scratch, DQ_MOE_STATIC_SCRATCH_BYTES, stream);
}

}  // extern "C"
