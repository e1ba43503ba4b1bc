// MoE grouped GEMV: y[t] = sum_k p[t,k] * W_down[e] ( silu(W_gate[e] x[t]) * (W_up[e] x[t]) ),  e = ids[t,k].
//
// The reference has no such kernel: its serving plugins refuse fused-MoE layers
// (integration/vllm_plugin/config.py:107-112) and pack_model refuses expert banks
// (runtime/linear.py:442-456).  What it does define is the weight format of a bank --
// a stacked tensor [E, out, in] folds to rows, expert e owning rows [e*out, (e+1)*out)
// (quant/tensor.py:253-255; shapes from graph/experts.py:35-43: gate_up [E, 2I, H] with
// the gate rows first, down [E, H, I]) -- and this file computes on exactly that.
//
// Three launches, all on the caller's stream, no host round trip:
//   1. gate_up  grid (row-tile pairs, slots), one slot per expert that COULD be active
//               (min(E, tokens * topk)).  Every CTA first works out the routing itself from
//               topk_ids -- which expert is the slot-th one with a token, and which
//               assignments are its (in ascending order) -- a few hundred cycles of shared-
//               memory work instead of a launch and a round trip through global memory.
//               CTAs of empty slots exit.  The expert's packed rows for the CTA's tile travel
//               to shared memory ONCE (16-byte cp.async) and are reused for all of its tokens,
//               eight at a time: the tokens are the 8 columns of the m16n8k16 accumulator,
//               exactly like the activation rows of the dense GEMV (dq_gemv_mma.cu), gathered
//               by index while staging.  A warp computes its slice of 16 gate rows and the
//               matching 16 up rows; h = silu(g) * u, rounded to the activation dtype, goes
//               to scratch.
//   2. down     same machinery over the down bank with h as the activation; the fp32
//               result of every assignment goes to scratch.  Routing and the down weights
//               depend on topk_ids only, so this kernel computes the one and requests the
//               other BEFORE griddepcontrol.wait, while gate_up is still running.
//   3. combine  y[t] = sum_k p[t,k] * d[t,k] in slot order -- a fixed order, so the layer is
//               bit-identical run to run (no atomics on floats anywhere).
// ids outside [0, num_experts) are skipped, which is how an expert-parallel rank passes
// "not mine".
#include <algorithm>
#include <cmath>
#include <cstdlib>

#include "dq_gemv.cuh"
#include "dq_gemv_mma_stream.cuh"
#include "dq_mma_plan.cuh"
#include "dq_mma_stage.cuh"

namespace dq {
namespace {

constexpr int kMoeWarps = 8;
constexpr int kMoeThreads = kMoeWarps * kWarp;
constexpr int kMaxAssign = DQ_MOE_MAX_TOKENS * 16;

struct MoeArgs {
  const void* act;          // gate_up: x [tokens, K]; down: h [assignments, K]
  const uint32_t* packed;   // the bank, [E * rows_per_expert(*2), words_per_row]
  const void* scales;
  const void* offsets;      // may be null
  void* out;                // gate_up: h [assignments, inter] act dtype; down: d [assignments, hidden] fp32
  const int32_t* ids;       // [assignments] expert of every (token, slot), minus first_expert
  int first_expert;         // ids are global; this call holds experts [first_expert, first_expert + num_experts)
  int by_assignment;        // 1: slot s IS assignment s (few tokens: no routing to work out, an expert may be read twice)
  int assignments, num_experts;
  int act_dtype, meta_dtype;
  int topk;
  int rows;                 // output rows per expert of this launch (inter, or hidden)
  int words_per_row, num_groups, in_features;
  int steps;                // padded K / 128
  int kw, rw;               // warps: rw row tiles x kw slices of the reduction axis
  int spw;                  // steps per slice, a multiple of CH
  int nb;                   // ring stages (of CH steps per warp)
  int tokens;               // of the whole call
  int m_cap;                // activation rows staged at once (<= 8)
  int m_stride_u4;
  uint32_t magic;
};

// Shared memory of moe_grouped_kernel, in order.
struct MoeSmem {
  size_t ring_w, ring_m, red, ids, counts, list, misc, stage, total;
};

template <int BITS, int CH>
__host__ __device__ inline MoeSmem moe_smem(const MoeArgs& a, bool gate_up) {
  const int halves = gate_up ? 2 : 1;
  const int na = BITS == 8 ? 32 : 16;
  auto up16 = [](size_t v) { return (v + 15) / 16 * 16; };
  MoeSmem m = {};
  size_t at = 0;
  m.ring_w = at, at += static_cast<size_t>(a.nb) * CH * 2 * kMoeThreads * (4 * BITS);
  m.ring_m = at, at += static_cast<size_t>(a.nb) * CH * 2 * kMoeThreads;
  // partial sums of the slices of the reduction axis: two buffers, alternating per item
  m.red = at, at += a.kw > 1 ? 2 * static_cast<size_t>(halves) * kMoeWarps * 128 * 4 : 0;
  m.ids = at, at = up16(at + static_cast<size_t>(a.assignments) * 4);
  m.counts = at, at = up16(at + static_cast<size_t>(a.num_experts) * 4);
  m.list = at, at = up16(at + static_cast<size_t>(DQ_MOE_MAX_TOKENS) * 4);
  m.misc = at, at += 64 * 4;  // [0] expert, [1] count, [8..15] row map, [16..47] ballot counts
  m.stage = at;
  at += (static_cast<size_t>(a.m_cap) * a.m_stride_u4 + na) * 16 + static_cast<size_t>(a.steps) * 64 + 16;
  m.total = at;
  return m;
}

__device__ __forceinline__ void moe_wait_pending(int n) {
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

// One CTA: one active expert (grid.y = slot), a strided share of its row tiles (grid.x).
// The plumbing is that of the tiled dense kernel (dq_gemv_mma_tile.cuh): 8 warps as rw row
// tiles x kw slices of the reduction axis, every warp streaming ITS slice of ITS tiles
// through a private cp.async ring of `nb` stages of CH steps, partial sums of the slices
// added in a fixed order.  GATE_UP: an item is 16 gate rows plus the matching 16 up rows per
// row tile, and the output is silu(g) * u.
template <int BITS, bool XBF16, int CH, bool GATE_UP, int CTAS>
__global__ void __launch_bounds__(kMoeThreads, CTAS) moe_grouped_kernel(const __grid_constant__ MoeArgs a) {
  using Plan = MmaPlan<BITS>;
  constexpr int NA = Plan::kARegs;
  constexpr int QU = NA / 4;
  constexpr int UNIT = 4 * BITS;
  constexpr int STEP_WORDS = 4 * BITS;
  constexpr int H = GATE_UP ? 2 : 1;
  constexpr int STAGE_W = CH * 2 * UNIT * kMoeThreads;
  constexpr int STAGE_M = CH * 2 * kMoeThreads;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const MoeSmem lay = moe_smem<BITS, CH>(a, GATE_UP);
  unsigned char* ring_w = smem_raw + lay.ring_w;
  unsigned char* ring_m = smem_raw + lay.ring_m;
  float* red = reinterpret_cast<float*>(smem_raw + lay.red);
  int* ids_s = reinterpret_cast<int*>(smem_raw + lay.ids);
  int* cnt = reinterpret_cast<int*>(smem_raw + lay.counts);
  int* list = reinterpret_cast<int*>(smem_raw + lay.list);
  int* misc = reinterpret_cast<int*>(smem_raw + lay.misc);
  int* row_map = misc + 8;
  int* ballots = misc + 16;
  uint4* xb = reinterpret_cast<uint4*>(smem_raw + lay.stage);
  float* xsum = reinterpret_cast<float*>(xb + a.m_cap * a.m_stride_u4 + NA);
  float* xneg = xsum + a.steps * 8;

  const int tid = threadIdx.x;
  const int lane = tid & (kWarp - 1);
  const int warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int slot = blockIdx.y;

  // gate_up: topk_ids come from the previous kernel; and only once every CTA of this grid
  // is past that wait may the down kernel start (its routing and weight requests run ahead
  // of ITS wait).  down: nothing it needs before the wait is written by gate_up.
  if (GATE_UP) {
    pdl_wait_prior_grid();
  }
  pdl_launch_dependents();

  // ---- routing, by every CTA for itself ----
  if (a.by_assignment) {
    // few tokens: a slot per assignment, nothing to count or rank
    if (tid == 0) {
      const int mine = __ldcg(a.ids + slot) - a.first_expert;
      misc[0] = (mine >= 0 && mine < a.num_experts) ? mine : -1;
      misc[1] = 1;
      list[0] = slot;
    }
    __syncthreads();
  } else {
  for (int i = tid; i < a.num_experts; i += kMoeThreads) cnt[i] = 0;
  for (int i = tid; i < a.assignments; i += kMoeThreads) ids_s[i] = __ldcg(a.ids + i) - a.first_expert;
  if (tid == 0) misc[0] = -1;
  __syncthreads();
  for (int i = tid; i < a.assignments; i += kMoeThreads) {
    const int e = ids_s[i];
    if (e >= 0 && e < a.num_experts) atomicAdd(&cnt[e], 1);  // integer count: order-independent
  }
  __syncthreads();
  if (warp == 0) {  // the slot-th expert (ascending id) that has a token
    int seen = 0;
    for (int base = 0; base < a.num_experts; base += kWarp) {
      const int e = base + lane;
      const bool active = e < a.num_experts && cnt[e] > 0;
      const unsigned mask = __ballot_sync(0xffffffffu, active);
      const int before = __popc(mask & ((1u << lane) - 1u));
      if (active && seen + before == slot) {
        misc[0] = e;
        misc[1] = min(cnt[e], DQ_MOE_MAX_TOKENS);
      }
      seen += __popc(mask);
      if (seen > slot) break;
    }
  }
  __syncthreads();
  }
  const int e = misc[0];
  if (e < 0) return;  // fewer active experts than slots
  const int count = misc[1];

  // ---- this warp's sequence of ring stages: (token chunk, item, half, chunk of CH steps) ----
  const int kw = a.kw, rw = a.rw, spw = a.spw, nb = a.nb;
  const int rwi = warp / kw;
  const int kwi = warp - rwi * kw;
  const int s_begin = kwi * spw;
  const int nchunks = spw / CH;
  const int tiles = (a.rows + 15) / 16;
  const int items = (tiles + rw - 1) / rw;
  const int ntc = (count + a.m_cap - 1) / a.m_cap;  // token chunks
  const int64_t expert_row0 = static_cast<int64_t>(e) * a.rows * H;
  const bool has_off = a.offsets != nullptr;
  // The cursor is kept as running pointers (integer instructions issue at half rate and the
  // decode needs that pipe): what depends on the lane, the row tile or the half is resolved
  // once per (item, half), a stage costs a pointer bump per source row, copies use immediates.
  constexpr int PIECES = 2 * UNIT;       // 16-byte pieces of one (step, row half) block
  constexpr int PER_ROW = UNIT / 4;      // pieces per row
  constexpr int NSRC = (PIECES + kWarp - 1) / kWarp;
  constexpr int STEP_BYTES = STEP_WORDS * 4;
  const uint32_t ring_w_s = static_cast<uint32_t>(__cvta_generic_to_shared(ring_w)) + (tid - lane) * UNIT + lane * 16;
  const uint32_t ring_m_s = static_cast<uint32_t>(__cvta_generic_to_shared(ring_m)) + tid * (CH * 2);
  const bool meta_lane = has_off || (t & 1) == 0;
  const unsigned short* meta_arr = reinterpret_cast<const unsigned short*>((t & 1) ? a.offsets : a.scales);
  bool pf_lane[NSRC];
#pragma unroll
  for (int i = 0; i < NSRC; ++i) pf_lane[i] = (PIECES % kWarp == 0) || (i * kWarp + lane < PIECES);
  const unsigned char* pf_src[2][NSRC];
  const unsigned short* pf_meta = nullptr;
  int pf_tc = 0, pf_item = blockIdx.x, pf_half = 0, pf_chunk = 0;
  bool pf_live = false;
  auto pf_point = [&]() {  // start of an (item, half)
    const int tile = pf_item * rw + rwi;
    pf_live = pf_tc < ntc && pf_item < items && tile < tiles;
    if (pf_live) {
      const int row0 = static_cast<int>(expert_row0) + pf_half * a.rows + tile * 16;
      const int last = static_cast<int>(expert_row0) + (pf_half + 1) * a.rows - 1;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int i = 0; i < NSRC; ++i) {
          const int piece = i * kWarp + lane;
          const int pg = piece / PER_ROW;
          const int part = piece - pg * PER_ROW;
          const int row = min(row0 + h * 8 + pg, last);
          pf_src[h][i] = reinterpret_cast<const unsigned char*>(a.packed + static_cast<int64_t>(row) * a.words_per_row +
                                                                 part * 4) + s_begin * STEP_BYTES;
        }
      }
      const int row = min(row0 + g + ((t & 2) ? 8 : 0), last);
      pf_meta = meta_arr + static_cast<int64_t>(row) * a.num_groups + s_begin;
    }
  };
  pf_point();
  uint32_t pf_w = ring_w_s, pf_m = ring_m_s;
  const uint32_t pf_w_end = ring_w_s + nb * STAGE_W;
  auto prefetch_stage = [&]() {
    if (pf_tc < ntc && pf_item < items) {
      if (pf_live) {
#pragma unroll
        for (int j = 0; j < CH; ++j) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int i = 0; i < NSRC; ++i) {
              if (pf_lane[i]) {
                stream::cp_async_n<16>(pf_w + (j * 2 + h) * (UNIT * kMoeThreads) + i * (kWarp * 16), pf_src[h][i] + j * STEP_BYTES);
              }
            }
          }
        }
        if constexpr (CH >= 2) {  // (a single step's metadata is 2 bytes: read in the loop instead)
          if (meta_lane) stream::cp_async_n<CH * 2>(pf_m, pf_meta);
        }
      }
      if (++pf_chunk == nchunks) {
        pf_chunk = 0;
        if (++pf_half == H) {
          pf_half = 0;
          pf_item += gridDim.x;
          if (pf_item >= items) {
            pf_item = blockIdx.x;
            ++pf_tc;
          }
        }
        pf_point();
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int i = 0; i < NSRC; ++i) pf_src[h][i] += CH * STEP_BYTES;
        }
        pf_meta += CH;
      }
    }
    pf_w += STAGE_W;
    pf_m += STAGE_M;
    if (pf_w == pf_w_end) {
      pf_w = ring_w_s;
      pf_m = ring_m_s;
    }
    stream::cp_async_commit();  // an empty group keeps the wait arithmetic uniform
  };
  for (int i = 0; i < nb; ++i) prefetch_stage();

  // ---- the expert's assignments in ascending order (so results do not depend on timing) ----
  if (!a.by_assignment) {
  for (int base = 0; base < a.assignments; base += kMoeThreads) {
    const int i = base + tid;
    const bool mine = i < a.assignments && ids_s[i] == e;
    const unsigned mask = __ballot_sync(0xffffffffu, mine);
    if (lane == 0) ballots[(base / kMoeThreads) * kMoeWarps + warp] = __popc(mask);
  }
  __syncthreads();
  for (int base = 0; base < a.assignments; base += kMoeThreads) {
    const int i = base + tid;
    const bool mine = i < a.assignments && ids_s[i] == e;
    const unsigned mask = __ballot_sync(0xffffffffu, mine);
    if (mine) {
      int rank = __popc(mask & ((1u << lane) - 1u));
      const int upto = (base / kMoeThreads) * kMoeWarps + warp;
      for (int k = 0; k < upto; ++k) rank += ballots[k];
      if (rank < DQ_MOE_MAX_TOKENS) list[rank] = i;
    }
  }
  }

  if (!GATE_UP) {
    pdl_wait_prior_grid();  // h
  }

  GemvArgs stage = {};
  stage.x = a.act;
  stage.x_dtype = a.act_dtype;
  stage.in_features = a.in_features;
  const bool mbf = a.meta_dtype == DQ_BF16;
  const uint32_t magic = a.magic;
  const unsigned char* ring_w_mine = ring_w + tid * UNIT;
  const unsigned char* ring_m_quad = ring_m + (tid & ~3) * (CH * 2);
  const float* xsum_w = xsum + s_begin * 8 + 2 * t;
  const float* xneg_w = xneg + s_begin * 8 + 2 * t;

  int parity = 0;
  const unsigned char* wslot = ring_w_mine;  // ring slot being consumed
  const unsigned char* mslot = ring_m_quad;
  const unsigned char* const wslot_end = ring_w_mine + nb * STAGE_W;
  for (int tc = 0; tc < ntc; ++tc) {
    const int c0 = tc * a.m_cap;
    const int m = min(a.m_cap, count - c0);
    __syncthreads();  // list is complete; the previous chunk is done with row_map / xb
    if (tid < 8) {
      const int aid = list[min(c0 + tid, count - 1)];
      row_map[tid] = GATE_UP ? aid / a.topk : aid;  // x is per token, h per assignment
    }
    __syncthreads();
    stage.m = m;
    stage_activation<BITS, XBF16>(stage, a.steps, a.m_stride_u4, xb, xsum, xneg, tid, kMoeThreads, row_map);
    __syncthreads();
    const bool b_live = g < m;
    const uint4* xb_lane = (b_live ? xb + g * a.m_stride_u4 + t : xb + m * a.m_stride_u4) + (b_live ? s_begin * QU * 4 : 0);
    const int xb_step_u4 = b_live ? QU * 4 : 0;

    for (int item = blockIdx.x; item < items; item += gridDim.x, parity ^= 1) {
      const int tile = item * rw + rwi;
      const bool live = tile < tiles;
      float acc[H][4];
#pragma unroll
      for (int h = 0; h < H; ++h) {
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[h][i] = 0.0f;
        for (int chunk = 0; chunk < nchunks; ++chunk) {
          moe_wait_pending(nb - 1);  // groups complete in issue order: all but the nb-1 youngest are done
          __syncwarp();              // copies of other lanes (units, the quad's metadata) are visible
          if (live) {
            const unsigned char* wsrc = wslot;
            const unsigned char* msrc = mslot;
            uint32_t mc[4][CH >= 2 ? CH / 2 : 1];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              if (has_off || (i & 1) == 0) {
                if constexpr (CH == 1) {
                  const int row0 = static_cast<int>(expert_row0) + h * a.rows;
                  const int row = min(row0 + tile * 16 + g + ((i & 2) ? 8 : 0), row0 + a.rows - 1);
                  const unsigned short* arr = reinterpret_cast<const unsigned short*>((i & 1) ? a.offsets : a.scales);
                  mc[i][0] = __ldg(arr + static_cast<int64_t>(row) * a.num_groups + s_begin + chunk);
                } else if constexpr (CH == 4) {
                  const uint2 v = *reinterpret_cast<const uint2*>(msrc + i * (CH * 2));
                  mc[i][0] = v.x, mc[i][1] = v.y;
                } else {
                  mc[i][0] = *reinterpret_cast<const uint32_t*>(msrc + i * (CH * 2));
                }
              }
            }
#pragma unroll
            for (int j = 0; j < CH; ++j) {
              const int sl = chunk * CH + j;
              uint32_t wa[BITS], wb[BITS];
              stream::read_unit<BITS>(wsrc + (j * 2 + 0) * (UNIT * kMoeThreads), wa);
              stream::read_unit<BITS>(wsrc + (j * 2 + 1) * (UNIT * kMoeThreads), wb);
              uint32_t aa[NA], ab[NA];
              decode_unit<BITS>(wa, magic, aa);
              decode_unit<BITS>(wb, magic, ab);
              unbias_fragments<XBF16, NA>(aa);
              unbias_fragments<XBF16, NA>(ab);
              const uint4* bsrc = xb_lane + sl * xb_step_u4;
              float d[4], f[4];
#pragma unroll
              for (int q = 0; q < QU; ++q) {
                const uint4 b = bsrc[q * 4];
                if (q == 0) {
                  mma_16816<XBF16, true>(d, aa[0], ab[0], aa[1], ab[1], b.x, b.y);
                  mma_16816<XBF16, true>(f, aa[2], ab[2], aa[3], ab[3], b.z, b.w);
                } else {
                  mma_16816<XBF16, false>(d, aa[4 * q], ab[4 * q], aa[4 * q + 1], ab[4 * q + 1], b.x, b.y);
                  mma_16816<XBF16, false>(f, aa[4 * q + 2], ab[4 * q + 2], aa[4 * q + 3], ab[4 * q + 3], b.z, b.w);
                }
              }
#pragma unroll
              for (int i = 0; i < 4; ++i) d[i] += f[i];
              auto meta_f32 = [&](int i) -> float {
                const uint32_t reg = mc[i][j / 2];
                if (mbf) return __uint_as_float((j & 1) ? (reg & 0xFFFF0000u) : (reg << 16));
                const __half2 hh = *reinterpret_cast<const __half2*>(&reg);
                return (j & 1) ? __high2float(hh) : __low2float(hh);
              };
              const float2 xs2 = *reinterpret_cast<const float2*>(xsum_w + sl * 8);
              const float2 xn2 = *reinterpret_cast<const float2*>(xneg_w + sl * 8);
              const float sc_a = meta_f32(0), sc_b = meta_f32(2);
              acc[h][0] = fmaf(sc_a, d[0] + xn2.x, acc[h][0]);
              acc[h][1] = fmaf(sc_a, d[1] + xn2.y, acc[h][1]);
              acc[h][2] = fmaf(sc_b, d[2] + xn2.x, acc[h][2]);
              acc[h][3] = fmaf(sc_b, d[3] + xn2.y, acc[h][3]);
              if (has_off) {
                const float of_a = meta_f32(1), of_b = meta_f32(3);
                acc[h][0] = fmaf(of_a, xs2.x, acc[h][0]);
                acc[h][1] = fmaf(of_a, xs2.y, acc[h][1]);
                acc[h][2] = fmaf(of_b, xs2.x, acc[h][2]);
                acc[h][3] = fmaf(of_b, xs2.y, acc[h][3]);
              }
            }
          }
          wslot += STAGE_W;
          mslot += STAGE_M;
          if (wslot == wslot_end) {
            wslot = ring_w_mine;
            mslot = ring_m_quad;
          }
          __syncwarp();      // every lane is done with the slot just consumed:
          prefetch_stage();  // refill it
        }
      }
      // sum the slices of the reduction axis in a fixed order (buffers alternate: one barrier per item)
      if (kw > 1) {
        float* rbuf = red + parity * (H * kMoeWarps * 128);
#pragma unroll
        for (int h = 0; h < H; ++h) {
          float* mine = rbuf + ((h * kw + kwi) * rw + rwi) * 128;
          *reinterpret_cast<float2*>(mine + g * 8 + 2 * t) = make_float2(acc[h][0], acc[h][1]);
          *reinterpret_cast<float2*>(mine + (g + 8) * 8 + 2 * t) = make_float2(acc[h][2], acc[h][3]);
        }
        __syncthreads();
        if (kwi == 0) {
#pragma unroll
          for (int h = 0; h < H; ++h) {
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[h][i] = 0.0f;
            for (int k = 0; k < kw; ++k) {
              const float* part = rbuf + ((h * kw + k) * rw + rwi) * 128;
              const float2 pa = *reinterpret_cast<const float2*>(part + g * 8 + 2 * t);
              const float2 pb = *reinterpret_cast<const float2*>(part + (g + 8) * 8 + 2 * t);
              acc[h][0] += pa.x, acc[h][1] += pa.y, acc[h][2] += pb.x, acc[h][3] += pb.y;
            }
          }
        }
      }
      if (kwi == 0 && live) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int mm = 2 * t + (i & 1);
          const int row = tile * 16 + g + ((i & 2) ? 8 : 0);
          if (mm < m && row < a.rows) {
            const int aid = list[c0 + mm];
            if constexpr (GATE_UP) {
              const float gate = acc[0][i], up = acc[H - 1][i];
              const float hval = (gate / (1.0f + __expf(-gate))) * up;
              store_f32(a.out, static_cast<int64_t>(aid) * a.rows + row, a.act_dtype, hval);
            } else {
              reinterpret_cast<float*>(a.out)[static_cast<int64_t>(aid) * a.rows + row] = acc[0][i];
            }
          }
        }
      }
    }
  }
  stream::cp_async_wait<0>();
}

// ---- few tokens: the down projection token by token, the combine folded in ----
//
// With a handful of tokens a layer is a chain of launch latencies, not a stream of bytes, and
// almost every assignment has an expert to itself.  One CTA = (16 output rows, one token):
// warp k takes the token's k-th expert -- its 16 rows over the whole reduction axis, with
// h[token, k] as the activation -- and the cross-warp sum that the sliced kernels need anyway
// IS the combine: y[token, rows] = sum over k, in slot order, of p[token, k] * (partial of warp
// k).  No per-assignment fp32 scratch, no combine launch.  A warp's whole share (a few steps)
// is requested before the dependency wait; topk_ids are inputs of the layer, so the addresses
// do not depend on the gate_up launch.  An expert shared by two tokens is read twice (the
// second time from L2): the host takes this path only for token counts at which that is rare.
struct MoeTokenArgs {
  const void* h;           // [assignments, inter] in act_dtype (gate_up's output)
  const uint32_t* packed;  // the down bank, [E * hidden, words_per_row]
  const void* scales;
  const void* offsets;     // may be null
  const int32_t* ids;      // [assignments], global numbers
  int first_expert;        // this call holds experts [first_expert, first_expert + num_experts)
  const float* weights;    // [assignments] routing weights
  void* y;                 // [tokens, hidden]
  int y_dtype, act_dtype, meta_dtype;
  int topk, num_experts;
  int hidden, inter;
  int words_per_row, num_groups;
  int steps;               // padded inter / 128, even, <= kTokenMaxSteps
  int m_stride_u4;
  uint32_t magic;
};
constexpr int kTokenMaxSteps = 8;

template <int BITS>
__host__ __device__ inline size_t moe_token_smem(int steps) {
  const int na = BITS == 8 ? 32 : 16;
  const size_t ring_w = static_cast<size_t>(steps) * 2 * (4 * BITS) * kMoeThreads;
  const size_t ring_m = static_cast<size_t>(steps) * 2 * kMoeThreads;
  const size_t red = static_cast<size_t>(kMoeWarps) * 128 * 4 + kMoeWarps * 4;
  const size_t stride = static_cast<size_t>(steps) * na + 4;
  const size_t stage = steps * 256 + (stride + na) * 16 + steps * 64;
  return ring_w + ring_m + red + kMoeWarps * stage + 16;
}

template <int BITS, bool XBF16>
__global__ void __launch_bounds__(kMoeThreads, 2) moe_down_token_kernel(const __grid_constant__ MoeTokenArgs a) {
  using Plan = MmaPlan<BITS>;
  constexpr int NA = Plan::kARegs;
  constexpr int QU = NA / 4;
  constexpr int UNIT = 4 * BITS;
  constexpr int STEP_BYTES = 4 * BITS * 4;
  constexpr int CH = 2;
  constexpr int STAGE_W = CH * 2 * UNIT * kMoeThreads;
  constexpr int STAGE_M = CH * 2 * kMoeThreads;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int steps = a.steps, nstages = steps / CH;
  unsigned char* ring_w = smem_raw;
  unsigned char* ring_m = ring_w + static_cast<size_t>(nstages) * STAGE_W;
  float* red = reinterpret_cast<float*>(ring_m + static_cast<size_t>(nstages) * STAGE_M);
  float* wts = red + kMoeWarps * 128;
  const int tid = threadIdx.x;
  const int lane = tid & (kWarp - 1);
  const int warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const size_t stage_one = static_cast<size_t>(steps) * 256 + (static_cast<size_t>(a.m_stride_u4) + NA) * 16 +
                           static_cast<size_t>(steps) * 64;
  unsigned char* mine = reinterpret_cast<unsigned char*>(wts + kMoeWarps) + 8 + warp * stage_one;
  mine = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(mine) + 15) & ~static_cast<uintptr_t>(15));
  unsigned short* raw = reinterpret_cast<unsigned short*>(mine);
  uint4* xb = reinterpret_cast<uint4*>(mine + steps * 256);
  float* xsum = reinterpret_cast<float*>(xb + a.m_stride_u4 + NA);
  float* xneg = xsum + steps * 8;

  const int tile = blockIdx.x, token = blockIdx.y;
  const int aid = token * a.topk + warp;
  // (inputs of the whole layer: readable before the dependency wait)
  const int e = warp < a.topk ? __ldg(a.ids + aid) - a.first_expert : -1;
  const bool live = e >= 0 && e < a.num_experts;
  if (lane == 0) wts[warp] = live ? __ldg(a.weights + aid) : 0.0f;
  pdl_launch_dependents();

  // ---- request this warp's whole share: 16 rows of its expert, every step ----
  constexpr int PIECES = 2 * UNIT;
  constexpr int PER_ROW = UNIT / 4;
  constexpr int NSRC = (PIECES + kWarp - 1) / kWarp;
  const bool has_off = a.offsets != nullptr;
  const uint32_t ring_w_s = static_cast<uint32_t>(__cvta_generic_to_shared(ring_w)) + (tid - lane) * UNIT + lane * 16;
  const uint32_t ring_m_s = static_cast<uint32_t>(__cvta_generic_to_shared(ring_m)) + tid * (CH * 2);
  if (live) {
    const int64_t row0 = static_cast<int64_t>(e) * a.hidden + tile * 16;
    const int64_t last = static_cast<int64_t>(e) * a.hidden + a.hidden - 1;
    const bool meta_lane = has_off || (t & 1) == 0;
    const unsigned short* meta_arr = reinterpret_cast<const unsigned short*>((t & 1) ? a.offsets : a.scales);
    const int64_t mrow = min(row0 + g + ((t & 2) ? 8 : 0), last);
    const unsigned short* meta = meta_arr + mrow * a.num_groups;
    for (int s = 0; s < nstages; ++s) {
#pragma unroll
      for (int j = 0; j < CH; ++j) {
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
#pragma unroll
          for (int i = 0; i < NSRC; ++i) {
            const int piece = i * kWarp + lane;
            if ((PIECES % kWarp == 0) || piece < PIECES) {
              const int pg = piece / PER_ROW;
              const int part = piece - pg * PER_ROW;
              const int64_t row = min(row0 + hh * 8 + pg, last);
              const unsigned char* src = reinterpret_cast<const unsigned char*>(a.packed + row * a.words_per_row + part * 4) +
                                         (s * CH + j) * STEP_BYTES;
              stream::cp_async_n<16>(ring_w_s + s * STAGE_W + (j * 2 + hh) * (UNIT * kMoeThreads) + i * (kWarp * 16), src);
            }
          }
        }
      }
      if (meta_lane) stream::cp_async_n<CH * 2>(ring_m_s + s * STAGE_M, meta + s * CH);
      stream::cp_async_commit();
    }
  }
  stage_zero_fill<BITS, false>(1, steps, a.m_stride_u4, xb, xsum, xneg, lane, kWarp);

  pdl_wait_prior_grid();  // h

  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  if (live) {
    GemvArgs stage = {};
    stage.x = static_cast<const unsigned char*>(a.h) + static_cast<size_t>(aid) * a.inter * 2;
    stage.x_dtype = a.act_dtype;
    stage.in_features = a.inter;
    stage.m = 1;
    stage_warp_slice<BITS, XBF16, false>(stage, 0, steps, a.m_stride_u4, raw, xb, xsum, xneg, lane, true);
    const bool mbf = a.meta_dtype == DQ_BF16;
    const uint32_t magic = a.magic;
    const unsigned char* wslot = ring_w + tid * UNIT;
    const unsigned char* mslot = ring_m + (tid & ~3) * (CH * 2);
    const bool b_live = g < 1;
    const uint4* xb_lane = b_live ? xb + t : xb + a.m_stride_u4;
    const int xb_step_u4 = b_live ? QU * 4 : 0;
    const float* xsum_w = xsum + 2 * t;
    const float* xneg_w = xneg + 2 * t;
    for (int s = 0; s < nstages; ++s) {
      moe_wait_pending(nstages - 1 - s);  // groups complete in issue order
      __syncwarp();
      uint32_t mc[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (has_off || (i & 1) == 0) mc[i] = *reinterpret_cast<const uint32_t*>(mslot + i * (CH * 2));
      }
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        const int sl = s * CH + j;
        uint32_t wa[BITS], wb[BITS];
        stream::read_unit<BITS>(wslot + (j * 2 + 0) * (UNIT * kMoeThreads), wa);
        stream::read_unit<BITS>(wslot + (j * 2 + 1) * (UNIT * kMoeThreads), wb);
        uint32_t aa[NA], ab[NA];
        decode_unit<BITS>(wa, magic, aa);
        decode_unit<BITS>(wb, magic, ab);
        unbias_fragments<XBF16, NA>(aa);
        unbias_fragments<XBF16, NA>(ab);
        const uint4* bsrc = xb_lane + sl * xb_step_u4;
        float d[4], f[4];
#pragma unroll
        for (int q = 0; q < QU; ++q) {
          const uint4 b = bsrc[q * 4];
          if (q == 0) {
            mma_16816<XBF16, true>(d, aa[0], ab[0], aa[1], ab[1], b.x, b.y);
            mma_16816<XBF16, true>(f, aa[2], ab[2], aa[3], ab[3], b.z, b.w);
          } else {
            mma_16816<XBF16, false>(d, aa[4 * q], ab[4 * q], aa[4 * q + 1], ab[4 * q + 1], b.x, b.y);
            mma_16816<XBF16, false>(f, aa[4 * q + 2], ab[4 * q + 2], aa[4 * q + 3], ab[4 * q + 3], b.z, b.w);
          }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) d[i] += f[i];
        auto meta_f32 = [&](int i) -> float {
          const uint32_t reg = mc[i];
          if (mbf) return __uint_as_float((j & 1) ? (reg & 0xFFFF0000u) : (reg << 16));
          const __half2 hh2 = *reinterpret_cast<const __half2*>(&reg);
          return (j & 1) ? __high2float(hh2) : __low2float(hh2);
        };
        const float2 xs2 = *reinterpret_cast<const float2*>(xsum_w + sl * 8);
        const float2 xn2 = *reinterpret_cast<const float2*>(xneg_w + sl * 8);
        const float sc_a = meta_f32(0), sc_b = meta_f32(2);
        acc[0] = fmaf(sc_a, d[0] + xn2.x, acc[0]);
        acc[1] = fmaf(sc_a, d[1] + xn2.y, acc[1]);
        acc[2] = fmaf(sc_b, d[2] + xn2.x, acc[2]);
        acc[3] = fmaf(sc_b, d[3] + xn2.y, acc[3]);
        if (has_off) {
          const float of_a = meta_f32(1), of_b = meta_f32(3);
          acc[0] = fmaf(of_a, xs2.x, acc[0]);
          acc[1] = fmaf(of_a, xs2.y, acc[1]);
          acc[2] = fmaf(of_b, xs2.x, acc[2]);
          acc[3] = fmaf(of_b, xs2.y, acc[3]);
        }
      }
      wslot += STAGE_W;
      mslot += STAGE_M;
    }
  }
  // ---- the combine: the token is column 0 of the accumulator (lanes t == 0: rows g and g + 8) ----
  if (t == 0) {
    red[warp * 128 + g] = acc[0];
    red[warp * 128 + 8 + g] = acc[2];
  }
  __syncthreads();
  if (tid < 16) {
    const int row = tile * 16 + tid;
    if (row < a.hidden) {
      float sum = 0.0f;
      for (int k = 0; k < a.topk; ++k) sum = fmaf(wts[k], red[k * 128 + tid], sum);  // slot order, like moe_combine_kernel
      store_f32(a.y, static_cast<int64_t>(token) * a.hidden + row, a.y_dtype, sum);
    }
  }
}

__global__ void moe_combine_kernel(const float* __restrict__ d, const float* __restrict__ w,
                                   const int32_t* __restrict__ ids, int first_expert, int tokens, int topk, int hidden,
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
      const int e = ids[aid] - first_expert;
      if (e >= 0 && e < num_experts) {
        acc = fmaf(w[aid], d[static_cast<int64_t>(aid) * hidden + col], acc);
      }
    }
    store_f32(y, i, y_dtype, acc);
  }
}

struct ScratchLayout {
  size_t h, d, total;
};

ScratchLayout scratch_layout(int64_t tokens, int64_t topk, int64_t hidden, int64_t inter, int act_bytes) {
  auto up = [](size_t v) { return (v + 255) / 256 * 256; };
  ScratchLayout l = {};
  const size_t assignments = static_cast<size_t>(tokens * topk);
  size_t at = 0;
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

// Launch-shape overrides of the MoE launcher (tuning builds only, see tuning_int; 0 = the built-in choice).
#define DQ_MOE_KNOB(var, name) const int var = ::dq::tuning_int(name)

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
  note_kernel("moe_grouped_kernel");
  return DQ_OK;
}

template <int BITS, int CH, bool GATE_UP>
int32_t launch_grouped(MoeArgs a, int slots, cudaStream_t stream) {
  const DeviceInfo* dev = device_info();
  if (dev == nullptr) return DQ_ERR_CUDA;
  DQ_MOE_KNOB(force_nb, "DQ_B200_MOE_NB");
  DQ_MOE_KNOB(force_x_both, "DQ_B200_MOE_GRID_X");
  DQ_MOE_KNOB(force_x_one, GATE_UP ? "DQ_B200_MOE_GRID_X_UP" : "DQ_B200_MOE_GRID_X_DOWN");
  const int force_x = force_x_one > 0 ? force_x_one : force_x_both;
  // ring: as deep as keeps two CTAs on an SM (one, if a single stage is that large)
  a.nb = 1;
  const size_t one = moe_smem<BITS, CH>(a, GATE_UP).total;
  const size_t stage = static_cast<size_t>(CH) * 2 * kMoeThreads * (4 * BITS) + static_cast<size_t>(CH) * 2 * kMoeThreads;
  const size_t fixed = one - stage;
  // Two register builds, like the tiled dense kernel: three CTAs per SM (80 registers) when a
  // ring of two stages still fits beside the staged activation, else two (128 registers).
  DQ_MOE_KNOB(force_ctas, "DQ_B200_MOE_CTAS");
  const size_t per_sm = 228 * 1024, reserve = 1024;
  int ctas = force_ctas == 2 || force_ctas == 3 ? force_ctas : (a.tokens >= 32 ? 3 : 2);
  if (ctas == 3 && fixed + 2 * stage > per_sm / 3 - reserve) ctas = 2;
  size_t budget = per_sm / ctas - reserve;
  if (fixed + 2 * stage > budget) budget = static_cast<size_t>(dev->max_smem_optin);
  if (fixed + stage > budget) {
    return fail(DQ_ERR_UNSUPPORTED, "moe_gemv: in_features=%d needs %zu bytes of shared memory", a.in_features,
                fixed + stage);
  }
  // Two stages: measured faster than any deeper ring at every token count (16 tokens: 71 us
  // against 74 with four stages and 92 with six, which leaves one CTA per SM) -- a CTA's whole
  // share is a few dozen steps, and what a deeper ring requests at once only queues.
  a.nb = static_cast<int>(std::max<size_t>(1, std::min<size_t>(2, (budget - fixed) / stage)));
  if (force_nb > 0) a.nb = static_cast<int>(std::min<size_t>(force_nb, (static_cast<size_t>(dev->max_smem_optin) - fixed) / stage));
  const size_t smem = moe_smem<BITS, CH>(a, GATE_UP).total;
  // CTAs per expert (measured on B200, Qwen3-30B-A3B shape, 1..64 tokens).  Every CTA pays
  // for routing and for staging the activation rows of its expert, so a CTA gets at least
  // about a dozen steps per warp to do; beyond that, more and smaller CTAs even out the
  // experts' different loads.  With so few tokens that this leaves SMs idle, the grid is
  // widened to one full wave over the experts expected to be active
  // (E * (1 - (1 - 1/E)^A) under uniform routing).
  const int tiles = (a.rows + 15) / 16;
  const int items = static_cast<int>(ceil_div(tiles, a.rw));
  const double e_count = a.num_experts;
  const double active = a.by_assignment ? static_cast<double>(a.assignments)
                                        : std::max(1.0, e_count * (1.0 - std::pow(1.0 - 1.0 / e_count, a.assignments)));
  const int steps_per_item = (GATE_UP ? 2 : 1) * a.spw;
  const int items_per_cta = std::max(1, static_cast<int>(ceil_div(12, steps_per_item)));
  const int one_wave = static_cast<int>(std::ceil(static_cast<double>(ctas) * dev->sm_count / active));
  int grid_x = static_cast<int>(std::min<int64_t>(items, std::max<int64_t>(ceil_div(items, items_per_cta), one_wave)));
  grid_x = static_cast<int>(ceil_div(items, ceil_div(items, grid_x)));  // no CTA with one item more than the others need
  if (force_x > 0) grid_x = std::min(force_x, items);
  const dim3 grid(static_cast<unsigned>(grid_x), static_cast<unsigned>(slots));
  const char* what = GATE_UP ? "moe_gemv(gate_up)" : "moe_gemv(down)";
  if (a.act_dtype == DQ_BF16) {
    return ctas == 3 ? launch_pdl(moe_grouped_kernel<BITS, true, CH, GATE_UP, 3>, grid, kMoeThreads, smem, stream, a, what)
                     : launch_pdl(moe_grouped_kernel<BITS, true, CH, GATE_UP, 2>, grid, kMoeThreads, smem, stream, a, what);
  }
  return ctas == 3 ? launch_pdl(moe_grouped_kernel<BITS, false, CH, GATE_UP, 3>, grid, kMoeThreads, smem, stream, a, what)
                   : launch_pdl(moe_grouped_kernel<BITS, false, CH, GATE_UP, 2>, grid, kMoeThreads, smem, stream, a, what);
}

template <bool GATE_UP>
int32_t launch_bank(const dq_weight& w, const dq_geometry& g, MoeArgs a, int slots, cudaStream_t stream) {
  a.packed = static_cast<const uint32_t*>(w.packed);
  a.scales = w.scales;
  a.offsets = w.offsets;
  a.meta_dtype = w.meta_dtype;
  a.words_per_row = g.words_per_row;
  a.num_groups = g.num_groups;
  a.in_features = g.in_features;
  a.steps = g.words_per_row / (4 * w.bits);
  // 8 warps: kw slices of the reduction axis (each an even number of steps), the other
  // warps take neighbouring row tiles.
  DQ_MOE_KNOB(force_kw, "DQ_B200_MOE_KW");
  // Measured on B200 (Qwen3-30B-A3B shape): up to three tokens a layer is a chain of
  // latencies and four slices are fastest (18.4 us against 22.2 with two at one token); from
  // four tokens on, whole rows per warp and no cross-warp sum at all (16 tokens: 68 us
  // against 78 with two slices; 64 tokens: 107 against 124).
  const int want_kw = a.tokens <= 3 ? 4 : 1;
  int kw = 1;
  while (kw < want_kw && a.steps % (kw * 2) == 0 && (a.steps / (kw * 2)) % 2 == 0) kw *= 2;
  if (force_kw > 0 && a.steps % force_kw == 0) kw = force_kw;
  a.kw = kw;
  a.rw = kMoeWarps / kw;
  a.spw = a.steps / kw;
  const bool meta_words = a.num_groups % 2 == 0 && reinterpret_cast<uintptr_t>(a.scales) % 4 == 0 &&
                          reinterpret_cast<uintptr_t>(a.offsets) % 4 == 0;
  const bool pairs = a.spw % 2 == 0 && meta_words;  // stages of two steps; else single steps
  const int aregs = w.bits == 8 ? 32 : 16;
  a.m_stride_u4 = a.steps * aregs + 4;
  a.magic = a.act_dtype == DQ_BF16 ? 0x43004300u : 0x64006400u;
  switch (w.bits) {
    case 2:
      return pairs ? launch_grouped<2, 2, GATE_UP>(a, slots, stream) : launch_grouped<2, 1, GATE_UP>(a, slots, stream);
    case 3:
      return pairs ? launch_grouped<3, 2, GATE_UP>(a, slots, stream) : launch_grouped<3, 1, GATE_UP>(a, slots, stream);
    case 4:
      return pairs ? launch_grouped<4, 2, GATE_UP>(a, slots, stream) : launch_grouped<4, 1, GATE_UP>(a, slots, stream);
    default:
      return pairs ? launch_grouped<8, 2, GATE_UP>(a, slots, stream) : launch_grouped<8, 1, GATE_UP>(a, slots, stream);
  }
}

// *taken stays false (nothing launched) when the layer does not qualify: more tokens than the
// threshold, more than eight experts per token, a reduction axis longer than kTokenMaxSteps
// steps or with an odd number of them, metadata rows that are not whole 32-bit words.
int32_t launch_down_by_token(const dq_weight& w, const dq_geometry& g, const MoeArgs& base, const float* topk_w,
                             const void* h, void* y, int y_dtype, int hidden, int inter, cudaStream_t stream,
                             bool* taken) {
  *taken = false;
  const DeviceInfo* dev = device_info();
  if (dev == nullptr) return DQ_ERR_CUDA;
  // Up to this many tokens nearly every assignment has its expert to itself (128 experts,
  // top-8: 30 distinct experts for 32 assignments at four tokens), so reading per assignment
  // costs no extra bytes and saves the combine launch.  Measured with the threshold at 8 and 16
  // (us per layer): 5 tokens 35.9 against 34.9 with three launches, 6 tokens 38.7 against 41.2,
  // 8 tokens 52.6 against 41.5, 16 tokens 95.8 against 71.2.
  const int max_tokens = tuning_int("DQ_B200_MOE_BY_TOKEN_MAX", 4);
  const int steps = g.words_per_row / (4 * w.bits);
  if (base.tokens > max_tokens || base.topk > kMoeWarps || steps > kTokenMaxSteps || steps % 2 != 0 || steps == 0) {
    return DQ_OK;
  }
  if (g.num_groups != steps || g.num_groups % 2 != 0 || reinterpret_cast<uintptr_t>(w.scales) % 4 != 0 ||
      reinterpret_cast<uintptr_t>(w.offsets) % 4 != 0) {
    return DQ_OK;
  }
  MoeTokenArgs t = {};
  t.h = h;
  t.packed = static_cast<const uint32_t*>(w.packed);
  t.scales = w.scales;
  t.offsets = w.offsets;
  t.ids = base.ids;
  t.first_expert = base.first_expert;
  t.weights = topk_w;
  t.y = y;
  t.y_dtype = y_dtype;
  t.act_dtype = base.act_dtype;
  t.meta_dtype = w.meta_dtype;
  t.topk = base.topk;
  t.num_experts = base.num_experts;
  t.hidden = hidden;
  t.inter = inter;
  t.words_per_row = g.words_per_row;
  t.num_groups = g.num_groups;
  t.steps = steps;
  t.m_stride_u4 = steps * (w.bits == 8 ? 32 : 16) + 4;
  t.magic = base.act_dtype == DQ_BF16 ? 0x43004300u : 0x64006400u;
  const dim3 grid(static_cast<unsigned>(ceil_div(hidden, 16)), static_cast<unsigned>(base.tokens));
  auto run = [&](auto kernel, size_t smem) -> int32_t {
    if (smem > static_cast<size_t>(dev->max_smem_optin)) return DQ_OK;  // not taken
    if (smem > 48 * 1024) {
      DQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kMoeThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    DQ_CUDA(cudaLaunchKernelEx(&cfg, kernel, t));
    DQ_CHECK_LAUNCH("moe_gemv(down by token)");
    note_kernel("moe_down_token_kernel");
    *taken = true;
    return DQ_OK;
  };
  const bool xbf = base.act_dtype == DQ_BF16;
  switch (w.bits) {
    case 2:
      return xbf ? run(moe_down_token_kernel<2, true>, moe_token_smem<2>(steps)) : run(moe_down_token_kernel<2, false>, moe_token_smem<2>(steps));
    case 3:
      return xbf ? run(moe_down_token_kernel<3, true>, moe_token_smem<3>(steps)) : run(moe_down_token_kernel<3, false>, moe_token_smem<3>(steps));
    case 4:
      return xbf ? run(moe_down_token_kernel<4, true>, moe_token_smem<4>(steps)) : run(moe_down_token_kernel<4, false>, moe_token_smem<4>(steps));
    default:
      return xbf ? run(moe_down_token_kernel<8, true>, moe_token_smem<8>(steps)) : run(moe_down_token_kernel<8, false>, moe_token_smem<8>(steps));
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
      dq::scratch_layout(tokens, topk, hidden, inter, dq::dtype_size(act_dtype)).total);
  return DQ_OK;
}

int32_t dq_moe_gemv(const void* x, int32_t x_dtype, int64_t tokens, const int32_t* topk_ids, const float* topk_w,
                    int64_t topk, int64_t num_experts, const dq_weight* gate_up, const dq_weight* down,
                    int64_t hidden, int64_t inter, void* y, int32_t y_dtype, void* scratch, int64_t scratch_bytes,
                    void* stream) {
  return dq_moe_gemv_shard(x, x_dtype, tokens, topk_ids, topk_w, topk, 0, num_experts, gate_up, down, hidden, inter, y,
                           y_dtype, scratch, scratch_bytes, stream);
}

int32_t dq_moe_gemv_shard(const void* x, int32_t x_dtype, int64_t tokens, const int32_t* topk_ids, const float* topk_w,
                          int64_t topk, int64_t first_expert, int64_t num_experts, const dq_weight* gate_up,
                          const dq_weight* down, int64_t hidden, int64_t inter, void* y, int32_t y_dtype, void* scratch,
                          int64_t scratch_bytes, void* stream) {
  DQ_REQUIRE(first_expert >= 0 && first_expert < (1LL << 30), "moe_gemv: first_expert=%lld out of range",
             static_cast<long long>(first_expert));
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
      reinterpret_cast<uintptr_t>(gate_up->packed) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(down->packed) % 16 != 0 || (g_gu.words_per_row * 4) % 16 != 0 ||
      (g_dn.words_per_row * 4) % 16 != 0) {
    return dq::fail(DQ_ERR_UNSUPPORTED,
                    "moe_gemv: this build handles fp16/bf16 activations and metadata, 128-value groups and "
                    "16-byte aligned packed rows");
  }

  auto s = static_cast<cudaStream_t>(stream);
  const dq::ScratchLayout lay = dq::scratch_layout(tokens, topk, hidden, inter, dq::dtype_size(x_dtype));
  auto* base = static_cast<unsigned char*>(scratch);
  const int assignments = static_cast<int>(tokens * topk);
  const int slots = static_cast<int>(std::min<int64_t>(num_experts, assignments));
  dq::MoeArgs a = {};
  a.ids = topk_ids;
  a.first_expert = static_cast<int>(first_expert);
  a.assignments = assignments;
  a.num_experts = static_cast<int>(num_experts);
  // Activation rows staged at once: the eight columns of one mma.  An expert with more tokens
  // than that takes another pass over its (L2-resident) rows.
  a.m_cap = static_cast<int>(std::min<int64_t>(8, tokens));
  {
    DQ_MOE_KNOB(force_m_cap, "DQ_B200_MOE_M_CAP");
    if (force_m_cap >= 1 && force_m_cap <= 8) a.m_cap = static_cast<int>(std::min<int64_t>(force_m_cap, tokens));
  }
  a.topk = static_cast<int>(topk);
  a.tokens = static_cast<int>(tokens);
  a.act_dtype = x_dtype;
  // gate_up: x -> h
  a.act = x;
  a.out = base + lay.h;
  a.rows = static_cast<int>(inter);
  // Few tokens (the threshold of the by-token down projection): a slot per assignment, so no CTA
  // has to work out the routing before it can request its weights.
  a.by_assignment = tokens <= dq::tuning_int("DQ_B200_MOE_BY_TOKEN_MAX", 4) ? 1 : 0;
  if (const int32_t rc = dq::launch_bank<true>(*gate_up, g_gu, a, a.by_assignment ? assignments : slots, s)) return rc;
  a.by_assignment = 0;
  // Few tokens: the down projection token by token with the combine folded in (two launches a
  // layer instead of three).  Measured on B200, Qwen3-30B-A3B shape: see launch_down_by_token.
  {
    bool taken = false;
    if (const int32_t rc = dq::launch_down_by_token(*down, g_dn, a, topk_w, base + lay.h, y, y_dtype,
                                                    static_cast<int>(hidden), static_cast<int>(inter), s, &taken)) {
      return rc;
    }
    if (taken) return DQ_OK;
  }
  // down: h -> d
  a.act = base + lay.h;
  a.out = base + lay.d;
  a.rows = static_cast<int>(hidden);
  if (const int32_t rc = dq::launch_bank<false>(*down, g_dn, a, slots, s)) return rc;
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
                               topk_ids, static_cast<int>(first_expert), static_cast<int>(tokens), static_cast<int>(topk), static_cast<int>(hidden),
                               static_cast<int>(num_experts), y, y_dtype));
    DQ_CHECK_LAUNCH("moe_gemv(combine)");
    dq::note_kernel("moe_combine_kernel");
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
