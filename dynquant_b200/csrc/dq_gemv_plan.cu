// Whole-step plans: every packed GEMV of a decode step in ONE persistent kernel.
//
// A decode step of a packed model is a chain of small GEMVs (1-13 MB of weights each), every
// one waiting for the activation the previous one produced.  Launched one kernel per link the
// chain costs 4-7 us per link in fixed latencies (launch hand-over, cold instruction cache,
// slowest-CTA tail) while the bytes of a link are worth 0.2-2 us: the reference measures the
// same thing one level up, 20-45 us of host time per module around single-digit-microsecond
// kernels (experiments/four_point/RESULTS.md:884-906, runtime/ops.py:184-231 called once per
// module).  Here the job list of dq_gemv_sequence is compiled once into a device table and a
// single grid of one CTA per SM walks it:
//
//   * the table is a list of STAGES: up to four consecutive jobs that read the same
//     activation (q/k/v, gate/up) form one stage; the CTAs of the grid are split among a
//     stage's jobs in proportion to their work, and inside a job a CTA takes row-tile items
//     cta, cta + n, ... exactly like the tiled kernel (dq_gemv_mma_tile.cuh): 16 warps =
//     rw row tiles x kw slices of the reduction axis, slices summed in a fixed order;
//   * weights never depend on data, so every warp streams its own sequence of weight slots
//     (stage after stage, item after item) through a private cp.async ring that runs `nb`
//     slots AHEAD of its arithmetic, across stage boundaries: while stage j computes, the
//     weights of stages j+1.. are already landing in shared memory;
//   * stage j+1 may read its activation only when stage j has stored all of its outputs: every
//     CTA that worked on stage j adds 1 to the stage's counter (release) after its last store,
//     and the warps that stage the next activation poll that counter (acquire) -- a BOUNDED
//     spin.  When the bound runs out the kernel writes a status word, drains its copies and
//     returns; the host reports DQ_ERR_DEVICE.  Nothing ever spins without a limit;
//   * the last CTA to leave zeroes the counters, so a plan can be launched again (and
//     replayed from a CUDA graph) without any host-side reset.
//
// The grid must be resident at once (one CTA per SM, checked with the occupancy API at build
// time); if it is not -- another kernel holds SMs for longer than the spin bound -- the waits
// run out and the launch fails cleanly instead of hanging.
//
// Arithmetic is that of the other tensor-core kernels (dq_mma_plan.cuh, dq_mma_stage.cuh):
// results are bit-identical run to run, and identical to what a chain of separate launches of
// the tiled kernel with the same slicing would produce.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "dq_gemv.cuh"
#include "dq_gemv_mma_stream.cuh"
#include "dq_mma_plan.cuh"
#include "dq_mma_stage.cuh"

namespace dq {
namespace plank {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * kWarp;
constexpr int kTileRows = 16;
constexpr int kStepValues = 128;
constexpr int kSlotWeights = 2048;                  // bytes of packed words in one ring slot
constexpr int kSlotBytes = kSlotWeights + 256;      // + 8 bytes of scales/offsets per lane
constexpr int kMaxStageJobs = 4;
constexpr int kRedFloats = 2 * kWarps * 128;        // two buffers of one 16 x 8 partial per warp
constexpr int kDefaultSpinLimit = 1 << 21;          // polls of an L2 word: about a second

// One matrix of a stage.
struct PJob {
  const uint32_t* packed;
  const void* scales;
  const void* offsets;  // may be null
  const void* bias;     // may be null
  void* out;
  int64_t out_stride;
  int64_t out_col0;
  int rows, words_per_row, num_groups, bits;
  int tiles;      // ceil(rows / 16)
  int items;      // ceil(tiles / rw)
  int cta_begin;  // CTAs [cta_begin, cta_begin + cta_count) of the grid work on this job
  int cta_count;
};

// Up to four jobs that read one activation.
struct PStage {
  const void* x;
  int m, in_features, steps;
  int meta_bf16, out_dtype;
  int kw, spw;       // 16 warps = (16 / kw) row tiles x kw slices of `spw` steps
  int cs;            // steps per ring slot (1, 2 or 4; divides spw)
  int job_begin, njobs;
  int wait_stage;    // stage whose completion releases x, or -1
  int wait_target;   // value its counter reaches when complete
  int signal;        // 1: a later stage waits for this one
  int pad;
};

struct PlanParams {
  const PStage* stages;
  const PJob* jobs;
  unsigned int* counters;  // [nstages] completion counters, then [nstages] = CTAs that left, [nstages + 1] = status
  int nstages;
  int first_stage, last_stage;  // this launch runs stages [first_stage, last_stage)
  int njobs;
  int tables_in_smem;  // 1: every CTA keeps its own copy of the two tables in shared memory
  int nb;          // ring slots per warp
  int spin_limit;
  int area_bytes;  // bytes of the staged-activation area (the tables follow it in shared memory)
  uint32_t magic;
#ifdef DQ_PLAN_TRACE
  unsigned long long* trace;  // [nstages][2 CTAs][8] device timestamps (diagnostic builds only)
  int debug_flags;            // 1: arrive without fence/release, 2: poll with relaxed loads, 4: no waits (timing experiments only)
#endif  // 16-bit magic constant in both halves; a parameter so it stays a register operand
};

__device__ __forceinline__ unsigned int ld_acquire(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned int ld_relaxed(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_add(unsigned int* p, unsigned int v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

#ifdef DQ_PLAN_TRACE
__device__ int g_debug_relaxed_poll = 0;
#endif

// Bounded wait for *ctr >= target.  False when the bound ran out or another CTA already failed.
__device__ __forceinline__ bool wait_counter(const unsigned int* ctr, unsigned int target, const unsigned int* status,
                                             int limit) {
  for (int it = 0; it < limit; ++it) {
#ifdef DQ_PLAN_TRACE
    if (g_debug_relaxed_poll) {
      if (ld_relaxed(ctr) >= target) return true;
      continue;
    }
#endif
    if (ld_acquire(ctr) >= target) return true;
    if ((it & 63) == 63 && ld_relaxed(status) != 0u) return false;
  }
  return false;
}

#ifdef DQ_PLAN_TRACE
__device__ __forceinline__ void trace_point(const PlanParams& P, int stage, int point) {
  if (P.trace != nullptr && threadIdx.x == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1)) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    P.trace[(static_cast<size_t>(stage) * 2 + (blockIdx.x == 0 ? 0 : 1)) * 8 + point] = t;
  }
}
#define DQ_TRACE(stage, point) trace_point(P, stage, point)
#else
#define DQ_TRACE(stage, point)
#endif

__device__ __forceinline__ void wait_pending(int n) {
  switch (n) {
    case 0: stream::cp_async_wait<0>(); break;
    case 1: stream::cp_async_wait<1>(); break;
    case 2: stream::cp_async_wait<2>(); break;
    case 3: stream::cp_async_wait<3>(); break;
    case 4: stream::cp_async_wait<4>(); break;
    default: stream::cp_async_wait<5>(); break;
  }
}

// The arithmetic of one ring slot: `cs` steps of one 16-row tile against the staged activation.
template <int BITS, bool XBF16>
__device__ __forceinline__ void consume_slot(const unsigned char* slot, int cs, int hw0, bool has_off, bool mbf,
                                             uint32_t magic, const uint4* bsrc, int xb_step_u4, const float* xs,
                                             const float* xn, int lane, float* acc) {
  using Plan = MmaPlan<BITS>;
  constexpr int NA = Plan::kARegs;
  constexpr int QU = NA / 4;
  constexpr int UNIT = 4 * BITS;
  // scales / offsets of rows g and g + 8: arrays 0..3 of this lane's quad, 8 bytes apart
  const unsigned char* mq = slot + kSlotWeights + (lane & ~3) * 8;
  uint2 mc[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    mc[i] = make_uint2(0u, 0u);
    if (has_off || (i & 1) == 0) mc[i] = *reinterpret_cast<const uint2*>(mq + i * 8);
  }
  const unsigned char* w = slot + lane * UNIT;
#pragma unroll 1
  for (int j = 0; j < cs; ++j) {
    uint32_t wa[BITS], wb[BITS];
    stream::read_unit<BITS>(w, wa);
    stream::read_unit<BITS>(w + kWarp * UNIT, wb);
    uint32_t aa[NA], ab[NA];
    decode_unit<BITS>(wa, magic, aa);
    decode_unit<BITS>(wb, magic, ab);
    unbias_fragments<XBF16, NA>(aa);
    unbias_fragments<XBF16, NA>(ab);
    // two accumulators halve the chain of dependent mma
    float d[4], e[4];
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
#pragma unroll
    for (int i = 0; i < 4; ++i) d[i] += e[i];
    const int hw = hw0 + j;
    auto meta_f32 = [&](int i) -> float {
      const uint32_t reg = (hw & 2) ? mc[i].y : mc[i].x;
      if (mbf) return __uint_as_float((hw & 1) ? (reg & 0xFFFF0000u) : (reg << 16));
      const __half2 h = *reinterpret_cast<const __half2*>(&reg);
      return (hw & 1) ? __high2float(h) : __low2float(h);
    };
    const float2 xs2 = *reinterpret_cast<const float2*>(xs);
    const float2 xn2 = *reinterpret_cast<const float2*>(xn);
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
    w += 2 * kWarp * UNIT;
    bsrc += xb_step_u4;
    xs += 8;
    xn += 8;
  }
}

template <bool XBF16>
__device__ __forceinline__ void stage_for_bits(int bits, const GemvArgs& a, int steps, int m_stride_u4, uint4* xb,
                                               float* xsum, float* xneg, int tid) {
  switch (bits) {
    // (the zero fragments of absent rows are already written: prefilled)
    case 2: stage_units<2, XBF16, false>(a, 0, steps, m_stride_u4, xb, xsum, xneg, tid, kThreads, nullptr, true); break;
    case 3: stage_units<3, XBF16, false>(a, 0, steps, m_stride_u4, xb, xsum, xneg, tid, kThreads, nullptr, true); break;
    case 4: stage_units<4, XBF16, false>(a, 0, steps, m_stride_u4, xb, xsum, xneg, tid, kThreads, nullptr, true); break;
    default: stage_units<8, XBF16, false>(a, 0, steps, m_stride_u4, xb, xsum, xneg, tid, kThreads, nullptr, true); break;
  }
}

template <bool XBF16>
__global__ void __launch_bounds__(kThreads, 1) gemv_plan_kernel(const __grid_constant__ PlanParams P) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int s_abort;

  const int tid = threadIdx.x;
  const int lane = tid & (kWarp - 1);
  const int warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int cta = blockIdx.x;
  const int nb = P.nb;
  const uint32_t magic = P.magic;
  unsigned int* const status = P.counters + P.nstages + 1;

  unsigned char* const ring = smem + warp * nb * kSlotBytes;  // this warp's slots; nobody else touches them
  float* const red = reinterpret_cast<float*>(smem + kWarps * nb * kSlotBytes);
  unsigned char* const area = reinterpret_cast<unsigned char*>(red + kRedFloats);
  if (tid == 0) s_abort = 0;

  // The stage and job tables are read at every stage and item boundary, by both cursors: from
  // shared memory when they fit (a copy per CTA), so that no L2 round trip sits between two stages.
  const PStage* stages = P.stages;
  const PJob* jobs = P.jobs;
  if (P.tables_in_smem) {
    unsigned char* tables = area + P.area_bytes;
    const int stage_words = P.nstages * static_cast<int>(sizeof(PStage) / 4);
    const int job_words = P.njobs * static_cast<int>(sizeof(PJob) / 4);
    uint32_t* dst_s = reinterpret_cast<uint32_t*>(tables);
    uint32_t* dst_j = dst_s + stage_words;
    const uint32_t* src_s = reinterpret_cast<const uint32_t*>(P.stages);
    const uint32_t* src_j = reinterpret_cast<const uint32_t*>(P.jobs);
    for (int i = tid; i < stage_words; i += kThreads) dst_s[i] = src_s[i];
    for (int i = tid; i < job_words; i += kThreads) dst_j[i] = src_j[i];
    stages = reinterpret_cast<const PStage*>(dst_s);
    jobs = reinterpret_cast<const PJob*>(dst_j);
    __syncthreads();
  }

  // ---- prefetch cursor: this warp's sequence of (stage, item, chunk) slots, nb ahead ----
  int pf_stage = P.first_stage - 1, pf_item = 0, pf_items = 0, pf_stride = 1, pf_job = 0;
  int pf_chunk = 0, pf_nchunks = 1, pf_cs = 1, pf_bits = 2, pf_step0 = 0, pf_rw = 1, pf_rwi = 0;
  bool pf_valid = false, pf_meta_live = false;
  bool pf_seek_pending = false;  // the cursor finished an item and has not looked for the next one yet
  const unsigned char* pf_base = nullptr;  // the job's packed words
  uint32_t pf_off[4] = {0u, 0u, 0u, 0u};   // byte offset of each 16-byte piece this lane copies, at step 0 of the row
  uint32_t pf_piece[4] = {0u, 0u, 0u, 0u}; // which (row, part) of a tile's step each of them is, at this stage's width
  int pf_pieces = 0;                       // how many of them are real
  const unsigned short* pf_meta = nullptr; // this lane's metadata array at its row
  int pf_slot = 0;
  const uint32_t ring_s = static_cast<uint32_t>(__cvta_generic_to_shared(ring));

  auto pf_seek = [&]() {
    pf_valid = false;
#pragma unroll 1
    while (true) {
      if (pf_stage >= P.first_stage && pf_item < pf_items) {
        const PJob& J = jobs[pf_job];
        const int tile = pf_item * pf_rw + pf_rwi;
        const int tiles = J.tiles;
        if (tile < tiles) {
          const int rows = J.rows;
          const uint32_t row_bytes = static_cast<uint32_t>(J.words_per_row) * 4u;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            // pf_piece: (row of the tile << 8 | byte offset inside the row's step), resolved once per stage
            const int row = min(tile * kTileRows + static_cast<int>(pf_piece[i] >> 8), rows - 1);
            pf_off[i] = static_cast<uint32_t>(row) * row_bytes + (pf_piece[i] & 0xffu);
          }
          pf_base = reinterpret_cast<const unsigned char*>(reinterpret_cast<unsigned long long>(J.packed));
          const void* arr = (t & 1) ? reinterpret_cast<const void*>(reinterpret_cast<unsigned long long>(J.offsets))
                                    : reinterpret_cast<const void*>(reinterpret_cast<unsigned long long>(J.scales));
          pf_meta_live = arr != nullptr;
          const int mrow = min(tile * kTileRows + g + ((t & 2) ? 8 : 0), rows - 1);
          pf_meta = reinterpret_cast<const unsigned short*>(arr) + static_cast<int64_t>(mrow) * J.num_groups;
          pf_chunk = 0;
          pf_valid = true;
          return;
        }
        pf_item = pf_items;  // rows beyond the last tile: nothing further in this job for this warp
      }
      if (++pf_stage >= P.last_stage) {
        pf_stage = P.last_stage;
        pf_items = 0;
        return;
      }
      const PStage& S = stages[pf_stage];
      pf_items = 0;
      const int jb = S.job_begin, nj = S.njobs;
#pragma unroll 1
      for (int j = 0; j < nj; ++j) {
        const PJob& J = jobs[jb + j];
        const int cb = J.cta_begin, cc = J.cta_count;
        if (cta >= cb && cta < cb + cc) {
          const int kw = S.kw;
          pf_job = jb + j;
          pf_items = J.items;
          pf_item = cta - cb;
          pf_stride = cc;
          pf_bits = J.bits;
          pf_pieces = 0;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int pc = lane + i * kWarp;  // 16-byte pieces of one step of 16 rows: 16 * bits of them
            if (pc < 16 * pf_bits) {
              const int r = pc / pf_bits;
              pf_piece[i] = (static_cast<uint32_t>(r) << 8) | static_cast<uint32_t>((pc - r * pf_bits) * 16);
              pf_pieces = i + 1;
            }
          }
          pf_cs = S.cs;
          const int spw = S.spw;
          pf_nchunks = spw / pf_cs;
          pf_rw = kWarps / kw;
          pf_rwi = warp / kw;
          pf_step0 = (warp - pf_rwi * kw) * spw;
        }
      }
    }
  };

  // Request the slot at the cursor (if any) into ring slot pf_slot, move the cursor on.
  // The search for the next item reads the tables and resolves this lane's source addresses: a
  // few hundred instructions.  It is left pending when an item ends and done at the next
  // request -- or earlier, at a point off the chain between two stages (pf_catch_up).
  auto pf_catch_up = [&]() {
    if (pf_seek_pending) {
      pf_seek_pending = false;
      pf_seek();
    }
  };
  auto pf_issue = [&]() {
    pf_catch_up();
    if (pf_valid) {
      const uint32_t dst = ring_s + pf_slot * kSlotBytes;
      const int step_bytes = 16 * pf_bits;
      const int first = pf_step0 + pf_chunk * pf_cs;  // first step of the slot
      const unsigned char* src0 = pf_base + static_cast<uint32_t>(first * step_bytes);
      const int slot_step = 16 * step_bytes;  // bytes of one step of 16 rows in the slot
#pragma unroll 1
      for (int j = 0; j < pf_cs; ++j) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (i < pf_pieces) {
            stream::cp_async_n<16>(dst + j * slot_step + (lane + i * kWarp) * 16, src0 + pf_off[i] + j * step_bytes);
          }
        }
      }
      if (pf_meta_live) {
        // the slot's groups, as whole 4-byte words: one word when cs <= 2, two when cs == 4
        const unsigned short* msrc = pf_meta + (first & ~1);
        if (pf_cs == 4) {
          stream::cp_async_n<8>(dst + kSlotWeights + lane * 8, msrc);
        } else {
          stream::cp_async_n<4>(dst + kSlotWeights + lane * 8, msrc);
        }
      }
      if (++pf_chunk == pf_nchunks) {
        pf_item += pf_stride;
        pf_valid = false;
        pf_seek_pending = true;
      }
    }
    stream::cp_async_commit();  // an empty group keeps the wait arithmetic uniform
    if (++pf_slot == nb) pf_slot = 0;
  };

  pf_seek_pending = true;  // (the first request looks for the first item)
  for (int i = 0; i < nb; ++i) pf_issue();
  __syncthreads();  // s_abort is initialised

  int rd_slot = 0;
  int parity = 0;
  bool aborted = false;

#pragma unroll 1
  for (int s = P.first_stage; s < P.last_stage && !aborted; ++s) {
    const PStage& S = stages[s];
    // ---- which job of the stage is this CTA's ----
    const int jb = S.job_begin, nj = S.njobs;
    int my_job = -1, cta_rel = 0, cta_count = 1;
    for (int j = 0; j < nj; ++j) {
      const PJob& J = jobs[jb + j];
      const int cb = J.cta_begin, cc = J.cta_count;
      if (cta >= cb && cta < cb + cc) {
        my_job = jb + j;
        cta_rel = cta - cb;
        cta_count = cc;
      }
    }
    if (my_job < 0) continue;  // nothing of this stage is ours (and the prefetch cursor skipped it too)
    DQ_TRACE(s, 0);
    const PJob& J = jobs[my_job];
    const int bits = J.bits;
    const int items = J.items;
    const int tiles = J.tiles;
    const int kw = S.kw, spw = S.spw, cs = S.cs;
    const int rw = kWarps / kw;
    const int rwi = warp / kw;
    const int kwi = warp - rwi * kw;
    const int nchunks = spw / cs;
    const int steps = S.steps;
    const int m = S.m;
    const bool mbf = S.meta_bf16 != 0;
    GemvArgs a = {};
    a.x = reinterpret_cast<const void*>(reinterpret_cast<unsigned long long>(S.x));
    a.in_features = S.in_features;
    a.m = m;
    a.x_dtype = XBF16 ? DQ_BF16 : DQ_F16;
    a.out_dtype = S.out_dtype;
    a.bias = reinterpret_cast<const void*>(reinterpret_cast<unsigned long long>(J.bias));
    a.out = reinterpret_cast<void*>(reinterpret_cast<unsigned long long>(J.out));
    a.out_stride = J.out_stride;
    a.out_col0 = J.out_col0;
    a.rows = J.rows;
    const bool has_off = reinterpret_cast<unsigned long long>(J.offsets) != 0ull;

    // ---- staged activation of this stage, in the fragment order of this job's width ----
    const int NA = bits == 8 ? 32 : 16;
    const int QU = NA / 4;
    const int m_stride_u4 = steps * NA + 4;
    uint4* xb = reinterpret_cast<uint4*>(area);
    float* xsum = reinterpret_cast<float*>(xb + m * m_stride_u4 + NA);
    float* xneg = xsum + steps * 8;
    // zero fragments and zero sums of absent activation rows do not depend on the activation
    if (bits == 8) {
      stage_zero_fill<8, false>(m, steps, m_stride_u4, xb, xsum, xneg, tid, kThreads);
    } else {
      stage_zero_fill<4, false>(m, steps, m_stride_u4, xb, xsum, xneg, tid, kThreads);
    }
    const int wait_stage = S.wait_stage;
    const bool stager = warp * kWarp < m * steps * 4;  // this warp builds fragments (tasks go round-robin over threads)
    int ok = 1;
#ifdef DQ_PLAN_TRACE
    const bool skip_wait = (P.debug_flags & 4) != 0;  // (timing experiment: arithmetic without the chain)
#else
    constexpr bool skip_wait = false;
#endif
    if (stager && wait_stage >= P.first_stage && !skip_wait) {  // (an earlier launch's stages are complete: stream order)
      // it reads the activation: it waits, bounded, for the stage that produces it
      if (lane == 0) {
        ok = wait_counter(P.counters + wait_stage, static_cast<unsigned int>(S.wait_target), status, P.spin_limit) ? 1 : 0;
        if (!ok) {
          atomicCAS(status, 0u, 1u | (static_cast<unsigned int>(s) << 8));
          s_abort = 1;
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
    }
    if (stager && ok) stage_for_bits<XBF16>(bits, a, steps, m_stride_u4, xb, xsum, xneg, tid);
    DQ_TRACE(s, 1);
    __syncthreads();
    if (s_abort) {
      aborted = true;
      break;
    }
    DQ_TRACE(s, 2);

    const bool b_live = g < m;
    const int s_begin = kwi * spw;
    const uint4* xb_lane = b_live ? xb + g * m_stride_u4 + t + s_begin * QU * 4 : xb + m * m_stride_u4;
    const int xb_step_u4 = b_live ? QU * 4 : 0;
    const float* xsum_w = xsum + s_begin * 8 + 2 * t;
    const float* xneg_w = xneg + s_begin * 8 + 2 * t;

#pragma unroll 1
    for (int item = cta_rel; item < items; item += cta_count, parity ^= 1) {
      const int tile = item * rw + rwi;
      const bool live = tile < tiles;
      float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      if (live) {
        const uint4* bchunk = xb_lane;
        const float* xs_chunk = xsum_w;
        const float* xn_chunk = xneg_w;
#pragma unroll 1
        for (int chunk = 0; chunk < nchunks; ++chunk) {
          wait_pending(nb - 1);  // groups complete in issue order: all but the nb-1 youngest are done
          __syncwarp();          // pieces other lanes copied are visible
          const unsigned char* slot = ring + rd_slot * kSlotBytes;
          const int hw0 = cs == 1 ? ((s_begin + chunk) & 1) : 0;
          switch (bits) {
            case 2:
              consume_slot<2, XBF16>(slot, cs, hw0, has_off, mbf, magic, bchunk, xb_step_u4, xs_chunk, xn_chunk, lane, acc);
              break;
            case 3:
              consume_slot<3, XBF16>(slot, cs, hw0, has_off, mbf, magic, bchunk, xb_step_u4, xs_chunk, xn_chunk, lane, acc);
              break;
            case 4:
              consume_slot<4, XBF16>(slot, cs, hw0, has_off, mbf, magic, bchunk, xb_step_u4, xs_chunk, xn_chunk, lane, acc);
              break;
            default:
              consume_slot<8, XBF16>(slot, cs, hw0, has_off, mbf, magic, bchunk, xb_step_u4, xs_chunk, xn_chunk, lane, acc);
              break;
          }
          bchunk += xb_step_u4 * cs;
          xs_chunk += cs * 8;
          xn_chunk += cs * 8;
          if (++rd_slot == nb) rd_slot = 0;
          __syncwarp();  // every lane is done with the slot just consumed:
          pf_issue();    // refill it
        }
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
#pragma unroll 2
          for (int k = 0; k < kw; ++k) {
            const float* part = buf + (k * rw + rwi) * 128;
            const float2 pa = *reinterpret_cast<const float2*>(part + g * 8 + 2 * t);
            const float2 pb = *reinterpret_cast<const float2*>(part + (g + 8) * 8 + 2 * t);
            acc[0] += pa.x, acc[1] += pa.y, acc[2] += pb.x, acc[3] += pb.y;
          }
        }
      }
      if (kwi == 0 && live) {
        const int row_a = tile * kTileRows + g, row_b = row_a + 8;
        const int m0 = 2 * t;
        if (m0 < m) {
          if (row_a < a.rows) store_out(a, m0, row_a, acc[0]);
          if (row_b < a.rows) store_out(a, m0, row_b, acc[2]);
        }
        if (m0 + 1 < m) {
          if (row_a < a.rows) store_out(a, m0 + 1, row_a, acc[1]);
          if (row_b < a.rows) store_out(a, m0 + 1, row_b, acc[3]);
        }
      }
    }
    // ---- this CTA's share of the stage is stored: tell the stage that waits for it ----
    DQ_TRACE(s, 3);
    __syncthreads();  // (also: the staged activation and the partial-sum buffers are free again)
    DQ_TRACE(s, 4);
    if (tid == 0 && S.signal != 0) {
#ifdef DQ_PLAN_TRACE
      if (P.debug_flags & 1) {
        atomicAdd(P.counters + s, 1u);
      } else
#endif
      {
        red_release_add(P.counters + s, 1u);  // (release at GPU scope: cumulative over the CTA's stores, through the barrier)
      }
    }
    DQ_TRACE(s, 5);
    pf_catch_up();  // the stage is signalled: now is the cheap moment to look for this warp's next item
    DQ_TRACE(s, 6);
  }

  stream::cp_async_wait<0>();  // nothing of ours is still in flight when the CTA leaves
  __syncthreads();
  if (tid == 0) {
    // the last CTA out zeroes the counters: by then nobody polls them any more
    __threadfence();
    const unsigned int left = atomicAdd(P.counters + P.nstages, 1u);
    if (left == gridDim.x - 1) {
      __threadfence();
      for (int i = P.first_stage; i < P.last_stage; ++i) P.counters[i] = 0u;
      P.counters[P.nstages] = 0u;
    }
  }
}

}  // namespace plank
}  // namespace dq

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------

// One launch of a plan: a range of stages in the persistent kernel, or one long matrix handed to
// the streaming GEMV (a matrix that fills the machine many tiles deep gains nothing from the
// stage machinery and runs faster on the leaner kernel: dq_gemv_mma_stream.cuh).
struct PlanOp {
  int first_stage, last_stage;  // persistent kernel over [first_stage, last_stage) ...
  int job;                      // ... or, when >= 0, this job of the caller's list on its own
};

struct dq_plan {
  std::vector<dq::plank::PStage> stages;
  std::vector<dq::plank::PJob> jobs;
  std::vector<dq_gemv_job> user_jobs;
  std::vector<PlanOp> ops;
  dq::plank::PlanParams params;
  void* workspace;
  int64_t workspace_bytes;
  size_t stage_bytes, job_bytes;  // sizes of the two tables in the workspace
  int grid;
  size_t smem;
  int x_bf16;
  int device;
};

namespace dq {
namespace plank {
namespace {

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Relative cost of one 128-value step of one row tile, by width (8-bit fragments are twice as many).
double step_cost(int bits) { return bits == 8 ? 1.9 : (bits == 3 ? 1.1 : 1.0); }

struct Pick {
  int kw = 0, cs = 0;
  int cta_count[kMaxStageJobs] = {0, 0, 0, 0};
  double cost = 0.0;
};

// Largest slot depth (steps per slot) a slicing allows: divides spw, fits the slot, and the slot's
// metadata is a whole number of aligned 4- or 8-byte words in every job.
int pick_cs(const dq_gemv_job* jobs, int n, int spw) {
  int max_bits = 0;
  for (int i = 0; i < n; ++i) max_bits = std::max(max_bits, static_cast<int>(jobs[i].weight.bits));
  for (int cs = 4; cs >= 1; cs /= 2) {
    if (spw % cs != 0 || cs * 256 * max_bits > kSlotWeights) continue;
    const uintptr_t al = cs == 4 ? 8 : 4;
    bool ok = true;
    for (int i = 0; i < n && ok; ++i) {
      const dq_weight& w = jobs[i].weight;
      ok = (w.num_groups * 2) % static_cast<int64_t>(al) == 0 && reinterpret_cast<uintptr_t>(w.scales) % al == 0 &&
           reinterpret_cast<uintptr_t>(w.offsets) % al == 0;
    }
    if (ok) return cs;
  }
  return 0;
}

// Slicing of one stage and the split of the grid among its jobs.
Pick pick_shape(const dq_gemv_job* jobs, int n, int steps, int grid) {
  Pick best;
  for (int kw = kWarps; kw >= 1; kw /= 2) {
    if (steps % kw != 0) continue;
    const int spw = steps / kw, rw = kWarps / kw;
    const int cs = pick_cs(jobs, n, spw);
    if (cs == 0) continue;
    int64_t items[kMaxStageJobs];
    double per_item[kMaxStageJobs], weight[kMaxStageJobs], total = 0.0;
    for (int i = 0; i < n; ++i) {
      items[i] = ceil_div(ceil_div(jobs[i].weight.rows, kTileRows), rw);
      // in units of one step of all 16 warps of an SM (issue-bound, about a microsecond): a slot
      // costs a wait and a refill; a sliced item a barrier and a pass through shared memory
      per_item[i] = spw * step_cost(jobs[i].weight.bits) + 0.1 * (spw / cs) + (kw > 1 ? 0.35 : 0.05);
      weight[i] = items[i] * per_item[i];
      total += weight[i];
    }
    Pick p;
    p.kw = kw;
    p.cs = cs;
    int used = 0;
    for (int i = 0; i < n; ++i) {
      p.cta_count[i] = std::max(1, static_cast<int>(grid * weight[i] / total));
      p.cta_count[i] = static_cast<int>(std::min<int64_t>(p.cta_count[i], items[i]));
      used += p.cta_count[i];
    }
    auto cost_of = [&](int i) { return ceil_div(items[i], p.cta_count[i]) * per_item[i]; };
    // hand the remaining CTAs, one at a time, to the job that is slowest
    while (used < grid) {
      int worst = -1;
      for (int i = 0; i < n; ++i) {
        if (p.cta_count[i] < items[i] && (worst < 0 || cost_of(i) > cost_of(worst))) worst = i;
      }
      if (worst < 0) break;
      ++p.cta_count[worst];
      ++used;
    }
    if (used > grid) continue;  // more jobs than CTAs: not a shape this grid can run
    p.cost = 0.0;
    for (int i = 0; i < n; ++i) p.cost = std::max(p.cost, cost_of(i));
    if (best.kw == 0 || p.cost < best.cost - 1e-9) best = p;
  }
  return best;
}

}  // namespace
}  // namespace plank
}  // namespace dq

extern "C" {

int32_t dq_plan_workspace_bytes(int32_t num_jobs, int64_t* bytes) {
  using namespace dq::plank;
  DQ_REQUIRE(num_jobs >= 0 && bytes != nullptr, "plan_workspace_bytes: bad arguments");
  const size_t n = static_cast<size_t>(std::max(num_jobs, 1));
  *bytes = static_cast<int64_t>(align_up(n * sizeof(PStage), 256) + align_up(n * sizeof(PJob), 256) +
                                align_up((n + 2) * sizeof(unsigned int), 256));
  return DQ_OK;
}

int32_t dq_plan_create(const dq_gemv_job* jobs, int32_t num_jobs, void* workspace, int64_t workspace_bytes,
                       void* stream, dq_plan** out_plan) {
  using namespace dq;
  using namespace dq::plank;
  DQ_REQUIRE(out_plan != nullptr, "plan_create: null result pointer");
  *out_plan = nullptr;
  DQ_REQUIRE(num_jobs > 0 && jobs != nullptr, "plan_create: need at least one job");
  int64_t need = 0;
  dq_plan_workspace_bytes(num_jobs, &need);
  DQ_REQUIRE(workspace != nullptr && workspace_bytes >= need && reinterpret_cast<uintptr_t>(workspace) % 256 == 0,
             "plan_create: the workspace must be 256-byte aligned device memory of at least %lld bytes, got %lld",
             static_cast<long long>(need), static_cast<long long>(workspace_bytes));
  const DeviceInfo* dev = device_info();
  if (dev == nullptr) return DQ_ERR_CUDA;

  // ---- validation: what dq_gemv_sequence checks, plus what this kernel needs ----
  std::vector<dq_geometry> geo(num_jobs);
  for (int i = 0; i < num_jobs; ++i) {
    const dq_gemv_job& j = jobs[i];
    if (const int32_t rc = dq_resolve_geometry("plan_create", &j.weight, &geo[i])) return rc;
    DQ_REQUIRE(j.m >= 1 && j.m <= DQ_GEMV_MAX_ROWS,
               "plan_create: job %d has %lld activation rows; a plan takes 1..%d (more exceeds the kernel's limit)", i,
               static_cast<long long>(j.m), DQ_GEMV_MAX_ROWS);
    DQ_REQUIRE(j.x != nullptr && j.out != nullptr, "plan_create: job %d has a null activation or output pointer", i);
    DQ_REQUIRE(j.weight.rows > 0, "plan_create: job %d has no rows", i);
    DQ_REQUIRE(j.out_col0 >= 0 && j.out_stride >= j.out_col0 + j.weight.rows,
               "plan_create: job %d writes columns [%lld, %lld) of a row of %lld", i, static_cast<long long>(j.out_col0),
               static_cast<long long>(j.out_col0 + j.weight.rows), static_cast<long long>(j.out_stride));
    DQ_REQUIRE(dtype_ok(j.out_dtype), "plan_create: job %d: unsupported output dtype tag %d", i, j.out_dtype);
    auto unsupported = [&](const char* why) {
      return fail(DQ_ERR_UNSUPPORTED, "plan_create: job %d cannot run in a plan (%s); launch it with dq_gemv_sequence", i,
                  why);
    };
    if (j.x_dtype != DQ_BF16 && j.x_dtype != DQ_F16) return unsupported("the activation is not 16-bit");
    if (j.x_dtype != jobs[0].x_dtype) return unsupported("activation dtypes differ between jobs");
    if (j.weight.meta_dtype != DQ_BF16 && j.weight.meta_dtype != DQ_F16) return unsupported("scales are not 16-bit");
    if (geo[i].group_values != kStepValues) return unsupported("groups are not 128 values");
    if (reinterpret_cast<uintptr_t>(j.weight.packed) % 16 != 0 || (static_cast<int64_t>(geo[i].words_per_row) * 4) % 16 != 0) {
      return unsupported("packed rows are not 16-byte aligned");
    }
    if ((geo[i].in_features & 7) != 0 || reinterpret_cast<uintptr_t>(j.x) % 16 != 0) {
      return unsupported("the activation is not 16-byte aligned or in_features is not a multiple of 8");
    }
    if (static_cast<int64_t>(j.weight.rows) * geo[i].words_per_row * 4 >= (1LL << 32)) {
      return unsupported("the packed tensor is 4 GiB or more");
    }
    if (reinterpret_cast<uintptr_t>(j.weight.scales) % 4 != 0 || reinterpret_cast<uintptr_t>(j.weight.offsets) % 4 != 0 ||
        geo[i].num_groups % 2 != 0) {
      return unsupported("scale rows are not 4-byte aligned");
    }
  }

  dq_plan* plan = new (std::nothrow) dq_plan();
  DQ_REQUIRE(plan != nullptr, "plan_create: out of host memory");
  plan->grid = dev->sm_count;
  plan->device = dev->device;
  plan->x_bf16 = jobs[0].x_dtype == DQ_BF16 ? 1 : 0;

  // ---- stages: consecutive jobs that read the same activation ----
  plan->user_jobs.assign(jobs, jobs + num_jobs);
  std::vector<int> own_launch;  // per stage: the job it hands to the streaming GEMV, or -1
  size_t stage_area = 0;
  int i = 0;
  while (i < num_jobs) {
    const dq_gemv_job& head = jobs[i];
    int end = i + 1;
    while (end < num_jobs && end - i < kMaxStageJobs && jobs[end].x == head.x && jobs[end].m == head.m &&
           jobs[end].out_dtype == head.out_dtype && jobs[end].weight.meta_dtype == head.weight.meta_dtype &&
           geo[end].in_features == geo[i].in_features) {
      ++end;
    }
    const int n = end - i;
    const int steps = geo[i].words_per_row / (4 * head.weight.bits);
    const Pick pick = pick_shape(jobs + i, n, steps, plan->grid);
    if (pick.kw == 0) {
      delete plan;
      return fail(DQ_ERR_UNSUPPORTED, "plan_create: no slicing of jobs %d..%d fits the kernel; launch them with dq_gemv_sequence",
                  i, end - 1);
    }
    PStage S = {};
    S.x = head.x;
    S.m = static_cast<int>(head.m);
    S.in_features = geo[i].in_features;
    S.steps = steps;
    S.meta_bf16 = head.weight.meta_dtype == DQ_BF16 ? 1 : 0;
    S.out_dtype = head.out_dtype;
    S.kw = pick.kw;
    S.spw = steps / pick.kw;
    S.cs = pick.cs;
    S.job_begin = static_cast<int>(plan->jobs.size());
    S.njobs = n;
    const int sidx = static_cast<int>(plan->stages.size());
    S.wait_stage = sidx - 1;  // stream order: a stage may read what the one before it wrote
    S.wait_target = 0;
    S.signal = 0;
    int cta = 0, active = 0, max_bits = 0;
    for (int k = 0; k < n; ++k) {
      const dq_gemv_job& j = jobs[i + k];
      PJob J = {};
      J.packed = static_cast<const uint32_t*>(j.weight.packed);
      J.scales = j.weight.scales;
      J.offsets = j.weight.offsets;
      J.bias = j.bias;
      J.out = j.out;
      J.out_stride = j.out_stride;
      J.out_col0 = j.out_col0;
      J.rows = static_cast<int>(j.weight.rows);
      J.words_per_row = geo[i + k].words_per_row;
      J.num_groups = geo[i + k].num_groups;
      J.bits = j.weight.bits;
      J.tiles = static_cast<int>(ceil_div(J.rows, kTileRows));
      J.items = static_cast<int>(ceil_div(J.tiles, kWarps / pick.kw));
      J.cta_begin = cta;
      J.cta_count = pick.cta_count[k];
      cta += J.cta_count;
      active += std::min(J.cta_count, J.items);
      max_bits = std::max(max_bits, J.bits);
      plan->jobs.push_back(J);
    }
    S.pad = active;  // CTAs that arrive on this stage's counter (copied into the waiter below)
    plan->stages.push_back(S);
    const bool long_matrix = n == 1 && ceil_div(head.weight.rows, kTileRows) >= static_cast<int64_t>(dev->sm_count) * 8;
    own_launch.push_back(long_matrix ? i : -1);
    if (!long_matrix) {
      const int na = max_bits == 8 ? 32 : 16;
      const size_t area = (static_cast<size_t>(S.m) * (static_cast<size_t>(steps) * na + 4) + na) * 16 +
                          static_cast<size_t>(steps) * 64 + 16;
      stage_area = std::max(stage_area, area);
    }
    i = end;
  }
  const int total_stages = static_cast<int>(plan->stages.size());
  for (int s = 1; s < total_stages; ++s) plan->stages[s].wait_target = plan->stages[s - 1].pad;
  for (int s = 0; s < total_stages; ++s) {
    PStage& S = plan->stages[s];
    S.pad = 0;
    // a stage signals only a successor that runs in the same launch
    S.signal = (s + 1 < total_stages && own_launch[s] < 0 && own_launch[s + 1] < 0) ? 1 : 0;
  }
  for (int s = 0; s < total_stages;) {
    if (own_launch[s] >= 0) {
      plan->ops.push_back(PlanOp{s, s + 1, own_launch[s]});
      ++s;
      continue;
    }
    int e = s;
    while (e < total_stages && own_launch[e] < 0) ++e;
    plan->ops.push_back(PlanOp{s, e, -1});
    s = e;
  }

  // ---- shared memory: staged activation, partial sums, the weight ring -- and, when they fit
  // beside a ring of at least three slots, a copy of the two tables ----
  const size_t area_bytes = align_up(stage_area, 16);
  const size_t table_bytes = align_up(plan->stages.size() * sizeof(PStage) + plan->jobs.size() * sizeof(PJob), 16);
  const size_t fixed = kRedFloats * 4 + area_bytes + 1024;  // (+ the kernel's static shared memory)
  int nb = 0, tables = 0;
  const int order[6][2] = {{1, 4}, {1, 3}, {0, 4}, {0, 3}, {1, 2}, {0, 2}};  // (tables in smem, ring slots)
  for (const auto& cand : order) {
    const size_t need_smem = fixed + (cand[0] ? table_bytes : 0) + static_cast<size_t>(cand[1]) * kWarps * kSlotBytes;
    if (need_smem <= static_cast<size_t>(dev->max_smem_optin)) {
      tables = cand[0];
      nb = cand[1];
      break;
    }
  }
  if (nb == 0) {
    delete plan;
    return fail(DQ_ERR_UNSUPPORTED,
                "plan_create: the staged activation (%zu bytes) leaves no room for the weight ring; launch with dq_gemv_sequence",
                stage_area);
  }
  plan->smem = fixed + (tables ? table_bytes : 0) + static_cast<size_t>(nb) * kWarps * kSlotBytes;

  auto set_attr = [&](auto kernel) -> int32_t {
    DQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(plan->smem)));
    int per_sm = 0;
    DQ_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, plan->smem));
    if (per_sm < 1) return fail(DQ_ERR_UNSUPPORTED, "plan_create: the kernel does not fit an SM with %zu bytes of shared memory", plan->smem);
    return DQ_OK;
  };
  const int32_t rc_attr = plan->x_bf16 ? set_attr(gemv_plan_kernel<true>) : set_attr(gemv_plan_kernel<false>);
  if (rc_attr != DQ_OK) {
    delete plan;
    return rc_attr;
  }

  // ---- device tables ----
  plan->workspace = workspace;
  plan->workspace_bytes = workspace_bytes;
  plan->stage_bytes = plan->stages.size() * sizeof(PStage);
  plan->job_bytes = plan->jobs.size() * sizeof(PJob);
  unsigned char* base = static_cast<unsigned char*>(workspace);
  const size_t n = static_cast<size_t>(num_jobs);
  unsigned char* d_stages = base;
  unsigned char* d_jobs = base + align_up(n * sizeof(PStage), 256);
  unsigned char* d_counters = d_jobs + align_up(n * sizeof(PJob), 256);
  auto s = static_cast<cudaStream_t>(stream);
  auto copy = [&]() -> int32_t {
    DQ_CUDA(cudaMemcpyAsync(d_stages, plan->stages.data(), plan->stage_bytes, cudaMemcpyHostToDevice, s));
    DQ_CUDA(cudaMemcpyAsync(d_jobs, plan->jobs.data(), plan->job_bytes, cudaMemcpyHostToDevice, s));
    DQ_CUDA(cudaMemsetAsync(d_counters, 0, (plan->stages.size() + 2) * sizeof(unsigned int), s));
    DQ_CUDA(cudaStreamSynchronize(s));  // the host vectors may be edited (dq_plan_set_wait) once this returns
    return DQ_OK;
  };
  if (const int32_t rc = copy()) {
    delete plan;
    return rc;
  }
  plan->params.stages = reinterpret_cast<const PStage*>(d_stages);
  plan->params.jobs = reinterpret_cast<const PJob*>(d_jobs);
  plan->params.counters = reinterpret_cast<unsigned int*>(d_counters);
  plan->params.nstages = static_cast<int>(plan->stages.size());
  plan->params.first_stage = 0;
  plan->params.last_stage = plan->params.nstages;
  plan->params.njobs = static_cast<int>(plan->jobs.size());
  plan->params.tables_in_smem = tables;
  plan->params.area_bytes = static_cast<int>(area_bytes);
  plan->params.nb = nb;
  plan->params.spin_limit = kDefaultSpinLimit;
  plan->params.magic = plan->x_bf16 ? 0x43004300u : 0x64006400u;
  *out_plan = plan;
  return DQ_OK;
}

int32_t dq_plan_launch(dq_plan* plan, void* stream) {
  using namespace dq;
  using namespace dq::plank;
  DQ_REQUIRE(plan != nullptr, "plan_launch: null plan");
  auto s = static_cast<cudaStream_t>(stream);
  for (const PlanOp& op : plan->ops) {
    if (op.job >= 0) {
      if (const int32_t rc = dq_gemv_sequence(&plan->user_jobs[op.job], 1, stream)) return rc;
      continue;
    }
    PlanParams params = plan->params;
    params.first_stage = op.first_stage;
    params.last_stage = op.last_stage;
    if (plan->x_bf16) {
      gemv_plan_kernel<true><<<plan->grid, kThreads, plan->smem, s>>>(params);
    } else {
      gemv_plan_kernel<false><<<plan->grid, kThreads, plan->smem, s>>>(params);
    }
    DQ_CHECK_LAUNCH("plan");
    note_kernel("gemv_plan_kernel");
  }
  return DQ_OK;
}

int32_t dq_plan_status(dq_plan* plan, void* stream) {
  using namespace dq;
  DQ_REQUIRE(plan != nullptr, "plan_status: null plan");
  auto s = static_cast<cudaStream_t>(stream);
  unsigned int word = 0;
  DQ_CUDA(cudaMemcpyAsync(&word, plan->params.counters + plan->params.nstages + 1, sizeof(word), cudaMemcpyDeviceToHost, s));
  DQ_CUDA(cudaStreamSynchronize(s));
  if (word != 0u) {
    // clear it, and the counters a broken-off run may have left behind, so the plan can run again
    DQ_CUDA(cudaMemsetAsync(plan->params.counters, 0, (plan->params.nstages + 2) * sizeof(unsigned int), s));
    DQ_CUDA(cudaStreamSynchronize(s));
    return fail(DQ_ERR_DEVICE,
                "plan: stage %u gave up waiting for the stage before it (%d polls); outputs of this run are incomplete",
                word >> 8, plan->params.spin_limit);
  }
  return DQ_OK;
}

int32_t dq_plan_set_wait(dq_plan* plan, int32_t stage, int32_t wait_target, int32_t spin_limit, void* stream) {
  using namespace dq;
  using namespace dq::plank;
  DQ_REQUIRE(plan != nullptr, "plan_set_wait: null plan");
  DQ_REQUIRE(stage >= 0 && stage < plan->params.nstages, "plan_set_wait: stage %d of %d", stage, plan->params.nstages);
  DQ_REQUIRE(spin_limit > 0, "plan_set_wait: the spin limit must be positive");
  auto s = static_cast<cudaStream_t>(stream);
  if (wait_target >= 0) plan->stages[stage].wait_target = wait_target;
  plan->params.spin_limit = spin_limit;
  DQ_CUDA(cudaMemcpyAsync(const_cast<PStage*>(plan->params.stages) + stage, &plan->stages[stage], sizeof(PStage),
                          cudaMemcpyHostToDevice, s));
  DQ_CUDA(cudaStreamSynchronize(s));
  return DQ_OK;
}

int32_t dq_plan_describe(const dq_plan* plan, dq_plan_info* info) {
  using namespace dq;
  DQ_REQUIRE(plan != nullptr && info != nullptr, "plan_describe: null argument");
  info->num_stages = plan->params.nstages;
  info->num_jobs = static_cast<int32_t>(plan->jobs.size());
  info->grid = plan->grid;
  info->threads = dq::plank::kThreads;
  info->ring_slots = plan->params.nb;
  info->launches = static_cast<int32_t>(plan->ops.size());
  info->shared_bytes = static_cast<int64_t>(plan->smem);
  return DQ_OK;
}

int32_t dq_plan_stage_shape(const dq_plan* plan, int32_t stage, int32_t* k_slices, int32_t* slot_steps,
                            int32_t* cta_counts /* [4] */) {
  using namespace dq;
  DQ_REQUIRE(plan != nullptr && stage >= 0 && stage < plan->params.nstages, "plan_stage_shape: bad arguments");
  const auto& S = plan->stages[stage];
  if (k_slices != nullptr) *k_slices = S.kw;
  if (slot_steps != nullptr) *slot_steps = S.cs;
  if (cta_counts != nullptr) {
    for (int k = 0; k < dq::plank::kMaxStageJobs; ++k) cta_counts[k] = k < S.njobs ? plan->jobs[S.job_begin + k].cta_count : 0;
  }
  return DQ_OK;
}

void dq_plan_destroy(dq_plan* plan) { delete plan; }

#ifdef DQ_PLAN_TRACE
// Diagnostic builds only: device buffer of nstages * 2 * 8 timestamps (see trace_point).
__attribute__((visibility("default"))) void dq_plan_set_trace(dq_plan* plan, unsigned long long* buffer) {
  plan->params.trace = buffer;
}
__attribute__((visibility("default"))) void dq_plan_set_debug(dq_plan* plan, int flags) {
  plan->params.debug_flags = flags;
  const int relaxed = (flags & 2) ? 1 : 0;
  cudaMemcpyToSymbol(dq::plank::g_debug_relaxed_poll, &relaxed, sizeof(int));
}
#endif

}  // extern "C"
