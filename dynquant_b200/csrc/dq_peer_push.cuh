// The all-gather of a column-sharded stage folded into the GEMV launch that produces it.
//
// A column-sharded layer computes [m, rows/world] on every rank and every rank needs all of it.
// Done as a separate exchange launch that costs about as much as the small GEMV itself.  Here
// the GEMV kernel's own CTAs, right after storing their output rows, copy those rows into every
// rank's window through peer-mapped pointers (ordinary st.global: nothing is ever READ from a
// peer, no TMA, no multicast), and the launch's last CTA raises this rank's flag in every window
// and then waits -- BOUNDED -- until every rank's flag of the same epoch is up in its own window.
// When the launch completes, the gathered output of the stage is complete on this GPU, so the
// next launch in the stream (whatever it is) may read it: no separate exchange launch, no
// change to the consumer.
//
// Window layout is the host's: byte offsets of this exchange's data (two halves chosen by the
// epoch's parity, each `world` pieces in rank order, so that a rank running one step ahead does
// not overwrite what a slower rank's stream still reads), of its u32[world] flags, of its local
// u32[2] state {epoch, arrived CTAs} and of the window's status word.  Epochs only grow; nothing
// is reset between launches except the arrival counter, by the last CTA itself.
#pragma once

#include "dq_gemv.cuh"

namespace dq {
namespace peerpush {

constexpr int kMaxWorld = 8;  // windows travel by value in the launch arguments

struct Push {
  unsigned char* window[kMaxWorld];  // every rank's window as mapped on this GPU; [rank] is the local one
  int64_t data_off;                  // this exchange's data: [2 halves][world][piece_bytes]
  int64_t piece_bytes;               // one rank's piece: the launch's whole [m, out_stride] output buffer
  int flags_off;                     // u32[world] in every window: epoch of the last piece that arrived from each rank
  int state_off;                     // u32[2] in the local window: {epoch of the last exchange, CTAs arrived}
  int status_off;                    // u32 in the local window: nonzero once a wait ran out
  int world, rank;
  int spin_limit;
  int enabled;
};

#ifdef __CUDACC__

__device__ __forceinline__ void st_relaxed_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned int ld_relaxed_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Epoch of the exchange this launch performs.  Call after the dependency wait (the previous
// launch on this exchange has completed and recorded its epoch) and before `arrive`: the last
// CTA records the new epoch only after every CTA has arrived, i.e. after every CTA has read it.
__device__ __forceinline__ unsigned int next_epoch(const Push& P) {
  return *reinterpret_cast<const volatile unsigned int*>(P.window[P.rank] + P.state_off) + 1u;
}

// Rows [row_lo, row_hi) of job `a` -- already stored to a.out by this CTA, and made visible to
// it by a CTA barrier -- into every rank's window, all activation rows.  All threads of the CTA.
__device__ __forceinline__ void push_rows(const Push& P, const GemvArgs& a, unsigned int epoch, int row_lo, int row_hi,
                                          int tid, int nthreads) {
  if (row_hi <= row_lo) return;
  const int es = a.out_dtype == DQ_F32 ? 4 : 2;
  const int64_t pitch = a.out_stride * es;                    // bytes between activation rows of the piece
  const int64_t lo = (a.out_col0 + row_lo) * static_cast<int64_t>(es);
  const int nbytes = (row_hi - row_lo) * es;
  const int64_t slot = P.data_off + ((epoch & 1u) ? P.piece_bytes * P.world : 0) + P.piece_bytes * P.rank;
  const unsigned char* src = static_cast<const unsigned char*>(a.out);
  if (((lo | pitch | nbytes) & 3) == 0) {
    const int n = nbytes >> 2, per_rank = n * a.m, total = per_rank * P.world;
    for (int i = tid; i < total; i += nthreads) {
      const int p = i / per_rank, r = i - p * per_rank;
      const int mi = r / n, u = r - mi * n;
      const int64_t off = mi * pitch + lo + 4 * u;
      *reinterpret_cast<unsigned int*>(P.window[p] + slot + off) = *reinterpret_cast<const unsigned int*>(src + off);
    }
  } else {
    const int n = nbytes >> 1, per_rank = n * a.m, total = per_rank * P.world;
    for (int i = tid; i < total; i += nthreads) {
      const int p = i / per_rank, r = i - p * per_rank;
      const int mi = r / n, u = r - mi * n;
      const int64_t off = mi * pitch + lo + 2 * u;
      *reinterpret_cast<unsigned short*>(P.window[p] + slot + off) = *reinterpret_cast<const unsigned short*>(src + off);
    }
  }
}

// The first WARP of every CTA (all 32 lanes), after a CTA barrier that follows the CTA's pushes.
// The barrier orders the CTA's stores before lane 0, which adds to the counter with release /
// acquire semantics at GPU scope, so the launch's last CTA has every CTA's stores in its
// causality order; its SYSTEM-scope fence followed by the flag stores is then a release of all of
// them to whoever acquires a flag.  (A system-scope fence in every CTA instead was measured:
// 3 us per stage slower, same results.)  Then lane p of the last CTA's warp polls, a bounded
// number of times, for rank p's flag -- all ranks at once.
__device__ __forceinline__ void arrive(const Push& P, unsigned int epoch, unsigned int ctas, int lane) {
  unsigned char* mine = P.window[P.rank];
  unsigned int* state = reinterpret_cast<unsigned int*>(mine + P.state_off);
  unsigned int before = 0;
  if (lane == 0) {
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(before) : "l"(state + 1) : "memory");
  }
  before = __shfl_sync(0xffffffffu, before, 0);
  if (before != ctas - 1u) return;
  if (lane == 0) {
    state[1] = 0u;
    state[0] = epoch;
    asm volatile("fence.acq_rel.sys;" ::: "memory");
  }
  __syncwarp();
  unsigned int* status = reinterpret_cast<unsigned int*>(mine + P.status_off);
  bool ok = true;
  if (lane < P.world) {
    st_relaxed_sys(reinterpret_cast<unsigned int*>(P.window[lane] + P.flags_off) + P.rank, epoch);
    const unsigned int* flag = reinterpret_cast<const unsigned int*>(mine + P.flags_off) + lane;
    ok = false;
    for (int it = 0; it < P.spin_limit; ++it) {
      // (>= as a signed distance: epochs wrap after 2^32 exchanges)
      if (static_cast<int>(ld_relaxed_sys(flag) - epoch) >= 0) {
        ok = static_cast<int>(ld_acquire_sys(flag) - epoch) >= 0;  // (one acquire once the flag is up)
        break;
      }
      if ((it & 255) == 255 && *reinterpret_cast<volatile unsigned int*>(status) != 0u) break;
    }
    if (!ok) atomicCAS(status, 0u, 1u | (static_cast<unsigned int>(lane) << 8));  // the host reads the status word
  }
}

#endif  // __CUDACC__

}  // namespace peerpush
}  // namespace dq
