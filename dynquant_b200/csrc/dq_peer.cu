// Exchanges of the sharded paths over peer memory: plain stores into the other GPUs' buffers
// through NVLink-mapped pointers, a release flag per source, a BOUNDED wait on the way in.
//
// The sharded decode paths exchange very little -- the 12-250 KB output slabs of a column-sharded
// layer, a few token rows of an expert layer -- and exchange it often.  A library collective
// issued from the host costs more than the kernels between two of them; these two kernels are
// launched like any other kernel of the library (and captured in the step's CUDA graph):
//
//   peer_all_gather      every rank holds `bytes`; afterwards every rank holds all of them, in
//                        rank order.  CTA group p of rank r stores r's piece into rank p's
//                        buffer, fences, raises flag[r] in p's buffer, waits for flag[p] in its
//                        own buffer and copies p's piece to the caller's output.
//   peer_reduce_scatter  every rank holds fp32 partial rows for every rank's elements; rank r
//                        ends up with the sum over source ranks of the rows that are r's, added
//                        in rank order (bit-identical from run to run).  Same push / flag / wait,
//                        then a second, purely local kernel adds the slots.
//
// No TMA, no multicast, no library kernel ever sees a peer pointer: remote memory is only
// WRITTEN, with ordinary st.global; everything that is read is local.  Flags carry a
// monotonically increasing epoch, so nothing has to be reset; pieces land in one of two halves
// of the buffer chosen by the epoch's parity, so a rank that runs one exchange ahead cannot
// overwrite what a slower rank is still copying out (it cannot run two ahead: the next
// exchange needs the slower rank's piece).  A wait that runs out of polls sets the buffer's
// status word and the kernel returns; dq_peer_status reports DQ_ERR_DEVICE.
#include <algorithm>

#include "dq_common.cuh"

namespace dq {
namespace peer {

constexpr int kThreads = 256;
constexpr int kMaxWorld = 64;
constexpr int kMaxCtasPerPeer = 8;
constexpr int kMaxParts = 4;
// header of every exchange buffer (bytes)
constexpr int kFlagsAt = 0;        // u32 [world]: epoch of the last piece that arrived from each source
constexpr int kEpochsAt = 1024;    // u32 [world]: epoch this rank last used towards each destination
constexpr int kArrivedAt = 2048;   // u32 [world]: CTAs of a group that have pushed their part (reset by the last)
constexpr int kStatusAt = 3072;    // u32: nonzero once a wait ran out
constexpr int kHeaderBytes = 4096;

struct Args {
  unsigned char* const* buffers;  // [world] every rank's buffer, as mapped here
  int64_t half_bytes;             // bytes of one parity half of the data area
  int world, rank;
  int ctas_per_peer;
  int spin_limit;
  const unsigned char* src;       // what this rank contributes (all-gather: one piece; reduce-scatter: world pieces)
  int64_t piece_bytes;
  unsigned char* out;             // all-gather: [world * piece_bytes]
  int scatter;                    // 1: piece p of src goes to rank p (reduce-scatter); 0: the one piece goes to everyone
  // all-gather of several tensors in one exchange: the piece is their concatenation (every part a
  // multiple of 16 bytes); part i comes from part_src[i] and rank p's copy of it goes to
  // part_out[i] + p * part_bytes[i].  parts == 0: the single src / out above.
  int parts;
  const unsigned char* part_src[kMaxParts];
  unsigned char* part_out[kMaxParts];
  int64_t part_bytes[kMaxParts];
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_relaxed_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Copy [lo, hi) bytes (16-byte aligned bounds except the very end) with this CTA's threads.
__device__ __forceinline__ void copy_span(unsigned char* dst, const unsigned char* src, int64_t lo, int64_t hi) {
  const int64_t vec_hi = lo + ((hi - lo) / 16) * 16;
  for (int64_t at = lo + static_cast<int64_t>(threadIdx.x) * 16; at < vec_hi; at += static_cast<int64_t>(kThreads) * 16) {
    *reinterpret_cast<uint4*>(dst + at) = *reinterpret_cast<const uint4*>(src + at);
  }
  for (int64_t at = vec_hi + threadIdx.x; at < hi; at += kThreads) dst[at] = src[at];
}

// Push, signal, wait.  Grid = world * ctas_per_peer CTAs; group p = CTAs [p * cpp, (p + 1) * cpp).
// gather (scatter == 0): afterwards piece p has been copied to out + p * piece_bytes.
// scatter: afterwards slot p of this rank's current half holds rank p's partial rows for this rank
// (the caller's second kernel adds the slots).
__global__ void __launch_bounds__(kThreads) peer_exchange_kernel(const Args a) {
  __shared__ unsigned int s_epoch;
  __shared__ int s_ok;
  const int p = blockIdx.x / a.ctas_per_peer;
  const int c = blockIdx.x - p * a.ctas_per_peer;
  unsigned char* mine = a.buffers[a.rank];
  unsigned char* theirs = a.buffers[p];
  unsigned int* epochs = reinterpret_cast<unsigned int*>(mine + kEpochsAt);
  unsigned int* arrived = reinterpret_cast<unsigned int*>(mine + kArrivedAt);
  unsigned int* status = reinterpret_cast<unsigned int*>(mine + kStatusAt);
  if (threadIdx.x == 0) s_epoch = epochs[p] + 1u;
  __syncthreads();
  const unsigned int epoch = s_epoch;
  const int64_t half = (epoch & 1u) ? a.half_bytes : 0;
  // this CTA's share of the piece: whole 16-byte words
  const int64_t words = (a.piece_bytes + 15) / 16;
  const int64_t lo = std::min<int64_t>(a.piece_bytes, (words * c / a.ctas_per_peer) * 16);
  const int64_t hi = std::min<int64_t>(a.piece_bytes, (words * (c + 1) / a.ctas_per_peer) * 16);

  // ---- push: my piece (gather) or my partial rows for rank p (scatter) into p's buffer, slot [rank] ----
  unsigned char* slot = theirs + kHeaderBytes + half + static_cast<int64_t>(a.rank) * a.piece_bytes;
  if (a.parts == 0) {
    const unsigned char* src = a.src + (a.scatter ? static_cast<int64_t>(p) * a.piece_bytes : 0);
    copy_span(slot, src, lo, hi);
  } else {
    int64_t at = 0;  // offset of the part inside the piece
    for (int i = 0; i < a.parts; ++i) {
      const int64_t from = max(lo, at), to = min(hi, at + a.part_bytes[i]);
      if (from < to) copy_span(slot + at, a.part_src[i], from - at, to - at);
      at += a.part_bytes[i];
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // Ordering without a fence per thread: the barrier above orders the CTA's stores before this
    // thread; the counter is added with release / acquire semantics at GPU scope (cumulative over
    // what each CTA's thread 0 has observed), and the flag is stored with release at SYSTEM scope.
    bool last = true;
    if (a.ctas_per_peer > 1) {
      unsigned int before;
      asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(before) : "l"(&arrived[p]) : "memory");
      last = before == static_cast<unsigned int>(a.ctas_per_peer) - 1u;
    }
    if (last) {
      // the last CTA of the group: everything of this piece is on its way, and every CTA of the
      // group has read the epoch (it did so before pushing) -- record it for the next exchange
      if (a.ctas_per_peer > 1) arrived[p] = 0u;
      epochs[p] = epoch;
      st_release_sys(reinterpret_cast<unsigned int*>(theirs + kFlagsAt) + a.rank, epoch);
    }
    // ---- wait, bounded, for rank p's piece of the same epoch in my own buffer ----
    const unsigned int* flag = reinterpret_cast<const unsigned int*>(mine + kFlagsAt) + p;
    int ok = 0;
    for (int it = 0; it < a.spin_limit; ++it) {
      if (ld_relaxed_sys(flag) >= epoch) {
        ok = ld_acquire_sys(flag) >= epoch ? 1 : 0;  // (one acquire once the flag is up)
        break;
      }
      if ((it & 255) == 255 && *reinterpret_cast<volatile unsigned int*>(status) != 0u) break;
    }
    if (!ok) atomicCAS(status, 0u, 1u | (static_cast<unsigned int>(p) << 8));
    s_ok = ok;
  }
  __syncthreads();
  if (s_ok && !a.scatter) {
    const unsigned char* got = mine + kHeaderBytes + half + static_cast<int64_t>(p) * a.piece_bytes;
    if (a.parts == 0) {
      copy_span(a.out + static_cast<int64_t>(p) * a.piece_bytes, got, lo, hi);
    } else {
      int64_t at = 0;
      for (int i = 0; i < a.parts; ++i) {
        const int64_t from = max(lo, at), to = min(hi, at + a.part_bytes[i]);
        if (from < to) copy_span(a.part_out[i] + static_cast<int64_t>(p) * a.part_bytes[i], got + at, from - at, to - at);
        at += a.part_bytes[i];
      }
    }
  }
}

// out[i] = sum over source ranks (in rank order) of slot[src][i], i < count; one rounding to out_dtype.
__global__ void __launch_bounds__(kThreads) peer_sum_kernel(const unsigned char* const* buffers, int rank, int world,
                                                            int64_t half_bytes, int64_t count, void* out, int out_dtype,
                                                            int dest_for_epoch) {
  const unsigned char* mine = buffers[rank];
  // the exchange that just ran recorded its epoch for every destination; they are all equal
  const unsigned int epoch = reinterpret_cast<const unsigned int*>(mine + kEpochsAt)[dest_for_epoch];
  const int64_t half = (epoch & 1u) ? half_bytes : 0;
  const float* slots = reinterpret_cast<const float*>(mine + kHeaderBytes + half);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(kThreads) + threadIdx.x; i < count;
       i += static_cast<int64_t>(gridDim.x) * kThreads) {
    float acc = 0.0f;
    for (int s = 0; s < world; ++s) acc += slots[static_cast<int64_t>(s) * count + i];
    store_f32(out, i, out_dtype, acc);
  }
}

int32_t check_group(const char* op, const dq_peer_group* g, int64_t piece_bytes) {
  DQ_REQUIRE(g != nullptr && g->buffers != nullptr, "%s: null peer group", op);
  DQ_REQUIRE(g->world >= 1 && g->world <= kMaxWorld && g->rank >= 0 && g->rank < g->world,
             "%s: rank %d of %d (at most %d ranks)", op, g->rank, g->world, kMaxWorld);
  DQ_REQUIRE(g->buffer_bytes > kHeaderBytes, "%s: the exchange buffer must exceed its %d-byte header", op, kHeaderBytes);
  const int64_t half = ((g->buffer_bytes - kHeaderBytes) / 2) / 16 * 16;
  DQ_REQUIRE(piece_bytes >= 0 && piece_bytes * g->world <= half,
             "%s: %d pieces of %lld bytes need %lld bytes per half of the exchange buffer, which has %lld", op, g->world,
             static_cast<long long>(piece_bytes), static_cast<long long>(piece_bytes * g->world),
             static_cast<long long>(half));
  return DQ_OK;
}

int32_t launch_exchange(const dq_peer_group* g, Args a, int64_t piece_bytes, int scatter, cudaStream_t stream) {
  a.buffers = reinterpret_cast<unsigned char* const*>(g->buffers);
  a.half_bytes = ((g->buffer_bytes - kHeaderBytes) / 2) / 16 * 16;
  a.world = g->world;
  a.rank = g->rank;
  a.ctas_per_peer = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(kMaxCtasPerPeer, piece_bytes / 16384)));
  a.spin_limit = g->spin_limit > 0 ? g->spin_limit : (1 << 22);
  a.piece_bytes = piece_bytes;
  a.scatter = scatter;
  peer_exchange_kernel<<<g->world * a.ctas_per_peer, kThreads, 0, stream>>>(a);
  DQ_CHECK_LAUNCH("peer exchange");
  return DQ_OK;
}

}  // namespace peer
}  // namespace dq

extern "C" {

int64_t dq_peer_header_bytes(void) { return dq::peer::kHeaderBytes; }

int32_t dq_peer_all_gather(const dq_peer_group* group, const void* src, int64_t bytes, void* out, void* stream) {
  using namespace dq;
  if (const int32_t rc = peer::check_group("peer_all_gather", group, bytes)) return rc;
  DQ_REQUIRE(bytes == 0 || (src != nullptr && out != nullptr), "peer_all_gather: null source or output");
  DQ_REQUIRE(bytes % 16 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0,
             "peer_all_gather: the piece must be a multiple of 16 bytes and both pointers 16-byte aligned");
  if (bytes == 0) return DQ_OK;
  peer::Args a = {};
  a.src = static_cast<const unsigned char*>(src);
  a.out = static_cast<unsigned char*>(out);
  return peer::launch_exchange(group, a, bytes, 0, static_cast<cudaStream_t>(stream));
}

int32_t dq_peer_all_gather_parts(const dq_peer_group* group, const void* const* srcs, const int64_t* bytes,
                                 void* const* outs, int32_t parts, void* stream) {
  using namespace dq;
  DQ_REQUIRE(parts >= 1 && parts <= peer::kMaxParts && srcs != nullptr && bytes != nullptr && outs != nullptr,
             "peer_all_gather_parts: 1..%d parts, got %d", peer::kMaxParts, parts);
  int64_t total = 0;
  for (int i = 0; i < parts; ++i) {
    DQ_REQUIRE(bytes[i] > 0 && bytes[i] % 16 == 0 && srcs[i] != nullptr && outs[i] != nullptr &&
                   reinterpret_cast<uintptr_t>(srcs[i]) % 16 == 0 && reinterpret_cast<uintptr_t>(outs[i]) % 16 == 0,
               "peer_all_gather_parts: part %d must be a positive multiple of 16 bytes with 16-byte aligned pointers", i);
    total += bytes[i];
  }
  if (const int32_t rc = peer::check_group("peer_all_gather_parts", group, total)) return rc;
  peer::Args a = {};
  a.parts = parts;
  for (int i = 0; i < parts; ++i) {
    a.part_src[i] = static_cast<const unsigned char*>(srcs[i]);
    a.part_out[i] = static_cast<unsigned char*>(outs[i]);
    a.part_bytes[i] = bytes[i];
  }
  return peer::launch_exchange(group, a, total, 0, static_cast<cudaStream_t>(stream));
}

int32_t dq_peer_reduce_scatter_f32(const dq_peer_group* group, const float* partial, int64_t count, void* out,
                                   int32_t out_dtype, void* stream) {
  using namespace dq;
  const int64_t bytes = count * 4;
  if (const int32_t rc = peer::check_group("peer_reduce_scatter", group, bytes)) return rc;
  DQ_REQUIRE(count == 0 || (partial != nullptr && out != nullptr), "peer_reduce_scatter: null source or output");
  DQ_REQUIRE(dtype_ok(out_dtype), "peer_reduce_scatter: unsupported output dtype tag %d", out_dtype);
  DQ_REQUIRE(count % 4 == 0 && reinterpret_cast<uintptr_t>(partial) % 16 == 0,
             "peer_reduce_scatter: count must be a multiple of 4 and the source 16-byte aligned");
  if (count == 0) return DQ_OK;
  auto s = static_cast<cudaStream_t>(stream);
  peer::Args a = {};
  a.src = reinterpret_cast<const unsigned char*>(partial);
  if (const int32_t rc = peer::launch_exchange(group, a, bytes, 1, s)) return rc;
  const int grid = static_cast<int>(std::min<int64_t>(148, ceil_div(count, peer::kThreads)));
  peer::peer_sum_kernel<<<grid, peer::kThreads, 0, s>>>(reinterpret_cast<const unsigned char* const*>(group->buffers),
                                                        group->rank, group->world,
                                                        ((group->buffer_bytes - peer::kHeaderBytes) / 2) / 16 * 16, count, out,
                                                        out_dtype, 0);
  DQ_CHECK_LAUNCH("peer sum");
  return DQ_OK;
}

int32_t dq_peer_status(const dq_peer_group* group, const void* local_buffer, void* stream) {
  using namespace dq;
  DQ_REQUIRE(group != nullptr && local_buffer != nullptr, "peer_status: null argument");
  auto s = static_cast<cudaStream_t>(stream);
  unsigned int word = 0;
  DQ_CUDA(cudaMemcpyAsync(&word, static_cast<const unsigned char*>(local_buffer) + peer::kStatusAt, sizeof(word),
                          cudaMemcpyDeviceToHost, s));
  DQ_CUDA(cudaStreamSynchronize(s));
  if (word != 0u) {
    return fail(DQ_ERR_DEVICE, "peer exchange: rank %d gave up waiting for the piece of rank %u (%d polls)", group->rank,
                word >> 8, group->spin_limit > 0 ? group->spin_limit : (1 << 22));
  }
  return DQ_OK;
}

}  // extern "C"
