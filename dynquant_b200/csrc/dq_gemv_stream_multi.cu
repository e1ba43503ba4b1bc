// Several long matrices that share an activation -- the gate and up projections of a large
// model's MLP -- in ONE launch of the streaming kernel's body.
//
// dq_gemv_shards / dq_gemv_sequence fuse up to four jobs that read the same activation into one
// launch.  The tiled kernel takes such a launch whatever the sizes, but on matrices large enough
// to be streams of bytes rather than chains of latencies it reaches half the bandwidth of the
// streaming kernel, which only took single matrices.  Here every job gets a range of CTAs in
// proportion to its bytes and runs the streaming body compiled for its width; a CTA belongs to
// one job.  Tiles are dealt as balanced runs inside a job's range (dq_gemv_mma_stream.cuh).
#include <algorithm>

#include "dq_gemv.cuh"
#include "dq_gemv_mma_stream.cuh"

namespace dq {
namespace streammulti {

constexpr int kMaxJobs = 4;

struct Job {
  GemvArgs a;
  stream::Params p;
  int bits;
  int plan16;     // 8-bit only: the fp16-operand fragment plan
  int cta_begin;  // CTAs [cta_begin, cta_begin + cta_count) of the grid work on this job
  int cta_count;
};

struct Launch {
  Job job[kMaxJobs];
  int njobs;
};

template <bool XBF16, bool MBF16>
__global__ void __launch_bounds__(stream::kThreads, 3) gemv_mma_stream_multi_kernel(const __grid_constant__ Launch L) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int j = 0;
#pragma unroll
  for (int i = 1; i < kMaxJobs; ++i) {
    if (i < L.njobs && static_cast<int>(blockIdx.x) >= L.job[i].cta_begin) j = i;
  }
  const Job& J = L.job[j];
  const unsigned int cta = blockIdx.x - J.cta_begin, ncta = J.cta_count;
  switch (J.bits) {
    case 2:
      stream::stream_body<2, XBF16, MBF16>(J.a, J.p, cta, ncta, smem_raw);
      break;
    case 3:
      stream::stream_body<3, XBF16, MBF16>(J.a, J.p, cta, ncta, smem_raw);
      break;
    case 4:
      stream::stream_body<4, XBF16, MBF16>(J.a, J.p, cta, ncta, smem_raw);
      break;
    default:
      if (J.plan16) {
        stream::stream_body<8, XBF16, MBF16, true>(J.a, J.p, cta, ncta, smem_raw);
      } else {
        stream::stream_body<8, XBF16, MBF16, false>(J.a, J.p, cta, ncta, smem_raw);
      }
      break;
  }
}

template <int BITS>
bool job_ok(const GemvArgs& a, int steps) {
  using C = stream::Cfg<BITS>;
  if (reinterpret_cast<uintptr_t>(a.packed) % 16 != 0 || (static_cast<int64_t>(a.words_per_row) * 4) % 16 != 0) return false;
  if (a.group_values != 128 || steps % C::P != 0 || a.num_groups % C::P != 0) return false;
  const auto align = static_cast<uintptr_t>(C::META_BYTES);
  return reinterpret_cast<uintptr_t>(a.scales) % align == 0 && reinterpret_cast<uintptr_t>(a.offsets) % align == 0;
}

template <int BITS>
size_t job_smem(const GemvArgs& a, int steps, bool plan16, int* m_stride_u4) {
  using C = stream::Cfg<BITS>;
  const int aregs = plan16 ? 16 : (BITS == 8 ? 32 : 16);
  *m_stride_u4 = steps * aregs + 4;
  return C::RING_BYTES + (static_cast<size_t>(a.m) * *m_stride_u4 + aregs) * 16 + static_cast<size_t>(steps) * 8 * 4 * 2;
}

}  // namespace streammulti

// Up to four matrices that share one activation, each long enough to be streamed, in one launch.
// *taken stays false (nothing launched) when the jobs do not qualify; the caller then tries the
// tiled kernel.
int32_t launch_gemv_stream_fused(const GemvArgs* jobs, const int* bits, int n, cudaStream_t stream_h, bool* taken) {
  using namespace streammulti;
  *taken = false;
  const DeviceInfo* dev = device_info();
  if (dev == nullptr) return DQ_ERR_CUDA;
  if (n < 2 || n > kMaxJobs) return DQ_OK;
  const GemvArgs& a0 = jobs[0];
  if (a0.x_dtype != DQ_BF16 && a0.x_dtype != DQ_F16) return DQ_OK;
  if (a0.meta_dtype != DQ_BF16 && a0.meta_dtype != DQ_F16) return DQ_OK;
  Launch L = {};
  L.njobs = n;
  int64_t total_tiles = 0;
  double weight[kMaxJobs], total_weight = 0.0;
  size_t smem = 0;
  for (int i = 0; i < n; ++i) {
    const GemvArgs& a = jobs[i];
    if (a.x != a0.x || a.m != a0.m || a.x_dtype != a0.x_dtype || a.meta_dtype != a0.meta_dtype ||
        a.in_features != a0.in_features || a.out_dtype != a0.out_dtype) {
      return DQ_OK;
    }
    const int steps = a.words_per_row / (4 * bits[i]);
    const bool ok = bits[i] == 2 ? job_ok<2>(a, steps) : bits[i] == 3 ? job_ok<3>(a, steps) : bits[i] == 4 ? job_ok<4>(a, steps) : job_ok<8>(a, steps);
    if (!ok) return DQ_OK;
    Job& J = L.job[i];
    J.a = a;
    J.bits = bits[i];
    J.plan16 = (bits[i] == 8 && (a.in_features & 7) == 0 && (reinterpret_cast<uintptr_t>(a.x) & 15) == 0) ? 1 : 0;
    J.p.steps = steps;
    J.p.tiles = static_cast<int>(ceil_div(a.rows, 16));
    J.p.magic = (J.plan16 || a.x_dtype != DQ_BF16) ? 0x64006400u : 0x43004300u;
    J.p.runs = 1;
    const size_t need = bits[i] == 2 ? job_smem<2>(a, steps, false, &J.p.m_stride_u4)
                        : bits[i] == 3 ? job_smem<3>(a, steps, false, &J.p.m_stride_u4)
                        : bits[i] == 4 ? job_smem<4>(a, steps, false, &J.p.m_stride_u4)
                                       : job_smem<8>(a, steps, J.plan16 != 0, &J.p.m_stride_u4);
    smem = std::max(smem, need);
    // every job a stream of its own: at least two row tiles per SM (and see the total below)
    if (J.p.tiles < 2 * dev->sm_count) return DQ_OK;
    total_tiles += J.p.tiles;
    weight[i] = static_cast<double>(J.p.tiles) * (bits[i] + 0.25);  // ~ bytes: codes + metadata per value
    total_weight += weight[i];
  }
  // The streaming body needs every resident warp busy (three CTAs of eight warps per SM, a ring of
  // two to three blocks each) to cover the memory latency: below a row tile per resident warp it is
  // a chain of latencies per warp and the tiled kernel, which slices the reduction axis over warps,
  // is faster (measured, the gate / up pair of a 14B model, 2 x 17408 x 5120 at 3 and 4 bits, 14.7
  // tiles per SM: the step of 40 such layers 3.22 ms here against 3.04 ms).  A build with rings of
  // six blocks and one CTA per SM -- the same bytes in flight from a third of the warps -- was
  // measured on such sizes too: within +-9 % of the tiled kernel on single matrices (14336 x 4096,
  // 17408 x 5120) and slower on the pair (35 against 29 us).  Those sizes sit at launch latency
  // plus the decode-bound streaming rate in either kernel.
  if (total_tiles < static_cast<int64_t>(dev->sm_count) * stream::kWarps * 3) return DQ_OK;
  if (smem > static_cast<size_t>(dev->max_smem_optin)) return DQ_OK;

  auto run = [&](auto kernel) -> int32_t {
    DQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    int per_sm = 0;
    DQ_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, stream::kThreads, smem));
    const int resident = std::max(1, per_sm) * dev->sm_count;
    // CTAs in proportion to the jobs' bytes, every job at least one, no job more CTAs than tiles
    int grid = 0;
    for (int i = 0; i < n; ++i) {
      int c = static_cast<int>(resident * weight[i] / total_weight);
      c = std::max(1, std::min(c, L.job[i].p.tiles));
      L.job[i].cta_begin = grid;
      L.job[i].cta_count = c;
      grid += c;
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
    cfg.numAttrs = pdl_enabled_for_rows() ? 1 : 0;
    DQ_CUDA(cudaLaunchKernelEx(&cfg, kernel, L));
    DQ_CHECK_LAUNCH("gemv");
    note_kernel("gemv_mma_stream_multi_kernel");
    *taken = true;
    return DQ_OK;
  };
  const bool xbf = a0.x_dtype == DQ_BF16, mbf = a0.meta_dtype == DQ_BF16;
  if (xbf && mbf) return run(gemv_mma_stream_multi_kernel<true, true>);
  if (xbf) return run(gemv_mma_stream_multi_kernel<true, false>);
  if (mbf) return run(gemv_mma_stream_multi_kernel<false, true>);
  return run(gemv_mma_stream_multi_kernel<false, false>);
}

}  // namespace dq
