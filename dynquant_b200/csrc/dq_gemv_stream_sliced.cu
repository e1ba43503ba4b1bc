// The streaming kernel's body on matrices of too few rows to be a stream for it: the reduction
// axis sliced over a thread-block cluster (gemv_mma_stream_sliced_kernel, dq_gemv_mma_stream.cuh).
//
// The streaming kernel gives a warp whole rows, so it needs eight row tiles per SM and warp to fill
// the machine; below that the tiled kernel slices the reduction axis over the eight warps of ONE
// CTA (8, 4 or 2 ways, even slices), which leaves a down-projection such as 5120 x 17408 with 160
// CTAs of eight warps on 148 SMs -- a third of the warps the streaming kernel keeps resident, and the
// decode needs them.  Here the slices are CTAs of a cluster: a group of eight row tiles x up to
// eight slices of whole blocks in any proportion, two CTAs per SM, every CTA staging only its own
// part of the activation; the slices' sums meet in the cluster's first CTA through distributed
// shared memory in slice order.
#include <algorithm>
#include <map>
#include <mutex>
#include <tuple>

#include "dq_gemv.cuh"
#include "dq_gemv_mma_stream.cuh"

namespace dq {
namespace {

// Clusters of `slices` CTAs with `smem` bytes each that the device holds at once, per kernel build.
template <typename Kernel>
int active_clusters(int tag, Kernel kernel, int slices, size_t smem) {
  static std::mutex mu;
  static std::map<std::tuple<int, int, size_t>, int> cache;
  const auto key = std::make_tuple(tag, slices, smem);
  {
    std::lock_guard<std::mutex> lock(mu);
    const auto it = cache.find(key);
    if (it != cache.end()) return it->second;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1, static_cast<unsigned>(slices));
  cfg.blockDim = dim3(stream::kThreads);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = static_cast<unsigned>(slices);
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess ||
      cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
    (void)cudaGetLastError();
    n = 0;
  }
  std::lock_guard<std::mutex> lock(mu);
  cache[key] = n;
  return n;
}

template <int BITS>
int32_t launch_sliced(const GemvArgs& a, const DeviceInfo& dev, cudaStream_t stream_h, bool* taken) {
  using C = stream::Cfg<BITS>;
  const int steps = a.words_per_row / (4 * BITS);
  if (reinterpret_cast<uintptr_t>(a.packed) % 16 != 0 || (static_cast<int64_t>(a.words_per_row) * 4) % 16 != 0) return DQ_OK;
  if (a.group_values != 128 || steps % C::P != 0 || a.num_groups != steps || a.in_features != steps * 128) return DQ_OK;
  const auto align = static_cast<uintptr_t>(C::META_BYTES);
  if (reinterpret_cast<uintptr_t>(a.scales) % align != 0 || reinterpret_cast<uintptr_t>(a.offsets) % align != 0 ||
      (static_cast<int64_t>(a.num_groups) * 2) % C::META_BYTES != 0) {
    return DQ_OK;
  }
  if ((reinterpret_cast<uintptr_t>(a.x) & 15) != 0) return DQ_OK;  // a slice of x starts on a step: stays 16-byte aligned
  const bool plan16 = BITS == 8;  // the fp16-operand plan (see launch_stream, dq_gemv_mma.cu)
  const int aregs = plan16 ? 16 : (BITS == 8 ? 32 : 16);
  const int nblocks = steps / C::P;
  const int tiles = static_cast<int>(ceil_div(a.rows, 16));
  const int row_groups = static_cast<int>(ceil_div(tiles, stream::kWarps));
  stream::Params p = {};
  p.steps = steps;
  p.tiles = tiles;
  p.magic = (plan16 || a.x_dtype != DQ_BF16) ? 0x64006400u : 0x43004300u;
  auto smem_for = [&](int slices) {
    const int slice_steps = static_cast<int>(ceil_div(nblocks, slices)) * C::P;
    const size_t stride = static_cast<size_t>(slice_steps) * aregs + 4;
    const size_t need = C::RING_BYTES + (static_cast<size_t>(a.m) * stride + aregs) * 16 + static_cast<size_t>(slice_steps) * 8 * 4 * 2;
    // At least 80 KB: two CTAs per SM, not three.  With one activation row three would fit, and the
    // CTAs of a cluster are then placed so unevenly over the SMs that the launch is slower and its
    // time erratic in the slice count (measured at 2 / 3 / 4 / 8 bits, one row: 5120 x 17408 17 / 24 /
    // 23 / 31 us with three per SM, 14 / 20 / 17 / 21 with two; 3584 x 18944 17 / 23 / 22 / 30 against
    // 13 / 18 / 15 / 18; one per SM is level with two except on 10240 x 5120, 23 against 13 at 8 bits).
    return std::max(need, static_cast<size_t>(tuning_int("DQ_B200_SLICED_MIN_SMEM_KB", 80)) << 10);
  };
  auto run = [&](auto kernel, int tag) -> int32_t {
    // The largest slice count (two blocks a slice at least) whose clusters are all resident at once,
    // then the smallest with the same longest slice.
    const int forced = tuning_int("DQ_B200_STREAM_SLICES", 0);
    int slices = 0;
    const int max_slices = std::min(8, nblocks / 2);
    if (forced > 1) {
      slices = std::min(forced, std::max(1, nblocks));
      if (slices < 2 || active_clusters(tag, kernel, slices, smem_for(slices)) < 1) return DQ_OK;
    } else {
      for (int s = max_slices; s >= 2 && slices == 0; --s) {
        const size_t smem = smem_for(s);
        if (smem <= static_cast<size_t>(dev.max_smem_optin) && active_clusters(tag, kernel, s, smem) >= row_groups) slices = s;
      }
      if (slices == 0) return DQ_OK;
      while (slices > 2 && ceil_div(nblocks, slices - 1) == ceil_div(nblocks, slices)) --slices;
    }
    const size_t smem = smem_for(slices);
    if (smem > static_cast<size_t>(dev.max_smem_optin)) return DQ_OK;
    DQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(row_groups), static_cast<unsigned>(slices));
    cfg.blockDim = dim3(stream::kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream_h;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = static_cast<unsigned>(slices);
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled_for_rows() ? 2 : 1;
    DQ_CUDA(cudaLaunchKernelEx(&cfg, kernel, a, p));
    DQ_CHECK_LAUNCH("gemv");
    note_kernel("gemv_mma_stream_sliced_kernel");
    *taken = true;
    return DQ_OK;
  };
  const bool xbf = a.x_dtype == DQ_BF16, mbf = a.meta_dtype == DQ_BF16;
  const int tag = BITS * 4 + (xbf ? 2 : 0) + (mbf ? 1 : 0);
  constexpr bool P16 = BITS == 8;
  if (xbf && mbf) return run(stream::gemv_mma_stream_sliced_kernel<BITS, true, true, P16>, tag);
  if (xbf) return run(stream::gemv_mma_stream_sliced_kernel<BITS, true, false, P16>, tag);
  if (mbf) return run(stream::gemv_mma_stream_sliced_kernel<BITS, false, true, P16>, tag);
  return run(stream::gemv_mma_stream_sliced_kernel<BITS, false, false, P16>, tag);
}

}  // namespace

// One matrix, one to eight activation rows.  *taken stays false (nothing launched) when the matrix
// or the activation does not qualify or no slice count fits the device in one wave.
int32_t launch_gemv_stream_sliced(const GemvArgs& a, int bits, cudaStream_t stream_h, bool* taken) {
  *taken = false;
  const DeviceInfo* dev = device_info();
  if (dev == nullptr) return DQ_ERR_CUDA;
  if (a.m < 1 || a.m > 8) return DQ_OK;
  if (a.x_dtype != DQ_BF16 && a.x_dtype != DQ_F16) return DQ_OK;
  if (a.meta_dtype != DQ_BF16 && a.meta_dtype != DQ_F16) return DQ_OK;
  if ((a.in_features & 7) != 0) return DQ_OK;
  switch (bits) {
    case 2:
      return launch_sliced<2>(a, *dev, stream_h, taken);
    case 3:
      return launch_sliced<3>(a, *dev, stream_h, taken);
    case 4:
      return launch_sliced<4>(a, *dev, stream_h, taken);
    default:
      return launch_sliced<8>(a, *dev, stream_h, taken);
  }
}

}  // namespace dq
