// Achievable-bandwidth probes: a read-only pass and a copy over a caller-owned buffer.
//
// The reference quotes every GEMV figure against the bandwidth the card actually delivers,
// measured in the same session by a large read (`src.sum()`) and a large copy
// (packages/dynquant-core/src/dynquant/commands/bench.py:95-120, achievable_bandwidth).
// These two kernels are that measurement for this library, so that a benchmark can report
// the packed GEMV against a read-only stream issued from the same process, the same
// clocks and the same launch path instead of against a number measured elsewhere.
//
// Both kernels move 16 bytes per thread per load, eight independent loads in flight per
// thread, and a grid of a whole number of waves (SM count x resident CTAs); they are the
// shape of traffic the streaming GEMV kernel issues, minus the arithmetic.
#include <algorithm>

#include "dq_common.cuh"

namespace dq {
namespace {

constexpr int kProbeThreads = 256;
constexpr int kProbeUnroll = 8;
constexpr int kProbeCtasPerSm = 8;

__device__ __forceinline__ uint4 load_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Reads `vectors` 16-byte vectors and adds the XOR of all words read by a CTA, as an
// integer, to *sink.  The XOR keeps every load live at one integer instruction per 16 bytes.
__global__ void __launch_bounds__(kProbeThreads)
    probe_read_kernel(const uint4* __restrict__ src, int64_t vectors, unsigned long long* sink) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kProbeThreads;
  int64_t i = static_cast<int64_t>(blockIdx.x) * kProbeThreads + threadIdx.x;
  uint32_t acc = 0;
  for (; i + (kProbeUnroll - 1) * stride < vectors; i += kProbeUnroll * stride) {
    uint4 v[kProbeUnroll];
#pragma unroll
    for (int u = 0; u < kProbeUnroll; ++u) v[u] = load_stream(src + i + u * stride);
#pragma unroll
    for (int u = 0; u < kProbeUnroll; ++u) acc ^= v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
  }
  for (; i < vectors; i += stride) {
    const uint4 v = load_stream(src + i);
    acc ^= v.x ^ v.y ^ v.z ^ v.w;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc ^= __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ uint32_t warp_acc[kProbeThreads / 32];
  if ((threadIdx.x & 31) == 0) warp_acc[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t total = 0;
#pragma unroll
    for (int w = 0; w < kProbeThreads / 32; ++w) total ^= warp_acc[w];
    atomicXor(sink, static_cast<unsigned long long>(total));  // XOR commutes: order-free
  }
}

__global__ void __launch_bounds__(kProbeThreads)
    probe_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int64_t vectors) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kProbeThreads;
  int64_t i = static_cast<int64_t>(blockIdx.x) * kProbeThreads + threadIdx.x;
  for (; i + (kProbeUnroll - 1) * stride < vectors; i += kProbeUnroll * stride) {
    uint4 v[kProbeUnroll];
#pragma unroll
    for (int u = 0; u < kProbeUnroll; ++u) v[u] = load_stream(src + i + u * stride);
#pragma unroll
    for (int u = 0; u < kProbeUnroll; ++u) __stcs(dst + i + u * stride, v[u]);
  }
  for (; i < vectors; i += stride) __stcs(dst + i, load_stream(src + i));
}

int probe_grid(const DeviceInfo* dev, int64_t vectors) {
  const int64_t wave = static_cast<int64_t>(dev->sm_count) * kProbeCtasPerSm;
  return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(wave, ceil_div(vectors, kProbeThreads))));
}

}  // namespace
}  // namespace dq

extern "C" int32_t dq_probe_read(const void* src, int64_t bytes, uint64_t* sink, void* stream) {
  DQ_REQUIRE(bytes >= 0 && bytes % 16 == 0, "probe_read: size must be a multiple of 16 bytes, got %lld",
             static_cast<long long>(bytes));
  if (bytes == 0) return DQ_OK;
  DQ_REQUIRE(src != nullptr && sink != nullptr, "probe_read: null pointer");
  DQ_REQUIRE(reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(sink) % 8 == 0,
             "probe_read: the buffer must be 16-byte aligned and the sink 8-byte aligned");
  const dq::DeviceInfo* dev = dq::device_info();
  if (dev == nullptr) return DQ_ERR_CUDA;
  const int64_t vectors = bytes / 16;
  dq::probe_read_kernel<<<dq::probe_grid(dev, vectors), dq::kProbeThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), vectors, reinterpret_cast<unsigned long long*>(sink));
  DQ_CHECK_LAUNCH("probe_read");
  return DQ_OK;
}

extern "C" int32_t dq_probe_copy(void* dst, const void* src, int64_t bytes, void* stream) {
  DQ_REQUIRE(bytes >= 0 && bytes % 16 == 0, "probe_copy: size must be a multiple of 16 bytes, got %lld",
             static_cast<long long>(bytes));
  if (bytes == 0) return DQ_OK;
  DQ_REQUIRE(src != nullptr && dst != nullptr, "probe_copy: null pointer");
  DQ_REQUIRE(reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0,
             "probe_copy: both buffers must be 16-byte aligned");
  const char* s = static_cast<const char*>(src);
  const char* d = static_cast<const char*>(dst);
  DQ_REQUIRE(d + bytes <= s || s + bytes <= d, "probe_copy: the buffers overlap");
  const dq::DeviceInfo* dev = dq::device_info();
  if (dev == nullptr) return DQ_ERR_CUDA;
  const int64_t vectors = bytes / 16;
  dq::probe_copy_kernel<<<dq::probe_grid(dev, vectors), dq::kProbeThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), vectors);
  DQ_CHECK_LAUNCH("probe_copy");
  return DQ_OK;
}
