// Shared host/device helpers for the sm_100a kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>

#include "dynquant_b200.h"

namespace dq {

constexpr int kWarp = 32;

// ---- error plumbing --------------------------------------------------------

// Message of the last failed call on this thread (dq_last_error()).
char* error_buffer();
constexpr int kErrorBufferSize = 1024;

inline int32_t fail(dq_status status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), kErrorBufferSize, fmt, ap);
  va_end(ap);
  return static_cast<int32_t>(status);
}

#define DQ_REQUIRE(cond, ...)                        \
  do {                                               \
    if (!(cond)) {                                   \
      return ::dq::fail(DQ_ERR_INVALID, __VA_ARGS__); \
    }                                                \
  } while (0)

#define DQ_CUDA(call)                                                                     \
  do {                                                                                    \
    const cudaError_t dq_err__ = (call);                                                  \
    if (dq_err__ != cudaSuccess) {                                                        \
      return ::dq::fail(DQ_ERR_CUDA, "%s failed: %s (%s:%d)", #call,                      \
                        cudaGetErrorString(dq_err__), __FILE__, __LINE__);                \
    }                                                                                     \
  } while (0)

// Checked right after a launch, like the reference's DYNQUANT_CHECK_LAUNCH
// (csrc/include/dynquant/common.cuh:26-38): configuration errors surface here,
// not at some later synchronisation.
#define DQ_CHECK_LAUNCH(what)                                                             \
  do {                                                                                    \
    ::dq::count_launch();                                                                 \
    const cudaError_t dq_err__ = cudaGetLastError();                                      \
    if (dq_err__ != cudaSuccess) {                                                        \
      return ::dq::fail(DQ_ERR_CUDA, "%s: kernel launch failed: %s", what,                \
                        cudaGetErrorString(dq_err__));                                    \
    }                                                                                     \
  } while (0)

// ---- host-side helpers -----------------------------------------------------

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

inline int dtype_size(int32_t dtype) { return dtype == DQ_F32 ? 4 : 2; }

inline const char* dtype_name(int32_t dtype) {
  switch (dtype) {
    case DQ_F16:
      return "Half";
    case DQ_BF16:
      return "BFloat16";
    case DQ_F32:
      return "Float";
    default:
      return "?";
  }
}

inline bool dtype_ok(int32_t dtype) { return dtype == DQ_F16 || dtype == DQ_BF16 || dtype == DQ_F32; }

// Values in the smallest run of whole words, per width (16 / 32 / 8 / 4).
inline int values_per_block(int bits) {
  switch (bits) {
    case 2:
      return 16;
    case 3:
      return 32;
    case 4:
      return 8;
    case 8:
      return 4;
    default:
      return 0;
  }
}

struct DeviceInfo {
  int device;
  int sm_count;
  int max_smem_optin;  // bytes per CTA
};
// Cached per device; returns nullptr and sets the error on failure.
const DeviceInfo* device_info();

// Launch-shape overrides used by the sweeps that chose the built-in heuristics.  They exist only in
// a tuning build (-DDQ_TUNING, `python -m dynquant_b200.build --tuning`), where they are read from
// the environment at every launch; a normal build returns the fallback and reads nothing.  The
// switches a user may need (DQ_B200_GEMV_PATH, DQ_B200_NO_PDL, DYNQUANT_GEMV_SCALAR) are not here.
inline int tuning_int(const char* name, int fallback = 0) {
#ifdef DQ_TUNING
  const char* v = std::getenv(name);
  return v != nullptr ? std::atoi(v) : fallback;
#else
  (void)name;
  return fallback;
#endif
}

// Process-wide count of the kernels this library has launched (dq_launch_count).
void count_launch();
// Name of the kernel the calling thread launched last (dq_last_kernel): lets a test prove which
// of the kernels a shape was dispatched to.
void note_kernel(const char* name);

// ---- device-side dtype helpers ---------------------------------------------

#ifdef __CUDACC__

// Element `i` of an array of the tagged dtype, widened to fp32 (exact).
__device__ __forceinline__ float load_f32(const void* __restrict__ p, int64_t i, int dtype) {
  if (dtype == DQ_F16) {
    return __half2float(__ldg(reinterpret_cast<const __half*>(p) + i));
  }
  if (dtype == DQ_BF16) {
    const unsigned short raw = __ldg(reinterpret_cast<const unsigned short*>(p) + i);
    return __uint_as_float(static_cast<uint32_t>(raw) << 16);
  }
  return __ldg(reinterpret_cast<const float*>(p) + i);
}

// One rounding (nearest-even) to the tagged dtype.
__device__ __forceinline__ void store_f32(void* __restrict__ p, int64_t i, int dtype, float v) {
  if (dtype == DQ_F16) {
    reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
  } else if (dtype == DQ_BF16) {
    reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  } else {
    reinterpret_cast<float*>(p)[i] = v;
  }
}

__device__ __forceinline__ uint32_t round_to_16(float v, int dtype) {
  if (dtype == DQ_F16) {
    return __half_as_ushort(__float2half_rn(v));
  }
  return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}

// Two values rounded (nearest-even) to the tagged 16-bit dtype and packed, `lo` in the low half:
// one conversion instruction for the pair.
__device__ __forceinline__ uint32_t round_pair_to_16(float lo, float hi, int dtype) {
  if (dtype == DQ_F16) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  const __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&b);
}

// Streaming 128-bit load: weights are read exactly once, so keep them out of L1.
__device__ __forceinline__ uint4 ldg_stream_128(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ uint32_t ldg_stream_32(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

// Programmatic dependent launch.  Both are no-ops unless the launch carries the
// programmatic-stream-serialization attribute.
__device__ __forceinline__ void pdl_wait_prior_grid() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

#endif  // __CUDACC__

}  // namespace dq
