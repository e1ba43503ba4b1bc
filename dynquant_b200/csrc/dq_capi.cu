// Metadata entry points, error plumbing and the host-side geometry check that
// every operator runs first.
//
// dq_resolve_geometry keeps the rules and the wording of the reference's
// resolve_geometry (packages/dynquant-kernels/csrc/include/dynquant/geometry.h:63-132):
// nothing is derived by guesswork, everything is either passed in or implied
// by a shape, and every implication is checked.
#include <atomic>
#include <mutex>

#include "dq_common.cuh"

namespace dq {

char* error_buffer() {
  static thread_local char buffer[kErrorBufferSize] = {0};
  return buffer;
}

namespace {
std::atomic<int64_t> g_launches{0};
}
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
namespace {
thread_local const char* t_last_kernel = "";
}
void note_kernel(const char* name) { t_last_kernel = name; }
const char* last_kernel() { return t_last_kernel; }
int64_t launches_so_far() { return g_launches.load(std::memory_order_relaxed); }

const DeviceInfo* device_info() {
  constexpr int kMaxDevices = 64;
  static DeviceInfo cache[kMaxDevices];
  static bool ready[kMaxDevices] = {false};
  static std::mutex mu;
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess || device < 0 || device >= kMaxDevices) {
    fail(DQ_ERR_CUDA, "cudaGetDevice failed: %s", cudaGetErrorString(err));
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!ready[device]) {
    DeviceInfo info = {};
    info.device = device;
    err = cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, device);
    if (err == cudaSuccess) {
      err = cudaDeviceGetAttribute(&info.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin,
                                   device);
    }
    if (err != cudaSuccess) {
      fail(DQ_ERR_CUDA, "cudaDeviceGetAttribute failed: %s", cudaGetErrorString(err));
      return nullptr;
    }
    cache[device] = info;
    ready[device] = true;
  }
  return &cache[device];
}

}  // namespace dq

extern "C" {

int64_t dq_launch_count(void) { return dq::launches_so_far(); }
const char* dq_last_kernel(void) { return dq::last_kernel(); }


int32_t dq_abi_version(void) { return DQ_ABI_VERSION; }
int32_t dq_built_with_cuda(void) { return 1; }
const char* dq_compiled_architectures(void) { return "sm_100a"; }
int32_t dq_gemv_max_rows(void) { return DQ_GEMV_MAX_ROWS; }
int32_t dq_moe_max_tokens(void) { return DQ_MOE_MAX_TOKENS; }
const char* dq_last_error(void) { return dq::error_buffer(); }

int32_t dq_resolve_geometry(const char* op, const dq_weight* w, dq_geometry* out) {
  if (op == nullptr) op = "dynquant";
  DQ_REQUIRE(w != nullptr && out != nullptr, "%s: null weight descriptor", op);
  const int vpb = dq::values_per_block(w->bits);
  DQ_REQUIRE(vpb > 0, "%s: unsupported bit width %d; expected one of {2, 3, 4, 8}", op, w->bits);
  DQ_REQUIRE(dq::dtype_ok(w->meta_dtype), "%s: unsupported scales dtype tag %d", op, w->meta_dtype);
  DQ_REQUIRE(w->rows >= 0 && w->words_per_row >= 0,
             "%s: packed must be 2-D [rows, words], got [%lld, %lld]", op,
             static_cast<long long>(w->rows), static_cast<long long>(w->words_per_row));
  DQ_REQUIRE(w->in_features > 0, "%s: in_features must be positive, got %lld", op,
             static_cast<long long>(w->in_features));
  DQ_REQUIRE(w->group_values > 0,
             "%s: group_values must be a resolved positive count, got %lld. The per-row sentinel "
             "(-1) is the caller's to resolve.",
             op, static_cast<long long>(w->group_values));
  DQ_REQUIRE(w->num_groups > 0, "%s: scales has zero groups", op);
  DQ_REQUIRE(w->words_per_row % w->num_groups == 0,
             "%s: %lld words per row is not divisible by %lld groups; the checkpoint is inconsistent",
             op, static_cast<long long>(w->words_per_row), static_cast<long long>(w->num_groups));
  const int64_t words_per_group = w->words_per_row / w->num_groups;
  const int64_t group_bits = w->group_values * w->bits;
  DQ_REQUIRE(words_per_group * 32 >= group_bits,
             "%s: a group of %lld values at %d-bit needs %lld words but only %lld are stored", op,
             static_cast<long long>(w->group_values), w->bits,
             static_cast<long long>((group_bits + 31) / 32), static_cast<long long>(words_per_group));
  if (w->num_groups > 1) {
    DQ_REQUIRE(group_bits % 32 == 0,
               "%s: group_values=%lld at %d-bit occupies %lld bits, not a whole number of words, so "
               "group 1 would begin mid-word. group_values must be a multiple of %d unless the whole "
               "row is one group.",
               op, static_cast<long long>(w->group_values), w->bits,
               static_cast<long long>(group_bits), DQ_GROUP_SIZE_ALIGNMENT);
    DQ_REQUIRE(words_per_group * 32 == group_bits,
               "%s: %lld words per group does not match %lld bits of payload", op,
               static_cast<long long>(words_per_group), static_cast<long long>(group_bits));
    DQ_REQUIRE(w->num_groups * w->group_values >= w->in_features,
               "%s: %lld groups of %lld cover %lld values, short of in_features=%lld", op,
               static_cast<long long>(w->num_groups), static_cast<long long>(w->group_values),
               static_cast<long long>(w->num_groups * w->group_values),
               static_cast<long long>(w->in_features));
  } else {
    DQ_REQUIRE(w->group_values == w->in_features,
               "%s: a single group must span the row exactly; got group_values=%lld for "
               "in_features=%lld",
               op, static_cast<long long>(w->group_values), static_cast<long long>(w->in_features));
  }
  DQ_REQUIRE(w->rows == 0 || (w->packed != nullptr && w->scales != nullptr),
             "%s: null packed or scales pointer", op);
  DQ_REQUIRE(w->rows < (int64_t{1} << 31) && w->words_per_row < (int64_t{1} << 31) &&
                 w->in_features < (int64_t{1} << 31),
             "%s: tensor dimensions exceed 32-bit indexing", op);
  DQ_REQUIRE(reinterpret_cast<uintptr_t>(w->packed) % 4 == 0 &&
                 reinterpret_cast<uintptr_t>(w->scales) % dq::dtype_size(w->meta_dtype) == 0 &&
                 reinterpret_cast<uintptr_t>(w->offsets) % dq::dtype_size(w->meta_dtype) == 0,
             "%s: misaligned packed / scales / offsets pointer", op);

  out->group_values = static_cast<int32_t>(w->group_values);
  out->num_groups = static_cast<int32_t>(w->num_groups);
  out->words_per_group = static_cast<int32_t>(words_per_group);
  out->words_per_row = static_cast<int32_t>(w->words_per_row);
  out->in_features = static_cast<int32_t>(w->in_features);
  out->blocks_per_group = static_cast<int32_t>((w->group_values + vpb - 1) / vpb);
  out->blocks_per_row = out->num_groups * out->blocks_per_group;
  return DQ_OK;
}

}  // extern "C"
