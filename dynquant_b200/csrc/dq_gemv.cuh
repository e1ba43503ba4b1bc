// Argument block and output store shared by the GEMV kernels.
#pragma once

#include "dq_common.cuh"

namespace dq {

struct GemvArgs {
  const void* x;
  const uint32_t* packed;
  const void* scales;
  const void* offsets;  // may be null
  const void* bias;     // may be null; [rows] in out_dtype, indexed from out_col0
  void* out;
  int64_t out_stride;  // elements between consecutive activation rows of out
  int64_t out_col0;    // first output column this weight writes
  int x_dtype, meta_dtype, out_dtype;
  int m;     // real activation rows
  int rows;  // output features of this weight
  int words_per_row, num_groups, words_per_group, group_values, in_features;
  int chunks_per_row, chunks_per_group;  // fast path only
};

namespace peerpush {
struct Push;  // dq_peer_push.cuh
}

// Tensor-core path (dq_gemv_mma.cu).  Returns DQ_ERR_UNSUPPORTED without touching
// the error buffer when the geometry or dtype is not one it handles, so the
// caller can fall through to the SIMT kernels.
bool mma_path_supports(const GemvArgs& a, int bits);
// `push` (optional): the launch also replicates its output rows into every rank's window and
// ends with the bounded wait for the other ranks' rows; only the streaming and the tiled kernel
// do that, so with `push` every other geometry returns DQ_ERR_UNSUPPORTED, nothing launched.
int32_t launch_gemv_mma(const GemvArgs& a, int bits, cudaStream_t stream, const peerpush::Push* push = nullptr);
// Up to four matrices that share one activation, in ONE launch.  *taken is false (and nothing
// was launched) when the jobs do not qualify; the caller then launches them one by one.
int32_t launch_gemv_mma_fused(const GemvArgs* jobs, const int* bits, int n, cudaStream_t stream, bool* taken,
                              const peerpush::Push* push = nullptr);

// Two to four long matrices that share an activation in one launch of the streaming kernel's body
// (dq_gemv_stream_multi.cu).  *taken stays false, nothing launched, when they do not qualify.
int32_t launch_gemv_stream_fused(const GemvArgs* jobs, const int* bits, int n, cudaStream_t stream, bool* taken);
// One to eight activation rows against one matrix of too few rows for the streaming kernel: its
// body with the reduction axis sliced over a thread-block cluster (dq_gemv_stream_sliced.cu).
int32_t launch_gemv_stream_sliced(const GemvArgs& a, int bits, cudaStream_t stream, bool* taken);
// min_rows..64 activation rows against one matrix in one pass over the weights (dq_gemv_rows.cu).
// *taken stays false, nothing launched, when the matrix or the activation does not qualify.
int32_t launch_gemv_rows(const GemvArgs& a, int bits, cudaStream_t stream, bool* taken, int min_rows = 9);
// False when DQ_B200_GEMV_PATH=simt forces the SIMT kernels.
bool mma_enabled_for_rows();
// False when DQ_B200_NO_PDL drops the programmatic-dependent-launch attribute.
bool pdl_enabled_for_rows();

#ifdef __CUDACC__
__device__ __forceinline__ void store_out(const GemvArgs& a, int m, int row, float v) {
  const int64_t col = a.out_col0 + row;
  if (a.bias != nullptr) {
    v += load_f32(a.bias, col, a.out_dtype);
  }
  store_f32(a.out, static_cast<int64_t>(m) * a.out_stride + col, a.out_dtype, v);
}

#endif

}  // namespace dq
