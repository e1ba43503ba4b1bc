// CUDA implementations of torch.ops.dynquant.{gemv, dequant} in C++, over the C ABI.
//
// The operators' schemas are defined by the Python package (dynquant_b200/ops.py, the schema
// strings of the reference's bindings.cpp:209-214); this file only attaches the CUDA backend,
// the way the reference's own kernels do (TORCH_LIBRARY_IMPL(dynquant, CUDA, m),
// csrc/gemv/gemv.cu:760, csrc/quant/dequant.cu:169).  A call then costs one dispatcher hop and
// one C call instead of a Python function plus ctypes marshalling: the reference measures
// 20-45 us of host time per packed module per decode step (experiments/four_point/
// RESULTS.md:884-892), and this is the part of it a kernel library can remove.
//
// Checks and messages follow dynquant_b200/ops.py::weight_descriptor (the tensor-level half of
// resolve_geometry, csrc/include/dynquant/geometry.h:71-86); the arithmetic half runs in the
// library.  No CPU implementation is registered: CPU tensors reach the Python-side refusal.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "dynquant_b200.h"

namespace {

int32_t dtype_tag(at::ScalarType t, const char* what) {
  switch (t) {
    case at::kHalf: return DQ_F16;
    case at::kBFloat16: return DQ_BF16;
    case at::kFloat: return DQ_F32;
    default: TORCH_CHECK(false, what, ": unsupported dtype ", t, "; expected float16, bfloat16 or float32");
  }
  return -1;
}

dq_weight describe(const char* op, const at::Tensor& packed, const at::Tensor& scales,
                   const std::optional<at::Tensor>& offsets, int64_t bits, int64_t group_values, int64_t in_features) {
  TORCH_CHECK(packed.dim() == 2, op, ": packed must be 2-D [rows, words], got ", packed.sizes());
  TORCH_CHECK(packed.scalar_type() == at::kInt, op, ": packed must be int32 (unsigned bit patterns stored as int32), got ",
              packed.scalar_type());
  TORCH_CHECK(scales.dim() == 2, op, ": scales must be 2-D [rows, groups], got ", scales.sizes());
  TORCH_CHECK(packed.size(0) == scales.size(0), op, ": packed has ", packed.size(0), " rows but scales has ", scales.size(0));
  TORCH_CHECK(packed.is_contiguous() && scales.is_contiguous(), op, ": packed and scales must be contiguous");
  TORCH_CHECK(packed.is_cuda(), op, ": packed is on ", packed.device(), "; dynquant_b200 has only sm_100a kernels and no CPU fallback");
  TORCH_CHECK(scales.device() == packed.device(), op, ": scales is on ", scales.device(), " but packed is on ", packed.device());
  const void* off = nullptr;
  if (offsets.has_value() && offsets->defined()) {
    TORCH_CHECK(offsets->sizes() == scales.sizes(), op, ": offsets shape ", offsets->sizes(), " != scales shape ", scales.sizes());
    TORCH_CHECK(offsets->scalar_type() == scales.scalar_type(), op, ": offsets dtype ", offsets->scalar_type(), " != scales dtype ",
                scales.scalar_type());
    TORCH_CHECK(offsets->is_contiguous(), op, ": offsets must be contiguous");
    TORCH_CHECK(offsets->device() == packed.device(), op, ": offsets is on ", offsets->device(), " but packed is on ", packed.device());
    off = offsets->const_data_ptr();
  }
  dq_weight w = {};
  w.packed = packed.const_data_ptr();
  w.scales = scales.const_data_ptr();
  w.offsets = off;
  w.rows = packed.size(0);
  w.words_per_row = packed.size(1);
  w.num_groups = scales.size(1);
  w.group_values = group_values;
  w.in_features = in_features;
  w.bits = static_cast<int32_t>(bits);
  w.meta_dtype = dtype_tag(scales.scalar_type(), op);
  return w;
}

void check(int32_t rc) { TORCH_CHECK(rc == DQ_OK, dq_last_error()); }

at::Tensor gemv_cuda(const at::Tensor& x, const at::Tensor& packed, const at::Tensor& scales,
                     const std::optional<at::Tensor>& offsets, int64_t bits, int64_t group_values, int64_t in_features) {
  const c10::cuda::CUDAGuard guard(packed.device());
  const dq_weight w = describe("gemv", packed, scales, offsets, bits, group_values, in_features);
  dq_geometry g;
  check(dq_resolve_geometry("gemv", &w, &g));
  TORCH_CHECK(x.dim() == 2, "gemv: x must be 2-D [rows, in_features], got ", x.sizes());
  TORCH_CHECK(x.size(1) == in_features, "gemv: x has ", x.size(1), " columns but in_features is ", in_features);
  TORCH_CHECK(x.is_contiguous(), "gemv: x must be contiguous");
  TORCH_CHECK(x.device() == packed.device(), "gemv: x is on ", x.device(), " but packed is on ", packed.device());
  const int32_t tag = dtype_tag(x.scalar_type(), "gemv: x");
  at::Tensor out = at::empty({x.size(0), packed.size(0)}, x.options());
  check(dq_gemv(x.const_data_ptr(), tag, x.size(0), &w, out.data_ptr(), tag, at::cuda::getCurrentCUDAStream().stream()));
  return out;
}

at::Tensor dequant_cuda(const at::Tensor& packed, const at::Tensor& scales, const std::optional<at::Tensor>& offsets,
                        int64_t bits, int64_t group_values, int64_t in_features) {
  const c10::cuda::CUDAGuard guard(packed.device());
  const dq_weight w = describe("dequant", packed, scales, offsets, bits, group_values, in_features);
  dq_geometry g;
  check(dq_resolve_geometry("dequant", &w, &g));
  at::Tensor out = at::empty({packed.size(0), in_features}, scales.options());
  if (out.numel() == 0) return out;
  check(dq_dequant(&w, out.data_ptr(), w.meta_dtype, at::cuda::getCurrentCUDAStream().stream()));
  return out;
}

}  // namespace

TORCH_LIBRARY_IMPL(dynquant, CUDA, m) {
  m.impl("gemv", TORCH_FN(gemv_cuda));
  m.impl("dequant", TORCH_FN(dequant_cuda));
}
