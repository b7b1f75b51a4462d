// Python-side description of the work folded into a GEMM epilogue -> OdyEpilogue (ody_kernels.h), with every check that
// keeps a bad description from reaching a kernel.  Shared by the plain and the fused-collective GEMM bindings.
#pragma once
#include <torch/extension.h>

#include <stdexcept>
#include <string>

#include "ody_kernels.h"

namespace ody_epi {

inline void need(bool ok, const char* what) {
  if (!ok) throw std::runtime_error(std::string("gemm epilogue: ") + what);
}

// rope: None or (cos [rows, 64] fp32, sin [rows, 64] fp32, rot_cols, period_cols); residual: None or bf16 [res_rows, N].
// rows / res_rows: the output rows the kernel indexes the tables / the residual with.  Returns false when nothing is asked.
inline bool fill(const pybind11::object& rope, const c10::optional<at::Tensor>& residual, int64_t rows, int64_t res_rows,
                 int64_t N, const at::Device& dev, OdyEpilogue& e) {
  memset(&e, 0, sizeof(e));
  bool any = false;
  if (!rope.is_none()) {
    pybind11::tuple t = rope.cast<pybind11::tuple>();
    need(t.size() == 4, "rope = (cos, sin, rot_cols, period_cols)");
    at::Tensor cos = t[0].cast<at::Tensor>(), sin = t[1].cast<at::Tensor>();
    const int64_t rot = t[2].cast<int64_t>(), period = t[3].cast<int64_t>();
    need(cos.is_cuda() && sin.is_cuda() && cos.device() == dev && sin.device() == dev, "rope tables on another device");
    need(cos.scalar_type() == at::kFloat && sin.scalar_type() == at::kFloat && cos.is_contiguous() && sin.is_contiguous(),
         "rope tables: fp32 contiguous");
    need(cos.dim() == 2 && cos.size(1) == 64 && cos.size(0) == rows && sin.sizes() == cos.sizes(),
         "rope tables must be [output rows, 64] (head_dim 128)");
    need(period > 0 && period % 128 == 0 && rot >= 0 && rot % 128 == 0 && rot <= period && N % period == 0,
         "rope: columns, period and rotated columns disagree");
    need(period < (int64_t(1) << 31), "rope: period too large");
    e.rope_cos = cos.data_ptr<float>();
    e.rope_sin = sin.data_ptr<float>();
    e.rope_rot_cols = (int)rot;
    e.rope_period_cols = (int)period;
    any = true;
  }
  if (residual.has_value()) {
    const at::Tensor& r = residual.value();
    need(r.is_cuda() && r.device() == dev && r.scalar_type() == at::kBFloat16, "residual: bf16 on the operands' device");
    need(r.dim() == 2 && r.size(0) == res_rows && r.size(1) == N && r.stride(1) == 1 && r.stride(0) % 8 == 0,
         "residual must be [output rows, N] with packed columns");
    need((reinterpret_cast<uintptr_t>(r.data_ptr()) & 15) == 0, "residual: 16-byte aligned");
    e.residual = r.data_ptr();
    e.residual_ld = r.stride(0);
    any = true;
  }
  return any;
}

}  // namespace ody_epi
