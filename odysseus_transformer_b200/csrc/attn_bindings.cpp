// Python bindings of the attention kernels (flash_fwd.cu, flash_bwd.cu).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
namespace py = pybind11;

#include <stdexcept>
#include <string>

#include "ody_kernels.h"

int* ody_status_ptr(const at::Tensor& like);
void ody_count_launches(int64_t n);

namespace {

void req(bool c, const std::string& msg) {
  if (!c) throw std::runtime_error("odysseus_transformer_b200: " + msg);
}

void check_rows(const at::Tensor& t, const char* name) {
  req(t.is_cuda() && t.scalar_type() == at::kBFloat16, std::string(name) + " must be a CUDA bfloat16 tensor");
  req(t.dim() == 3 && t.size(2) == 128, std::string(name) + " must be [T, heads, 128]");
  req(t.stride(2) == 1 && t.stride(1) == 128 && t.stride(0) % 8 == 0, std::string(name) + ": heads must be packed (strides [row, 128, 1])");
}

std::vector<at::Tensor> attn_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, bool causal, double scale) {
  check_rows(q, "q"); check_rows(k, "k"); check_rows(v, "v");
  req(k.size(0) == v.size(0) && k.size(1) == v.size(1), "k/v shape mismatch");
  req(q.size(1) % k.size(1) == 0, "query heads must be a multiple of kv heads");
  req(!causal || q.size(0) == k.size(0), "causal attention needs Tq == Tk");
  c10::cuda::CUDAGuard guard(q.device());
  const int64_t Tq = q.size(0), Tk = k.size(0), H = q.size(1), Hkv = k.size(1);
  auto o = at::empty({Tq, H, 128}, q.options());
  auto lse = at::empty({H, Tq}, q.options().dtype(at::kFloat));
  int rc = ody_flash_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), (int)Tq, (int)Tk,
                         (int)H, (int)Hkv, q.stride(0), k.stride(0), v.stride(0), o.stride(0), causal ? 1 : 0, (float)scale,
                         ody_status_ptr(q), at::cuda::getCurrentCUDAStream().stream());
  req(rc == 0, "flash_fwd failed with code " + std::to_string(rc));
  ody_count_launches(1);
  return {o, lse};
}

std::vector<at::Tensor> attn_bwd(const at::Tensor& dO, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                 const at::Tensor& o, const at::Tensor& lse, bool causal, double scale,
                                 const c10::optional<at::Tensor>& dq_out, const c10::optional<at::Tensor>& dk_out,
                                 const c10::optional<at::Tensor>& dv_out) {
  check_rows(dO, "dO"); check_rows(q, "q"); check_rows(k, "k"); check_rows(v, "v"); check_rows(o, "o");
  req(lse.is_cuda() && lse.scalar_type() == at::kFloat && lse.is_contiguous(), "lse must be contiguous fp32");
  req(lse.dim() == 2 && lse.size(0) == q.size(1) && lse.size(1) == q.size(0), "lse must be [H, Tq]");
  req(dO.sizes() == q.sizes() && o.sizes() == q.sizes(), "dO / o shape mismatch");
  req(!causal || q.size(0) == k.size(0), "causal attention needs Tq == Tk");
  c10::cuda::CUDAGuard guard(q.device());
  const int64_t Tq = q.size(0), Tk = k.size(0), H = q.size(1), Hkv = k.size(1);
  at::Tensor dq = dq_out.has_value() ? dq_out.value() : at::empty({Tq, H, 128}, q.options());
  at::Tensor dk = dk_out.has_value() ? dk_out.value() : at::empty({Tk, Hkv, 128}, q.options());
  at::Tensor dv = dv_out.has_value() ? dv_out.value() : at::empty({Tk, Hkv, 128}, q.options());
  check_rows(dq, "dq"); check_rows(dk, "dk"); check_rows(dv, "dv");
  req(dq.size(0) == Tq && dq.size(1) == H && dk.size(0) == Tk && dk.size(1) == Hkv && dv.size(0) == Tk && dv.size(1) == Hkv,
      "gradient output shape mismatch");
  auto ws = at::empty({ody_flash_bwd_workspace_bytes((int)Tq, (int)H)}, q.options().dtype(at::kByte));
  int rc = ody_flash_bwd(dO.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(),
                         dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), (int)Tq, (int)Tk, (int)H, (int)Hkv,
                         dO.stride(0), q.stride(0), k.stride(0), v.stride(0), o.stride(0), dq.stride(0), dk.stride(0),
                         dv.stride(0), causal ? 1 : 0, (float)scale, ody_status_ptr(q),
                         at::cuda::getCurrentCUDAStream().stream());
  req(rc == 0, "flash_bwd failed with code " + std::to_string(rc));
  ody_count_launches(3);
  return {dq, dk, dv};
}

}  // namespace

void ody_register_attention(pybind11::module& m) {
  m.def("attn_fwd", &attn_fwd);
  m.def("attn_fwd_set_trace", [](const c10::optional<at::Tensor>& t) {
    if (t.has_value()) { req(t.value().is_cuda() && t.value().scalar_type() == at::kLong && t.value().numel() >= 48 * 8, "trace: int64 [48*8]"); ody_flash_fwd_set_trace((long long*)t.value().data_ptr()); }
    else ody_flash_fwd_set_trace(nullptr);
  });
  m.def("attn_bwd_set_trace", [](const c10::optional<at::Tensor>& t) {
    if (t.has_value()) { req(t.value().is_cuda() && t.value().scalar_type() == at::kLong && t.value().numel() >= 48 * 8, "trace: int64 [48*8]"); ody_flash_bwd_set_trace((long long*)t.value().data_ptr()); }
    else ody_flash_bwd_set_trace(nullptr);
  });
  m.def("attn_bwd", &attn_bwd, py::arg("dO"), py::arg("q"), py::arg("k"), py::arg("v"), py::arg("o"), py::arg("lse"),
        py::arg("causal"), py::arg("scale"), py::arg("dq_out") = py::none(), py::arg("dk_out") = py::none(),
        py::arg("dv_out") = py::none());
}
