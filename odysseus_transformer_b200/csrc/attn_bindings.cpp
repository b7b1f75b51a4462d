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

// The backward launchers build V's tensor map from k's row count and head count: a shorter or narrower v would be
// read past its end.  Every tensor must also live on q's device, where the kernels run.
void check_kv_and_devices(const at::Tensor& dO, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                          const at::Tensor& o, const at::Tensor& lse) {
  req(k.size(0) == v.size(0) && k.size(1) == v.size(1), "k / v shape mismatch");
  req(k.size(1) > 0 && q.size(1) % k.size(1) == 0, "query heads must be a multiple of kv heads");
  const auto dev = q.get_device();
  req(dO.get_device() == dev && k.get_device() == dev && v.get_device() == dev && o.get_device() == dev &&
          lse.get_device() == dev, "all attention tensors must be on q's device");
}

std::vector<at::Tensor> attn_bwd(const at::Tensor& dO, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                 const at::Tensor& o, const at::Tensor& lse, bool causal, double scale,
                                 const c10::optional<at::Tensor>& dq_out, const c10::optional<at::Tensor>& dk_out,
                                 const c10::optional<at::Tensor>& dv_out) {
  check_rows(dO, "dO"); check_rows(q, "q"); check_rows(k, "k"); check_rows(v, "v"); check_rows(o, "o");
  req(lse.is_cuda() && lse.scalar_type() == at::kFloat && lse.is_contiguous(), "lse must be contiguous fp32");
  req(lse.dim() == 2 && lse.size(0) == q.size(1) && lse.size(1) == q.size(0), "lse must be [H, Tq]");
  req(dO.sizes() == q.sizes() && o.sizes() == q.sizes(), "dO / o shape mismatch");
  check_kv_and_devices(dO, q, k, v, o, lse);
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

// Split forms for the Ulysses exchange.  Destination tensors may live in a peer's symmetric memory; they are only
// ever written by this package's own kernels.
void check_split(const std::vector<at::Tensor>& d, int64_t rows, int64_t heads, const char* name) {
  req(!d.empty() && d.size() <= 8, std::string(name) + ": 1..8 destinations");
  for (const auto& t : d) {
    check_rows(t, name);
    req(t.size(0) == rows && t.size(1) == heads && t.stride(0) == d[0].stride(0), std::string(name) + ": destination shape / pitch mismatch");
  }
}

// attn_fwd that ALSO stores output rows [d * rows, (d + 1) * rows) to dests[d] ([rows, H, 128])
std::vector<at::Tensor> attn_fwd_split(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, bool causal, double scale,
                                       const std::vector<at::Tensor>& dests) {
  check_rows(q, "q"); check_rows(k, "k"); check_rows(v, "v");
  req(k.size(0) == v.size(0) && k.size(1) == v.size(1) && q.size(1) % k.size(1) == 0, "q/k/v shape mismatch");
  req(!causal || q.size(0) == k.size(0), "causal attention needs Tq == Tk");
  const int64_t Tq = q.size(0), Tk = k.size(0), H = q.size(1), Hkv = k.size(1);
  const int64_t rows = dests.empty() ? 0 : dests[0].size(0);
  check_split(dests, rows, H, "o destination");
  req(rows % 128 == 0 && rows * (int64_t)dests.size() == Tq, "o destinations must tile the query rows in multiples of 128");
  c10::cuda::CUDAGuard guard(q.device());
  auto o = at::empty({Tq, H, 128}, q.options());
  auto lse = at::empty({H, Tq}, q.options().dtype(at::kFloat));
  void* ptr[8];
  for (size_t i = 0; i < dests.size(); ++i) ptr[i] = dests[i].data_ptr();
  int rc = ody_flash_fwd_ex(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), (int)Tq, (int)Tk, (int)H,
                            (int)Hkv, q.stride(0), k.stride(0), v.stride(0), o.stride(0), causal ? 1 : 0, (float)scale, nullptr, ptr,
                            (int)dests.size(), (int)rows, dests[0].stride(0), ody_status_ptr(q),
                            at::cuda::getCurrentCUDAStream().stream());
  req(rc == 0, "flash_fwd (split) failed with code " + std::to_string(rc));
  ody_count_launches(1);
  return {o, lse};
}

// attn_bwd whose gradients go, split by rows, to dq_dests[d] [rows, H, 128] and dk_dests[d] / dv_dests[d] [rows, Hkv, 128]
void attn_bwd_split(const at::Tensor& dO, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& o,
                    const at::Tensor& lse, bool causal, double scale, const std::vector<at::Tensor>& dq_dests,
                    const std::vector<at::Tensor>& dk_dests, const std::vector<at::Tensor>& dv_dests) {
  check_rows(dO, "dO"); check_rows(q, "q"); check_rows(k, "k"); check_rows(v, "v"); check_rows(o, "o");
  req(lse.is_cuda() && lse.scalar_type() == at::kFloat && lse.is_contiguous(), "lse must be contiguous fp32");
  req(lse.dim() == 2 && lse.size(0) == q.size(1) && lse.size(1) == q.size(0), "lse must be [H, Tq]");
  req(dO.sizes() == q.sizes() && o.sizes() == q.sizes(), "dO / o shape mismatch");
  check_kv_and_devices(dO, q, k, v, o, lse);
  const int64_t Tq = q.size(0), Tk = k.size(0), H = q.size(1), Hkv = k.size(1);
  req(Tq == Tk, "split backward needs Tq == Tk");
  const int64_t rows = dq_dests.empty() ? 0 : dq_dests[0].size(0);
  check_split(dq_dests, rows, H, "dq destination");
  check_split(dk_dests, rows, Hkv, "dk destination");
  check_split(dv_dests, rows, Hkv, "dv destination");
  req(dq_dests.size() == dk_dests.size() && dq_dests.size() == dv_dests.size(), "destination count mismatch");
  req(rows % 128 == 0 && rows * (int64_t)dq_dests.size() == Tq, "destinations must tile the rows in multiples of 128");
  c10::cuda::CUDAGuard guard(q.device());
  void *pq[8], *pk[8], *pv[8];
  for (size_t i = 0; i < dq_dests.size(); ++i) { pq[i] = dq_dests[i].data_ptr(); pk[i] = dk_dests[i].data_ptr(); pv[i] = dv_dests[i].data_ptr(); }
  auto ws = at::empty({ody_flash_bwd_workspace_bytes((int)Tq, (int)H)}, q.options().dtype(at::kByte));
  int rc = ody_flash_bwd_ex(dO.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), nullptr,
                            nullptr, nullptr, ws.data_ptr(), (int)Tq, (int)Tk, (int)H, (int)Hkv, dO.stride(0), q.stride(0), k.stride(0),
                            v.stride(0), o.stride(0), dq_dests[0].stride(0), dk_dests[0].stride(0), dv_dests[0].stride(0),
                            causal ? 1 : 0, (float)scale, pq, pk, pv, (int)dq_dests.size(), (int)rows, ody_status_ptr(q),
                            at::cuda::getCurrentCUDAStream().stream());
  req(rc == 0, "flash_bwd (split) failed with code " + std::to_string(rc));
  ody_count_launches(3);
}

}  // namespace

void ody_register_attention(pybind11::module& m) {
  m.def("attn_fwd", &attn_fwd);
  m.def("attn_fwd_split", &attn_fwd_split);
  m.def("attn_bwd_split", &attn_bwd_split);
  m.def("attn_fwd_set_trace", [](const c10::optional<at::Tensor>& t) {
    if (t.has_value()) req(t.value().is_cuda() && t.value().scalar_type() == at::kLong && t.value().numel() >= 64 * 16, "trace: int64 [64*16]");
    req(ody_flash_fwd_set_trace(t.has_value() ? (long long*)t.value().data_ptr() : nullptr) == 0,
        "attn_fwd_set_trace needs a build with -DODY_ATTN_TRACE");
  });
  m.def("attn_bwd_set_variant", [](int64_t v) { req(ody_flash_bwd_set_variant((int)v) == 0, "attn_bwd_set_variant: 0 fused, 1 split"); });
  m.def("attn_fwd_set_kslice", [](bool on) { req(ody_flash_fwd_set_kslice(on ? 1 : 0) == 0, "attn_fwd_set_kslice"); });
  m.def("attn_fwd_ctas", [](int64_t Tq, int64_t H) { return (int64_t)ody_flash_fwd_ctas((int)Tq, (int)H); });
  m.def("attn_bwd_set_trace", [](const c10::optional<at::Tensor>& t) {
    if (t.has_value()) { req(t.value().is_cuda() && t.value().scalar_type() == at::kLong && t.value().numel() >= 96 * 8, "trace: int64 [96*8] (dK/dV kernel stamps, then dQ kernel stamps; only a build with -DODY_ATTN_TRACE records them)"); ody_flash_bwd_set_trace((long long*)t.value().data_ptr()); }
    else ody_flash_bwd_set_trace(nullptr);
  });
  m.def("attn_bwd", &attn_bwd, py::arg("dO"), py::arg("q"), py::arg("k"), py::arg("v"), py::arg("o"), py::arg("lse"),
        py::arg("causal"), py::arg("scale"), py::arg("dq_out") = py::none(), py::arg("dk_out") = py::none(),
        py::arg("dv_out") = py::none());
}
