// Python bindings (torch tensors -> raw-pointer launchers of ody_kernels.h).
// All kernels run on the current CUDA stream of the tensors' device.  A per-device status word
// receives the error code of any bounded in-kernel wait that gave up; `check_status()` reads it.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <map>
#include <sstream>
#include <stdexcept>
#include <string>
#include <mutex>

#include "ody_kernels.h"
#include "epilogue_arg.h"

namespace {

int64_t g_launches = 0;
std::map<int, at::Tensor> g_status;
std::mutex g_mu;

// Failures are reported with std::runtime_error (pybind11 maps it to RuntimeError) rather than
// c10::Error, whose backtrace capture crashed on the B200 hosts when raised from this module.
[[noreturn]] inline void ody_fail(const std::string& msg) { throw std::runtime_error("odysseus_transformer_b200: " + msg); }

#define ODY_CHECK(call, what)                                                                         \
  do {                                                                                                \
    int rc__ = (call);                                                                                \
    if (rc__ != 0) {                                                                                  \
      std::string m__ = std::string(what) + " failed with code " + std::to_string(rc__);              \
      if (rc__ > 0 && rc__ < 1000) m__ += std::string(" (") + cudaGetErrorString((cudaError_t)rc__) + ")"; \
      ody_fail(m__);                                                                                  \
    }                                                                                                 \
  } while (0)

template <class... A>
inline void ody_req(bool cond, const A&... parts) {
  if (!cond) {
    std::ostringstream o;
    (o << ... << parts);
    ody_fail(o.str());
  }
}

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

int* status_ptr(const at::Tensor& like) {
  std::lock_guard<std::mutex> g(g_mu);
  const int dev = like.get_device();
  auto it = g_status.find(dev);
  if (it == g_status.end()) {
    auto t = torch::zeros({16}, torch::dtype(torch::kInt32).device(like.device()));
    it = g_status.emplace(dev, t).first;
  }
  return it->second.data_ptr<int>();
}

void check_bf16(const at::Tensor& t, const char* name) {
  ody_req(t.is_cuda(), name, " must be a CUDA tensor");
  ody_req(t.scalar_type() == at::kBFloat16, name, " must be bfloat16");
}

// ------------------------------------------------------------------------------------------- GEMM
at::Tensor gemm(const at::Tensor& a, const at::Tensor& b, const c10::optional<at::Tensor>& out, int64_t layout,
                bool accumulate, const py::object& rope, const c10::optional<at::Tensor>& residual) {
  check_bf16(a, "a");
  check_bf16(b, "b");
  ody_req(a.dim() == 2 && b.dim() == 2, "gemm expects 2-D operands");
  ody_req(a.stride(1) == 1 && b.stride(1) == 1, "gemm operands must be row-major (last stride 1)");
  c10::cuda::CUDAGuard guard(a.device());
  int64_t M, N, K;
  if (layout == 0) { M = a.size(0); K = a.size(1); N = b.size(0); ody_req(b.size(1) == K, "K mismatch"); }
  else if (layout == 1) { M = a.size(0); K = a.size(1); N = b.size(1); ody_req(b.size(0) == K, "K mismatch"); }
  else { K = a.size(0); M = a.size(1); N = b.size(1); ody_req(b.size(0) == K, "K mismatch"); }
  at::Tensor c = out.has_value() ? out.value() : at::empty({M, N}, a.options());
  check_bf16(c, "out");
  ody_req(c.dim() == 2 && c.size(0) == M && c.size(1) == N && c.stride(1) == 1, "bad out shape");
  ody_req(!accumulate || out.has_value(), "accumulate needs out");
  if (M == 0 || N == 0) return c;
  OdyEpilogue epi;
  const bool has_epi = ody_epi::fill(rope, residual, M, M, N, a.device(), epi);
  ody_req(!has_epi || K > 0, "gemm: an epilogue needs K > 0");
  ody_req(!(accumulate && residual.has_value()), "gemm: accumulate and residual exclude each other");
  ody_req(rope.is_none() || layout == 0, "gemm: the rotary epilogue belongs to layout 0 (a forward projection)");
  if (K == 0) { if (!accumulate) c.zero_(); return c; }
  ODY_CHECK(ody_gemm_bf16_ex(a.data_ptr(), b.data_ptr(), c.data_ptr(), (int)M, (int)N, (int)K, a.stride(0), b.stride(0),
                             c.stride(0), (int)layout, accumulate ? 1 : 0, has_epi ? &epi : nullptr, status_ptr(a),
                             cur_stream()),
            "gemm");
  ++g_launches;
  return c;
}

// ------------------------------------------------------------------------------------------- RMSNorm
std::vector<at::Tensor> rmsnorm_fwd(const at::Tensor& x, const at::Tensor& w, double eps) {
  check_bf16(x, "x"); check_bf16(w, "w");
  ody_req(x.is_contiguous() && w.is_contiguous(), "rmsnorm: contiguous inputs required");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t dim = x.size(-1), rows = x.numel() / dim;
  auto y = at::empty_like(x);
  auto rstd = at::empty({rows}, x.options().dtype(at::kFloat));
  ODY_CHECK(ody_rmsnorm_fwd(x.data_ptr(), nullptr, w.data_ptr(), nullptr, y.data_ptr(), rstd.data_ptr<float>(), rows,
                            (int)dim, (float)eps, cur_stream()), "rmsnorm_fwd");
  ++g_launches;
  return {y, rstd};
}

std::vector<at::Tensor> add_rmsnorm_fwd(const at::Tensor& x, const at::Tensor& delta, const at::Tensor& w, double eps) {
  check_bf16(x, "x"); check_bf16(delta, "delta"); check_bf16(w, "w");
  ody_req(x.is_contiguous() && delta.is_contiguous() && w.is_contiguous(), "add_rmsnorm: contiguous inputs required");
  ody_req(x.sizes() == delta.sizes(), "add_rmsnorm: shape mismatch");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t dim = x.size(-1), rows = x.numel() / dim;
  auto s = at::empty_like(x);
  auto y = at::empty_like(x);
  auto rstd = at::empty({rows}, x.options().dtype(at::kFloat));
  ODY_CHECK(ody_rmsnorm_fwd(x.data_ptr(), delta.data_ptr(), w.data_ptr(), s.data_ptr(), y.data_ptr(),
                            rstd.data_ptr<float>(), rows, (int)dim, (float)eps, cur_stream()), "add_rmsnorm_fwd");
  ++g_launches;
  return {s, y, rstd};
}

std::vector<at::Tensor> rmsnorm_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& w,
                                    const at::Tensor& rstd, const c10::optional<at::Tensor>& ds) {
  check_bf16(dy, "dy"); check_bf16(x, "x"); check_bf16(w, "w");
  ody_req(dy.is_contiguous() && x.is_contiguous() && w.is_contiguous(), "rmsnorm_bwd: contiguous inputs required");
  ody_req(x.dim() >= 1 && x.size(-1) > 0, "rmsnorm_bwd: x must have a non-empty last dim");
  const int64_t dim = x.size(-1), rows = x.numel() / dim;
  ody_req(dy.sizes() == x.sizes(), "rmsnorm_bwd: dy and x must have the same shape");
  ody_req(w.numel() == dim, "rmsnorm_bwd: w must have x's last dim");
  ody_req(rstd.is_cuda() && rstd.scalar_type() == at::kFloat && rstd.is_contiguous() && rstd.numel() == rows,
          "rmsnorm_bwd: rstd must be a contiguous fp32 CUDA tensor with one entry per row");
  ody_req(dy.get_device() == x.get_device() && w.get_device() == x.get_device() && rstd.get_device() == x.get_device(),
          "rmsnorm_bwd: all tensors must be on x's device");
  c10::cuda::CUDAGuard guard(x.device());
  auto dx = at::empty_like(x);
  auto dw = at::empty({dim}, x.options().dtype(at::kFloat));
  const int nb = ody_rmsnorm_bwd_blocks(rows, (int)dim);
  auto partial = at::empty({nb, dim}, x.options().dtype(at::kFloat));
  const void* dsp = nullptr;
  if (ds.has_value()) {
    check_bf16(ds.value(), "ds");
    ody_req(ds.value().is_contiguous() && ds.value().sizes() == x.sizes() && ds.value().get_device() == x.get_device(),
            "rmsnorm_bwd: ds must match x");
    dsp = ds.value().data_ptr();
  }
  ODY_CHECK(ody_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), dsp, dx.data_ptr(),
                            dw.data_ptr<float>(), partial.data_ptr<float>(), rows, (int)dim, cur_stream()), "rmsnorm_bwd");
  g_launches += 2;
  return {dx, dw};
}

// ------------------------------------------------------------------------------------------- RoPE
std::vector<at::Tensor> rope_tables(const at::Tensor& pos, int64_t head_dim, double theta) {
  ody_req(pos.is_cuda() && pos.scalar_type() == at::kLong && pos.is_contiguous(), "positions: contiguous int64 CUDA");
  c10::cuda::CUDAGuard guard(pos.device());
  const int64_t T = pos.numel();
  auto opt = pos.options().dtype(at::kFloat);
  auto c = at::empty({T, head_dim / 2}, opt), s = at::empty({T, head_dim / 2}, opt);
  ODY_CHECK(ody_rope_tables(pos.data_ptr<int64_t>(), c.data_ptr<float>(), s.data_ptr<float>(), T, (int)head_dim,
                            (float)theta, cur_stream()), "rope_tables");
  ++g_launches;
  return {c, s};
}

void rope_inplace_(at::Tensor x, int64_t n_rot, const at::Tensor& cos, const at::Tensor& sin, bool inverse) {
  check_bf16(x, "x");
  ody_req(x.dim() == 3 && x.stride(2) == 1 && x.stride(1) == x.size(2), "rope: x must be [T, heads, hd] with packed heads");
  ody_req(cos.is_contiguous() && sin.is_contiguous() && cos.scalar_type() == at::kFloat, "rope tables: fp32 contiguous");
  ody_req(cos.size(0) == x.size(0) && cos.size(1) * 2 == x.size(2), "rope tables shape");
  ody_req(n_rot <= x.size(1));
  c10::cuda::CUDAGuard guard(x.device());
  ODY_CHECK(ody_rope_inplace(x.data_ptr(), cos.data_ptr<float>(), sin.data_ptr<float>(), x.size(0), (int)n_rot,
                             (int)x.size(2), x.stride(0), inverse ? 1 : 0, cur_stream()), "rope_inplace");
  ++g_launches;
}

// src [T, heads, hd] -> dst [T, heads, hd] (src may be dst): heads in groups of `period` (0 = one group of all heads), the
// first n_rot of each group rotated, the rest copied when dst is another tensor.  Rows may be strided, heads packed.
void rope_grouped_(const at::Tensor& src, at::Tensor dst, int64_t n_rot, int64_t period, const at::Tensor& cos,
                   const at::Tensor& sin, bool inverse) {
  check_bf16(src, "src");
  check_bf16(dst, "dst");
  ody_req(src.dim() == 3 && src.stride(2) == 1 && src.stride(1) == src.size(2), "rope: src must be [T, heads, hd] with packed heads");
  ody_req(dst.dim() == 3 && dst.stride(2) == 1 && dst.stride(1) == dst.size(2), "rope: dst must be [T, heads, hd] with packed heads");
  ody_req(src.sizes() == dst.sizes() && src.device() == dst.device(), "rope: src and dst differ in shape or device");
  ody_req(cos.is_contiguous() && sin.is_contiguous() && cos.scalar_type() == at::kFloat && sin.scalar_type() == at::kFloat,
          "rope tables: fp32 contiguous");
  ody_req(cos.size(0) == src.size(0) && cos.size(1) * 2 == src.size(2) && sin.sizes() == cos.sizes(), "rope tables shape");
  ody_req(cos.device() == src.device() && sin.device() == src.device(), "rope tables on another device");
  const int64_t per = period > 0 ? period : src.size(1);
  ody_req(per > 0 && src.size(1) % per == 0 && n_rot >= 0 && n_rot <= per, "rope: heads, period and n_rot disagree");
  ody_req((((uintptr_t)src.data_ptr()) & 15) == 0 && (((uintptr_t)dst.data_ptr()) & 15) == 0, "rope: 16-byte aligned tensors");
  c10::cuda::CUDAGuard dev_guard(src.device());
  ODY_CHECK(ody_rope(src.data_ptr(), dst.data_ptr(), cos.data_ptr<float>(), sin.data_ptr<float>(), src.size(0),
                     (int)src.size(1), (int)per, (int)n_rot, (int)src.size(2), src.stride(0), dst.stride(0),
                     inverse ? 1 : 0, cur_stream()), "rope");
  ++g_launches;
}

at::Tensor rope_apply(const at::Tensor& x, const at::Tensor& cos, const at::Tensor& sin, bool inverse) {
  auto y = x.contiguous().clone();
  rope_inplace_(y, y.size(1), cos, sin, inverse);
  return y;
}

// ------------------------------------------------------------------------------------------- SwiGLU
at::Tensor swiglu_fwd(const at::Tensor& gu) {
  check_bf16(gu, "gate_up");
  ody_req(gu.is_contiguous() && gu.dim() == 2);
  c10::cuda::CUDAGuard guard(gu.device());
  const int64_t T = gu.size(0), I = gu.size(1) / 2;
  auto h = at::empty({T, I}, gu.options());
  ODY_CHECK(ody_swiglu_fwd(gu.data_ptr(), h.data_ptr(), T, I, cur_stream()), "swiglu_fwd");
  ++g_launches;
  return h;
}

at::Tensor swiglu_bwd(const at::Tensor& dh, const at::Tensor& gu) {
  check_bf16(gu, "gate_up"); check_bf16(dh, "dh");
  ody_req(gu.is_contiguous() && dh.is_contiguous());
  c10::cuda::CUDAGuard guard(gu.device());
  const int64_t T = gu.size(0), I = gu.size(1) / 2;
  auto dgu = at::empty_like(gu);
  ODY_CHECK(ody_swiglu_bwd(dh.data_ptr(), gu.data_ptr(), dgu.data_ptr(), T, I, cur_stream()), "swiglu_bwd");
  ++g_launches;
  return dgu;
}

// ------------------------------------------------------------------------------------------- cross-entropy
std::vector<at::Tensor> ce_fwd(const at::Tensor& logits, const at::Tensor& targets, int64_t ignore_index) {
  check_bf16(logits, "logits");
  ody_req(logits.is_contiguous() && logits.dim() == 2 && targets.scalar_type() == at::kLong && targets.is_contiguous());
  c10::cuda::CUDAGuard guard(logits.device());
  const int64_t T = logits.size(0), V = logits.size(1);
  auto opt = logits.options().dtype(at::kFloat);
  auto loss = at::empty({T}, opt), lse = at::empty({T}, opt);
  ODY_CHECK(ody_ce_fwd(logits.data_ptr(), targets.data_ptr<int64_t>(), loss.data_ptr<float>(), lse.data_ptr<float>(), T, V,
                       ignore_index, cur_stream()), "ce_fwd");
  ++g_launches;
  return {loss, lse};
}

void ce_bwd_(at::Tensor logits, const at::Tensor& targets, const at::Tensor& lse, const at::Tensor& scale,
             int64_t ignore_index) {
  check_bf16(logits, "logits");
  ody_req(logits.is_contiguous() && scale.is_cuda() && scale.scalar_type() == at::kFloat);
  c10::cuda::CUDAGuard guard(logits.device());
  const int64_t T = logits.size(0), V = logits.size(1);
  for (int64_t r0 = 0; r0 < T; r0 += 32768) {   // grid.y limit
    const int64_t n = std::min<int64_t>(32768, T - r0);
    ODY_CHECK(ody_ce_bwd((char*)logits.data_ptr() + r0 * V * 2, targets.data_ptr<int64_t>() + r0,
                         lse.data_ptr<float>() + r0, scale.data_ptr<float>(), n, V, ignore_index, cur_stream()), "ce_bwd");
    ++g_launches;
  }
}

// ------------------------------------------------------------------------------------------- AdamW
void adamw_step(at::Tensor master, at::Tensor m, at::Tensor v, const at::Tensor& grad, at::Tensor param, double lr,
                double beta1, double beta2, double eps, double weight_decay, int64_t step, double grad_scale,
                const c10::optional<at::Tensor>& guard) {
  check_bf16(grad, "grad"); check_bf16(param, "param");
  const float* gp = nullptr;
  if (guard.has_value()) {
    const at::Tensor& g = guard.value();
    ody_req(g.is_cuda() && g.scalar_type() == at::kFloat && g.numel() >= 1 && g.get_device() == master.get_device(),
            "adamw guard must be a float32 CUDA tensor on the optimizer's device");
    gp = g.data_ptr<float>();
  }
  ody_req(master.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat);
  ody_req(master.is_contiguous() && m.is_contiguous() && v.is_contiguous() && grad.is_contiguous() && param.is_contiguous());
  c10::cuda::CUDAGuard dev_guard(master.device());
  ODY_CHECK(ody_adamw(master.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), grad.data_ptr(), param.data_ptr(),
                      master.numel(), (float)lr, (float)beta1, (float)beta2, (float)eps, (float)weight_decay, (int)step,
                      (float)grad_scale, gp, cur_stream()), "adamw");
  ++g_launches;
}

// ------------------------------------------------------------------------------------------- attention merge
void attn_merge_(at::Tensor out, at::Tensor lse, const at::Tensor& o, const at::Tensor& l, int64_t row0) {
  check_bf16(o, "o");
  ody_req(out.scalar_type() == at::kFloat && lse.scalar_type() == at::kFloat && l.scalar_type() == at::kFloat);
  ody_req(out.is_contiguous() && lse.is_contiguous() && o.is_contiguous() && l.is_contiguous());
  c10::cuda::CUDAGuard guard(out.device());
  ODY_CHECK(ody_attn_merge(out.data_ptr<float>(), lse.data_ptr<float>(), o.data_ptr(), l.data_ptr<float>(), o.size(0),
                           (int)o.size(1), (int)o.size(2), row0, out.size(0), cur_stream()), "attn_merge");
  ++g_launches;
}

// dst [T, C] (row pitch free) += sum of srcs; srcs[i] [rows_i, C] lands on rows begins[i] ..., summed in fp32
void sum_rows_(at::Tensor dst, const std::vector<at::Tensor>& srcs, const std::vector<int64_t>& begins) {
  ody_req(dst.is_cuda() && dst.scalar_type() == at::kBFloat16 && dst.dim() == 2 && dst.stride(1) == 1);
  ody_req(srcs.size() == begins.size() && srcs.size() <= 8);
  c10::cuda::CUDAGuard guard(dst.device());
  const void* ptr[8];
  int64_t ld[8], rows[8];
  for (size_t i = 0; i < srcs.size(); ++i) {
    const at::Tensor& t = srcs[i];
    ody_req(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 2 && t.stride(1) == 1 && t.size(1) == dst.size(1));
    ptr[i] = t.data_ptr(); ld[i] = t.stride(0); rows[i] = t.size(0);
  }
  ODY_CHECK(ody_sum_rows(dst.data_ptr(), dst.stride(0), dst.size(0), dst.size(1), ptr, ld, begins.data(), rows, (int)srcs.size(),
                         cur_stream()), "sum_rows");
  ++g_launches;
}

// merge attention partials over disjoint key sets in one pass -> (out [T, H, hd] bf16, lse [H, T] fp32)
std::vector<at::Tensor> attn_merge_parts(const std::vector<at::Tensor>& os, const std::vector<at::Tensor>& ls,
                                         const std::vector<int64_t>& begins, int64_t T) {
  ody_req(!os.empty() && os.size() <= 8 && os.size() == ls.size() && os.size() == begins.size());
  const int64_t H = os[0].size(1), hd = os[0].size(2);
  c10::cuda::CUDAGuard guard(os[0].device());
  const void* op[8];
  const float* lp[8];
  int64_t rows[8];
  for (size_t i = 0; i < os.size(); ++i) {
    check_bf16(os[i], "o");
    ody_req(os[i].is_contiguous() && os[i].dim() == 3 && os[i].size(1) == H && os[i].size(2) == hd);
    ody_req(ls[i].scalar_type() == at::kFloat && ls[i].is_contiguous() && ls[i].size(0) == H && ls[i].size(1) == os[i].size(0));
    op[i] = os[i].data_ptr(); lp[i] = ls[i].data_ptr<float>(); rows[i] = os[i].size(0);
  }
  auto out = at::empty({T, H, hd}, os[0].options());
  auto lse = at::empty({H, T}, ls[0].options());
  ODY_CHECK(ody_attn_merge_parts(out.data_ptr(), lse.data_ptr<float>(), T, (int)H, (int)hd, op, lp, begins.data(), rows,
                                 (int)os.size(), cur_stream()), "attn_merge_parts");
  ++g_launches;
  return {out, lse};
}

// ------------------------------------------------------------------------------------------- status
int64_t status(int64_t device) {
  at::Tensor t;
  {
    std::lock_guard<std::mutex> g(g_mu);
    auto it = g_status.find((int)device);
    if (it == g_status.end()) return 0;
    t = it->second;
  }
  return t.cpu().data_ptr<int>()[0];
}

// The device-resident status words themselves (int32[16], word 0 = first error code), creating them if needed:
// lets a training step fold the status into a collective or an optimizer guard without a host read.
at::Tensor status_tensor(const at::Tensor& like) {
  ody_req(like.is_cuda(), "status_tensor needs a CUDA tensor");
  status_ptr(like);
  std::lock_guard<std::mutex> g(g_mu);
  return g_status.find(like.get_device())->second;
}

void clear_status(int64_t device) {
  std::lock_guard<std::mutex> g(g_mu);
  auto it = g_status.find((int)device);
  if (it != g_status.end()) it->second.zero_();
}

int64_t launch_count() { return g_launches; }
void reset_launch_count() { g_launches = 0; }
void add_launches(int64_t n) { g_launches += n; }

}  // namespace

int* ody_status_ptr(const at::Tensor& like) { return status_ptr(like); }
void ody_count_launches(int64_t n) { g_launches += n; }

// attention (defined in attn_bindings.cpp)
void ody_register_attention(pybind11::module& m);
void ody_register_comm(pybind11::module& m);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &gemm, py::arg("a"), py::arg("b"), py::arg("out") = py::none(), py::arg("layout") = 0,
        py::arg("accumulate") = false, py::arg("rope") = py::none(), py::arg("residual") = py::none());
  m.def("gemm_set_variant", [](int64_t v) { ODY_CHECK(ody_gemm_set_variant((int)v), "gemm_set_variant (0 auto, 1 one CTA, 2 CTA pairs)"); });
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("add_rmsnorm_fwd", &add_rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("rope_tables", &rope_tables);
  m.def("rope_inplace_", &rope_inplace_);
  m.def("rope_grouped_", &rope_grouped_);
  m.def("rope_apply", &rope_apply);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("ce_fwd", &ce_fwd);
  m.def("ce_bwd_", &ce_bwd_);
  m.def("adamw_step", &adamw_step, py::arg("master"), py::arg("m"), py::arg("v"), py::arg("grad"), py::arg("param"),
        py::arg("lr"), py::arg("beta1"), py::arg("beta2"), py::arg("eps"), py::arg("weight_decay"), py::arg("step"),
        py::arg("grad_scale"), py::arg("guard") = py::none());
  m.def("attn_merge_", &attn_merge_);
  m.def("sum_rows_", &sum_rows_);
  m.def("attn_merge_parts", &attn_merge_parts);
  m.def("status", &status);
  m.def("clear_status", &clear_status);
  m.def("status_tensor", &status_tensor);
  m.def("launch_count", &launch_count);
  m.def("reset_launch_count", &reset_launch_count);
  m.def("add_launches", &add_launches);
  ody_register_attention(m);
  ody_register_comm(m);
}
