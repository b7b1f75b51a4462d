// Python bindings of the fused compute+collective GEMM (gemm_comm.cu).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <stdexcept>
#include <string>

#include "ody_kernels.h"
#include "epilogue_arg.h"
namespace py = pybind11;

int* ody_status_ptr(const at::Tensor& like);
void ody_count_launches(int64_t n);

namespace {

void req(bool c, const std::string& msg) {
  if (!c) throw std::runtime_error("odysseus_transformer_b200: " + msg);
}

template <class T>
T get(const py::dict& d, const char* k) { return d[k].cast<T>(); }

void fill_ptrs(const py::dict& d, const char* key, void** dst, int n) {
  auto v = d[key].cast<std::vector<int64_t>>();
  req((int)v.size() == n, std::string(key) + ": need one pointer per rank");
  for (int i = 0; i < n; ++i) dst[i] = reinterpret_cast<void*>(v[i]);
}

// gather descriptions are dicts built by comm.symm.GatherSlot: consume_desc() for the operand a GEMM reads,
// push_desc() for the shard a launch delivers.  scatter: ScatterSlot.describe().
void fill_gather_desc(const py::dict& d, OdyGatherDesc& gd, std::vector<at::Tensor>& keep, bool need_shard) {
  memset(&gd, 0, sizeof(gd));
  gd.n_ranks = get<int>(d, "n_ranks");
  req(gd.n_ranks >= 2 && gd.n_ranks <= 8, "gather: 2..8 ranks");
  gd.rank = get<int>(d, "rank");
  gd.chunk_rows = get<int>(d, "chunk_rows");
  gd.cols = get<int>(d, "cols");
  if (need_shard) {
    at::Tensor shard = get<at::Tensor>(d, "shard");
    req(shard.is_cuda() && shard.scalar_type() == at::kBFloat16 && shard.dim() == 2 && shard.stride(1) == 1, "gather shard: bf16 [rows, cols]");
    req(shard.size(0) == gd.chunk_rows && shard.size(1) == gd.cols, "gather shard shape");
    keep.push_back(shard);
    gd.shard = shard.data_ptr();
    gd.shard_ld = shard.stride(0);
  }
  fill_ptrs(d, "gathered_ptrs", gd.gathered_peer, gd.n_ranks);
  fill_ptrs(d, "flags_ptrs", (void**)gd.flags_peer, gd.n_ranks);
  fill_ptrs(d, "counters_ptrs", (void**)gd.counters_peer, gd.n_ranks);
  fill_ptrs(d, "free_ptrs", (void**)gd.free_peer, gd.n_ranks);
  at::Tensor gdone = get<at::Tensor>(d, "gemm_done");
  keep.push_back(gdone);
  gd.gemm_done = reinterpret_cast<uint32_t*>(gdone.data_ptr());
  if (d.contains("stats") && !d["stats"].is_none()) {
    at::Tensor st = get<at::Tensor>(d, "stats");
    req(st.is_cuda() && st.scalar_type() == at::kLong && st.is_contiguous() && st.numel() >= 4 * 148, "stats: int64 [>=148*4]");
    gd.stats = st.data_ptr();
  }
  gd.n_cta = get<int>(d, "n_cta");
  gd.push_total = get<uint32_t>(d, "push_total");
  gd.consume_total = get<uint32_t>(d, "consume_total");
  gd.epoch = get<uint32_t>(d, "epoch");
  gd.prev_epoch = get<uint32_t>(d, "prev_epoch");
  gd.uses = get<uint32_t>(d, "uses");
  gd.which = d.contains("which") ? get<int>(d, "which") : 0;
  gd.dest_first = d.contains("dest_first") ? get<int>(d, "dest_first") : 0;
  gd.dest_count = d.contains("dest_count") ? get<int>(d, "dest_count") : 0;
}

void check_heads(const at::Tensor& t, const char* name) {
  req(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 3 && t.size(2) == 128 && t.stride(2) == 1 &&
          t.stride(1) == 128 && t.stride(0) % 8 == 0,
      std::string(name) + " must be CUDA bf16 [T, heads, 128] with packed heads");
}

// Attention forward (as attn_fwd) whose comm warps deliver push["shard"] (the packed local K|V rows) to the ring
// peers named by push["dest_first"/"dest_count"] while the tiles run.
std::vector<at::Tensor> attn_fwd_push(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, bool causal, double scale,
                                      const py::dict& push) {
  check_heads(q, "q"); check_heads(k, "k"); check_heads(v, "v");
  req(k.size(0) == v.size(0) && k.size(1) == v.size(1) && q.size(1) % k.size(1) == 0, "q/k/v shape mismatch");
  req(!causal || q.size(0) == k.size(0), "causal attention needs Tq == Tk");
  c10::cuda::CUDAGuard guard(q.device());
  OdyGatherDesc pd;
  std::vector<at::Tensor> keep;
  fill_gather_desc(push, pd, keep, true);
  req((pd.shard_ld % 8) == 0 && ((uintptr_t)pd.shard & 15) == 0, "push shard alignment");
  const int64_t Tq = q.size(0), Tk = k.size(0), H = q.size(1), Hkv = k.size(1);
  auto o = at::empty({Tq, H, 128}, q.options());
  auto lse = at::empty({H, Tq}, q.options().dtype(at::kFloat));
  int rc = ody_flash_fwd_push(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), (int)Tq, (int)Tk,
                              (int)H, (int)Hkv, q.stride(0), k.stride(0), v.stride(0), o.stride(0), causal ? 1 : 0, (float)scale,
                              &pd, ody_status_ptr(q), at::cuda::getCurrentCUDAStream().stream());
  req(rc == 0, "flash_fwd_push failed with code " + std::to_string(rc));
  ody_count_launches(1);
  return {o, lse};
}

void wait_shard(const py::dict& slot, int64_t src) {
  OdyGatherDesc d;
  std::vector<at::Tensor> keep;
  fill_gather_desc(slot, d, keep, false);
  c10::cuda::CUDAGuard guard(keep[0].device());
  int rc = ody_wait_shard(&d, (int)src, ody_status_ptr(keep[0]), at::cuda::getCurrentCUDAStream().stream());
  req(rc == 0, "wait_shard failed with code " + std::to_string(rc));
  ody_count_launches(1);
}

void signal_free(const py::dict& slot) {
  OdyGatherDesc d;
  std::vector<at::Tensor> keep;
  fill_gather_desc(slot, d, keep, false);
  c10::cuda::CUDAGuard guard(keep[0].device());
  int rc = ody_signal_free(&d, at::cuda::getCurrentCUDAStream().stream());
  req(rc == 0, "signal_free failed with code " + std::to_string(rc));
  ody_count_launches(1);
}

// epoch words in symmetric memory: base / ptrs are raw device addresses; `like` names the device
void wait_flags(const at::Tensor& like, int64_t base, int64_t mask, int64_t target) {
  c10::cuda::CUDAGuard guard(like.device());
  int rc = ody_wait_flags(reinterpret_cast<const uint32_t*>(base), (uint32_t)mask, (uint32_t)target, ody_status_ptr(like),
                          at::cuda::getCurrentCUDAStream().stream());
  req(rc == 0, "wait_flags failed with code " + std::to_string(rc));
  ody_count_launches(1);
}

void signal_flags(const at::Tensor& like, const std::vector<int64_t>& ptrs, int64_t mask, int64_t index, int64_t value) {
  c10::cuda::CUDAGuard guard(like.device());
  req(ptrs.size() >= 1 && ptrs.size() <= 8, "signal_flags: 1..8 ranks");
  uint32_t* p[8];
  for (size_t i = 0; i < ptrs.size(); ++i) p[i] = reinterpret_cast<uint32_t*>(ptrs[i]);
  int rc = ody_signal_flags(p, (int)ptrs.size(), (uint32_t)mask, (int)index, (uint32_t)value, at::cuda::getCurrentCUDAStream().stream());
  req(rc == 0, "signal_flags failed with code " + std::to_string(rc));
  ody_count_launches(1);
}

at::Tensor gemm_comm(const at::Tensor& a, const at::Tensor& b, const c10::optional<at::Tensor>& out, int64_t layout,
                     const py::object& gather, const py::object& push, const py::object& scatter, const py::object& rope,
                     const c10::optional<at::Tensor>& residual) {
  req(a.is_cuda() && b.is_cuda() && a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16, "bf16 CUDA operands");
  req(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1, "row-major 2-D operands");
  c10::cuda::CUDAGuard guard(a.device());
  int64_t M, N, K;
  if (layout == 0) { M = a.size(0); K = a.size(1); N = b.size(0); req(b.size(1) == K, "K mismatch"); }
  else if (layout == 1) { M = a.size(0); K = a.size(1); N = b.size(1); req(b.size(0) == K, "K mismatch"); }
  else { K = a.size(0); M = a.size(1); N = b.size(1); req(b.size(0) == K, "K mismatch"); }
  OdyGatherDesc gd, pd;
  OdyScatterDesc sd;
  const OdyGatherDesc* gdp = nullptr;
  const OdyGatherDesc* pdp = nullptr;
  const OdyScatterDesc* sdp = nullptr;
  std::vector<at::Tensor> keep;
  if (!gather.is_none()) { fill_gather_desc(gather.cast<py::dict>(), gd, keep, false); gdp = &gd; }
  if (!push.is_none()) { req(gdp != nullptr, "push needs a gather GEMM"); fill_gather_desc(push.cast<py::dict>(), pd, keep, true); pdp = &pd; }
  at::Tensor c;
  if (!scatter.is_none()) {
    py::dict d = scatter.cast<py::dict>();
    memset(&sd, 0, sizeof(sd));
    sd.n_ranks = get<int>(d, "n_ranks");
    req(sd.n_ranks >= 2 && sd.n_ranks <= 8, "scatter: 2..8 ranks");
    fill_ptrs(d, "stage_ptrs", sd.stage_peer, sd.n_ranks);
    fill_ptrs(d, "arrived_ptrs", (void**)sd.arrived_peer, sd.n_ranks);
    fill_ptrs(d, "consumed_ptrs", (void**)sd.consumed_peer, sd.n_ranks);
    at::Tensor rc = get<at::Tensor>(d, "reduce_counter");
    sd.reduce_counter = reinterpret_cast<uint32_t*>(rc.data_ptr());
    c = get<at::Tensor>(d, "out");
    req(c.is_cuda() && c.scalar_type() == at::kBFloat16 && c.dim() == 2 && c.stride(1) == 1, "scatter out: bf16 [rows, N]");
    sd.out = c.data_ptr();
    sd.out_ld = c.stride(0);
    sd.rank = get<int>(d, "rank");
    sd.chunk_rows = get<int>(d, "chunk_rows");
    sd.epoch = get<uint32_t>(d, "epoch");
    sd.prev_epoch = get<uint32_t>(d, "prev_epoch");
    sd.arrived_target = get<uint32_t>(d, "arrived_target");
    sd.uses = get<uint32_t>(d, "uses");
    sd.mode = d.contains("mode") ? get<int>(d, "mode") : 1;
    if (sd.mode == 2) {
      sd.a2a_cols = get<int>(d, "a2a_cols");
      sd.a2a_ld = get<int64_t>(d, "a2a_ld");
      sd.a2a_row0 = get<int64_t>(d, "a2a_row0");
      sd.a2a_col0 = get<int64_t>(d, "a2a_col0");
    } else {
      req(c.size(0) == sd.chunk_rows && c.size(1) == N && (int64_t)sd.chunk_rows * sd.n_ranks == M, "scatter shapes");
    }
    sdp = &sd;
  } else {
    c = out.has_value() ? out.value() : at::empty({M, N}, a.options());
    req(c.dim() == 2 && c.size(0) == M && c.size(1) == N && c.stride(1) == 1 && c.scalar_type() == at::kBFloat16, "bad out");
  }
  req(gdp != nullptr || sdp != nullptr, "gemm_comm needs a gather or a scatter description");
  OdyEpilogue epi;
  const bool reduces = sdp != nullptr && sd.mode != 2;
  req(rope.is_none() || (!reduces && layout == 0), "gemm_comm: the rotary epilogue belongs to a layout-0 product that is not reduced");
  req(!residual.has_value() || sdp == nullptr || reduces, "gemm_comm: no residual in the all-to-all epilogue");
  const bool has_epi = ody_epi::fill(rope, residual, M, reduces ? sd.chunk_rows : M, N, a.device(), epi);
  int rc = ody_gemm_comm_ex(a.data_ptr(), b.data_ptr(), c.data_ptr(), (int)M, (int)N, (int)K, a.stride(0), b.stride(0),
                            c.stride(0), (int)layout, gdp, pdp, sdp, has_epi ? &epi : nullptr, ody_status_ptr(a),
                            at::cuda::getCurrentCUDAStream().stream());
  req(rc == 0, "gemm_comm failed with code " + std::to_string(rc));
  ody_count_launches(1);
  return c;
}

void push_shard(const py::dict& push) {
  OdyGatherDesc pd;
  std::vector<at::Tensor> keep;
  fill_gather_desc(push, pd, keep, true);
  c10::cuda::CUDAGuard guard(keep[0].device());
  int rc = ody_push_shard(&pd, ody_status_ptr(keep[0]), at::cuda::getCurrentCUDAStream().stream());
  req(rc == 0, "push_shard failed with code " + std::to_string(rc));
  ody_count_launches(1);
}

// dst / src are raw device addresses (possibly of a peer's symmetric memory)

}  // namespace

void ody_register_comm(pybind11::module& m) {
  m.def("push_shard", &push_shard);
  m.def("attn_fwd_push", &attn_fwd_push);
  m.def("wait_shard", &wait_shard);
  m.def("wait_flags", &wait_flags);
  m.def("signal_flags", &signal_flags);
  m.def("signal_free", &signal_free);
  m.def("set_push_order", [](bool unit_major) { req(ody_set_push_order(unit_major ? 1 : 0) == 0, "set_push_order failed"); });
  m.def("set_wait_accumulator", [](const py::object& acc) {
    if (acc.is_none()) { req(ody_set_wait_accumulator(nullptr) == 0, "set_wait_accumulator failed"); return; }
    at::Tensor t = acc.cast<at::Tensor>();
    req(t.is_cuda() && t.scalar_type() == at::kLong && t.is_contiguous() && t.numel() >= 4, "wait accumulator: int64 CUDA tensor [>= 4]");
    c10::cuda::CUDAGuard guard(t.device());
    req(ody_set_wait_accumulator(reinterpret_cast<unsigned long long*>(t.data_ptr())) == 0, "set_wait_accumulator failed");
  });
  m.def("set_peer_wait_limit", [](int64_t cycles) { req(ody_set_peer_wait_limit(cycles) == 0, "set_peer_wait_limit failed"); });
  m.def("gemm_comm", &gemm_comm, py::arg("a"), py::arg("b"), py::arg("out"), py::arg("layout"), py::arg("gather"),
        py::arg("push"), py::arg("scatter"), py::arg("rope") = py::none(), py::arg("residual") = py::none());
}
