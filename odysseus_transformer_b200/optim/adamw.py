"""Sharded AdamW with fp32 master weights over one flat buffer per rank.

The reference calls ``torch.optim.AdamW(model.parameters(), lr)`` on bf16 parameters, so its moments
are bf16 and there is no master copy (reference ``train.py:167,224-225``), and FSDP decides what is
sharded.  Here every parameter a rank holds is *already* its shard (tensor-parallel slice, ZeRO-3
slice, or a small replicated norm weight), so the optimizer is purely local:

* all parameters are re-pointed into one flat low-precision buffer, their gradients into a second
  flat buffer exposed as ``p.main_grad`` (the GEMM kernels write wgrads straight into it), and the
  fp32 master / exp_avg / exp_avg_sq live in three flat fp32 buffers;
* parameters that are replicated over some group (norm weights; attention weights across ring
  blocks in the Odysseus x ring hybrid) are laid out contiguously per group so one all-reduce per
  group sums their gradients before the step;
* the step is ONE fused kernel over the flat buffers on CUDA (``adamw_k`` in ``csrc/elementwise.cu``), or
  the same arithmetic in PyTorch elsewhere;
* ``step(guard=t)`` hands the kernel a device word: when it is non-zero at run time (a kernel of this step
  reported a failed wait) nothing is updated, without the host having to look first;
* ``cpu_offload=True`` (the reference's ``--cpu-offload``, reference ``train.py:123-125,142-144``, which asks
  FSDP for ``CPUOffload(offload_params=True)``) keeps the fp32 master weights and both moments in pinned
  host memory - 12 of the 16 bytes per parameter - and runs the update on the CPU: gradients go device ->
  host, the new bf16 parameters host -> device, once per step.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional

import torch

from ..comm import torch_backend as C
from ..ops import native, torch_ref
from ..parallel.linear import wait_pending_grad_comm


class ShardedAdamW:
    def __init__(self, params: Iterable[torch.nn.Parameter], lr: float = 2e-5, betas=(0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 0.01, master_dtype: torch.dtype = torch.float32,
                 cpu_offload: bool = False):
        params = [p for p in params if p.requires_grad]
        if not params:
            raise ValueError("no parameters")
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.step_count = 0
        # group replicated parameters by their sync group so each group is one contiguous range
        def key(p):
            g = getattr(p, "grad_sync_group", None)
            return 0 if g is None or C.group_size(g) == 1 else id(g)
        order: Dict[int, List[torch.nn.Parameter]] = {}
        for p in params:
            order.setdefault(key(p), []).append(p)
        self.params: List[torch.nn.Parameter] = []
        self.sync_ranges = []   # (group, start, end)
        dev, dt = params[0].device, params[0].dtype
        off = 0
        self._offsets = []
        for k, plist in order.items():
            start = off
            for p in plist:
                if p.device != dev or p.dtype != dt:
                    raise ValueError("all parameters must share one device and dtype")
                self.params.append(p)
                self._offsets.append(off)
                off += (p.numel() + 7) // 8 * 8        # keep every view 16-byte aligned
            if k != 0:
                self.sync_ranges.append((plist[0].grad_sync_group, start, off))
        self.numel = off
        self.flat_param = torch.zeros(off, dtype=dt, device=dev)
        self.flat_grad = torch.zeros(off, dtype=dt, device=dev)
        for p, o in zip(self.params, self._offsets):
            view = self.flat_param[o:o + p.numel()].view(p.shape)
            view.copy_(p.data)
            p.data = view
            p.main_grad = self.flat_grad[o:o + p.numel()].view(p.shape)
            p._grad_written = False
            p.grad = None
        self.cpu_offload = bool(cpu_offload)
        if self.cpu_offload:
            pin = dev.type == "cuda"
            host = lambda dtype: torch.zeros(off, dtype=dtype, device="cpu", pin_memory=pin)   # noqa: E731
            self.master = host(master_dtype)
            self.master.copy_(self.flat_param)
            self.exp_avg, self.exp_avg_sq = host(master_dtype), host(master_dtype)
            self._host_grad, self._host_param = host(dt), host(dt)
        else:
            self.master = self.flat_param.to(master_dtype)
            self.exp_avg = torch.zeros(off, dtype=master_dtype, device=dev)
            self.exp_avg_sq = torch.zeros(off, dtype=master_dtype, device=dev)

    # ------------------------------------------------------------------ step
    def sync_grads(self) -> None:
        """Finish gradient reduce-scatters in flight and sum replicated parameters' gradients."""
        wait_pending_grad_comm()
        for p in self.params:
            if not p._grad_written:
                if p.grad is not None:          # a gradient that came through plain autograd
                    p.main_grad.copy_(p.grad)
                    p.grad = None
                else:
                    p.main_grad.zero_()
        for group, s, e in self.sync_ranges:
            C.all_reduce_(self.flat_grad[s:e], group)

    def step(self, grad_scale: float = 1.0, guard: Optional[torch.Tensor] = None) -> None:
        """One AdamW update of every shard.  ``guard``: optional fp32 tensor on the parameters' device; a
        non-zero first element makes the update a no-op (decided on the device, no host read)."""
        self.sync_grads()
        self.step_count += 1
        b1, b2 = self.betas
        if self.cpu_offload:
            self._host_grad.copy_(self.flat_grad)          # device -> pinned host (synchronises)
            host_guard = guard.detach().to("cpu") if guard is not None else None
            torch_ref.adamw_step_(self.master, self.exp_avg, self.exp_avg_sq, self._host_grad, self._host_param,
                                  self.lr, b1, b2, self.eps, self.weight_decay, self.step_count, grad_scale, host_guard)
            if host_guard is None or float(host_guard.reshape(-1)[0]) == 0.0:
                self.flat_param.copy_(self._host_param, non_blocking=True)
        elif native.use_native(self.flat_param):
            native.lib().adamw_step(self.master, self.exp_avg, self.exp_avg_sq, self.flat_grad, self.flat_param,
                                    self.lr, b1, b2, self.eps, self.weight_decay, self.step_count, grad_scale, guard)
        else:
            torch_ref.adamw_step_(self.master, self.exp_avg, self.exp_avg_sq, self.flat_grad, self.flat_param,
                                  self.lr, b1, b2, self.eps, self.weight_decay, self.step_count, grad_scale, guard)

    def zero_grad(self) -> None:
        """Gradients are overwritten by the next backward; only the per-step flags are reset."""
        for p in self.params:
            p._grad_written = False
            p.grad = None

    def grad_norm(self) -> torch.Tensor:
        """Local (this rank's shards) gradient 2-norm squared, fp32 - callers all-reduce if needed."""
        return self.flat_grad.float().pow(2).sum()

    # ------------------------------------------------------------------ checkpoint sidecar
    def state_dict(self) -> Dict[str, object]:
        return {"step": self.step_count, "lr": self.lr, "betas": self.betas, "eps": self.eps,
                "weight_decay": self.weight_decay, "master": self.master, "exp_avg": self.exp_avg,
                "exp_avg_sq": self.exp_avg_sq, "numel": self.numel}

    def load_state_dict(self, sd: Dict[str, object]) -> None:
        if sd["numel"] != self.numel:
            raise ValueError(f"optimizer shard has {self.numel} elements, checkpoint has {sd['numel']} "
                             "(resume with the same mode and world size, or load weights only)")
        self.step_count = int(sd["step"])
        self.master.copy_(sd["master"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        self.flat_param.copy_(self.master.to(self.flat_param.dtype))   # also host -> device when offloaded

    def bytes_held(self) -> int:
        return sum(t.numel() * t.element_size() for t in
                   (self.flat_param, self.flat_grad, self.master, self.exp_avg, self.exp_avg_sq))
