"""Training driver: the reference's ``train.py`` re-done on this package's model, modes and kernels.

CLI flags are the reference's (reference ``train.py:243-263``; dashed and underscored spellings are
both accepted), plus ``--ulysses-degree / --ring-degree`` for the hybrid mesh, ``--model-config`` for
synthetic random-init runs, ``--backend {fused,library,auto}``, ``--jsonl``, ``--save`` and ``--load``.

Per step, as in the reference (reference ``train.py:184-235``): a random ``[1, L+1]`` token batch is
drawn on the CPU, split into inputs and shifted targets, sliced for this rank's mode and copied to
the device, then forward, loss, backward, optimizer step.  Rank 0 prints parameter count, allocated /
reserved GB and the loss in the reference's format, and at the end
``"{mode} {L//1024}K {world} Time taken: {elapsed:.2f} seconds"`` over the steps after warm-up.

What differs on purpose: ``loss.backward()`` is seeded with 1 (the reference seeds it with the loss
value, reference ``train.py:222``); the loss is the global mean over all tokens; elapsed time is
also measured on the device and reduced as the max over ranks; there is no FSDP - every large weight
is tensor-parallel or ZeRO-3 sharded by the model itself and the optimizer keeps fp32 masters.
"""
from __future__ import annotations

import argparse
import contextlib
import dataclasses
import os
import time
from typing import Dict, Optional

import torch
import torch.distributed as dist

from .config import PARALLEL_MODES, ModelConfig, TrainConfig, get_model_config
from .mesh import ParallelContext, init_parallel_context
from .ops import native
from .optim.adamw import ShardedAdamW
from .parallel.apply import build_model, prepare_attn_inputs
from .utils import checkpoint as ckpt
from .utils.buffers import set_global_memory_buffer
from .utils.health import Heartbeat, guarded_collective
from .utils.log_utils import get_logger, rank_log
from .utils.metrics import DeviceTimer, JsonlWriter, PhaseTimers, exposed_comm_ms, max_over_ranks, memory_gb, train_flops_per_token
from .utils.profiler import init_prof, nvtx_range


def set_seed(seed: int) -> None:
    import random
    import numpy as np
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


class Trainer:
    """Model + optimizer + one-step API for a given mode on the current mesh.

    ``train_step(batch)`` is the call a user makes: ``batch`` is a host tensor ``[1, L+1]`` of token
    ids (pinned memory recommended); it returns the device scalar holding this step's global-mean
    loss.  ``train_step_device`` takes already-sliced device tensors.

    Failure handling: the kernels' bounded waits report into a per-device status word.  Every step
    sums that word over the ranks together with the loss (one small all-reduce), hands the sum to the
    optimizer kernel as its guard - a step with a failed wait anywhere updates no weight on any rank -
    and copies it to pinned host memory without synchronising.  The next ``train_step*`` call (or
    ``check_status``) raises ``KernelStatusError`` once that copy has landed."""

    def __init__(self, cfg: ModelConfig, mode: Optional[str], ctx: ParallelContext, seq_length: int,
                 lr: float = 2e-5, weight_decay: float = 0.01, betas=(0.9, 0.999), eps: float = 1e-8,
                 dtype: torch.dtype = torch.bfloat16, seed: int = 42, ulysses_degree: int = 0,
                 ring_degree: int = 1, state_dict: Optional[Dict[str, torch.Tensor]] = None,
                 grad_checkpoint: bool = False, use_zero2: bool = False, cpu_offload: bool = False,
                 use_zero3_linear: bool = True, time_phases: bool = False, loss_chunk_rows: Optional[int] = None):
        self.cfg, self.mode, self.ctx, self.seq_length = cfg, mode, ctx, seq_length
        self.ulysses_degree, self.ring_degree = ulysses_degree, ring_degree
        set_global_memory_buffer(ctx.device)
        if ctx.world_size > 1 and ctx.device.type == "cuda" and native.get_backend() != "library" and dtype == torch.bfloat16:
            from .comm import symm
            symm.setup_fused_comm(ctx, cfg, max(1, seq_length // ctx.world_size), mode=mode)
        if loss_chunk_rows is None:
            loss_chunk_rows = default_loss_chunk_rows(cfg, seq_length, ctx.world_size, mode, dtype)
        self.loss_chunk_rows = loss_chunk_rows
        self.model = build_model(cfg, mode, ctx, dtype=dtype, device=ctx.device, seed=seed, state_dict=state_dict,
                                 use_zero3_linear=use_zero3_linear, loss_chunk_rows=loss_chunk_rows)
        if grad_checkpoint:
            self.model.gradient_checkpointing_enable()
        if use_zero2:
            self.model.zero3.keep_gathered = True
        self.optimizer = ShardedAdamW(self.model.parameters(), lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                      cpu_offload=cpu_offload)
        self._status_reads = []          # (step, event or None, host tensor) awaiting a look
        self.phases = PhaseTimers(ctx.device) if time_phases else None
        self.global_tokens = seq_length * (ctx.world_size if mode in (None, "dp") else 1)
        self.position_ids = torch.arange(seq_length).unsqueeze(0)
        self.steps_done = 0
        self.last_h2d_bytes = 0

    def shard_batch(self, batch: torch.Tensor) -> Dict[str, torch.Tensor]:
        """Host ``[1, L+1]`` batch -> this rank's device tensors (the step's host-to-device copy)."""
        input_ids, target_ids = batch[:, :-1], batch[:, 1:]
        out = prepare_attn_inputs(self.mode, input_ids, self.position_ids, target_ids, self.ctx.rank,
                                  self.ctx.world_size, self.ctx.device, self.ulysses_degree, self.ring_degree)
        self.last_h2d_bytes = sum(t.numel() * t.element_size() for t in out.values() if t is not None)
        return out

    def train_step_device(self, local_input_ids, local_position_ids, local_target_ids) -> torch.Tensor:
        self.check_status(block=False)
        with self._phase("forward"):
            loss = self.model(local_input_ids, local_position_ids, labels=local_target_ids,
                              global_tokens=self.global_tokens)
        with self._phase("backward"):
            loss.backward()
        # [loss, kernel status] summed over the ranks in one collective, before the optimizer looks at it
        dev = self.ctx.device
        status = native.status_tensor(dev)
        parts = [loss.detach().float().reshape(1)]
        if status is not None:
            parts.append(status.reshape(-1)[:1].float())
        health = torch.cat(parts)
        if self.ctx.world_size > 1:
            guarded_collective(dist.all_reduce, health, group=self.ctx.world_group,
                               on_timeout="loss / status all-reduce")
        guard = health[1:2] if status is not None else None
        with self._phase("optimizer"):
            self.optimizer.step(guard=guard)
            self.optimizer.zero_grad()
        if guard is not None:
            self._queue_status_read(guard)
        self.steps_done += 1
        return health[0]

    def _phase(self, name: str):
        """NVTX range around a phase of the step, plus a device timer when ``time_phases`` was asked for."""
        if self.phases is None:
            return nvtx_range(name)
        stack = contextlib.ExitStack()
        stack.enter_context(nvtx_range(name))
        stack.enter_context(self.phases.phase(name))
        return stack

    def phase_summary(self, reset: bool = False) -> Dict[str, float]:
        """ms per phase since the last reset, each the max over ranks (empty without ``time_phases``)."""
        if self.phases is None:
            return {}
        out = self.phases.summary(self.ctx.world_group)
        if reset:
            self.phases = PhaseTimers(self.ctx.device)
        return out

    def _queue_status_read(self, guard: torch.Tensor) -> None:
        if guard.is_cuda:
            host = torch.empty(1, dtype=torch.float32, pin_memory=True)
            host.copy_(guard, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            self._status_reads.append((self.steps_done, ev, host))
        else:
            self._status_reads.append((self.steps_done, None, guard.detach().clone()))

    def check_status(self, block: bool = True) -> None:
        """Raise ``KernelStatusError`` if a finished step reported a failed device-side wait.  ``block=False``
        looks only at steps whose status has already reached the host (no synchronisation)."""
        while self._status_reads:
            step, ev, host = self._status_reads[0]
            if ev is not None:
                if block:
                    ev.synchronize()
                elif not ev.query():
                    return
            self._status_reads.pop(0)
            st = int(host[0])
            if st != 0:
                self._status_reads.clear()
                if self.ctx.device.type == "cuda" and native.available():
                    native.lib().clear_status(self.ctx.device.index or 0)
                raise native.KernelStatusError(
                    st, f"in training step {step} (sum over ranks); that step's optimizer update was skipped on every rank")

    def train_step(self, batch: torch.Tensor) -> torch.Tensor:
        s = self.shard_batch(batch)
        return self.train_step_device(s["local_input_ids"], s["local_position_ids"], s["local_target_ids"])


def default_loss_chunk_rows(cfg: ModelConfig, seq_length: int, world_size: int, mode: Optional[str], dtype) -> int:
    """Tokens per lm_head + loss chunk, or 0 to form the local ``[t, V]`` logits in one piece: chunking starts
    once those logits would pass 2 GiB, in pieces of about 1 GiB (a multiple of 128 rows)."""
    t = seq_length if mode in (None, "dp") else max(1, seq_length // max(1, world_size))
    esize = torch.empty((), dtype=dtype).element_size()
    if t * cfg.vocab_size * esize <= (2 << 30):
        return 0
    return max(128, ((1 << 30) // (cfg.vocab_size * esize)) // 128 * 128)


def _dtype(name: str) -> torch.dtype:
    return {"bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16}[name]


def resolve_model_config(args) -> ModelConfig:
    if args.use_cfg_init_model:
        cfg = get_model_config("llama2-3b-gqa")
    elif args.model_config:
        cfg = get_model_config(args.model_config)
    elif args.model and os.path.isdir(args.model):
        cfg = ckpt.load_hf_config(args.model)
    else:
        name = {"meta-llama/Llama-2-7b-hf": "llama2-7b", "meta-llama/Meta-Llama-3-8B": "llama3-8b"}.get(args.model, args.model)
        cfg = get_model_config(name)
    if args.rope_theta is not None:
        cfg = cfg.replace(rope_theta=float(args.rope_theta))
    return cfg


def main(args) -> Dict[str, float]:
    assert args.batch_size == 1, "Only batch size 1 is supported (sequence parallelism folds the batch dim)"
    native.set_backend(args.backend)
    ctx = init_parallel_context(args.parallel_mode, args.ulysses_degree, args.ring_degree, backend=args.backend)
    rank, world, dev = ctx.rank, ctx.world_size, ctx.device
    set_seed(args.seed)
    cfg = resolve_model_config(args)
    state_dict = None
    src = args.load or (args.model if (args.model and os.path.isdir(args.model) and not args.use_cfg_init_model
                                       and not args.model_config) else None)
    if src:
        state_dict = ckpt.load_hf_state_dict_file(src)
    trainer = Trainer(cfg, args.parallel_mode, ctx, args.seq_length, lr=args.learning_rate, dtype=_dtype(args.dtype),
                      seed=args.seed, ulysses_degree=args.ulysses_degree, ring_degree=args.ring_degree,
                      state_dict=state_dict, grad_checkpoint=args.grad_checkpoint, use_zero2=args.use_zero2,
                      cpu_offload=args.cpu_offload, use_zero3_linear=args.use_ody_zero3, time_phases=bool(args.jsonl),
                      loss_chunk_rows=args.loss_chunk_rows)
    log = get_logger()
    start_step = 0
    # the data stream is a function of the RNG state: seed it for a fresh run, restore it for a resumed one
    set_seed(args.seed)
    if args.load and os.path.exists(os.path.join(args.load, f"train_state_rank{rank}.pt")):
        start_step = ckpt.load_train_state(args.load, trainer.optimizer, rank)
        rank_log(rank, log, f"resumed optimizer, step {start_step} and RNG state from {args.load}")
    if rank == 0:
        print(f"{cfg.num_parameters() / 1e9:.2f}B parameters; mode {args.parallel_mode} on {world} rank(s); "
              f"backend {native.get_backend()}")
        m = memory_gb(dev)
        print(f"After init model and optimizer, CUDA memory allocated: {m['allocated']:.2f} GB, reserved: {m['reserved']:.2f} GB")
        if args.parallel_mode in ("odysseus", "tpsp", "ulysses", "ring") and args.seq_length % world == 0:
            from .utils.memory import estimate_memory
            est = estimate_memory(cfg, args.parallel_mode, args.seq_length, world, trainer.ctx.inner_size, trainer.ctx.ring_size,
                                  args.grad_checkpoint, trainer.loss_chunk_rows, args.use_ody_zero3,
                                  native.get_backend() == "fused")
            print(f"Estimated peak allocated: {est['peak_allocated']:.1f} GB (states {est['states']:.1f}, saved activations "
                  f"{est['saved_activations']:.1f}, logits {est['logits']:.1f}, backward transients "
                  f"{est['backward_transients']:.1f}); communication heap {est['comm_heap']:.1f} GB on top")
    hb = None
    if world > 1 and args.heartbeat_timeout > 0:
        hb = Heartbeat(dist.distributed_c10d._get_default_store(), rank, world, args.heartbeat_timeout)
    writer = JsonlWriter(args.jsonl, rank)
    warmup = args.warmup_iterations
    timer = DeviceTimer(dev)
    elapse, timed_steps, exposed_sum = 0.0, 0, 0.0
    loss_val = float("nan")
    with init_prof(args.use_profiler) as prof:
        for step in range(start_step, args.max_train_steps):
            if hb is not None:
                hb.barrier(step)
            timed = (step - start_step) > warmup       # a resumed run warms up again
            if timed:
                t0 = time.time()
                timer.start()
            batch = torch.randint(cfg.vocab_size, (args.batch_size, args.seq_length + 1))
            loss = trainer.train_step(batch)
            if rank == 0:
                m = memory_gb(dev)
                print(f"CUDA memory allocated: {m['allocated']:.2f} GB, reserved: {m['reserved']:.2f} GB")
                loss_val = loss.item()
                print(f"step {step}, loss: {loss_val}")
                trainer.check_status(block=True)       # rank 0 has just synchronised anyway
            if timed:
                timer.stop()
                elapse += time.time() - t0
                timed_steps += 1
            if prof is not None:
                prof.step()
            rec = {"step": step, "loss": loss_val}
            if args.jsonl:      # every rank takes part in the max-over-ranks reductions
                rec["exposed_comm_ms"] = exposed_comm_ms(ctx, reset=True)
                rec["phase_ms"] = trainer.phase_summary(reset=True)
                if timed:
                    exposed_sum += rec["exposed_comm_ms"]
            writer.write(**rec, **memory_gb(dev))
    trainer.check_status(block=True)
    dev_ms = max_over_ranks(timer.elapsed_ms(), dev)
    tok_s = timed_steps * args.seq_length / (dev_ms / 1e3) if dev_ms > 0 else 0.0
    flops = train_flops_per_token(cfg, args.seq_length) * tok_s / max(1, world)
    if rank == 0:
        print(f"{args.parallel_mode} {args.seq_length // 1024}K {world} Time taken: {elapse:.2f} seconds")
        m = memory_gb(dev)
        print(f"device time (max over ranks) {dev_ms / 1e3:.3f} s over {timed_steps} steps; {tok_s:.0f} tokens/s; "
              f"peak allocated {m['peak_allocated']:.2f} GB, peak reserved {m['peak_reserved']:.2f} GB")
    peak = max_over_ranks(memory_gb(dev)["peak_allocated"], dev)
    writer.write(final=True, mode=args.parallel_mode, model=cfg.name, seq_length=args.seq_length, world=world,
                 inner_degree=ctx.inner_size, ring_degree=ctx.ring_size, backend=native.get_backend(),
                 grad_checkpoint=bool(args.grad_checkpoint), timed_steps=timed_steps, elapsed_s=elapse,
                 device_s=dev_ms / 1e3, tokens_per_s=tok_s, model_tflops_per_gpu=flops / 1e12,
                 exposed_comm_ms_per_step=(exposed_sum / timed_steps) if timed_steps else None,
                 peak_allocated_gb_max_over_ranks=peak, **memory_gb(dev))
    writer.close()
    if args.save:
        ckpt.save_hf_checkpoint(trainer.model, args.save)
        ckpt.save_train_state(args.save, trainer.optimizer, args.max_train_steps, rank)
    return {"loss": loss_val, "elapsed_s": elapse, "device_s": dev_ms / 1e3, "tokens_per_s": tok_s}


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="Sequence-parallel Llama training on B200 (Odysseus / TP-SP / Ulysses / ring)")
    d = TrainConfig()
    p.add_argument("--batch-size", "--batch_size", type=int, default=d.batch_size)
    p.add_argument("--seed", type=int, default=d.seed)
    p.add_argument("--max-train-steps", "--max_train_steps", type=int, default=d.max_train_steps)
    p.add_argument("--learning-rate", "--learning_rate", type=float, default=d.learning_rate)
    p.add_argument("--rope-theta", "--rope_theta", type=float, default=None)
    p.add_argument("--model", type=str, default="meta-llama/Llama-2-7b-hf")
    p.add_argument("--seq-length", "--seq_length", type=int, default=d.seq_length)
    p.add_argument("--cpu-offload", "--cpu_offload", action="store_true", default=False)
    p.add_argument("--grad-checkpoint", "--grad_checkpoint", action="store_true", default=False)
    p.add_argument("--use_zero2", "--use-zero2", action="store_true", default=False)
    p.add_argument("--use_ody_zero3", "--use-ody-zero3", action="store_true", default=True)
    p.add_argument("--no_ody_zero3", "--no-ody-zero3", dest="use_ody_zero3", action="store_false",
                   help="odysseus mode: keep the MLP weights whole on every rank and all-reduce their gradients "
                        "(the reference's flag is store_true with default True and cannot be switched off, train.py:255)")
    p.add_argument("--use_profiler", "--use-profiler", action="store_true", default=False)
    p.add_argument("--use_cfg_init_model", "--use-cfg-init-model", action="store_true", default=False)
    p.add_argument("--parallel_mode", "--parallel-mode", type=str, choices=list(PARALLEL_MODES))
    # additions
    p.add_argument("--ulysses-degree", "--ulysses_degree", type=int, default=0)
    p.add_argument("--ring-degree", "--ring_degree", type=int, default=1)
    p.add_argument("--model-config", "--model_config", type=str, default=None,
                   help="named synthetic architecture (tiny, llama2-7b, llama3-8b, ...); random-init weights")
    p.add_argument("--backend", type=str, default="auto", choices=["auto", "fused", "library"])
    p.add_argument("--dtype", type=str, default="bf16", choices=["bf16", "fp32", "fp16"])
    p.add_argument("--warmup-iterations", "--warmup_iterations", type=int, default=d.warmup_iterations)
    p.add_argument("--heartbeat-timeout", "--heartbeat_timeout", type=float, default=0.0)
    p.add_argument("--loss-chunk-rows", "--loss_chunk_rows", type=int, default=None,
                   help="tokens per lm_head + cross-entropy chunk (0 = whole logits; default: chunk beyond 2 GiB of logits)")
    p.add_argument("--jsonl", type=str, default=None)
    p.add_argument("--save", type=str, default=None)
    p.add_argument("--load", type=str, default=None)
    return p


def cli() -> None:
    """Console entry point (``odysseus-train``): the same flags as ``python train.py``."""
    main(build_parser().parse_args())


if __name__ == "__main__":
    cli()
