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
from .utils.health import Heartbeat
from .utils.metrics import DeviceTimer, JsonlWriter, max_over_ranks, memory_gb
from .utils.profiler import init_prof


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
    loss.  ``train_step_device`` takes already-sliced device tensors."""

    def __init__(self, cfg: ModelConfig, mode: Optional[str], ctx: ParallelContext, seq_length: int,
                 lr: float = 2e-5, weight_decay: float = 0.01, betas=(0.9, 0.999), eps: float = 1e-8,
                 dtype: torch.dtype = torch.bfloat16, seed: int = 42, ulysses_degree: int = 0,
                 ring_degree: int = 1, state_dict: Optional[Dict[str, torch.Tensor]] = None,
                 grad_checkpoint: bool = False, use_zero2: bool = False):
        self.cfg, self.mode, self.ctx, self.seq_length = cfg, mode, ctx, seq_length
        self.ulysses_degree, self.ring_degree = ulysses_degree, ring_degree
        set_global_memory_buffer(ctx.device)
        if ctx.world_size > 1 and ctx.device.type == "cuda" and native.get_backend() != "library" and dtype == torch.bfloat16:
            from .comm import symm
            symm.setup_fused_comm(ctx, cfg, max(1, seq_length // ctx.world_size), mode=mode)
        self.model = build_model(cfg, mode, ctx, dtype=dtype, device=ctx.device, seed=seed, state_dict=state_dict)
        if grad_checkpoint:
            self.model.gradient_checkpointing_enable()
        if use_zero2:
            self.model.zero3.keep_gathered = True
        self.optimizer = ShardedAdamW(self.model.parameters(), lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
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
        loss = self.model(local_input_ids, local_position_ids, labels=local_target_ids,
                          global_tokens=self.global_tokens)
        loss.backward()
        self.optimizer.step()
        self.optimizer.zero_grad()
        self.steps_done += 1
        loss = loss.detach()
        if self.ctx.world_size > 1:
            loss = loss.clone()
            dist.all_reduce(loss, group=self.ctx.world_group)
        return loss

    def train_step(self, batch: torch.Tensor) -> torch.Tensor:
        s = self.shard_batch(batch)
        return self.train_step_device(s["local_input_ids"], s["local_position_ids"], s["local_target_ids"])


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
    if args.cpu_offload:
        raise NotImplementedError("--cpu-offload: parameters are sharded 1/N by construction; offload is not provided")
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
                      state_dict=state_dict, grad_checkpoint=args.grad_checkpoint, use_zero2=args.use_zero2)
    start_step = 0
    if args.load and os.path.exists(os.path.join(args.load, f"train_state_rank{rank}.pt")):
        start_step = ckpt.load_train_state(args.load, trainer.optimizer, rank)
    if rank == 0:
        print(f"{cfg.num_parameters() / 1e9:.2f}B parameters; mode {args.parallel_mode} on {world} rank(s); "
              f"backend {native.get_backend()}")
        m = memory_gb(dev)
        print(f"After init model and optimizer, CUDA memory allocated: {m['allocated']:.2f} GB, reserved: {m['reserved']:.2f} GB")
    hb = None
    if world > 1 and args.heartbeat_timeout > 0:
        hb = Heartbeat(dist.distributed_c10d._get_default_store(), rank, world, args.heartbeat_timeout)
    writer = JsonlWriter(args.jsonl, rank)
    set_seed(args.seed)
    warmup = args.warmup_iterations
    timer = DeviceTimer(dev)
    elapse, timed_steps = 0.0, 0
    loss_val = float("nan")
    with init_prof(args.use_profiler) as prof:
        for step in range(start_step, args.max_train_steps):
            if hb is not None:
                hb.barrier(step)
            timed = step > warmup
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
            if timed:
                timer.stop()
                elapse += time.time() - t0
                timed_steps += 1
            if prof is not None:
                prof.step()
            writer.write(step=step, loss=loss_val, **memory_gb(dev))
    dev_ms = max_over_ranks(timer.elapsed_ms(), dev)
    tok_s = timed_steps * args.seq_length / (dev_ms / 1e3) if dev_ms > 0 else 0.0
    if rank == 0:
        print(f"{args.parallel_mode} {args.seq_length // 1024}K {world} Time taken: {elapse:.2f} seconds")
        m = memory_gb(dev)
        print(f"device time (max over ranks) {dev_ms / 1e3:.3f} s over {timed_steps} steps; {tok_s:.0f} tokens/s; "
              f"peak allocated {m['peak_allocated']:.2f} GB, peak reserved {m['peak_reserved']:.2f} GB")
    writer.write(final=True, mode=args.parallel_mode, seq_length=args.seq_length, world=world, elapsed_s=elapse,
                 device_s=dev_ms / 1e3, tokens_per_s=tok_s, **memory_gb(dev))
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
    p.add_argument("--jsonl", type=str, default=None)
    p.add_argument("--save", type=str, default=None)
    p.add_argument("--load", type=str, default=None)
    return p


if __name__ == "__main__":
    main(build_parser().parse_args())
