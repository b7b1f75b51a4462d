"""Worker for the multi-GPU tests: run under torch.distributed.run, one rank per GPU.

Usage: mgpu_worker.py MODE CONFIG SEQLEN ULYSSES RING BACKEND [ITERS [VARIANT]]
Every rank builds the model in MODE (bf16), runs ITERS forward + backward passes on its shard (the later ones reuse
every buffer, slot and epoch counter of the fused paths), exports loss and HF-layout gradients; rank 0 compares
them with a single-GPU fp32 run of the same (bf16-rounded) weights in plain PyTorch.
VARIANT: none | zero2 (gathered ZeRO-3 weights kept for backward) | gradckpt (activation checkpointing) |
chunked (lm_head + loss in row chunks)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    mode, cfg_name, L, U, R, backend = sys.argv[1], sys.argv[2], int(sys.argv[3]), int(sys.argv[4]), int(sys.argv[5]), sys.argv[6]
    iters = int(sys.argv[7]) if len(sys.argv) > 7 else 2
    variant = sys.argv[8] if len(sys.argv) > 8 else "none"
    from odysseus_transformer_b200.config import get_model_config
    from odysseus_transformer_b200.mesh import ParallelContext, init_parallel_context
    from odysseus_transformer_b200.ops import native
    from odysseus_transformer_b200.parallel.apply import build_model, prepare_attn_inputs
    from odysseus_transformer_b200.utils.debug import export_hf_grads
    native.set_backend(backend)
    ctx = init_parallel_context(mode, U, R, backend=backend, timeout_s=120)
    if backend == "fused":
        from odysseus_transformer_b200.comm import symm
        symm.setup_fused_comm(ctx)
    rank, world, dev = ctx.rank, ctx.world_size, ctx.device
    cfg = get_model_config(cfg_name)
    g = torch.Generator().manual_seed(0)
    batch = torch.randint(cfg.vocab_size, (1, L + 1), generator=g)
    pos = torch.arange(L).unsqueeze(0)
    model = build_model(cfg, mode, ctx, dtype=torch.bfloat16, device=dev, seed=0,
                        loss_chunk_rows=128 if variant == "chunked" else 0)
    if variant == "zero2":
        model.zero3.keep_gathered = True
    if variant == "gradckpt":
        model.gradient_checkpointing_enable()
    s = prepare_attn_inputs(mode, batch[:, :-1], pos, batch[:, 1:], rank, world, dev, U, R)
    gt = L * (world if mode == "dp" else 1)
    for it in range(iters):   # later iterations exercise buffer / flag / epoch reuse
        for p in model.parameters():
            p.grad = None
        loss = model(s["local_input_ids"], s["local_position_ids"], labels=s["local_target_ids"], global_tokens=gt)
        loss.backward()
    total = loss.detach().float().clone()
    dist.all_reduce(total)
    grads = export_hf_grads(model)
    torch.cuda.synchronize()
    native.check_status(dev.index)
    ok = True
    if rank == 0:
        native.set_backend("library")
        from odysseus_transformer_b200.models.llama import random_hf_state_dict
        sd = {k: v.float() for k, v in random_hf_state_dict(cfg, 0, dev, torch.bfloat16).items()}   # the same rounded weights
        ref = build_model(cfg, None, ParallelContext(device=dev), dtype=torch.float32, device=dev, seed=None, state_dict=sd)
        rl = ref(batch[:, :-1].to(dev), pos.to(dev), labels=batch[:, 1:].to(dev))
        rl.backward()
        rg = export_hf_grads(ref)
        dl = abs(total.item() - rl.item())
        worst, worst_k = 0.0, None
        for k, v in rg.items():
            rel = ((grads[k].float() - v.float()).norm() / (v.float().norm() + 1e-6)).item()
            if rel > worst:
                worst, worst_k = rel, k
        from odysseus_transformer_b200.ops import fused_comm
        print(f"FUSED {fused_comm.stats}", flush=True)
        print(f"RESULT mode={mode} backend={backend} variant={variant} iters={iters} loss={total.item():.5f} "
              f"ref_fp32={rl.item():.5f} dloss={dl:.2e} worst_rel_grad={worst:.3e} ({worst_k})", flush=True)
        ok = dl < 3e-3 and worst < 3e-2
        if backend == "fused" and fused_comm.stats["gather"] + fused_comm.stats["scatter"] == 0:
            print("fused backend requested but no fused collective kernel ran", flush=True)
            ok = False
        if backend == "fused" and mode == "ulysses" and ctx.inner_size > 1 and cfg.head_dim == 128 and L // world % 128 == 0 \
                and fused_comm.stats.get("ulysses", 0) == 0:
            print("fused backend requested but the Ulysses exchanges ran as separate all-to-alls", flush=True)
            ok = False
        if backend == "fused" and ctx.ring_size > 1 and cfg.head_dim == 128 and fused_comm.stats.get("ring", 0) == 0:
            print("fused backend requested but ring attention ran the all-gather composition", flush=True)
            ok = False
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.broadcast(flag, 0)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1 else 1)


if __name__ == "__main__":
    main()
