"""Plain-PyTorch implementations of every hot op: forward and hand-derived backward.

These run on CPU (fp32 parity tests over gloo) and on CUDA as the "library" baseline path, and
they are the numerical oracle for the sm_100a kernels in ``csrc/``.  Each function mirrors the
argument list of its native counterpart so ``ops.functional`` can switch between the two.

Semantics follow the model the reference trains (HF Llama, reference ``train.py:66-86``):
RMSNorm with fp32 statistics, rotate-half RoPE, SwiGLU ``silu(gate) * up``, causal softmax
attention with grouped KV heads, token-level cross-entropy.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

# ----------------------------------------------------------------------------- RMSNorm


def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """y = x * rsqrt(mean(x^2) + eps) * w ; returns (y, rstd[T] fp32)."""
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1) + eps)
    y = (xf * rstd.unsqueeze(-1) * w.float()).to(x.dtype)
    return y, rstd


def rmsnorm_bwd(dy: torch.Tensor, x: torch.Tensor, w: torch.Tensor, rstd: torch.Tensor):
    """Returns (dx in x.dtype, dw fp32)."""
    xf, dyf, wf = x.float(), dy.float(), w.float()
    xhat = xf * rstd.unsqueeze(-1)
    g = dyf * wf
    dw = (dyf * xhat).sum(0)
    c = (g * xhat).mean(-1, keepdim=True)
    dx = (g - xhat * c) * rstd.unsqueeze(-1)
    return dx.to(x.dtype), dw


def add_rmsnorm_fwd(x: torch.Tensor, delta: torch.Tensor, w: torch.Tensor, eps: float):
    """Residual add fused with the norm: s = x + delta ; y = rmsnorm(s). Returns (s, y, rstd)."""
    s = (x.float() + delta.float()).to(x.dtype)
    y, rstd = rmsnorm_fwd(s, w, eps)
    return s, y, rstd


# ----------------------------------------------------------------------------- RoPE


def rope_tables(positions: torch.Tensor, head_dim: int, theta: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables [T, head_dim/2] in fp32 for integer positions [T]."""
    half = head_dim // 2
    inv_freq = 1.0 / (theta ** (torch.arange(0, half, device=positions.device, dtype=torch.float32) * 2.0 / head_dim))
    ang = positions.to(torch.float32).unsqueeze(-1) * inv_freq.unsqueeze(0)
    return ang.cos(), ang.sin()


def rope_apply(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, inverse: bool = False) -> torch.Tensor:
    """Rotate-half RoPE on x [T, H, hd] with tables [T, hd/2]; ``inverse`` applies the transpose
    rotation, which is the backward of the forward map."""
    half = x.shape[-1] // 2
    xf = x.float()
    x1, x2 = xf[..., :half], xf[..., half:]
    c = cos.unsqueeze(1)
    s = sin.unsqueeze(1)
    if inverse:
        s = -s
    y = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)
    return y.to(x.dtype)


# ----------------------------------------------------------------------------- SwiGLU


def swiglu_fwd(gu: torch.Tensor) -> torch.Tensor:
    """gu [T, 2i] laid out [gate | up] -> silu(gate) * up  [T, i]."""
    i = gu.shape[-1] // 2
    g, u = gu[..., :i].float(), gu[..., i:].float()
    return (torch.nn.functional.silu(g) * u).to(gu.dtype)


def swiglu_bwd(dh: torch.Tensor, gu: torch.Tensor) -> torch.Tensor:
    i = gu.shape[-1] // 2
    g, u = gu[..., :i].float(), gu[..., i:].float()
    dhf = dh.float()
    sig = torch.sigmoid(g)
    silu = g * sig
    dg = dhf * u * (sig * (1.0 + g * (1.0 - sig)))
    du = dhf * silu
    return torch.cat([dg, du], dim=-1).to(gu.dtype)


# ----------------------------------------------------------------------------- cross-entropy


def cross_entropy_fwd(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100):
    """Per-row loss and log-sum-exp, both fp32 [T]; ignored rows give loss 0."""
    lf = logits.float()
    lse = torch.logsumexp(lf, dim=-1)
    valid = targets != ignore_index
    tgt = targets.clamp_min(0)
    picked = lf.gather(-1, tgt.unsqueeze(-1)).squeeze(-1)
    loss = torch.where(valid, lse - picked, torch.zeros_like(lse))
    return loss, lse


def cross_entropy_bwd_(logits: torch.Tensor, targets: torch.Tensor, lse: torch.Tensor, scale,
                       ignore_index: int = -100) -> torch.Tensor:
    """Overwrites ``logits`` with d(loss_sum * scale)/dlogits = (softmax - onehot) * scale."""
    valid = (targets != ignore_index)
    tgt = targets.clamp_min(0)
    lf = logits.float()
    p = torch.exp(lf - lse.unsqueeze(-1))
    p.scatter_add_(-1, tgt.unsqueeze(-1), -torch.ones_like(p[..., :1]))
    p = p * (valid.unsqueeze(-1).to(p.dtype) * scale)
    logits.copy_(p.to(logits.dtype))
    return logits


# ----------------------------------------------------------------------------- attention blocks


def _expand_kv(k: torch.Tensor, n_q_heads: int) -> torch.Tensor:
    rep = n_q_heads // k.shape[1]
    return k if rep == 1 else k.repeat_interleave(rep, dim=1)


def attn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool,
             scale: Optional[float] = None, q_chunk: int = 2048):
    """Softmax attention block. q [Tq,H,hd], k/v [Tk,Hkv,hd]; ``causal`` needs Tq == Tk.

    Returns out [Tq,H,hd] (q.dtype) and lse [H,Tq] fp32 (natural log)."""
    Tq, H, hd = q.shape
    Tk = k.shape[0]
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    kf = _expand_kv(k, H).float().permute(1, 2, 0)      # [H, hd, Tk]
    vf = _expand_kv(v, H).float().permute(1, 0, 2)      # [H, Tk, hd]
    out = torch.empty(Tq, H, hd, dtype=q.dtype, device=q.device)
    lse = torch.empty(H, Tq, dtype=torch.float32, device=q.device)
    for s in range(0, Tq, q_chunk):
        e = min(Tq, s + q_chunk)
        qf = q[s:e].float().permute(1, 0, 2)            # [H, c, hd]
        sc = torch.matmul(qf, kf) * scale               # [H, c, Tk]
        if causal:
            rows = torch.arange(s, e, device=q.device).unsqueeze(-1)
            cols = torch.arange(Tk, device=q.device).unsqueeze(0)
            sc = sc.masked_fill((cols > rows).unsqueeze(0), float("-inf"))
        l = torch.logsumexp(sc, dim=-1)
        p = torch.exp(sc - l.unsqueeze(-1))
        out[s:e] = torch.matmul(p, vf).permute(1, 0, 2).to(q.dtype)
        lse[:, s:e] = l
    return out, lse


def attn_bwd(do: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor,
             lse: torch.Tensor, causal: bool, scale: Optional[float] = None, q_chunk: int = 2048,
             delta: Optional[torch.Tensor] = None):
    """Backward of one attention block given the *final* (o, lse) of the rows of q.

    P = exp(S*scale - lse); dV = P^T dO; dP = dO V^T; dS = P * (dP - delta); dQ = dS K * scale;
    dK = dS^T Q * scale, with delta = rowsum(dO * O).  Returns fp32 (dq, dk, dv); dk/dv have
    Hkv heads (summed over the query heads of each group)."""
    Tq, H, hd = q.shape
    Tk, Hkv, _ = k.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    kf = _expand_kv(k, H).float().permute(1, 0, 2)      # [H, Tk, hd]
    vf = _expand_kv(v, H).float().permute(1, 0, 2)
    dq = torch.empty(Tq, H, hd, dtype=torch.float32, device=q.device)
    dk = torch.zeros(H, Tk, hd, dtype=torch.float32, device=q.device)
    dv = torch.zeros(H, Tk, hd, dtype=torch.float32, device=q.device)
    if delta is None:
        delta = (do.float() * o.float()).sum(-1).transpose(0, 1)   # [H, Tq]
    for s in range(0, Tq, q_chunk):
        e = min(Tq, s + q_chunk)
        qf = q[s:e].float().permute(1, 0, 2)
        dof = do[s:e].float().permute(1, 0, 2)
        sc = torch.matmul(qf, kf.transpose(1, 2)) * scale
        if causal:
            rows = torch.arange(s, e, device=q.device).unsqueeze(-1)
            cols = torch.arange(Tk, device=q.device).unsqueeze(0)
            sc = sc.masked_fill((cols > rows).unsqueeze(0), float("-inf"))
        p = torch.exp(sc - lse[:, s:e].unsqueeze(-1))
        dv += torch.matmul(p.transpose(1, 2), dof)
        dp = torch.matmul(dof, vf.transpose(1, 2))
        ds = p * (dp - delta[:, s:e].unsqueeze(-1)) * scale
        dq[s:e] = torch.matmul(ds, kf).permute(1, 0, 2)
        dk += torch.matmul(ds.transpose(1, 2), qf)
    rep = H // Hkv
    dk = dk.view(Hkv, rep, Tk, hd).sum(1).permute(1, 0, 2).contiguous()
    dv = dv.view(Hkv, rep, Tk, hd).sum(1).permute(1, 0, 2).contiguous()
    return dq, dk, dv


def merge_attn(out_a: torch.Tensor, lse_a: torch.Tensor, out_b: torch.Tensor, lse_b: torch.Tensor):
    """Combine two partial attention results over disjoint key sets (fp32 out [T,H,hd], lse [H,T])."""
    lse = torch.logaddexp(lse_a, lse_b)
    wa = torch.exp(lse_a - lse).transpose(0, 1).unsqueeze(-1)
    wb = torch.exp(lse_b - lse).transpose(0, 1).unsqueeze(-1)
    return out_a * wa + out_b * wb, lse


# ----------------------------------------------------------------------------- AdamW


def adamw_step_(master: torch.Tensor, m: torch.Tensor, v: torch.Tensor, grad: torch.Tensor,
                param_out: Optional[torch.Tensor], lr: float, beta1: float, beta2: float, eps: float,
                weight_decay: float, step: int, grad_scale: float = 1.0,
                guard: Optional[torch.Tensor] = None) -> None:
    """Decoupled-weight-decay Adam on an fp32 master shard; writes the low-precision copy.
    A non-zero ``guard`` (first element) leaves everything untouched, like the CUDA kernel's guard word."""
    if guard is not None and float(guard.reshape(-1)[0]) != 0.0:
        return
    g = grad.float() * grad_scale
    master.mul_(1.0 - lr * weight_decay)
    m.mul_(beta1).add_(g, alpha=1.0 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    master.addcdiv_(m, denom, value=-lr / bc1)
    if param_out is not None:
        param_out.copy_(master.to(param_out.dtype))
