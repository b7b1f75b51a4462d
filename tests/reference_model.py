"""Independent single-process Llama used as the oracle: plain nn.functional ops + causal SDPA,
consuming the HF-named state dict directly.  Shares no code with the package's ops."""
import torch
import torch.nn.functional as Fn


def _rms(x, w, eps):
    v = x.float().pow(2).mean(-1, keepdim=True)
    return (x.float() * torch.rsqrt(v + eps)).to(x.dtype) * w


def _rope(x, pos, theta):
    # x [B, H, T, hd], HF rotate-half
    hd = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
    f = pos.float()[:, None] * inv[None, :]
    emb = torch.cat([f, f], -1)
    cos, sin = emb.cos()[None, None], emb.sin()[None, None]
    x1, x2 = x[..., : hd // 2], x[..., hd // 2:]
    rot = torch.cat([-x2, x1], -1)
    return (x.float() * cos + rot.float() * sin).to(x.dtype)


def reference_loss(cfg, sd, input_ids, targets):
    """input_ids, targets: [L] long.  Returns mean CE over L tokens; sd tensors need requires_grad."""
    L = input_ids.shape[0]
    H, Hkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    pos = torch.arange(L)
    x = sd["model.embed_tokens.weight"][input_ids]
    for n in range(cfg.num_hidden_layers):
        p = f"model.layers.{n}."
        h = _rms(x, sd[p + "input_layernorm.weight"], cfg.rms_norm_eps)
        q = (h @ sd[p + "self_attn.q_proj.weight"].t()).view(1, L, H, hd).transpose(1, 2)
        k = (h @ sd[p + "self_attn.k_proj.weight"].t()).view(1, L, Hkv, hd).transpose(1, 2)
        v = (h @ sd[p + "self_attn.v_proj.weight"].t()).view(1, L, Hkv, hd).transpose(1, 2)
        q, k = _rope(q, pos, cfg.rope_theta), _rope(k, pos, cfg.rope_theta)
        if Hkv != H:
            k = k.repeat_interleave(H // Hkv, dim=1)
            v = v.repeat_interleave(H // Hkv, dim=1)
        a = Fn.scaled_dot_product_attention(q, k, v, is_causal=True)
        a = a.transpose(1, 2).reshape(L, H * hd)
        x = x + a @ sd[p + "self_attn.o_proj.weight"].t()
        h = _rms(x, sd[p + "post_attention_layernorm.weight"], cfg.rms_norm_eps)
        g = h @ sd[p + "mlp.gate_proj.weight"].t()
        u = h @ sd[p + "mlp.up_proj.weight"].t()
        x = x + (Fn.silu(g) * u) @ sd[p + "mlp.down_proj.weight"].t()
    h = _rms(x, sd["model.norm.weight"], cfg.rms_norm_eps)
    logits = h @ sd["lm_head.weight"].t()
    return Fn.cross_entropy(logits.float(), targets), logits
