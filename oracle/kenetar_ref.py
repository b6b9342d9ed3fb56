"""Plain restatement of the Kenetar decoder (test infrastructure; nothing under vllm_neuron_b200/ imports it).

Kenetar is a hybrid decoder with post-norm residual branches:  x += N1(mixer(x));  x += N2(ff(x))  where
N(y) = y / sqrt(mean(y^2) + eps) * (1 + w).  The token embedding is scaled and a hashed bigram row is added.  Mixers:
a gated delta-rule recurrence behind short causal convolutions, or latent attention (queries and keys / values through
low-rank latents, one rotated key part shared by the heads, YaRN-scaled rotary angles, a per-head sigmoid output gate).
Feed-forward: a dense gated unit (tanh-GELU) or a mixture of SiLU experts whose router takes the `top` largest
logits and weighs the experts' OUTPUTS by the softmax over the chosen logits.  One function per mechanism, whole sequences,
no cache: a token's output depends on earlier tokens only, so every way of cutting a sequence into engine steps must
reproduce `forward` on the full list.  `dtype` float64 gives the reference values.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rms_unit(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def offset_rms_norm(x, w, eps):
    """Weight stored around zero."""
    return rms_unit(x, eps) * (1 + w)


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def embed_tokens(tokens, W, e):
    """Scaled token row + bigram row hashed from (previous, current); the first token takes the table's last row."""
    t = torch.tensor(tokens, dtype=torch.int64)
    x = W["embed"][t] * e["scale"]
    b = e.get("bigram")
    if b:
        prev = torch.cat([t.new_zeros(1), t[:-1]])
        row = (prev * b["mul_prev"] + t * b["mul_cur"]) % b["buckets"]
        row[0] = b["buckets"]
        x = x + W["bigram"][row]
    return x


def short_conv_silu(u, w):
    """u [T, C]; w [C, taps], the last column multiplies the current token; zeros before the start; no bias."""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.cat([u.new_zeros(taps - 1, C), u])
    out = u.new_zeros(T, C)
    for j in range(taps):
        out = out + pad[j : j + T] * w[:, j]
    return F.silu(out)


def gated_delta_rule(q, k, v, beta, g):
    """q, k [T, H, D]; v [T, H, P]; beta, g [T, H].  Per head, token by token:
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q  (the read-out sees the token's own write)."""
    T, H, D = q.shape
    S = q.new_zeros(H, D, v.shape[-1])
    o = v.new_zeros(v.shape)
    for t in range(T):
        S = g[t, :, None, None] * S
        u = beta[t, :, None] * (v[t] - torch.einsum("hdp,hd->hp", S, k[t]))
        S = S + k[t, :, :, None] * u[:, None, :]
        o[t] = torch.einsum("hdp,hd->hp", S, q[t])
    return o


def delta_mixer(h, W, p, m, eps):
    H, G, D, P = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = short_conv_silu(h @ W[p + "q"].T, W[p + "q.conv"]).view(T, G, D)
    k = short_conv_silu(h @ W[p + "k"].T, W[p + "k.conv"]).view(T, G, D)
    v = short_conv_silu(h @ W[p + "v"].T, W[p + "v.conv"]).view(T, H, P)
    unit = lambda a: a / torch.sqrt(a.pow(2).sum(-1, keepdim=True) + 1e-6)
    q = (unit(q) * D ** -0.5).repeat_interleave(H // G, dim=1)
    k = unit(k).repeat_interleave(H // G, dim=1)
    beta = torch.sigmoid(h @ W[p + "b"].T)
    g = torch.exp(-torch.exp(W[p + "A_log"]) * F.softplus(h @ W[p + "a"].T + W[p + "dt_bias"]))
    o = gated_delta_rule(q, k, v, beta, g)
    o = rms_unit(o, eps) * W[p + "norm"] * F.silu(h @ W[p + "g"].T).view(T, H, P)
    return o.reshape(T, H * P) @ W[p + "o"].T


def yarn_angles(rot, positions, dtype):
    """Per-pair rotary frequency with YaRN's blend between the plain and the stretched one -> (cos, sin) [T, dims/2],
    both multiplied by the attention factor 0.1 ln(factor) + 1."""
    dims, base = rot["dims"], rot["base"]
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2 * i / dims)
    mscale = 1.0
    s = rot.get("scaling")
    if s:
        corr = lambda turns: dims * math.log(s["original"] / (2 * math.pi * turns)) / (2 * math.log(base))
        lo = max(math.floor(corr(s["fast"])), 0)
        hi = min(math.ceil(corr(s["slow"])), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
        f = f / s["factor"] * ramp + f * (1 - ramp)
        mscale = 0.1 * math.log(s["factor"]) + 1
    a = torch.as_tensor(positions, dtype=torch.float64)[:, None] * f
    return (torch.cos(a) * mscale).to(dtype), (torch.sin(a) * mscale).to(dtype)


def rotate_pairs(x, cos, sin):
    """x [T, ..., dims] with (2i, 2i+1) pairs; cos, sin [T, dims/2]."""
    u, v = x[..., 0::2], x[..., 1::2]
    while cos.dim() < u.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    return torch.stack([u * cos - v * sin, v * cos + u * sin], dim=-1).flatten(-2)


def latent_attention(h, W, p, m, eps):
    H, D, R, P, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    cq = rms_unit(h @ W[p + "dq"].T, eps) * W[p + "dq.norm"]
    q = (cq @ W[p + "uq"].T).view(T, H, D + R)
    kv = h @ W[p + "dkv"].T
    c = rms_unit(kv[:, :C], eps) * W[p + "dkv.norm"]
    cos, sin = yarn_angles(m["rot"], range(T), h.dtype)
    n = m["rot"]["dims"]  # the first n of the rotated part turn, the rest passes
    k_rot = torch.cat([rotate_pairs(kv[:, C : C + n], cos, sin), kv[:, C + n :]], dim=-1)
    q_rot = torch.cat([rotate_pairs(q[..., D : D + n], cos, sin), q[..., D + n :]], dim=-1)
    k = (c @ W[p + "uk"].T).view(T, H, D)
    v = (c @ W[p + "uv"].T).view(T, H, P)
    s = (torch.einsum("ihd,jhd->hij", q[..., :D], k) + torch.einsum("ihr,jr->hij", q_rot, k_rot)) * m["scale"]
    causal = torch.arange(T)[:, None] >= torch.arange(T)[None, :]
    pr = torch.softmax(s.masked_fill(~causal, -math.inf), dim=-1)
    o = torch.einsum("hij,jhd->ihd", pr, v) * torch.sigmoid(h @ W[p + "g"].T)[:, :, None]
    return o.reshape(T, H * P) @ W[p + "o"].T


def dense_ff(h, W, p):
    return (gelu_tanh(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def softmax_topk_moe(h, W, p, f):
    E, top = f["router"]["experts"], f["router"]["top"]
    z = h @ W[p + "router"].T + W[p + "router.b"]
    val, idx = z.topk(top, dim=-1)
    wt = torch.softmax(val, dim=-1)
    out = torch.zeros_like(h)
    for e in range(E):
        for c in range(top):
            rows = (idx[:, c] == e).nonzero().flatten()
            if rows.numel():
                a = h[rows]
                y = (F.silu(a @ W[f"{p}e{e}.gate"].T) * (a @ W[f"{p}e{e}.up"].T)) @ W[f"{p}e{e}.down"].T
                out[rows] += wt[rows, c, None] * y
    return out


def forward(cfg, W, tokens, dtype=torch.float64, want_layers=False):
    """tokens: list[int] of ONE sequence -> logits [T, vocab] (and, with want_layers, x as each layer leaves it)."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    x = embed_tokens(tokens, W, cfg["embedding"])
    streams = []
    for li, L in enumerate(cfg["layers"]):
        p = f"l{li}."
        if L["type"] == "delta":
            y = delta_mixer(x, W, p + "mix.", L["mixer"], eps)
        elif L["type"] == "latent_attention":
            y = latent_attention(x, W, p + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + offset_rms_norm(y, W[p + "norm1"], eps)
        f = L.get("mlp")
        if f:
            y = dense_ff(x, W, p + "mlp.") if f["kind"] == "dense" else softmax_topk_moe(x, W, p + "mlp.", f)
            x = x + offset_rms_norm(y, W[p + "norm2"], eps)
        streams.append(x)
    logits = offset_rms_norm(x, W["final.norm"], eps) @ W["head"].T * cfg.get("logit_scale", 1.0)
    return (logits, torch.stack(streams)) if want_layers else logits
