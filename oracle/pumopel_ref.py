"""Plain restatement of the Pumopel decoder (test infrastructure; nothing under vllm_neuron_b200/ imports it).

Pumopel is a hybrid decoder: every layer is  x += N1b(mixer(N1(x)));  x += N2b(ff(N2(x)))  with Dynamic-Tanh norms
N(x) = gain * tanh(a x) + shift, a mixer that is either a Mamba-2 state-space layer or sliding-window attention without
positional rotation, with a per-head softmax sink and value mixing across layers, and a mixture-of-experts feed-forward
whose routing weight scales the expert's INPUT.  One function per mechanism, whole sequences at a time, no cache: a
token's output depends on the tokens before it only, so prefill, chunked prefill and decode of the product path must all
reproduce `forward` on the full token list.  `dtype` float64 gives the reference values; weights come as a
name -> tensor dictionary under the checkpoint's tensor names.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def dyt(x, W, name):
    """Dynamic Tanh, elementwise: gain * tanh(a * x) + shift."""
    return torch.tanh(W[name + ".alpha"] * x) * W[name] + W[name + ".b"]


def rms_unit(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def causal_conv_silu(u, w, b):
    """u [T, C]; w [C, taps] (last column multiplies the current token); zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.cat([u.new_zeros(taps - 1, C), u])
    out = b.clone().expand(T, C).clone()
    for j in range(taps):
        out = out + pad[j : j + T] * w[:, j]
    return F.silu(out)


def selective_scan(x, B, C, dt_raw, dt_bias, A_log, D, S0=None):
    """x [T, H, P]; B, C [T, H, N] (already expanded per head); dt_raw [T, H].  Returns y [T, H, P]."""
    T, H, P = x.shape
    dt = F.softplus(dt_raw + dt_bias)                       # no clamp
    decay = torch.exp(-torch.exp(A_log) * dt)
    S = x.new_zeros(H, B.shape[-1], P) if S0 is None else S0.clone()
    y = x.new_zeros(T, H, P)
    for t in range(T):
        S = decay[t, :, None, None] * S + dt[t, :, None, None] * B[t, :, :, None] * x[t, :, None, :]
        y[t] = torch.einsum("hnp,hn->hp", S, C[t]) + D[:, None] * x[t]
    return y


def mamba2_mixer(h, W, p, m, eps):
    """h [T, width].  m: heads, vdim, state, groups, conv, norm_groups."""
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    T = h.shape[0]
    proj = h @ W[p + "in"].T
    z, xBC, dt = proj.split([inner, inner + 2 * G * N, H], dim=-1)
    xBC = causal_conv_silu(xBC, W[p + "conv"], W[p + "conv.b"])
    x, B, C = xBC.split([inner, G * N, G * N], dim=-1)
    x = x.view(T, H, P)
    B = B.view(T, G, N).repeat_interleave(H // G, dim=1)   # head h reads group h // (H / G)
    C = C.view(T, G, N).repeat_interleave(H // G, dim=1)
    y = selective_scan(x, B, C, dt, W[p + "dt_bias"], W[p + "A_log"], W[p + "D"])
    y = y.reshape(T, inner) * F.silu(z)                     # gate first, normalise second
    ng = m["norm_groups"]
    y = rms_unit(y.view(T, ng, inner // ng), eps).reshape(T, inner) * W[p + "norm"]
    return y @ W[p + "o"].T


def sink_window_attention(q, k, v, sink, scale, window):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] of one sequence -> [T, H * Dv].  query i attends keys i - window < j <= i;
    the softmax runs over those scores and one extra per-head logit `sink` that is dropped afterwards."""
    T, H, _ = q.shape
    G = k.shape[1]
    kk = k.repeat_interleave(H // G, dim=1)
    vv = v.repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = (i - j >= 0) & (i - j < window)
    s = s.masked_fill(~seen, -math.inf)
    sk = sink.to(s.dtype)[:, None, None].expand(H, T, 1)
    pr = torch.softmax(torch.cat([s, sk], dim=-1), dim=-1)[..., :T]
    return torch.einsum("hij,jhd->ihd", pr, vv).reshape(T, H * v.shape[-1])


def swa_sink_attention(h, W, p, m, v_first):
    """Sliding-window attention, no rotation, softmax with a per-head sink logit in the denominator.
    Returns (output, the values this layer cached)."""
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ W[p + "q"].T).view(T, H, D)
    k = (h @ W[p + "k"].T).view(T, G, D)
    v = (h @ W[p + "v"].T).view(T, G, Dv)
    if m.get("v_mix") and v_first is not None:
        lam = W[p + "vmix"]
        v = (1 - lam) * v + lam * v_first
    o = sink_window_attention(q, k, v, W[p + "sink"], m["scale"], m["mask"]["size"] if m.get("mask") else T + 1)
    return o @ W[p + "o"].T, v


def clamped_glu_expert(h, W, p, limit):
    g = (h @ W[p + "gate"].T).clamp(max=limit)
    u = (h @ W[p + "up"].T).clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ W[p + "down"].T


def moe_ff(h, W, p, f):
    """Sigmoid router, top-k by score, weights = scores (not renormalised), weight applied to the expert's input."""
    E, top = f["router"]["experts"], f["router"]["top"]
    s = torch.sigmoid(h @ W[p + "router"].T)
    val, idx = s.topk(top, dim=-1)
    out = torch.zeros_like(h)
    for e in range(E):
        for c in range(top):
            rows = (idx[:, c] == e).nonzero().flatten()
            if rows.numel():
                out[rows] += clamped_glu_expert(val[rows, c, None] * h[rows], W, f"{p}e{e}.", f["expert"]["limit"])
    if f.get("shared"):
        out = out + clamped_glu_expert(h, W, p + "shared.", f["shared"]["limit"])
    return out


def forward(cfg, W, tokens, dtype=torch.float64, want_layers=False):
    """tokens: list[int] of ONE sequence -> logits [T, vocab] (and, with want_layers, x as each layer leaves it)."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    v_first = None
    streams = []
    for li, L in enumerate(cfg["layers"]):
        p = f"l{li}."
        h = dyt(x, W, p + "norm1")
        if L["type"] == "mamba2":
            y = mamba2_mixer(h, W, p + "mix.", L["mixer"], eps)
        elif L["type"] == "attention":
            y, v = swa_sink_attention(h, W, p + "mix.", L["mixer"], v_first)
            if L["mixer"].get("v_mix") and v_first is None:
                v_first = v
        else:
            raise ValueError(L["type"])
        x = x + dyt(y, W, p + "norm1b")
        if L.get("mlp"):
            x = x + dyt(moe_ff(dyt(x, W, p + "norm2"), W, p + "mlp.", L["mlp"]), W, p + "norm2b")
        streams.append(x)
    logits = dyt(x, W, "final.norm") @ W["head"].T
    return (logits, torch.stack(streams)) if want_layers else logits
