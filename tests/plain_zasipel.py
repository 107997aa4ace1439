"""A plain, slow implementation of the Zasipel design in torch on the CPU: the oracle of the tests.

One function per mechanism, written from the design's equations in 64-bit, whole sequences at a time (a state can
be carried, so that a sequence may also be walked token by token), no cache and no batching.  It shares no code
with the package.

Notation: ``h`` a sublayer's input [T, width]; ``W x`` is ``x @ W.T`` for a weight stored [out, in]; positions
count from 0.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def rms_norm(x, w, eps):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


# ---------------------------------------------------------------- short causal convolution
def short_conv(x, w, history=None):
    """x [T, C]; w [C, taps], the last column weighs the current token; ``history`` [taps - 1, C]: the inputs just
    before x (zeros at the start of a sequence).  Returns (y [T, C], the last taps - 1 inputs)."""
    T, C = x.shape
    taps = w.shape[1]
    if history is None:
        history = x.new_zeros((taps - 1, C))
    full = torch.cat([history, x], 0)                       # row i + taps - 1 is token i
    y = x.new_zeros((T, C))
    for d in range(taps):                                   # d tokens back
        y += full[taps - 1 - d: taps - 1 - d + T] * w[:, taps - 1 - d]
    return y, full[full.shape[0] - (taps - 1):]


# ---------------------------------------------------------------- the delta rule
def delta_rule(q, k, v, beta, g, S=None):
    """q, k [T, H, dk] (already per value head), v [T, H, dv], beta [T, H], g [T, H] (one decay a head) or
    [T, H, dk] (one per key channel: row i of S).  S [H, dk, dv] carried.  Returns (o [T, H, dv], S)."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    if S is None:
        S = q.new_zeros((H, dk, dv))
    o = q.new_zeros((T, H, dv))
    for t in range(T):
        gt = g[t][:, None, None] if g.dim() == 2 else g[t][:, :, None]
        S = gt * S
        read = torch.einsum("hkv,hk->hv", S, k[t])
        u = beta[t][:, None] * (v[t] - read)
        S = S + torch.einsum("hk,hv->hkv", k[t], u)
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o, S


def unit(x):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def gated_delta(h, t: Dict[str, torch.Tensor], m: dict, eps, channel: bool, state=None):
    """The gated delta-rule mixer.  ``channel`` False: one decay a head (``a``), output gate silu(W_g h);
    True: a decay per head and key channel through two thin matrices (``a1``, ``a2``), output gate
    sigmoid(W_g2 W_g1 h).  ``state``: dict with ``S`` and the convolutions' histories, carried."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    state = dict(state or {})
    out = {}
    for name in ("q", "k", "v"):
        y, state["conv_" + name] = short_conv(h @ t[name].T, t[name + ".conv"], state.get("conv_" + name))
        out[name] = silu(y)
    rep = H // G
    q = unit(out["q"].reshape(T, G, dk)).repeat_interleave(rep, 1) * dk ** -0.5
    k = unit(out["k"].reshape(T, G, dk)).repeat_interleave(rep, 1)
    v = out["v"].reshape(T, H, dv)
    beta = torch.sigmoid(h @ t["b"].T)
    if channel:
        a = (h @ t["a1"].T) @ t["a2"].T + t["dt_bias"]
        g = torch.exp(-torch.exp(t["A_log"])[None, :, None] * softplus(a).reshape(T, H, dk))
        gate = torch.sigmoid((h @ t["g1"].T) @ t["g2"].T)
    else:
        a = h @ t["a"].T + t["dt_bias"]
        g = torch.exp(-torch.exp(t["A_log"])[None, :] * softplus(a))
        gate = silu(h @ t["g"].T)
    o, state["S"] = delta_rule(q, k, v, beta, g, state.get("S"))
    o = rms_norm(o, t["norm"], eps) * gate.reshape(T, H, dv)
    return o.reshape(T, H * dv) @ t["o"].T, state


# ---------------------------------------------------------------- attention with a window and a sink
def rotate_pairs(x, positions, base, dims):
    """x [T, heads, D]: (x[2i], x[2i + 1]), i < dims / 2, turned by positions * base^(-2i / dims); the rest pass."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=F64)
    ang = positions.to(F64)[:, None] * base ** (-2.0 * i / dims)[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    u, w = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - w * s
    out[..., 1:dims:2] = w * c + u * s
    return out


def sink_softmax(s, visible):
    """p_j = exp(s_j) / (1 + sum over visible j' of exp(s_j')): a sink of score 0 without a value."""
    s = s.masked_fill(~visible, -math.inf)
    mx = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)
    e = torch.exp(s - mx)
    return e / (torch.exp(-mx) + e.sum(-1, keepdim=True))


def window_attention(h, t: Dict[str, torch.Tensor], m: dict, eps, keys=None, start=0):
    """Grouped-query attention with biases, partial rotation, weightless RMS norm of q and k behind the rotation,
    a sliding window and a sink.  ``keys``: (k, v) of the tokens before ``start`` (carried).  Returns (y, keys)."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(start, start + T)
    q = (h @ t["q"].T + t["q.b"]).reshape(T, H, D)
    k = (h @ t["k"].T + t["k.b"]).reshape(T, G, D)
    v = (h @ t["v"].T + t["v.b"]).reshape(T, G, V)
    q = rms_norm(rotate_pairs(q, pos, m["rot"]["base"], m["rot"]["dims"]), None, eps)
    k = rms_norm(rotate_pairs(k, pos, m["rot"]["base"], m["rot"]["dims"]), None, eps)
    if keys is not None:
        k, v = torch.cat([keys[0], k], 0), torch.cat([keys[1], v], 0)
    rep = H // G
    kk, vv = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * m["scale"]
    i = pos[:, None]
    j = torch.arange(k.shape[0])[None, :]
    visible = (i - j >= 0) & (i - j < m["mask"]["size"])
    p = sink_softmax(s, visible[None])
    o = torch.einsum("hij,jhv->ihv", p, vv).reshape(T, H * V)
    return o @ t["o"].T + t["o.b"], (k, v)


# ---------------------------------------------------------------- feed-forward
def expert(h, t, name):
    return (silu(h @ t[name + ".gate"].T) * (h @ t[name + ".up"].T)) @ t[name + ".down"].T


def table_moe(h, tokens, t: Dict[str, torch.Tensor], f: dict):
    """Each token id names its experts in a table; each counts 1 / top; a shared expert is added."""
    top = f["router"]["top"]
    table = t["table"]
    out = torch.zeros_like(h)
    for i, tok in enumerate(tokens):
        for e in table[tok].tolist():
            out[i] += expert(h[i:i + 1], t, f"e{e}")[0] / top
    if f.get("shared"):
        out = out + expert(h, t, "shared")
    return out


# ---------------------------------------------------------------- the model
def sub(W, prefix):
    return {k[len(prefix):]: v for k, v in W.items() if k.startswith(prefix)}


def as64(W):
    return {k: (v.to(F64) if v.is_floating_point() else v) for k, v in W.items()}


def mixer(kind, h, t, m, eps, state, start):
    state = dict(state or {})
    if kind == "channel_delta":
        y, state["delta"] = gated_delta(h, t, m, eps, True, state.get("delta"))
        return y, state
    if kind == "parallel":
        left, state["keys"] = window_attention(h, sub(t, "left."), m["left"], eps, state.get("keys"), start)
        right, state["delta"] = gated_delta(h, sub(t, "right."), m["right"], eps, False, state.get("delta"))
        return 0.5 * (rms_norm(left, t["left.out"], eps) + rms_norm(right, t["right.out"], eps)), state
    raise ValueError(kind)


def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int], state: Optional[list] = None, start: int = 0,
            layers_out: Optional[list] = None):
    """Logits [T, vocab] of ``tokens`` at positions start.. (64-bit) and the state to go on from."""
    W = as64(W)
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens)]
    state = list(state) if state is not None else [None] * len(cfg["layers"])
    for i, l in enumerate(cfg["layers"]):
        t = sub(W, f"l{i}.")
        a, state[i] = mixer(l["type"], x, sub(t, "mix."), l["mixer"], eps, state[i], start)
        x = x + rms_norm(a, t["norm1"], eps)
        if l.get("mlp"):
            x = x + rms_norm(table_moe(x, tokens, sub(t, "mlp."), l["mlp"]), t["norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, W["final.norm"], eps) @ W["head"].T, state


def logits(cfg, W, tokens):
    return forward(cfg, W, tokens)[0]
