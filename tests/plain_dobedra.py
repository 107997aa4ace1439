"""A plain, slow implementation of the Dobedra design in torch on the CPU: the oracle of the tests.

One function per mechanism, written from the design's equations in 64-bit (or any dtype handed in),
whole sequences at a time, no cache and no batching.  It shares no code with the package.

Notation: ``h`` a layer's normed input [T, width]; ``W x`` is ``x @ W.T`` for a weight stored [out, in].
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_pairs(v, positions, base, dims):
    """v [T, ..., D]: elements (2i, 2i + 1), i < dims / 2, turn by the angle p * base^(-2i / dims); the rest pass."""
    out = v.clone()
    T = v.shape[0]
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    a = positions.to(torch.float64)[:, None] * f[None, :]                 # [T, dims/2]
    shape = [T] + [1] * (v.dim() - 2) + [dims // 2]
    c, s = a.cos().reshape(shape).to(v.dtype), a.sin().reshape(shape).to(v.dtype)
    u, w = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - w * s
    out[..., 1:dims:2] = w * c + u * s
    return out


def latent_kv(h, positions, W_dkv, w_norm, kv_rank, rot, eps):
    """What a layer with a down projection of its own leaves for the keys: the normed latent [T, kv_rank] and the
    rotated shared key part [T, rot_dim]."""
    d = h @ W_dkv.T
    c = rms_norm(d[:, :kv_rank], w_norm, eps)
    kr = rotate_pairs(d[:, kv_rank:], positions, rot["base"], rot["dims"])
    return c, kr


def latent_attention(h, positions, c, kr, t: Dict[str, torch.Tensor], m: dict, eps):
    """h [T, width] of one sequence from position 0; c, kr: the latents and rotated key parts of the same tokens."""
    T = h.shape[0]
    H, D, P, V = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    cq = rms_norm(h @ t["dq"].T, t["dq.norm"], eps)
    q = (cq @ t["uq"].T).reshape(T, H, D + P)
    qn, qr = q[..., :D], rotate_pairs(q[..., D:], positions, m["rot"]["base"], m["rot"]["dims"])
    kn = (c @ t["uk"].T).reshape(T, H, D)
    v = (c @ t["uv"].T).reshape(T, H, V)
    s = (torch.einsum("thd,jhd->htj", qn, kn) + torch.einsum("thp,jp->htj", qr, kr)) * m["scale"]
    mask = positions[None, :, None] >= positions[None, None, :]
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("htj,jhv->thv", p, v).reshape(T, H * V)
    return o @ t["o"].T


def dense_ff(h, t):
    return (gelu_tanh(h @ t["gate"].T) * (h @ t["up"].T)) @ t["down"].T


def relu2_expert(h, up, down):
    return (torch.relu(h @ up.T) ** 2) @ down.T


def router_margin(z, top):
    """How far the router's choice is from going the other way: the gap between the ``top``-th and the next logit
    (infinite when every expert is chosen)."""
    if top >= z.shape[-1]:
        return torch.full(z.shape[:-1], float("inf"), dtype=z.dtype)
    v = torch.sort(z, dim=-1, descending=True).values
    return v[..., top - 1] - v[..., top]


def moe_ff(h, t, mlp: dict, margins=None):
    """``margins`` (a list) receives each token's ``router_margin``."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ t["router"].T
    if margins is not None:
        margins.append(router_margin(z, top))
    s = torch.softmax(z, dim=-1)
    w, idx = torch.topk(s, top, dim=-1)
    out = torch.zeros_like(h)
    for e in range(E):
        chose = (idx == e)                                               # [T, top]
        rows = chose.any(-1).nonzero().flatten()
        if rows.numel():
            weight = (w * chose)[rows].sum(-1, keepdim=True)
            out[rows] += weight * relu2_expert(h[rows], t[f"e{e}.up"], t[f"e{e}.down"])
    if mlp.get("shared"):
        g = torch.sigmoid(h @ t["shared.sg"].T)                            # [T, 1]
        out = out + g * relu2_expert(h, t["shared.up"], t["shared.down"])
    return out


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config: dict, tensors: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64, streams=None,
            margins=None):
    """Logits [T, vocab] of one sequence; ``streams`` (a list) receives the residual after every layer, ``margins``
    (a list) the router margins [T] of every routed layer."""
    W = {k: v.to(dtype) for k, v in tensors.items()}
    eps = config["norm"]["eps"]
    pos = torch.arange(len(tokens))
    x = W["embed"][torch.tensor(tokens)]
    kept = {}
    for i, layer in enumerate(config["layers"]):
        pre = f"l{i}."
        m = layer["mixer"]
        if layer["type"] != "latent_attention":
            raise ValueError(layer["type"])
        h1 = layer_norm(x, W[pre + "norm1"], W[pre + "norm1.b"], eps)
        mix = sub(W, pre + "mix.")
        if "kv_from" in m and m["kv_from"] is not None:
            c, kr = kept[m["kv_from"]]
        else:
            c, kr = kept[i] = latent_kv(h1, pos, mix["dkv"], mix["dkv.norm"], m["kv_rank"], m["rot"], eps)
        y = latent_attention(h1, pos, c, kr, mix, m, eps) * W[pre + "ls1"]
        if layer.get("mlp"):
            f = sub(W, pre + "mlp.")
            h2 = layer_norm(x, W[pre + "norm2"], W[pre + "norm2.b"], eps)
            ff = dense_ff(h2, f) if layer["mlp"]["kind"] == "dense" else moe_ff(h2, f, layer["mlp"], margins)
            y = y + ff * W[pre + "ls2"]
        x = x + y
        if streams is not None:
            streams.append(x.clone())
    f = layer_norm(x, W["final.norm"], W["final.norm.b"], eps)
    logits = f @ W["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits
