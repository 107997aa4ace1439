"""The gated delta rule: a recurrent mixer.  Per head a matrix S [key channels, value channels] in 32-bit is carried
from token to token of a request:

    S <- g * S;   u = beta * (v - S^T k);   S <- S + k u^T;   o = S^T q

q, k, v come from projections followed by a short causal convolution per channel and silu; q and k are unit vectors
per head (q also times dk^-1/2); ``beta = sigmoid(W_b x)``; the decay ``g = exp(-exp(A_log) * softplus(a + dt_bias))``
is one number per head (``decay = "head"``, ``a = W_a x``) or one per head and key channel (``decay = "channel"``,
``a = W_a2 W_a1 x`` through a thin middle).  The output is ``o / rms(o) * w * act(gate)`` per head, with
``gate = W_g x`` (or ``W_g2 W_g1 x``) and act silu or sigmoid, then the output projection.

Data flow of one step (prompt portions and decoded tokens alike):
  P = x [W_q; W_k; W_v; W_b; W_a | W_a1; W_g | W_g1]^T      one stacked product
  a, gate = thin second products where the design has them
  q, k, v, beta, g = delta_prep(P, a, convolution history)    32-bit; the history then moves on
  o = delta_recurrence(q, k, v, beta, g, S)                    32-bit, S in place
  y = delta_post(o, w, gate);  out = y W_o^T
What a request keeps is one row of a fixed-size state: S of every head, then the last ``taps - 1`` inputs of the
convolutions.  Everything reads the step's slots and fresh flags from the device, so steps replay as CUDA graphs.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import delta_ops
from .base import MIXERS, BuildEnv, CacheBinding, Mixer, StateNeed, StepContext
from .linear import Linear
from .spec import TensorDecl


def _up8(n: int) -> int:
    return (n + 7) // 8 * 8


@MIXERS.register("gated_delta")
class GatedDelta(Mixer):
    """params: ``num_heads`` (value heads), ``num_kv_heads`` (query/key heads; value head h uses h // (heads / kv_heads)),
    ``key_dim``, ``value_dim``, ``conv`` (taps of the short convolutions), ``eps`` (of the output norm), ``decay``
    ("head" or "channel"), ``gate`` ("silu" or "sigmoid"), ``decay_rank`` / ``gate_rank`` (the thin middle of the
    decay's / gate's projection; 0: one matrix; -1: whatever the file holds), and the tensor names ``q_proj``,
    ``k_proj``, ``v_proj`` (their convolutions: the name + ``conv_suffix``), ``beta_proj``, ``A_log``, ``dt_bias``,
    ``norm``, ``o_proj``, ``decay_proj`` / ``gate_proj`` (with a thin middle: the names of the two matrices as a pair).
    ``out_float32``: the output projection's result stays 32-bit (for an arrangement that norms it before it joins the
    stream)."""

    graph_capturable = True

    def __init__(self, params, env: BuildEnv, prefix=""):
        super().__init__(params, env, prefix)
        p = self.params
        self.hidden = env.hidden_size
        self.H, self.G = int(p["num_heads"]), int(p["num_kv_heads"])
        self.dk, self.dv = int(p["key_dim"]), int(p["value_dim"])
        self.taps = int(p["conv"])
        self.eps = float(p["eps"])
        self.per_channel = p.get("decay", "head") == "channel"
        self.sigmoid_gate = p.get("gate", "silu") == "sigmoid"
        self.decay_rank, self.gate_rank = int(p.get("decay_rank", 0)), int(p.get("gate_rank", 0))
        self.out_float32 = bool(p.get("out_float32", False))
        if p.get("decay", "head") not in ("head", "channel") or p.get("gate", "silu") not in ("silu", "sigmoid"):
            raise ValueError("gated_delta: decay is head or channel, gate is silu or sigmoid")
        if self.H % self.G or min(self.H, self.G, self.dk, self.dv, self.taps) <= 0:
            raise ValueError(f"gated_delta: heads {self.H} / kv heads {self.G} / sizes {self.dk}, {self.dv}, taps {self.taps}")
        n = lambda key, default: prefix + p.get(key, default)
        pair = lambda key, default: tuple(prefix + x for x in p.get(key, default))
        self.names = {"q": n("q_proj", "q"), "k": n("k_proj", "k"), "v": n("v_proj", "v"), "b": n("beta_proj", "b"),
                      "A_log": n("A_log", "A_log"), "dt_bias": n("dt_bias", "dt_bias"), "norm": n("norm", "norm"),
                      "o": n("o_proj", "o")}
        self.conv_suffix = p.get("conv_suffix", ".conv")
        self.decay_names = pair("decay_proj", ("a1", "a2")) if self.decay_rank else (n("decay_proj", "a"),)
        self.gate_names = pair("gate_proj", ("g1", "g2")) if self.gate_rank else (n("gate_proj", "g"),)
        self.nq, self.nv = self.G * self.dk, self.H * self.dv
        self.nd = self.H * self.dk if self.per_channel else self.H
        self.channels = 2 * self.nq + self.nv
        self.state_size = self.H * self.dk * self.dv
        self.proj: Optional[Linear] = None

    def declare(self) -> List[TensorDecl]:
        h, t = self.hidden, self.taps
        N = self.names
        d = []
        for key, rows in (("q", self.nq), ("k", self.nq), ("v", self.nv)):
            d += [TensorDecl(N[key], (rows, h)), TensorDecl(N[key] + self.conv_suffix, (rows, t))]
        d += [TensorDecl(N["b"], (self.H, h)), TensorDecl(N["A_log"], (self.H,)), TensorDecl(N["norm"], (self.dv,), init="ones"),
              TensorDecl(N["dt_bias"], (self.nd,)), TensorDecl(N["o"], (h, self.nv))]
        for names, rank, rows in ((self.decay_names, self.decay_rank, self.nd), (self.gate_names, self.gate_rank, self.nv)):
            if rank:
                d += [TensorDecl(names[0], (rank, h)), TensorDecl(names[1], (rows, rank))]
            else:
                d.append(TensorDecl(names[0], (rows, h)))
        return d

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        N = self.names
        first = [tensors[N["q"]], tensors[N["k"]], tensors[N["v"]], tensors[N["b"]],
                 tensors[self.decay_names[0]], tensors[self.gate_names[0]]]
        for names, rank in ((self.decay_names, self.decay_rank), (self.gate_names, self.gate_rank)):
            if rank and tensors[names[0]].shape[0] != tensors[names[1]].shape[1]:
                raise ValueError(f"{names[0]} has {tensors[names[0]].shape[0]} rows, {names[1]} has "
                                 f"{tensors[names[1]].shape[1]} columns: the thin middle must agree")
        dt = torch.float32 if any(t.dtype == torch.float32 for t in first) else first[0].dtype
        # one stacked matrix; every part starts at a multiple of 8 rows (zero rows between), so that views of the
        # product's columns keep the alignment the tensor-core products want
        parts, self.col, at = [], [], 0
        for t in first:
            self.col.append(at)
            parts.append(t.to(dt))
            pad = _up8(t.shape[0]) - t.shape[0]
            if pad:
                parts.append(t.new_zeros((pad, t.shape[1]), dtype=dt))
            at += _up8(t.shape[0])
        self.width = [t.shape[0] for t in first]
        self.proj = Linear(torch.cat(parts, dim=0))
        self.decay_up = Linear(tensors[self.decay_names[1]]) if self.decay_rank else None
        self.gate_up = Linear(tensors[self.gate_names[1]]) if self.gate_rank else None
        self.o = Linear(tensors[N["o"]])
        f32 = lambda t: t.to(torch.float32).contiguous()
        self.conv_w = torch.cat([f32(tensors[N[x] + self.conv_suffix]) for x in ("q", "k", "v")], dim=0).contiguous()
        self.A_log, self.dt_bias, self.norm_w = f32(tensors[N["A_log"]]), f32(tensors[N["dt_bias"]]), f32(tensors[N["norm"]])

    def cache_need(self):
        return StateNeed((self.state_size + (self.taps - 1) * self.channels,), torch.float32)

    def kernel_libraries(self):
        libs = ["delta_rule"] + self.proj.kernel_libraries() + self.o.kernel_libraries()
        for l in (self.decay_up, self.gate_up):
            if l is not None:                               # their input is the 32-bit stacked product: the 32-bit product
                libs += l.kernel_libraries() + ["gemm_f32"]
        return libs

    def forward(self, x, ctx: StepContext, cache: CacheBinding):
        T = x.shape[0]
        # the stacked product's result stays 32-bit: what enters the recurrence is then rounded nowhere behind x itself
        # (its columns feed convolutions, unit norms and exponentials, where a bfloat16 rounding travels far)
        P = self.proj(x, out_dtype=torch.float32)
        cq, ck, cv, cb, ca, cg = self.col
        A = P[:, ca:ca + self.width[4]]
        if self.decay_up is not None:
            A = self.decay_up(A)
        gate = P[:, cg:cg + self.width[5]]
        if self.gate_up is not None:
            gate = self.gate_up(gate)
        B = ctx.cu_seqlens.numel() - 1
        slots, fresh = ctx.state_slots[:B], ctx.state_fresh[:B]
        state = cache.state
        q, k, v, beta, decay = delta_ops.prep(P, (cq, ck, cv, cb), A, self.conv_w, self.A_log, self.dt_bias, state,
                                              self.state_size, ctx.cu_seqlens, slots, fresh, self.H, self.G, self.dk,
                                              self.dv, self.taps, self.per_channel)
        o = delta_ops.recurrence(q, k, v, beta, decay, state, ctx.cu_seqlens, slots, fresh, self.per_channel)
        y = torch.empty((T, self.nv), dtype=x.dtype, device=x.device)
        delta_ops.post(o, self.norm_w, gate, self.eps, self.sigmoid_gate, y)
        return self.o(y, out_dtype=torch.float32 if self.out_float32 else None)
