"""Zasipel as a list of parts.

Every layer has its norms on the sublayers' outputs: ``x += norm1(mixer(x)); x += norm2(ff(x))`` (RMS norms with a
weight), the sublayers reading ``x`` itself.  A ``parallel`` layer's mixer is two mixers side by side whose outputs
are each RMS-normed over the width (weights ``mix.left.out`` / ``mix.right.out``) and averaged: on the left
grouped-query attention with biases, a rotation of the first ``rot.dims`` elements of a head (pairs 2i, 2i + 1), a
weightless RMS norm of q and k behind the rotation, a sliding window and a sink in the softmax; on the right a gated
delta rule with one decay a head and a silu output gate.  A ``channel_delta`` layer's mixer is the delta rule with a
decay per key channel and a sigmoid output gate, both through thin projections.  The feed-forward is a mixture of
gated silu experts chosen by a table over the token ids (each choice weighs 1 / top) plus a shared expert, or absent.
RMS norm, head.  Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.model_config import DeltaRuleSizes, WindowAttentionSizes, ZasipelConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _window_attention(a: WindowAttentionSizes, cfg: ZasipelConfig, at: str) -> PartSpec:
    position = PartSpec("rope", {"head_dim": a.dim, "rotary_dim": a.rot_dims, "theta": a.rot_base,
                                 "max_positions": cfg.max_positions, "style": "interleaved"})
    return PartSpec("gqa_attention", {
        "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim, "v_dim": a.vdim, "scale": a.scale,
        "window": a.window, "sink": True, "qk_norm": True, "qk_norm_order": "after", "qk_norm_weight": False,
        "eps": cfg.norm_eps, "bias": True, "bias_suffix": ".b", "position": position, "out_float32": True,
        "q_proj": at + "q", "k_proj": at + "k", "v_proj": at + "v", "o_proj": at + "o"})


def _delta_rule(r: DeltaRuleSizes, cfg: ZasipelConfig, at: str, channel: bool) -> PartSpec:
    p = {"num_heads": r.heads, "num_kv_heads": r.kv_heads, "key_dim": r.dim, "value_dim": r.vdim, "conv": r.conv,
         "eps": cfg.norm_eps, "out_float32": True, "q_proj": at + "q", "k_proj": at + "k", "v_proj": at + "v", "beta_proj": at + "b",
         "A_log": at + "A_log", "dt_bias": at + "dt_bias", "norm": at + "norm", "o_proj": at + "o"}
    if channel:
        p.update(decay="channel", gate="sigmoid", decay_rank=r.decay_rank, gate_rank=r.gate_rank,
                 decay_proj=(at + "a1", at + "a2"), gate_proj=(at + "g1", at + "g2"))
    else:
        p.update(decay="head", gate="silu", decay_proj=at + "a", gate_proj=at + "g")
    return PartSpec("gated_delta", p)


def zasipel_spec(cfg: ZasipelConfig) -> ModelSpec:
    def rms(name: str, optional: bool = False) -> PartSpec:
        return PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "weight": name, "optional": optional})

    layers = []
    for i, l in enumerate(cfg.layers):
        if l.type == "parallel":
            mixer = PartSpec("parallel_mixers", {
                "left": _window_attention(l.left, cfg, "mix.left."), "right": _delta_rule(l.right, cfg, "mix.right.", False),
                "left_out": "mix.left.out", "right_out": "mix.right.out", "eps": cfg.norm_eps, "coef": 0.5})
        else:
            mixer = _delta_rule(l.right, cfg, "mix.", True)
        f = l.mlp
        if f is None:
            ff = PartSpec("none")
        else:
            ff = PartSpec("moe", {"num_experts": f.experts, "top_k": f.top, "expert_size": f.ff, "shared_size": f.shared_ff,
                                  "activation": "silu", "gated": True, "routing": "table", "vocab_size": cfg.vocab,
                                  "table": "mlp.table", "expert_gate": "mlp.e{e}.gate", "expert_up": "mlp.e{e}.up",
                                  "expert_down": "mlp.e{e}.down", "shared_gate_up": "mlp.shared.gate",
                                  "shared_up": "mlp.shared.up", "shared_down": "mlp.shared.down"})
        layers.append(LayerSpec(prefix=f"l{i}.", block="postnorm_residual", mixer=mixer, mixer_norm=rms("norm1"),
                                feed_forward=ff, feed_forward_norm=rms("norm2", optional=f is None)))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding_tensor="embed", layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(cfg.layers))),
        final_norm=rms("final.norm"), lm_head_tensor="head", tie_word_embeddings=False, eos_token_ids=cfg.eos_token_ids)


register_architecture("Zasipel", ZasipelConfig.from_dict, zasipel_spec)
