"""Dobedra as a list of parts.

Every layer is parallel: ``x += ls1 * mixer(LN1(x)) + ls2 * ff(LN2(x))`` with two layer norms (weight and bias)
of the same ``x`` and a per-channel layer scale on each branch.  The mixer is attention over a cached latent
(``latent_attention``); a layer may read the latents of an earlier layer (``kv_from``) instead of keeping its
own.  The feed-forward is a gated dense one (tanh-gelu gate) or a mixture of relu-squared experts with a softmax
router (weights not renormalised) and a sigmoid-gated shared expert, or absent.  Layer norm, head, soft-capped
logits.  Tensor names: ``embed``, ``l<i>.norm1[.b]``, ``l<i>.norm2[.b]``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``l<i>.ls1``, ``l<i>.ls2``, ``final.norm[.b]``, ``head``.
"""
from __future__ import annotations

from ..config.model_config import DobedraConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def dobedra_spec(cfg: DobedraConfig) -> ModelSpec:
    def layer_norm(name: str, optional: bool = False) -> PartSpec:
        return PartSpec("layernorm", {"size": cfg.width, "eps": cfg.norm_eps, "weight": name, "bias": name + ".b",
                                      "optional": optional})

    layers = []
    for i, l in enumerate(cfg.layers):
        m = l.mixer
        position = PartSpec("rope", {"head_dim": m.rot_dim, "rotary_dim": m.rot_dims, "theta": m.rot_base,
                                     "max_positions": cfg.max_positions, "style": "interleaved"})
        mixer = PartSpec("latent_attention", {
            "num_heads": m.heads, "nope_dim": m.dim, "rope_dim": m.rot_dim, "v_dim": m.vdim, "kv_rank": m.kv_rank,
            "q_rank": m.q_rank, "scale": m.scale, "eps": cfg.norm_eps, "position": position,
            "own_kv": m.kv_from is None,
            "q_down": "mix.dq", "q_norm": "mix.dq.norm", "q_up": "mix.uq", "kv_down": "mix.dkv",
            "kv_norm": "mix.dkv.norm", "k_up": "mix.uk", "v_up": "mix.uv", "o_proj": "mix.o"})
        f = l.mlp
        if f is None:
            ff = PartSpec("none")
        elif f.kind == "dense":
            ff = PartSpec("gated_mlp", {"intermediate_size": f.ff, "activation": "gelu_tanh", "gate_proj": "mlp.gate",
                                        "up_proj": "mlp.up", "down_proj": "mlp.down"})
        else:
            ff = PartSpec("moe", {"num_experts": f.experts, "top_k": f.top, "expert_size": f.ff,
                                  "shared_size": f.shared_ff, "activation": "relu2", "scoring": "softmax",
                                  "renormalize": False, "shared_gate": "sigmoid", "router": "mlp.router",
                                  "expert_up": "mlp.e{e}.up", "expert_down": "mlp.e{e}.down",
                                  "shared_up": "mlp.shared.up", "shared_down": "mlp.shared.down",
                                  "shared_gate_proj": "mlp.shared.sg"})
        layers.append(LayerSpec(
            prefix=f"l{i}.", block="parallel_residual", mixer=mixer, mixer_norm=layer_norm("norm1"),
            feed_forward=ff, feed_forward_norm=layer_norm("norm2", optional=f is None),
            extras={"mixer_scale": "ls1", "feed_forward_scale": "ls2"}))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding_tensor="embed", layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i, cache_from=l.mixer.kv_from) for i, l in enumerate(cfg.layers)),
        final_norm=PartSpec("layernorm", {"size": cfg.width, "eps": cfg.norm_eps, "weight": "final.norm",
                                          "bias": "final.norm.b"}),
        lm_head_tensor="head", tie_word_embeddings=False, eos_token_ids=cfg.eos_token_ids,
        logit_softcap=cfg.logit_softcap)


register_architecture("Dobedra", DobedraConfig.from_dict, dobedra_spec)
