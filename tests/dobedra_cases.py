"""Tiny Dobedra configurations for the tests: they differ from one another in every size and option, and use
values that are easy to confuse when they happen to be equal (head size against value size against latent size,
one expert per token, one head, a rotation over fewer elements than the rotated part holds)."""
from __future__ import annotations

import json
import os
from typing import Dict

import torch


def mixer(heads, dim, rot_dim, vdim, kv_rank, q_rank, base=10000.0, rot_dims=None, kv_from=None, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "rot": {"base": base, "dims": rot_dims or rot_dim},
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=0):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(m, mlp):
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


# sizes the tensor-core paths take (multiples of 16); experts not a power of two, one expert per token in one
# layer; a layer without feed-forward; the dense layer not first; latents shared with a layer that is not the neighbour
MA = mixer(3, 16, 16, 32, 32, 40, base=500.0)
DOBEDRA_A = {"architecture": "Dobedra", "vocab": 300, "width": 64, "norm": {"eps": 1e-5}, "logit_softcap": 8.0,
             "layers": [layer(MA, moe(5, 1, 24, shared=40)),
                        layer(dict(MA, kv_from=0), dense(96)),
                        layer(mixer(2, 32, 16, 16, 48, 24, base=77.0), None),
                        layer(dict(MA, kv_from=0), moe(8, 3, 16))]}
# one head; value size, head size and latent size all different; a wider model; eps and cap different
MB = mixer(5, 48, 32, 16, 64, 56, base=1e6, scale=0.07)
DOBEDRA_B = {"architecture": "Dobedra", "vocab": 515, "width": 128, "norm": {"eps": 3e-6}, "logit_softcap": 30.0,
             "layers": [layer(mixer(1, 64, 16, 80, 32, 16, base=3000.0), dense(160)),
                        layer(MB, moe(6, 2, 48, shared=24)),
                        layer(dict(MB, kv_from=1), moe(3, 3, 40, shared=56))]}
# sizes no vector load or tensor-core tile divides; a rotation over fewer elements than the rotated part holds
MC = mixer(2, 12, 6, 20, 24, 20, base=100.0, rot_dims=4)
DOBEDRA_C = {"architecture": "Dobedra", "vocab": 331, "width": 72, "norm": {"eps": 1e-6}, "logit_softcap": 12.0,
             "layers": [layer(MC, moe(4, 2, 28, shared=12)), layer(dict(MC, kv_from=0), dense(100)),
                        layer(mixer(3, 10, 2, 6, 14, 10, base=50.0), moe(7, 1, 20))]}
# a width no 16-byte load or tensor-core tile divides (every product and the grouped products take their plain paths in
# bfloat16 too), many heads over a small latent
MD = mixer(9, 20, 12, 28, 36, 44, base=2000.0)
DOBEDRA_D = {"architecture": "Dobedra", "vocab": 257, "width": 100, "norm": {"eps": 2e-6}, "logit_softcap": 20.0,
             "layers": [layer(MD, dense(52)), layer(dict(MD, kv_from=0), moe(5, 2, 36, shared=20))]}
CONFIGS = {"A": DOBEDRA_A, "B": DOBEDRA_B, "C": DOBEDRA_C, "D": DOBEDRA_D}


def write_model(path: str, cfg: dict, seed: int, dtype: torch.dtype, sharp: float = 6.0, std: float = 0.08) -> str:
    """Random weights with the query up-projections scaled by ``sharp``, so that the attention of a token rests on
    few keys (often far ones) instead of averaging hundreds: a key that is lost or one too many then moves the
    logits.  Biases and layer scales vary around their neutral values."""
    from dinfer_b200.weights.random_init import model_declarations, random_tensor
    from dinfer_b200.weights.safetensors_io import write_safetensors
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    tensors = []
    for d in model_declarations(cfg):
        t = random_tensor(d, seed, std, 0.3, torch.float32)
        if d.name.endswith("mix.uq"):
            t = t * sharp
        if d.name.endswith(".b"):
            t = t * 2.0
        if d.name.endswith("router"):
            t = t * 4.0                                  # spread the experts' scores
        tensors.append((d.name, t.to(torch.bfloat16).to(dtype)))     # the same values in every dtype
    write_safetensors(os.path.join(path, "model.safetensors"), tensors, metadata={"format": "pt"})
    return path


def load_weights(model_dir: str) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file
    return load_file(os.path.join(model_dir, "model.safetensors"))


def decided_tokens(cfg: dict, W: Dict[str, torch.Tensor], n: int, rng, margin: float = 0.15):
    """``n`` random tokens none of which leaves a router undecided: wherever the gap between the last chosen and the
    first rejected expert's logit is below ``margin`` (reduced precision could then choose differently, which is a
    property of the weights, not a fault), the tokens from there on are drawn again.  Earlier positions do not
    depend on later tokens, so the sequence settles from the front."""
    import plain_dobedra as P
    toks = [rng.randrange(cfg["vocab"]) for _ in range(n)]
    for _ in range(40 * n):
        m = []
        P.forward(cfg, W, toks, margins=m)
        if not m:
            return toks
        low = (torch.stack(m).min(0).values < margin).nonzero().flatten()
        if not low.numel():
            return toks
        p = int(low[0])
        toks[p:] = [rng.randrange(cfg["vocab"]) for _ in range(n - p)]
    raise RuntimeError("no decided sequence found")
