"""Tiny Zasipel configurations for the tests.  They differ from one another in every size and option and use values
that are easy to confuse when they happen to be equal or 1: key size against value size, heads against key heads,
one expert per token, a window shorter than a page, a rotation over the whole head, a convolution of one tap
(no history), thin middles of odd rank, a model without any attention layer."""
from __future__ import annotations

import json
import os
from typing import Dict

import torch


def left(heads, kv_heads, dim, vdim, window, rot_dims, base=10000.0, scale=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window},
            "rot": {"base": base, "dims": rot_dims}, "scale": scale if scale is not None else dim ** -0.5}


def delta(heads, kv_heads, dim, vdim, conv, decay_rank=None, gate_rank=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}
    if decay_rank:
        m.update(decay_rank=decay_rank, gate_rank=gate_rank)
    return m


def moe(experts, top, ff, shared=0):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def parallel(l, r, mlp):
    return {"type": "parallel", "mixer": {"left": l, "right": r}, "mlp": mlp}


def channel(m, mlp):
    return {"type": "channel_delta", "mixer": m, "mlp": mlp}


# a recurrent layer first; fewer key heads than value heads in both forms; a rotation over the whole head; one expert
# per token; a layer without feed-forward; no shared expert in one layer
ZASIPEL_A = {"architecture": "Zasipel", "vocab": 300, "width": 64, "norm": {"eps": 1e-5},
             "layers": [channel(delta(4, 2, 16, 24, 3, 8, 12), moe(5, 1, 24, shared=40)),
                        parallel(left(4, 2, 32, 32, 20, 32, base=500.0, scale=0.2), delta(2, 1, 64, 16, 4), moe(6, 3, 16)),
                        parallel(left(2, 2, 16, 8, 9, 6), delta(4, 4, 8, 8, 2), None),
                        channel(delta(2, 2, 32, 16, 4, 4, 4), moe(3, 3, 8, shared=8))]}
# a window shorter than a page; one key head for six query heads; a state of 128 key channels; values no tile divides
ZASIPEL_B = {"architecture": "Zasipel", "vocab": 515, "width": 128, "norm": {"eps": 3e-6},
             "layers": [parallel(left(6, 1, 48, 16, 7, 8, base=1e6, scale=0.11), delta(3, 3, 128, 40, 2), moe(4, 2, 48, shared=24)),
                        channel(delta(2, 2, 24, 128, 5, 16, 8), moe(7, 2, 40, shared=56)),
                        parallel(left(2, 1, 64, 128, 50, 16, base=77.0), delta(6, 2, 16, 48, 3), moe(2, 1, 64))]}
# sizes no vector load or tensor-core tile divides; a convolution of one tap; thin middles of odd rank
ZASIPEL_C = {"architecture": "Zasipel", "vocab": 331, "width": 72, "norm": {"eps": 1e-6},
             "layers": [parallel(left(3, 3, 10, 6, 33, 4, base=100.0), delta(1, 1, 12, 20, 1), moe(4, 2, 28, shared=12)),
                        channel(delta(3, 1, 20, 12, 4, 5, 7), moe(7, 1, 20)),
                        parallel(left(9, 3, 6, 14, 1, 2, base=50.0), delta(3, 3, 20, 4, 6), None)]}
# no attention layer at all (the engine then has no paged cache), a width of 100
ZASIPEL_D = {"architecture": "Zasipel", "vocab": 257, "width": 100, "norm": {"eps": 2e-6},
             "layers": [channel(delta(5, 5, 12, 12, 4, 9, 9), moe(5, 2, 36, shared=20)),
                        channel(delta(2, 1, 40, 36, 3, 8, 24), None)]}
# head sizes the tensor-core attention kernels take (64 in groups of two, keys and values alike)
ZASIPEL_E = {"architecture": "Zasipel", "vocab": 400, "width": 256, "norm": {"eps": 1e-5},
             "layers": [parallel(left(4, 2, 64, 64, 40, 32, base=5000.0, scale=0.3), delta(4, 2, 64, 64, 4), moe(8, 2, 64, shared=128)),
                        parallel(left(8, 2, 128, 128, 100, 64, base=5000.0, scale=0.2), delta(2, 2, 128, 128, 4), moe(4, 2, 128))]}
CONFIGS = {"A": ZASIPEL_A, "B": ZASIPEL_B, "C": ZASIPEL_C, "D": ZASIPEL_D, "E": ZASIPEL_E}


def write_model(path: str, cfg: dict, seed: int, dtype: torch.dtype, sharp: float = 5.0, std: float = 0.08) -> str:
    """Random weights shaped so that faults show: attention queries scaled by ``sharp`` (a token's attention then
    rests on few keys, often old ones: a key lost or one too many moves the logits); decay biases drawn around -3 so
    that many heads and channels forget slowly and the state carries far tokens; convolution taps large enough that
    every tap matters; biases large enough to matter."""
    from dinfer_b200.weights.random_init import model_declarations, random_tensor
    from dinfer_b200.weights.safetensors_io import write_safetensors
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    tensors = []
    for d in model_declarations(cfg):
        if d.kind == "int":
            tensors.append((d.name, random_tensor(d, seed, std, 0.3, torch.float32)))
            continue
        t = random_tensor(d, seed, std, 0.3, torch.float32)
        if d.name.endswith("left.q"):
            t = t * sharp
        elif d.name.endswith(".conv"):
            t = t * 6.0
        elif d.name.endswith("dt_bias"):
            t = t * 12.0 - 3.0
        elif d.name.endswith("A_log"):
            t = t * 6.0
        elif d.name.endswith(".b") and len(d.shape) == 1:
            t = t * 3.0
        tensors.append((d.name, t.to(torch.bfloat16).to(dtype)))     # the same values in every dtype
    write_safetensors(os.path.join(path, "model.safetensors"), tensors, metadata={"format": "pt"})
    return path


def load_weights(model_dir: str) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file
    return load_file(os.path.join(model_dir, "model.safetensors"))
