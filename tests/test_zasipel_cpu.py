"""Zasipel on the CPU: the configuration reader and its refusals, the tensors the model declares, and the plain
implementation held to itself (a sequence walked in pieces against the same sequence whole; the window's and the
sink's meaning; the convolution's history)."""
import copy
import random

import pytest
import torch

import plain_zasipel as P
import zasipel_cases as C
from dinfer_b200.config.model_config import ConfigError, ZasipelConfig
from dinfer_b200.config.registry import resolve_architecture
from dinfer_b200.weights.random_init import model_declarations, random_tensor


@pytest.mark.parametrize("name", sorted(C.CONFIGS))
def test_config_round_trip_and_spec(name):
    cfg = C.CONFIGS[name]
    arch = resolve_architecture(cfg)
    typed = arch.parse_config(cfg)
    assert isinstance(typed, ZasipelConfig) and ZasipelConfig.from_dict(typed.to_dict()) == typed
    spec = arch.build_spec(typed)
    assert len(spec.layers) == len(cfg["layers"]) and spec.hidden_size == cfg["width"]
    for l, ls in zip(cfg["layers"], spec.layers):
        assert ls.block == "postnorm_residual"
        assert ls.mixer.kind == ("parallel_mixers" if l["type"] == "parallel" else "gated_delta")
        assert ls.feed_forward.kind == ("moe" if l["mlp"] else "none")


def test_declared_tensors():
    d = {t.name: t for t in model_declarations(C.ZASIPEL_A)}
    assert d["l0.mix.a1"].shape == (8, 64) and d["l0.mix.a2"].shape == (4 * 16, 8) and d["l0.mix.dt_bias"].shape == (64,)
    assert d["l0.mix.g2"].shape == (4 * 24, 12) and d["l0.mix.v.conv"].shape == (96, 3) and d["l0.mix.q"].shape == (32, 64)
    assert d["l1.mix.left.v"].shape == (64, 64) and d["l1.mix.left.q.b"].shape == (128,) and d["l1.mix.left.o.b"].shape == (64,)
    assert d["l1.mix.right.a"].shape == (2, 64) and d["l1.mix.right.dt_bias"].shape == (2,) and d["l1.mix.right.g"].shape == (32, 64)
    assert d["l1.mix.left.out"].shape == (64,) and d["l1.mlp.table"].shape == (300, 3) and d["l1.mlp.table"].kind == "int"
    assert "l1.mlp.shared.up" not in d and "l2.norm2" not in d and "l2.mlp.table" not in d and "l0.mlp.shared.gate" in d
    table = random_tensor(d["l1.mlp.table"], 3, 0.1, 0.0, torch.float32)
    assert table.dtype == torch.int32 and int(table.min()) >= 0 and int(table.max()) < 6
    assert all(len(set(row)) == 3 for row in table.tolist())
    # without the optional ranks the file decides the thin middles
    bare = copy.deepcopy(C.ZASIPEL_D)
    for l in bare["layers"]:
        del l["mixer"]["decay_rank"], l["mixer"]["gate_rank"]
    spec = resolve_architecture(bare).build_spec(ZasipelConfig.from_dict(bare))
    assert spec.layers[0].mixer.params["decay_rank"] == -1


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][0].update(type="attention"), "unknown type"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(heads=5), "multiple of kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=34), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["left"]["mask"].update(size=0), "must be positive"),
    (lambda c: c["layers"][0]["mixer"].update(conv=0), "must be positive"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "router.top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense", ff=8), "mixture of experts"),
    (lambda c: c["norm"].update(eps=0), "norm.eps"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][1]["mixer"].pop("right"), "right"),
])
def test_config_refusals(change, text):
    cfg = copy.deepcopy(C.ZASIPEL_A)
    change(cfg)
    with pytest.raises(ConfigError, match=text):
        ZasipelConfig.from_dict(cfg)


def _weights(cfg, seed=1):
    W = {}
    for d in model_declarations(cfg):
        t = random_tensor(d, seed, 0.3, 0.3, torch.float32)
        W[d.name] = t if d.kind == "int" else t.to(torch.float64)
    return W


@pytest.mark.parametrize("name", ["A", "C"])
def test_plain_in_pieces_equals_whole(name):
    """The plain implementation carries its state: pieces of 1, 2, 5 tokens give the logits of the whole."""
    cfg = C.CONFIGS[name]
    W = _weights(cfg)
    rng = random.Random(3)
    toks = [rng.randrange(cfg["vocab"]) for _ in range(41)]
    whole = P.logits(cfg, W, toks)
    state, at, rows = None, 0, []
    for n in [1, 2, 5, 1, 1, 13, 2, 16]:
        lg, state = P.forward(cfg, W, toks[at:at + n], state, start=at)
        rows.append(lg)
        at += n
    assert at == len(toks)
    assert torch.allclose(torch.cat(rows), whole, rtol=1e-9, atol=1e-9)


def test_plain_window_sink_and_history():
    m = C.left(2, 1, 8, 4, 3, 4)
    t = {k: torch.randn(s, dtype=torch.float64) for k, s in
         {"q": (16, 12), "q.b": (16,), "k": (8, 12), "k.b": (8,), "v": (4, 12), "v.b": (4,), "o": (12, 8), "o.b": (12,)}.items()}
    h = torch.randn(9, 12, dtype=torch.float64)
    y, _ = P.window_attention(h, t, m, 1e-6)
    h2 = h.clone()
    h2[2] += 5.0                                            # token 2 is outside the window of token 5 (sees 3, 4, 5) ...
    y2, _ = P.window_attention(h2, t, m, 1e-6)
    assert torch.equal(y[5:], y2[5:]) and not torch.allclose(y[4], y2[4])      # ... and inside that of token 4
    # the sink: weights sum to less than one, and to one half for a single key of score 0
    p = P.sink_softmax(torch.zeros(1, 1, 1, dtype=torch.float64), torch.ones(1, 1, 1, dtype=torch.bool))
    assert float(p) == 0.5
    # convolution: the last column weighs the current token, the history stands for the tokens before
    x = torch.randn(6, 3, dtype=torch.float64)
    w = torch.randn(3, 4, dtype=torch.float64)
    y, hist = P.short_conv(x, w)
    assert torch.allclose(y[0], x[0] * w[:, 3]) and torch.allclose(y[2], x[2] * w[:, 3] + x[1] * w[:, 2] + x[0] * w[:, 1])
    ya, ha = P.short_conv(x[:2], w)
    yb, hb = P.short_conv(x[2:], w, ha)
    assert torch.allclose(torch.cat([ya, yb]), y) and torch.equal(hb, hist) and torch.equal(hist, x[3:])


def test_random_model_folder(tmp_path):
    """The random-weights mode writes a folder the engine's own reader takes: every declared tensor, the experts'
    tables as int32 with rows of different entries."""
    from dinfer_b200.weights.loader import SafetensorsSource, verify
    from dinfer_b200.weights.random_init import write_random_model
    d = write_random_model(str(tmp_path / "m"), C.ZASIPEL_C, seed=3)
    src = SafetensorsSource(d)
    try:
        assert verify(src, model_declarations(C.ZASIPEL_C)) == []
        table = src.get("l1.mlp.table")
        assert table.dtype == torch.int32 and tuple(table.shape) == (331, 1) and int(table.max()) < 7
        assert src.dtype("l0.mix.right.q") == torch.bfloat16
    finally:
        src.close()
    # a file whose thin middles disagree with one another is refused when the part binds them
    from dinfer_b200.parts.base import BuildEnv
    from dinfer_b200.parts.delta_rule import GatedDelta
    part = GatedDelta({"num_heads": 2, "num_kv_heads": 1, "key_dim": 4, "value_dim": 4, "conv": 2, "eps": 1e-5,
                       "decay": "channel", "gate": "sigmoid", "decay_rank": -1, "gate_rank": -1},
                      BuildEnv(torch.device("cpu"), torch.float32, 8, 16), "")
    W = {t.name: torch.zeros([3 if n < 0 else n for n in t.shape]) for t in part.declare()}
    W["a2"] = torch.zeros(8, 5)
    with pytest.raises(ValueError, match="thin middle"):
        part.bind(W)
