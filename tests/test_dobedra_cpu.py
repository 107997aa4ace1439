"""Dobedra without a device: the configuration's reader, the list of parts it becomes, the tensors it declares,
and the plain implementation's own consistency (the absorbed form of latent attention against the expanded one)."""
import copy
import json

import pytest
import torch

import dobedra_cases as C
import plain_dobedra as P
from dinfer_b200.config.model_config import ConfigError, DobedraConfig
from dinfer_b200.config.registry import resolve_architecture
from dinfer_b200.weights.random_init import model_declarations


def test_config_reads_every_size_and_round_trips():
    for cfg in C.CONFIGS.values():
        c = DobedraConfig.from_dict(cfg)
        assert c.vocab == cfg["vocab"] and c.width == cfg["width"] and c.norm_eps == cfg["norm"]["eps"]
        assert len(c.layers) == len(cfg["layers"])
        for l, raw in zip(c.layers, cfg["layers"]):
            m = raw["mixer"]
            assert (l.mixer.heads, l.mixer.dim, l.mixer.rot_dim, l.mixer.vdim, l.mixer.kv_rank, l.mixer.q_rank) == \
                (m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"])
            assert l.mixer.scale == m["scale"] and l.mixer.rot_base == m["rot"]["base"] and l.mixer.kv_from == m.get("kv_from")
            assert (l.mlp is None) == (raw["mlp"] is None)
        again = DobedraConfig.from_dict(json.loads(json.dumps(c.to_dict())))
        assert again == c


@pytest.mark.parametrize("edit, text", [
    (lambda d: d["layers"][1]["mixer"].__setitem__("kv_from", 1), "kv_from"),
    (lambda d: d["layers"][1]["mixer"].__setitem__("kv_rank", 16), "kv_rank"),
    (lambda d: d["layers"][0]["mlp"]["router"].__setitem__("top", 9), "top"),
    (lambda d: d["layers"][0].__setitem__("type", "convolution"), "type"),
    (lambda d: d["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "rot.dims"),
    (lambda d: d.pop("norm"), "norm"),
    (lambda d: d["layers"][1]["mlp"].__setitem__("kind", "sparse"), "kind"),
])
def test_config_refusals(edit, text):
    d = copy.deepcopy(C.DOBEDRA_A)
    edit(d)
    with pytest.raises(ConfigError) as e:
        DobedraConfig.from_dict(d)
    assert text in str(e.value)


def test_registry_finds_the_design_by_either_key():
    assert resolve_architecture(C.DOBEDRA_A).name == "Dobedra"
    d = dict(C.DOBEDRA_A)
    d["architectures"] = [d.pop("architecture")]
    assert resolve_architecture(d).name == "Dobedra"


def test_spec_and_declared_tensors():
    arch = resolve_architecture(C.DOBEDRA_A)
    spec = arch.build_spec(arch.parse_config(C.DOBEDRA_A))
    assert [e.cache_from for e in spec.schedule] == [None, 0, None, 0]
    assert spec.logit_softcap == 8.0 and [l.block for l in spec.layers] == ["parallel_residual"] * 4
    names = {d.name: tuple(d.shape) for d in model_declarations(C.DOBEDRA_A)}
    assert names["l0.mix.dkv"] == (48, 64) and "l1.mix.dkv" not in names and "l3.mix.dkv.norm" not in names
    assert names["l0.mix.uq"] == (3 * 32, 40) and names["l2.mix.uv"] == (2 * 16, 48) and names["l2.mix.o"] == (64, 32)
    assert names["l0.mlp.e4.up"] == (24, 64) and "l0.mlp.e5.up" not in names and names["l0.mlp.shared.sg"] == (1, 64)
    assert "l3.mlp.shared.up" not in names and names["l3.mlp.router"] == (8, 64)
    assert names["l1.mlp.gate"] == (96, 64) and not any(n.startswith("l2.mlp") for n in names)
    assert "l2.norm2" not in names and "l2.ls2" not in names            # optional, not made for a layer without one
    assert names["final.norm.b"] == (64,) and names["head"] == (300, 64)


def test_plain_absorbed_form_equals_the_expanded_one():
    """The identity the engine's attention rests on, held on the plain side: scores against the latent with
    W_uk folded into the query, values as W_uv of the summed latents."""
    torch.manual_seed(0)
    m = C.MB
    H, D, Pd, V, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T, h = 9, 32
    t = {"dq": torch.randn(m["q_rank"], h), "dq.norm": torch.rand(m["q_rank"]) + 0.5, "uq": torch.randn(H * (D + Pd), m["q_rank"]),
         "uk": torch.randn(H * D, R), "uv": torch.randn(H * V, R), "o": torch.randn(h, H * V)}
    t = {k: v.double() for k, v in t.items()}
    x = torch.randn(T, h).double()
    pos = torch.arange(T)
    c, kr = P.latent_kv(x, pos, torch.randn(R + Pd, h).double(), torch.ones(R).double(), R, m["rot"], 1e-6)
    want = P.latent_attention(x, pos, c, kr, t, m, 1e-6)
    cq = P.rms_norm(x @ t["dq"].T, t["dq.norm"], 1e-6)
    q = (cq @ t["uq"].T).reshape(T, H, D + Pd)
    q_lat = torch.einsum("thd,hdr->thr", q[..., :D], t["uk"].reshape(H, D, R))
    qr = P.rotate_pairs(q[..., D:], pos, m["rot"]["base"], m["rot"]["dims"])
    s = (torch.einsum("thr,jr->htj", q_lat, c) + torch.einsum("thp,jp->htj", qr, kr)) * m["scale"]
    s = s.masked_fill(pos[None, :, None] < pos[None, None, :], float("-inf"))
    o_lat = torch.einsum("htj,jr->thr", torch.softmax(s, -1), c)
    got = torch.einsum("thr,hvr->thv", o_lat, t["uv"].reshape(H, V, R)).reshape(T, H * V) @ t["o"].T
    assert torch.allclose(got, want, rtol=1e-10, atol=1e-10)


def test_plain_model_runs_every_branch(tmp_path):
    for name, cfg in C.CONFIGS.items():
        d = C.write_model(str(tmp_path / name), cfg, 3, torch.float32)
        W = C.load_weights(d)
        streams = []
        lg = P.forward(cfg, W, list(range(1, 12)), streams=streams)
        assert lg.shape == (11, cfg["vocab"]) and torch.isfinite(lg).all() and len(streams) == len(cfg["layers"])
        assert float(lg.abs().max()) <= cfg["logit_softcap"]
        # causal: a later token changes no earlier row
        lg2 = P.forward(cfg, W, list(range(1, 11)) + [0])
        assert torch.allclose(lg[:10], lg2[:10], rtol=0, atol=1e-12) and not torch.allclose(lg[10], lg2[10], atol=1e-6)
