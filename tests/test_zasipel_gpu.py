"""Zasipel on the device: every new kernel alone against the plain implementation's function for it, then tiny
models that differ in every size replayed whole / with a decoded tail / in portions down to two tokens / mixed on a
pool that only holds the most demanding step, the trace runner as a process, and greedy generation through ``LLM``."""
import json
import math
import os
import random

import numpy as np
import pytest
import torch

import helpers as H
import plain_zasipel as P
import zasipel_cases as C

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F64 = torch.float64


def dev(t, dtype=None):
    return t.to("cuda", dtype or t.dtype).contiguous()


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device="cuda")


# ---------------------------------------------------------------- the norm that joins a branch to the stream
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("h", [72, 256, 1000])
def test_branch_norm(dtype, h):
    from dinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(h)
    dt = DT[dtype]
    a, b = (torch.randn(5, h, generator=g).to(dt) for _ in range(2))
    wa, wb, w = (1 + 0.3 * torch.randn(h, generator=g).to(dt) for _ in range(3))
    x = torch.randn(5, h, generator=g)
    tol = dict(rtol=1e-5, atol=1e-5)
    # one branch
    res, cast = dev(x), torch.empty(5, h, dtype=dt, device="cuda")
    ops.branch_norm(dev(a), dev(w), 1e-5, residual=res, cast=cast)
    want = x.to(F64) + P.rms_norm(a.to(F64), w.to(F64), 1e-5)
    assert torch.allclose(res.cpu().to(F64), want, **tol) and torch.equal(cast, res.to(dt))
    # two branches normed, averaged, normed again
    res = dev(x)
    ops.branch_norm(dev(a), dev(w), 1e-5, residual=res, inner=(dev(wa), dev(wb)), b=dev(b), coef=0.5, inner_eps=2e-5)
    y = 0.5 * (P.rms_norm(a.to(F64), wa.to(F64), 2e-5) + P.rms_norm(b.to(F64), wb.to(F64), 2e-5))
    assert torch.allclose(res.cpu().to(F64), x.to(F64) + P.rms_norm(y, w.to(F64), 1e-5), **tol)
    # the mean alone
    out = torch.empty(5, h, dtype=torch.float32, device="cuda")
    ops.branch_norm(dev(a), None, 0.0, out32=out, inner=(dev(wa), dev(wb)), b=dev(b), coef=0.5, inner_eps=2e-5)
    assert torch.allclose(out.cpu().to(F64), y, **tol)


# ---------------------------------------------------------------- attention: rotation, norm behind it, window, sink
def attention_case(dtype, H_, G, D, Dv, window, rot, seqs, block_size, scale, sharp_at=None, seed=0):
    """Requests given as (history, new tokens): the history is written to the cache by a first step, the new tokens
    run in a second one (all requests as one batch).  Returns (engine output, plain output) of the new tokens."""
    from dinfer_b200.kernels import ops
    from dinfer_b200.parts.rope import rope_table
    g = torch.Generator().manual_seed(seed)
    dt = DT[dtype]
    width = (H_ + G) * D + G * Dv
    total = [a + b for a, b in seqs]
    table = rope_table(rot, 300.0, max(total) + 1, "cuda")
    pages = [(n + block_size - 1) // block_size for n in total]
    order = list(range(sum(pages)))
    random.Random(seed).shuffle(order)                      # pages in no particular order
    tab = torch.full((len(seqs), max(pages)), -1, dtype=torch.int32)
    at = 0
    for b, n in enumerate(pages):
        tab[b, :n] = torch.tensor(order[at:at + n])
        at += n
    Dc = max(D, Dv)
    cache = torch.full((sum(pages), 2, G, block_size, Dc), float("nan"), dtype=dt, device="cuda")
    rows = [torch.randn(n, width, generator=g).to(dt) for n in total]
    if sharp_at is not None:                                # one key made to stand out for one query: it points
        b, qi, kj = sharp_at                                # the way the query's heads do (lengths do not matter,
        for hk in range(G):                                 # q and k are normed: only the direction does)
            rows[b][kj, (H_ + hk) * D:(H_ + hk + 1) * D] = rows[b][qi, hk * (H_ // G) * D:(hk * (H_ // G) + 1) * D]
    outs, wants = [], []
    for phase in (0, 1):
        lens = [(0, a) if phase == 0 else (a, a + b) for a, b in seqs]
        live = [i for i, (lo, hi) in enumerate(lens) if hi > lo]
        if not live:
            continue
        x = torch.cat([rows[i][lens[i][0]:lens[i][1]] for i in live]).cuda()
        pos = torch.cat([torch.arange(*lens[i]) for i in live]).to(torch.int32).cuda()
        cu = i32(np.concatenate([[0], np.cumsum([lens[i][1] - lens[i][0] for i in live])]))
        slots = torch.cat([tab[i][torch.arange(*lens[i]) // block_size] * block_size + torch.arange(*lens[i]) % block_size
                           for i in live]).to(torch.int32).cuda()
        ops.qkv_post_general(x, pos, H_, G, D, Dv, 1e-5, None, None, True, False, table, cache, slots, block_size,
                             interleaved=True)
        out = torch.empty(x.shape[0], H_ * Dv, dtype=dt, device="cuda")
        ops.attention_generic(x[:, :H_ * D], out, cache, dev(tab[live]), cu, pos, H_, G, D, scale, window, v_dim=Dv, sink=True)
        if phase == 1:
            outs = out.cpu().to(F64)
    m = {"heads": H_, "kv_heads": G, "dim": D, "vdim": Dv, "scale": scale, "mask": {"size": window},
         "rot": {"base": 300.0, "dims": rot}}
    eye = {"q": torch.eye(H_ * D, width, dtype=F64), "k": torch.eye(G * D, width, dtype=F64).roll(H_ * D, 1),
           "v": torch.eye(G * Dv, width, dtype=F64).roll((H_ + G) * D, 1), "o": torch.eye(H_ * Dv, dtype=F64)}
    eye.update({k + ".b": torch.zeros(v.shape[0], dtype=F64) for k, v in list(eye.items())})
    for i, (a, b) in enumerate(seqs):
        if b:
            wants.append(P.window_attention(rows[i].to(F64), eye, m, 1e-5)[0][a:])
    return outs, torch.cat(wants)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H_, G, D, Dv, window, rot, block_size", [
    (4, 2, 32, 32, 20, 32, 16), (6, 1, 48, 16, 7, 8, 16), (3, 3, 10, 6, 33, 4, 4), (2, 1, 64, 128, 50, 16, 64), (9, 3, 6, 14, 1, 2, 8)])
def test_attention_window_and_sink(dtype, H_, G, D, Dv, window, rot, block_size):
    """Prompts from position 0, portions behind a history and single decoded tokens in one batch; keys on both sides
    of page borders and of the window's edge."""
    seqs = [(0, 70), (37, 1), (64, 5), (0, 1), (window + 3, 1), (90, 2)]
    got, want = attention_case(dtype, H_, G, D, Dv, window, rot, seqs, block_size, D ** -0.5)
    tol = 1e-5 if dtype == "float32" else 3e-2
    assert torch.allclose(got, want, rtol=tol, atol=tol), float((got - want).abs().max())


@pytest.mark.parametrize("new", [1, 6])
@pytest.mark.parametrize("back", [-1, 0, 1])
def test_attention_key_at_the_windows_edge(new, back):
    """A key that dominates (it points the way the query does) just inside the window, on its edge and just outside, for the
    last token of a prompt portion and for a decoded token: outside it must leave no trace at all."""
    window, hist = 24, 61
    q_at = hist + new - 1
    k_at = q_at - window + 1 - back                          # back = 1: just outside
    seqs = [(hist, new), (30, 2)]
    got, want = attention_case("float32", 4, 2, 32, 16, window, 8, seqs, 16, 0.4, sharp_at=(0, q_at, k_at), seed=5)
    assert torch.allclose(got, want, rtol=1e-5, atol=1e-5), float((got - want).abs().max())
    plain, _ = attention_case("float32", 4, 2, 32, 16, window, 8, seqs, 16, 0.4, seed=5)
    moved = float((got[new - 1] - plain[new - 1]).abs().max())
    assert (moved > 1e-2) == (back <= 0), moved


@pytest.mark.parametrize("D, H_, G, block_size", [(64, 4, 2, 16), (128, 8, 2, 16), (64, 2, 2, 64), (128, 4, 1, 8), (32, 4, 4, 4)])
def test_tensor_core_attention_with_sink(D, H_, G, block_size):
    """The tensor-core kernels (tcgen05 prompt kernels with 64- and 128-key tiles, the TMA decode kernel with its key
    splits, the mma.sync kernel) with a window and the sink, against the plain-arithmetic kernel on the same cache:
    a prompt from position 0, a portion behind a history longer than the window, decoded tokens."""
    from dinfer_b200.kernels import attention_ops, ops
    g = torch.Generator().manual_seed(D + H_)
    window, scale = 150, 0.6 * D ** -0.5
    seqs = [(0, 300), (700, 1), (420, 140), (0, 1), (149, 1), (151, 1)]
    total = [a + b for a, b in seqs]
    pages = [(n + block_size - 1) // block_size for n in total]
    perm = torch.randperm(sum(pages), generator=g)
    tab = torch.full((len(seqs), max(pages)), -1, dtype=torch.int32)
    at = 0
    for b, n in enumerate(pages):
        tab[b, :n] = perm[at:at + n]
        at += n
    cache = torch.randn(sum(pages), 2, G, block_size, D, generator=g).to(torch.bfloat16).cuda()
    T = sum(b for _, b in seqs)
    q = torch.randn(T, H_ * D, generator=g).to(torch.bfloat16).cuda()
    pos = torch.cat([torch.arange(a, a + b) for a, b in seqs]).to(torch.int32).cuda()
    cu = i32(np.concatenate([[0], np.cumsum([b for _, b in seqs])]))
    seq_lens, table = i32(total), dev(tab)
    want = torch.empty(T, H_ * D, dtype=torch.bfloat16, device="cuda")
    ops.attention_generic(q, want, cache, table, cu, pos, H_, G, D, scale, window, sink=True)
    plain = torch.empty_like(want)
    ops.attention_generic(q, plain, cache, table, cu, pos, H_, G, D, scale, window, sink=False)
    assert float((want.float() - plain.float()).abs().max()) > 0.05          # the sink matters at these scores
    prompt_rows = torch.cat([torch.arange(int(cu[i]), int(cu[i + 1])) for i, (_, b) in enumerate(seqs) if b > 1]).cuda()
    decode_rows = torch.cat([torch.arange(int(cu[i]), int(cu[i + 1])) for i, (_, b) in enumerate(seqs) if b == 1]).cuda()
    group = H_ // G

    def close(got, rows, what):
        d = float((got[rows].float() - want[rows].float()).abs().max())
        assert d <= 2e-2, (what, d)

    for splits in (1, 4):
        got = torch.full_like(want, float("nan"))
        attention_ops.attention_tc(q, got, cache, table, cu, seq_lens, H_, G, D, scale, window, 300, True, True, splits, sink=True)
        close(got, torch.arange(T).cuda(), f"mma.sync kernel, {splits} splits")
    if attention_ops.decode_supported(torch.bfloat16, D, group, block_size) and block_size >= 8:
        for splits in (1, 2, 8):
            got = torch.full_like(want, float("nan"))
            attention_ops.attention_decode(q, got, cache, table, cu, seq_lens, H_, G, D, scale, window, splits, sink=True)
            close(got, decode_rows, f"decode kernel, {splits} splits")
    if attention_ops.umma_supported(torch.bfloat16, D, group, block_size):
        lens = [b for _, b in seqs]
        bound = attention_ops.umma_pair_bound(lens, group)
        for ks in (1, 2):
            got = torch.full_like(want, float("nan"))
            attention_ops.attention_umma(q, got, cache, table, cu, seq_lens, H_, G, D, scale, window, 300, ks, bound, sink=True)
            close(got, prompt_rows, f"tcgen05 kernel, keys shared {ks} ways")
        if attention_ops.umma64_supported(torch.bfloat16, D, group, block_size):
            got = torch.full_like(want, float("nan"))
            attention_ops.attention_umma64(q, got, cache, table, cu, seq_lens, H_, G, D, scale, window, 300, bound, sink=True)
            close(got, prompt_rows, "tcgen05 kernel with 64-key tiles")


# ---------------------------------------------------------------- the delta rule
def delta_inputs(T, H_, G, dk, dv, per_channel, seed):
    g = torch.Generator().manual_seed(seed)
    q = P.unit(torch.randn(T, G, dk, generator=g, dtype=F64)) * dk ** -0.5
    k = P.unit(torch.randn(T, G, dk, generator=g, dtype=F64))
    v = torch.randn(T, H_, dv, generator=g, dtype=F64)
    beta = torch.rand(T, H_, generator=g, dtype=F64)
    decay = torch.rand((T, H_, dk) if per_channel else (T, H_), generator=g, dtype=F64) * 0.2 + 0.8
    return q, k, v, beta, decay


@pytest.mark.parametrize("per_channel", [False, True])
@pytest.mark.parametrize("H_, G, dk, dv", [(4, 2, 16, 24), (3, 3, 128, 40), (2, 2, 24, 128), (1, 1, 12, 20), (2, 1, 64, 16), (5, 5, 200, 7),
                                          (2, 1, 32, 33), (1, 1, 256, 20)])
def test_delta_recurrence(H_, G, dk, dv, per_channel):
    """Three requests in one batch against each alone in the plain implementation; then the same tokens in portions
    (of 1, 2 and more tokens) through slots that another request has used before: the carried state is exact, so
    the two ways differ by the order of sums at most."""
    from dinfer_b200.kernels import delta_ops
    lens = [37, 1, 18]
    T = sum(lens)
    q, k, v, beta, decay = delta_inputs(T, H_, G, dk, dv, per_channel, dk + dv)
    f = lambda t: dev(t, torch.float32)
    state = torch.full((5, H_ * dk * dv + 3), float("nan"), dtype=torch.float32, device="cuda")
    cu = i32([0, 37, 38, 56])
    out = delta_ops.recurrence(f(q), f(k), f(v), f(beta), f(decay.reshape(T, -1) - 1), state, cu, i32([3, 0, 1]), i32([1, 1, 1]), per_channel)
    rep = H_ // G
    want, at = [], 0
    for n in lens:
        s = slice(at, at + n)
        o, S = P.delta_rule(q[s].repeat_interleave(rep, 1), k[s].repeat_interleave(rep, 1), v[s], beta[s], decay[s])
        want.append(o)
        at += n
    want = torch.cat(want)
    assert torch.allclose(out.cpu().to(F64), want, rtol=2e-5, atol=2e-5), float((out.cpu() - want).abs().max())
    assert torch.allclose(state[1, :H_ * dk * dv].cpu().to(F64).reshape(H_, dk, dv), S, rtol=2e-5, atol=2e-5)
    # request 0 again in portions, in slot 1 (used by request 2 above) and marked fresh only in its first step; with a
    # column's rows spread over 1, 2 or 4 times the lanes (what the kernel otherwise chooses by the batch's size)
    for widen in (0, 1, 2, 4):
        got, at = [], 0
        for n in (1, 2, 1, 9, 2, 22):
            s = slice(at, at + n)
            got.append(delta_ops.recurrence(f(q[s]), f(k[s]), f(v[s]), f(beta[s]), f(decay[s].reshape(n, -1) - 1), state,
                                            i32([0, n]), i32([1]), i32([int(at == 0)]), per_channel, widen=widen))
            at += n
        assert torch.allclose(torch.cat(got), out[:37], rtol=1e-5, atol=2e-6), widen


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("per_channel, taps, H_, G, dk, dv", [(False, 4, 2, 1, 64, 16), (True, 3, 4, 2, 16, 24), (True, 1, 1, 1, 12, 20), (False, 6, 3, 3, 20, 4)])
def test_delta_prep_and_post(dtype, per_channel, taps, H_, G, dk, dv):
    """Convolution with its history across steps of 1, 2 and more tokens (two requests, one of which sits a step
    out), unit vectors, beta, decay; the output norm with its gate."""
    from dinfer_b200.kernels import delta_ops
    g = torch.Generator().manual_seed(taps)
    dt = DT[dtype]
    nq, nv = G * dk, H_ * dv
    C_ = 2 * nq + nv
    nd = H_ * dk if per_channel else H_
    lens = {"a": 23, "b": 9}
    P_in = {r: torch.randn(n, C_ + H_ + 5, generator=g).to(dt) for r, n in lens.items()}      # q | k | v | (gap of 5) | b
    A_in = {r: torch.randn(n, nd, generator=g).to(dt) for r, n in lens.items()}
    conv_w = torch.randn(C_, taps, generator=g)
    A_log, dt_bias = torch.randn(H_, generator=g), torch.randn(nd, generator=g) - 1.0
    S0 = H_ * dk * dv
    state = torch.full((4, S0 + (taps - 1) * C_), float("nan"), dtype=torch.float32, device="cuda")
    steps = [[("a", 0, 1)], [("a", 1, 3), ("b", 0, 2)], [("b", 2, 3)], [("a", 3, 4), ("b", 3, 9)], [("a", 4, 23)]]
    got = {r: [] for r in lens}
    slot = {"a": 2, "b": 0}
    for entries in steps:
        Pm = torch.cat([P_in[r][lo:hi] for r, lo, hi in entries]).cuda()
        Am = torch.cat([A_in[r][lo:hi] for r, lo, hi in entries]).cuda()
        cu = i32(np.concatenate([[0], np.cumsum([hi - lo for _, lo, hi in entries])]))
        outs = delta_ops.prep(Pm, (0, nq, 2 * nq, C_ + 5), Am, dev(conv_w), dev(A_log), dev(dt_bias), state, S0, cu,
                              i32([slot[r] for r, _, _ in entries]), i32([int(lo == 0) for _, lo, _ in entries]),
                              H_, G, dk, dv, taps, per_channel)
        at = 0
        for r, lo, hi in entries:
            got[r].append([o[at:at + hi - lo].cpu().to(F64) for o in outs])
            at += hi - lo
    tol = dict(rtol=2e-5, atol=2e-5)
    for r, n in lens.items():
        x = P_in[r].to(F64)
        y = {}
        for name, lo, hi in (("q", 0, nq), ("k", nq, 2 * nq), ("v", 2 * nq, C_)):
            y[name] = P.silu(P.short_conv(x[:, lo:hi], conv_w[lo:hi].to(F64))[0])
        a = A_in[r].to(F64) + dt_bias.to(F64)
        decay = torch.exp(-torch.exp(A_log.to(F64)).repeat_interleave(dk if per_channel else 1) * P.softplus(a))
        want = [P.unit(y["q"].reshape(n, G, dk)) * dk ** -0.5, P.unit(y["k"].reshape(n, G, dk)), y["v"].reshape(n, H_, dv),
                torch.sigmoid(x[:, C_ + 5:]), decay - 1]              # the kernel hands the decay on as g - 1
        for j, w in enumerate(want):
            have = torch.cat([piece[j] for piece in got[r]])
            assert torch.allclose(have, w, **tol), (r, j, float((have - w).abs().max()))
    o = torch.randn(7, H_, dv, generator=g)
    gate = torch.randn(7, nv + 8, generator=g).to(dt)
    w = 1 + 0.2 * torch.randn(dv, generator=g)
    for sig in (False, True):
        yv = torch.empty(7, nv, dtype=dt, device="cuda")
        delta_ops.post(dev(o), dev(w), dev(gate)[:, 8:], 1e-5, sig, yv)
        zz = gate[:, 8:].to(F64).reshape(7, H_, dv)
        want = P.rms_norm(o.to(F64), w.to(F64), 1e-5) * (torch.sigmoid(zz) if sig else P.silu(zz))
        t = 1e-5 if dtype == "float32" else 1e-2
        assert torch.allclose(yv.cpu().to(F64).reshape(7, H_, dv), want, rtol=t, atol=t)


def test_delta_rule_remembers_a_far_token():
    """A value written 300 tokens back under a decay close to one, read by a query along the same key: it must come
    back almost whole, through the kernel as through the plain rule."""
    from dinfer_b200.kernels import delta_ops
    T, dk, dv = 320, 32, 16
    q, k, v, beta, decay = delta_inputs(T, 1, 1, dk, dv, False, 1)
    decay[:] = 0.9995
    beta[:] = 0.02
    k[7], beta[7], v[7] = 0.0, 1.0, 10.0
    k[7, 0, 3] = 1.0
    q[T - 1] = k[7] + 0.0
    f = lambda t: dev(t, torch.float32)
    state = torch.zeros((1, dk * dv), dtype=torch.float32, device="cuda")
    out = delta_ops.recurrence(f(q), f(k), f(v), f(beta), f(decay - 1), state, i32([0, T]), i32([0]), i32([1]), False)
    want, _ = P.delta_rule(q, k, v, beta, decay)
    assert float(want[-1].abs().min()) > 3.0
    assert torch.allclose(out.cpu().to(F64), want, rtol=1e-4, atol=1e-4)


# ---------------------------------------------------------------- the routed feed-forward with a table
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E, top, ff, shared, h", [(5, 1, 24, 40, 64), (6, 3, 16, 0, 64), (7, 2, 40, 56, 128), (3, 3, 20, 12, 100)])
def test_table_routed_experts(dtype, E, top, ff, shared, h):
    from dinfer_b200.parts.base import BuildEnv, StepContext
    from dinfer_b200.parts.moe import MoE
    from dinfer_b200.weights.random_init import random_tensor
    dt = DT[dtype]
    vocab = 50
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": E, "top": top}}
    if shared:
        f["shared"] = {"ff": shared}
    part = MoE({"num_experts": E, "top_k": top, "expert_size": ff, "shared_size": shared, "activation": "silu", "gated": True,
                "routing": "table", "vocab_size": vocab, "table": "table", "expert_gate": "e{e}.gate", "expert_up": "e{e}.up",
                "expert_down": "e{e}.down", "shared_gate_up": "shared.gate", "shared_up": "shared.up", "shared_down": "shared.down"},
               BuildEnv(torch.device("cuda"), dt, h, 64), "")
    W = {d.name: random_tensor(d, 4, 0.2, 0.0, torch.float32) for d in part.declare()}
    W = {k: (v if v.dtype == torch.int32 else v.to(torch.bfloat16).float()) for k, v in W.items()}
    part.bind({k: dev(v, None if v.dtype == torch.int32 else dt) for k, v in W.items()})
    for T in (1, 3, 40, 700):
        g = torch.Generator().manual_seed(T)
        toks = torch.randint(0, vocab, (T,), generator=g)
        x = torch.randn(T, h, generator=g).to(dt)
        ctx = StepContext(T, 1, None, None, None, [], None, None, T, T, T == 1)
        ctx.token_ids = dev(toks.to(torch.int32))
        got = part.forward(dev(x), ctx).cpu().to(F64)
        want = P.table_moe(x.to(F64), toks.tolist(), {k: (v if v.dtype == torch.int32 else v.to(F64)) for k, v in W.items()}, f)
        t = 1e-5 if dtype == "float32" else 3e-2
        assert torch.allclose(got, want, rtol=t, atol=t * float(want.abs().max())), (T, float((got - want).abs().max()))
    # a token a step has not read from the device yet: named by its row of the last sampling
    ctx = StepContext(2, 1, None, None, None, [], None, None, 2, 2, False)
    ctx.token_ids, ctx.prev_tokens = i32([-2, 7]), i32([9, 31])
    x = torch.randn(2, h).to(dt)
    got = part.forward(dev(x), ctx).cpu().to(F64)
    want = P.table_moe(x.to(F64), [31, 7], {k: (v if v.dtype == torch.int32 else v.to(F64)) for k, v in W.items()}, f)
    assert torch.allclose(got, want, rtol=3e-2, atol=3e-2 * float(want.abs().max()))


# ---------------------------------------------------------------- whole models
LENGTHS = {"A": {"a": 1, "b": 2, "c": 45, "d": 131, "e": 77},
           "B": {"a": 150, "b": 3, "c": 66, "d": 1, "e": 19},
           "C": {"a": 97, "b": 40, "c": 2, "d": 71},
           "D": {"a": 120, "b": 1, "c": 33, "d": 64},
           "E": {"a": 190, "b": 17, "c": 65, "d": 128}}


BF16_WORST, BF16_RMS = 0.3, 0.08


def rms_err(got, want):
    if not np.isfinite(got).all():
        return float("inf")
    return float(np.sqrt(np.mean((got.astype(np.float64) - want) ** 2) / np.mean(np.asarray(want) ** 2)))


class Oracle:
    def __init__(self, model_dir):
        self.cfg = json.load(open(os.path.join(model_dir, "config.json")))
        self.W = C.load_weights(model_dir)
        self._cache = {}

    def logits(self, ids):
        key = tuple(ids)
        if key not in self._cache:
            self._cache[key] = P.logits(self.cfg, self.W, list(ids)).numpy()
        return self._cache[key]


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    out = {}
    for name, cfg in C.CONFIGS.items():
        for dt in DT:
            out[(name, dt)] = C.write_model(str(tmp_path_factory.mktemp(f"zasipel{name}_{dt}")), cfg, 11 + ord(name), DT[dt])
    return out


_REQUESTS = {}


def requests(name, model_dirs):
    if name not in _REQUESTS:
        cfg, rng = C.CONFIGS[name], random.Random(7 + ord(name))
        oracle = Oracle(model_dirs[(name, "bfloat16")])
        tokens = {r: H.random_tokens(rng, n, cfg["vocab"]) for r, n in LENGTHS[name].items()}
        _REQUESTS[name] = (tokens, {r: oracle.logits(t) for r, t in tokens.items()})
    return _REQUESTS[name]


@pytest.mark.parametrize("block_size", [4, 16, 64])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(C.CONFIGS))
def test_replay_all_ways(model_dirs, name, dtype, block_size):
    """Every position of every request: whole / with a decoded tail long enough to pass page borders and windows /
    in portions down to two tokens / mixed with up to four live requests (some sitting steps out) on a pool and with
    state slots that only hold the most demanding step, so that pages and slots are freed and used again."""
    model_dir = model_dirs[(name, dtype)]
    rng = random.Random(99 + ord(name))
    lengths = LENGTHS[name]
    tokens, want = requests(name, model_dirs)
    schedules = {
        "whole": H.schedule_whole(lengths),
        "tail": H.schedule_tail(lengths, 70),
        "chunks": H.schedule_chunks(lengths, rng),
        "mixed": H.schedule_mixed(lengths, rng),
        "mixed2": H.schedule_mixed(dict(reversed(list(lengths.items()))), rng, max_live=3, decode_tail=40),
    }
    max_tokens = max(H.max_live_tokens(s, round_to=max(64, block_size)) for s in schedules.values())
    rp = H.LocalReplay(model_dir, dtype, max_tokens, block_size=block_size)
    worst, spread = {}, {}
    for sname, steps in schedules.items():
        got = H.run_schedule(rp, steps, tokens, tag=sname + "/")
        worst[sname] = max(H.rel_err(got[r], want[r]) for r in tokens)
        spread[sname] = max(rms_err(got[r], want[r]) for r in tokens)
    assert rp.close() == 0
    # 32-bit is the sharp test.  In bfloat16 a rounding can travel far in this design: at a sequence's first tokens
    # a recurrent mixer's output is (q . k) u with q . k near zero, and the norm behind it brings that back to unit
    # size, relative error included.  So the root mean square of the differences over a request is held to BF16_RMS
    # of the logits' own and the largest single difference to BF16_WORST of their largest (a fault gives about 1).
    if dtype == "float32":
        bad = {k: v for k, v in worst.items() if not v <= H.TOLERANCE[dtype]}
    else:
        bad = {k: (worst[k], spread[k]) for k in worst if not (worst[k] <= BF16_WORST and spread[k] <= BF16_RMS)}
    assert not bad, f"{name} {dtype} pages of {block_size}: {bad} (largest: {worst}; rms: {spread})"


def test_trace_runner_and_first_tokens(model_dirs, tmp_path):
    """Through ``bin/trace_run`` as a process: the first tokens of sequences (a request of one token, the first two
    positions of others), and a request that sits steps out while others come and go."""
    model_dir = model_dirs[("A", "float32")]
    cfg = C.CONFIGS["A"]
    rng = random.Random(5)
    tokens = {r: H.random_tokens(rng, n, cfg["vocab"]) for r, n in {"p": 1, "q": 2, "r": 70, "s": 45}.items()}
    oracle = Oracle(model_dir)
    rp = H.Replay(model_dir, "float32", str(tmp_path / "out"), 256)
    try:
        a = rp.step([{"id": "p", "tokens": tokens["p"], "want": [0]}, {"id": "r", "tokens": tokens["r"][:2], "want": [0, 1]}], ["p"])
        b = rp.step([{"id": "q", "tokens": tokens["q"], "want": [0, 1]}, {"id": "s", "tokens": tokens["s"][:40], "want": [39]}], ["q"])
        c = rp.step([{"id": "r", "tokens": tokens["r"][2:], "want": [67]}, {"id": "s", "tokens": tokens["s"][40:41], "want": [0]}], ["r"])
        d = rp.step([{"id": "s", "tokens": tokens["s"][41:], "want": [3]}], ["s"])
    finally:
        assert rp.close() == 0
    for got, want in ((a[0], oracle.logits(tokens["p"])[0]), (a[1:], oracle.logits(tokens["r"])[:2]),
                      (b[:2], oracle.logits(tokens["q"])), (b[2], oracle.logits(tokens["s"])[39]),
                      (c[0], oracle.logits(tokens["r"])[69]), (c[1], oracle.logits(tokens["s"])[40]),
                      (d[0], oracle.logits(tokens["s"])[44])):
        assert H.rel_err(np.asarray(got), np.asarray(want)) <= H.TOLERANCE["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "E"])
def test_greedy_generation_through_the_entry_point(model_dirs, name, dtype):
    """``LLM.generate``: scheduler, chunked prompts (a token budget below the prompts' lengths), decode steps replayed
    as CUDA graphs (the mixers' state is driven from device tensors), greedy sampling, tokens named by their sampling
    row while a step is scheduled ahead (the experts' table must follow them); more requests than run at once."""
    from dinfer_b200 import LLM, SamplingParams
    model_dir = model_dirs[(name, dtype)]
    cfg = C.CONFIGS[name]
    rng = random.Random(21)
    prompts = [H.random_tokens(rng, n, cfg["vocab"]) for n in (1, 5, 23, 40, 9, 31)]
    llm = LLM(model_dir, dtype=dtype, max_model_len=128, max_num_seqs=4, max_num_batched_tokens=16, block_size=16,
              num_blocks=40)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True))
    oracle = Oracle(model_dir)
    exact = total = 0
    for p, o in zip(prompts, outs):
        assert len(o.output_ids) == 40
        lg = oracle.logits(list(p) + list(o.output_ids))
        exact += sum(int(lg[len(p) - 1 + i].argmax()) == t for i, t in enumerate(o.output_ids))
        total += 40
    assert exact >= (0.9 if dtype == "bfloat16" else 0.99) * total, (exact, total)
    assert any(isinstance(k, int) for k in llm.runner._graphs)
