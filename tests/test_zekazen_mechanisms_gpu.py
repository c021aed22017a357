"""Each Zekazen mechanism alone on the GPU against the oracle's function of the same name: models of one layer
whose weights or inputs are made so that a fault shows (a key that holds nearly all of the weight, placed far
away, at page borders, just inside and just outside the window, in prompts and in decoding; a sink that holds
most of the weight; a state that has to come from hundreds of tokens back; routers whose groups decide), and
the kernels of the mechanisms called by themselves."""
import math

import pytest
import torch

import plain_zekazen as P
from zekazen_helpers import assert_rows_close, make_tensors, prompts, write_model

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]


def engine(tmp_path, cfg, tensors, dtype, tag, **kw):
    from zlm_b200 import Engine
    folder = write_model(tmp_path, cfg, tensors, tag)
    return Engine.from_pretrained(folder, dtype=dtype, max_tokens=kw.pop("max_tokens", 2048), **kw)


def one_layer(kind, mixer, mlp=None, width=64, vocab=96):
    return {"architecture": "Zekazen", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "layers": [{"type": kind, "mixer": mixer, "mlp": mlp}]}


# ---------------------------------------------------------------------------- attention: one key stands out
def peaked_attention(window, conv=1, heads=2, kv_heads=2, dim=16, vdim=24, scale=1.5):
    """A one-layer model in which token 1's key points exactly where token 2's query points (the same projection,
    the same embedding row, a convolution that only passes the newest value), so that among hundreds of other
    keys the one of token 1 holds nearly all of a token-2 query's weight, if it is inside the window."""
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "scale": scale}
    if window:
        mixer["mask"] = {"size": window}
    cfg = one_layer("attention", mixer)
    W = make_tensors(cfg, 11)
    # k_1 = W_k h_1 = W_q h_2 = q_2 with W_k's columns those of W_q moved by one and h_1 those of h_2 likewise (the
    # norm before the mixer has the weight 1): the same direction, while v_1 and v_2, and token 2's own key, differ
    assert kv_heads == heads
    W["l0.norm1"] = torch.ones_like(W["l0.norm1"])
    W["l0.mix.k"] = torch.roll(W["l0.mix.q"], 1, dims=1)
    for n in ("q", "k", "v"):
        c = torch.zeros_like(W[f"l0.mix.{n}.conv"])
        c[:, -1] = 1.0
        W[f"l0.mix.{n}.conv"] = c
    W["embed"][1] = torch.roll(W["embed"][2], 1, dims=0)
    return cfg, W


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [0, 9, 64, 70, 150])
def test_a_key_that_holds_the_weight_at_every_distance(tmp_path, dtype, window):
    """The key sits 1, 63, 64, 65 and several hundred tokens back, and just inside and just outside the window;
    the query is asked for inside a prompt, at the start of a portion, and decoded alone."""
    from zlm_b200 import StepEntry
    cfg, W = peaked_attention(window)
    ref = {n: t.double() for n, t in W.items()}
    eng = engine(tmp_path, cfg, W, dtype, f"peak{window}")
    dists = sorted({1, 63, 64, 65, 300} | ({window - 1, window, window + 1} if window else {500}))
    for d in [x for x in dists if x >= 1]:
        n = d + 40
        (p,) = prompts(cfg["vocab"] - 3, [n], seed=d)
        p = [t + 3 for t in p]                       # tokens 1 and 2 appear only where they are put
        i = n - 5
        p[i - d], p[i] = 1, 2
        want, *_ = P.forward(cfg, ref, p)
        inside = window == 0 or d < window
        # the oracle itself must show the difference that the test is after
        alone = P.forward(cfg, ref, p[:i - d] + [5] + p[i - d + 1:])[0][i]
        moved = float((want[i] - alone).norm() / want[i].norm())
        assert (moved > 0.2) == inside, f"distance {d}, window {window}: the test's key moves the logits by {moved:.3f}"
        for cut in (None, i, i - 1):
            s = eng.new_sequence()
            if cut is None:
                got = eng.step([StepEntry(s, p, [i])]).clone()
            else:
                eng.step([StepEntry(s, p[:cut], [])])
                if cut == i:
                    got = eng.step([StepEntry(s, [p[i]], [0])]).clone()         # decoded alone
                    eng.step([StepEntry(s, p[i + 1:], [])])
                else:
                    got = eng.step([StepEntry(s, p[cut:], [1])]).clone()         # second token of a portion
            eng.release(s)
            assert_rows_close(got[0], want[i].float(), dtype, f"window {window} distance {d} cut {cut}",
                              tol=2e-4 if dtype == "float32" else 6e-2)
    eng.check(sync=True)


@pytest.mark.parametrize("dtype", DTYPES)
def test_grouped_heads_read_their_own_kv_head(tmp_path, dtype):
    """6 query heads on 3 kv heads with different sizes of keys and values and a convolution of 4 taps."""
    from zlm_b200 import StepEntry
    cfg = one_layer("attention", {"heads": 6, "kv_heads": 3, "dim": 40, "vdim": 8, "conv": 4, "scale": 0.25,
                                  "mask": {"size": 33}})
    W = make_tensors(cfg, 12)
    ref = {n: t.double() for n, t in W.items()}
    eng = engine(tmp_path, cfg, W, dtype, "gqa")
    (p,) = prompts(cfg["vocab"], [150], seed=3)
    want = P.forward(cfg, ref, p)[0].float()
    s = eng.new_sequence()
    got = [eng.step([StepEntry(s, p[:100], list(range(100)))]).clone()]
    got += [eng.step([StepEntry(s, [p[t]], [0])]).clone() for t in range(100, 150)]
    assert_rows_close(torch.cat(got), want, dtype, "grouped heads")


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_sink_takes_its_share(tmp_path, dtype):
    """Scores far below zero: the sink holds nearly all of the weight and the mixer's output nearly vanishes;
    a softmax without it would give an average of the values."""
    from zlm_b200 import StepEntry
    cfg = one_layer("attention", {"heads": 1, "kv_heads": 1, "dim": 16, "vdim": 16, "conv": 1, "scale": 0.6})
    W = make_tensors(cfg, 13)
    W["l0.mix.k"] = -W["l0.mix.q"].clone()           # every key points away from the queries of its own token
    for n in ("q", "k", "v"):
        W[f"l0.mix.{n}.conv"] = torch.ones_like(W[f"l0.mix.{n}.conv"])
    W["embed"][:] = W["embed"][0] + 0.05 * W["embed"]      # all tokens nearly alike: all scores near -dim * scale
    W = {n: t.to(torch.bfloat16).float() for n, t in W.items()}
    ref = {n: t.double() for n, t in W.items()}
    eng = engine(tmp_path, cfg, W, dtype, "sink")
    (p,) = prompts(cfg["vocab"], [90], seed=4)
    want, after, _, _ = P.forward(cfg, ref, p)
    x0 = ref["embed"][torch.tensor(p)]
    assert float((after[0] - x0).norm() / x0.norm()) < 0.02          # the oracle's mixer adds next to nothing
    s = eng.new_sequence()
    got = [eng.step([StepEntry(s, p[:70], list(range(70)))]).clone()]
    got += [eng.step([StepEntry(s, [p[t]], [0])]).clone() for t in range(70, 90)]
    assert_rows_close(torch.cat(got), want.float(), dtype, "sink", tol=2e-4 if dtype == "float32" else 2e-2)


# ---------------------------------------------------------------------------- the convolution's state
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps", [2, 3, 4, 8])
def test_convolution_across_steps_of_every_length(tmp_path, dtype, taps):
    """Portions shorter than the taps (1, 2 tokens), one after the other, so that the history has to be shifted
    and not only replaced; two sequences side by side with different cuts."""
    from zlm_b200 import StepEntry
    cfg = one_layer("attention", {"heads": 2, "kv_heads": 2, "dim": 24, "vdim": 8, "conv": taps, "scale": 0.3,
                                  "mask": {"size": 50}})
    W = make_tensors(cfg, 14 + taps)
    ref = {n: t.double() for n, t in W.items()}
    eng = engine(tmp_path, cfg, W, dtype, f"conv{taps}")
    a, b = prompts(cfg["vocab"], [40, 40], seed=6)
    wa, wb = P.forward(cfg, ref, a)[0].float(), P.forward(cfg, ref, b)[0].float()
    cuts_a, cuts_b = [1, 1, 2, 1, 5, 2, 1, 1, 26], [3, 1, 1, 1, 2, 9, 1, 2, 20]
    sa, sb = eng.new_sequence(), eng.new_sequence()
    ga, gb, ia, ib = [], [], 0, 0
    for ca, cb in zip(cuts_a, cuts_b):
        out = eng.step([StepEntry(sa, a[ia:ia + ca], list(range(ca))), StepEntry(sb, b[ib:ib + cb], list(range(cb)))]).clone()
        ga.append(out[:ca]); gb.append(out[ca:])
        ia += ca; ib += cb
    assert_rows_close(torch.cat(ga), wa, dtype, f"{taps} taps, first sequence")
    assert_rows_close(torch.cat(gb), wb, dtype, f"{taps} taps, second sequence")
    # the slots are given back and taken again: the new sequences must not see the old histories
    eng.release(sa); eng.release(sb)
    sb2, sa2 = eng.new_sequence(), eng.new_sequence()
    out = eng.step([StepEntry(sa2, b[:2], [0, 1]), StepEntry(sb2, a[:1], [0])]).clone()
    assert_rows_close(out, torch.cat([wb[:2], wa[:1]]), dtype, f"{taps} taps, slots used again")


# ---------------------------------------------------------------------------- retention
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [(2, 16, 24, 16), (1, 48, 200, 20), (3, 72, 8, 0), (2, 128, 64, 128)])
def test_retention_state_from_far_back(tmp_path, dtype, sizes):
    """Decays close to 1: what the first tokens wrote into the state still decides the output hundreds of tokens
    later.  The prompt runs in pieces side by side, then in a portion on a state that is not zero, then token by
    token; key sizes that are no power of two, value sizes above and below a block's columns, rotation over a part
    of a head, over all of it and none."""
    from zlm_b200 import StepEntry
    heads, dim, vdim, dims = sizes
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "decay": [0.9995, 0.97, 0.999][:heads]}
    if dims:
        mixer["rot"] = {"base": 300.0, "dims": dims}
    cfg = one_layer("retention", mixer)
    W = make_tensors(cfg, 20 + dim)
    ref = {n: t.double() for n, t in W.items()}
    eng = engine(tmp_path, cfg, W, dtype, f"ret{dim}")
    (p,) = prompts(cfg["vocab"], [700], seed=8)
    want = P.forward(cfg, ref, p)[0]
    # the oracle itself: without the first 100 tokens the logits at the end are others
    late = P.forward(cfg, ref, p[100:])[0][-1]
    assert float((want[-1] - late).norm() / want[-1].norm()) > 0.01
    s = eng.new_sequence()
    got = [eng.step([StepEntry(s, p[:333], list(range(333)))]).clone()]
    got.append(eng.step([StepEntry(s, p[333:650], list(range(317)))]).clone())
    got += [eng.step([StepEntry(s, [p[t]], [0])]).clone() for t in range(650, 700)]
    assert_rows_close(torch.cat(got), want.float(), dtype, f"retention {sizes}")
    eng.release(s)
    # a slot that is used again starts from a zero state
    s = eng.new_sequence()
    got = eng.step([StepEntry(s, p[:5], list(range(5)))]).clone()
    assert_rows_close(got, want[:5].float(), dtype, f"retention {sizes}, slot used again")


def test_retention_pieces_equal_the_plain_walk():
    """The kernel alone: a step of three sequences (one shorter than a piece, one of several pieces and a rest, one
    of one token) from states that are not zero, in pieces and in one walk: the same outputs and states to rounding."""
    from zlm_b200.kernels import get_kernels
    k = get_kernels()
    dev = "cuda"
    H, D, V = 3, 40, 72
    lens = [37, 300, 1]
    T, R = sum(lens), len(lens)
    g = torch.Generator().manual_seed(2)
    proj = torch.randn(T, 2 * H * D + 2 * H * V, generator=g).to(dev)
    inv = torch.tensor([300.0 ** (-2.0 * i / 24) for i in range(12)], dtype=torch.float32, device=dev)
    decay = torch.tensor([0.999, 0.9, 0.97], dtype=torch.float32, device=dev)
    state0 = torch.randn(4, H, D, V, generator=g).to(dev)

    class Plan:
        pass
    plan = Plan()
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    plan.cu_seqlens = torch.tensor(cu, dtype=torch.int32, device=dev)
    plan.seq_slot = torch.tensor([2, 0, 3], dtype=torch.int32, device=dev)
    plan.seq_start = torch.tensor([5, 100, 64], dtype=torch.int32, device=dev)
    plan.R, plan.h_seq_new, plan.max_new = R, lens, max(lens)
    plan.scratch = lambda name, shape, dtype: torch.empty(shape, dtype=dtype, device=dev)
    outs = []
    for pieces in (False, True):
        st = state0.clone()
        o = torch.zeros(T, H * V, device=dev)
        k.retention(o, proj, 0, H * D, 2 * H * D, inv, 24, decay, st, plan, H, D, V, D ** -0.5, pieces=pieces)
        torch.cuda.synchronize()
        outs.append((o, st))
    assert_rows_close(outs[1][0], outs[0][0], "float32", "outputs", tol=1e-5)
    assert torch.allclose(outs[1][1], outs[0][1], rtol=1e-5, atol=1e-5)
    assert torch.equal(outs[0][1][1], state0[1])             # a slot that no sequence of the step uses is left alone


# ---------------------------------------------------------------------------- routing and experts
def route_inputs(E, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(40, 64, generator=g).to(torch.bfloat16).float()
    wr = (torch.randn(E, 64, generator=g) / 4).to(torch.bfloat16).float()
    corr = (0.05 * torch.randn(E, generator=g)).to(torch.bfloat16).float()
    return x, wr, corr


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("r", [
    {"experts": 12, "identity": 4, "top": 4, "scale": 1.5, "groups": {"count": 4, "keep": 2}},
    {"experts": 6, "identity": 0, "top": 1, "scale": 1.0, "groups": {"count": 3, "keep": 1}},
    {"experts": 5, "identity": 2, "top": 7, "scale": 0.5, "groups": {"count": 1, "keep": 1}},
    {"experts": 40, "identity": 8, "top": 6, "scale": 2.0, "groups": {"count": 48, "keep": 7}},
])
def test_router_kernels_against_the_oracle(dtype, r):
    """Both router kernels (logits inside, and the choice from logits that a product left) against the oracle's
    ``route``: groups of neighbours, the correction in the choice and not in the weight, identity experts among
    the choices, more groups than a warp has lanes."""
    from zlm_b200.kernels import get_kernels
    k = get_kernels()
    E = r["experts"] + r["identity"]
    x, wr, corr = route_inputs(E, 31 + E)
    idx_w, wgt_w, margin = P.route(x.double(), wr.double(), corr.double(), r)
    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    xd, wd, cd = x.cuda().to(dt), wr.cuda().to(dt), corr.cuda()
    T, top = x.shape[0], r["top"]
    for way in ("route", "choose"):
        idx = torch.zeros(T, top, dtype=torch.int32, device="cuda")
        wgt = torch.zeros(T, top, dtype=torch.float32, device="cuda")
        if way == "route":
            k.moe_route(idx, wgt, xd, wd, top, None, None, "softmax", False, cd, r["groups"]["count"], r["groups"]["keep"], r["scale"])
        else:
            logits = (xd.float() @ wd.float().T).contiguous()
            k.moe_choose(idx, wgt, logits, E, top, None, "softmax", False, cd, r["groups"]["count"], r["groups"]["keep"], r["scale"])
        torch.cuda.synchronize()
        clear = margin > 1e-4
        assert int(clear.sum()) > T // 2
        assert torch.equal(idx.cpu()[clear].long(), idx_w[clear]), way
        assert torch.allclose(wgt.cpu()[clear].double(), wgt_w[clear], rtol=1e-4, atol=1e-6), way


def test_groups_decide_the_choice():
    """Made logits: with one group kept the choice stays inside the group of the best single score although its
    second member is weak; choice scores below zero (a correction of -1) still beat a refused group (it counts as
    minus infinity, not as 0); the correction reorders experts 2 and 3 for the choice only."""
    from zlm_b200.kernels import get_kernels
    k = get_kernels()
    logits = torch.tensor([[3.0, 0.0, 2.9, 2.95, 0.0, 0.0]], device="cuda")           # groups (0,1) (2,3) (4,5)
    corr = torch.tensor([-1.0, -1.0, -1.02, -1.05, -1.0, -1.0], device="cuda")
    idx = torch.zeros(1, 2, dtype=torch.int32, device="cuda")
    wgt = torch.zeros(1, 2, device="cuda")
    k.moe_choose(idx, wgt, logits, 6, 2, None, "softmax", False, corr, 3, 1, 1.0)
    assert idx.tolist() == [[0, 1]]                    # group 0 has the best single score; its second member is weak
    s = torch.softmax(logits[0], 0)
    assert torch.allclose(wgt[0], s[:2])
    k.moe_choose(idx, wgt, logits, 6, 2, None, "softmax", False, corr, 3, 2, 1.0)
    assert idx.tolist() == [[0, 2]]                    # two groups kept: 0 and (2,3); the best two of those four
    k.moe_choose(idx, wgt, logits, 6, 2, None, "softmax", False, None, 1, 1, 1.0)
    assert idx.tolist() == [[0, 3]]                    # no correction, no groups: the two largest scores


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("r", [
    {"experts": 6, "identity": 2, "top": 3, "scale": 1.5, "groups": {"count": 4, "keep": 3}},
    {"experts": 3, "identity": 3, "top": 6, "scale": 1.0, "groups": {"count": 1, "keep": 1}},
    {"experts": 9, "identity": 0, "top": 1, "scale": 0.7, "groups": {"count": 3, "keep": 2}},
])
@pytest.mark.parametrize("tokens", [5, 150])
def test_experts_layer_against_the_oracle(tmp_path, dtype, r, tokens):
    """A model of one attention layer (a trivial one) and one routed feed-forward: every expert gated, identity
    experts adding their input, every expert chosen (top = all), one expert a token; few tokens and many."""
    from zlm_b200 import StepEntry
    cfg = one_layer("attention", {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "conv": 1, "scale": 0.1},
                    {"kind": "moe", "expert": {"ff": 40}, "router": r})
    W = make_tensors(cfg, 40 + r["experts"])
    ref = {n: t.double() for n, t in W.items()}
    eng = engine(tmp_path, cfg, W, dtype, f"moe{r['experts']}")
    (p,) = prompts(cfg["vocab"], [tokens], seed=9)
    want, _, _, margin = P.forward(cfg, ref, p)
    s = eng.new_sequence()
    got = eng.step([StepEntry(s, p, list(range(tokens)))]).clone()
    keep = margin >= (0.0 if dtype == "float32" else 0.008)          # (one layer: a close call stays at its position)
    assert int(keep.sum()) * 3 >= tokens
    assert_rows_close(got[keep.cuda()], want.float()[keep], dtype, f"experts {r}")


# ---------------------------------------------------------------------------- the small kernels alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("act", ["sigmoid", "silu"])
@pytest.mark.parametrize("norm", [False, True])
def test_head_gate_kernel(dtype, act, norm):
    from zlm_b200.kernels import get_kernels
    k = get_kernels()
    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    T, H, V, pad = 7, 3, 40, 48
    g = torch.Generator().manual_seed(5)
    for o_dt in ([torch.float32] if dtype == "float32" else [torch.float32, torch.bfloat16]):
        o = torch.randn(T, H, pad, generator=g).cuda().to(o_dt)
        gate = torch.randn(T, 10 + H * V, generator=g).cuda().to(dt)
        out = torch.zeros(T, H * V, device="cuda", dtype=dt)
        k.head_gate(out, o, gate[:, 10:], H, V, norm, 1e-5, act)
        x = o.double()[:, :, :V]
        if norm:
            x = P.unit_norm(x, 1e-5)
        z = gate.double()[:, 10:]
        want = x.reshape(T, H * V) * (torch.sigmoid(z) if act == "sigmoid" else P.silu(z))
        assert torch.allclose(out.double(), want, rtol=2e-2 if dtype == "bfloat16" else 1e-5, atol=1e-2 if dtype == "bfloat16" else 1e-5)
