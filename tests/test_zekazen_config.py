"""Zekazen without a GPU: the configuration (reading, refusing, writing back, lowering to parts), the
checkpoint's tensor names, and the oracle's own invariants (whole sequences against its incremental form)."""
import copy

import pytest
import torch

import plain_zekazen as P
from zekazen_helpers import ZEKA, ZEKA_A, make_tensors


def test_architecture_is_chosen_by_its_string_key():
    from zlm_b200 import ZekazenConfig
    from zlm_b200.registry import config_from_dict
    cfg = config_from_dict(ZEKA_A)
    assert isinstance(cfg, ZekazenConfig)
    assert cfg.to_dict() == ZEKA_A
    assert config_from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("name", sorted(ZEKA))
def test_lowering_names_parts_and_tensors(name):
    from zlm_b200.parts.model import DecoderModel
    from zlm_b200.registry import config_from_dict
    d = ZEKA[name]
    spec = config_from_dict(d).to_model_spec()
    assert [l.mixer.kind for l in spec.layers] == [{"retention": "retention", "attention": "conv_attention"}[l["type"]]
                                                   for l in d["layers"]]
    specs = DecoderModel(spec).param_specs()
    W = d["width"]
    want = {"embed": (d["vocab"], W), "final.norm": (W,), "head": (d["vocab"], W)}
    for i, l in enumerate(d["layers"]):
        m, p = l["mixer"], f"l{i}."
        want[p + "norm1"] = (W,)
        if l["type"] == "retention":
            q = k = m["heads"] * m["dim"]
            v = g = m["heads"] * m["vdim"]
        else:
            q, k, v, g = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"], m["heads"] * m["vdim"]
            for n, c in (("q", q), ("k", k), ("v", v)):
                want[f"{p}mix.{n}.conv"] = (c, m["conv"])
        for n, c in (("q", q), ("k", k), ("v", v), ("g", g)):
            want[p + "mix." + n] = (c, W)
        want[p + "mix.o"] = (W, g)
        mlp = l["mlp"]
        if mlp is None:
            continue
        want[p + "norm2"] = (W,)
        r = mlp["router"]
        want[p + "mlp.router"] = (r["experts"] + r["identity"], W)
        want[p + "mlp.correction"] = (r["experts"] + r["identity"],)
        for e in range(r["experts"]):
            want[f"{p}mlp.e{e}.gate"] = want[f"{p}mlp.e{e}.up"] = (mlp["expert"]["ff"], W)
            want[f"{p}mlp.e{e}.down"] = (W, mlp["expert"]["ff"])
    assert {n: tuple(s.shape) for n, s in specs.items()} == want


def _bad(change):
    d = copy.deepcopy(ZEKA_A)
    change(d)
    return d


@pytest.mark.parametrize("change, word", [
    (lambda d: d["layers"][0].update(type="lstm"), "type"),
    (lambda d: d["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=26), "rot.dims"),
    (lambda d: d["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda d: d["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda d: d["layers"][1]["mixer"].update(conv=9), "conv"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(count=3), "groups"),
    (lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(keep=1, count=8), "groups"),
    (lambda d: d["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda d: d.pop("width"), "width"),
    (lambda d: d["norm"].pop("eps"), "eps"),
])
def test_refusals_name_the_key(change, word):
    from zlm_b200.config.spec import ConfigError
    from zlm_b200.registry import config_from_dict
    with pytest.raises(ConfigError) as e:
        config_from_dict(_bad(change))
    assert word in str(e.value)


def test_optional_keys_have_the_plain_meaning():
    """No groups: one group that is kept; no identity: none; no mask: every earlier token; no rot: no rotation."""
    from zlm_b200.registry import config_from_dict
    d = copy.deepcopy(ZEKA_A)
    d["layers"][1]["mlp"]["router"].pop("groups")
    d["layers"][1]["mlp"]["router"].pop("identity")
    d["layers"][0]["mixer"].pop("rot")
    cfg = config_from_dict(d)
    assert (cfg.layers[1].mlp.groups, cfg.layers[1].mlp.keep, cfg.layers[1].mlp.identity) == (1, 1, 0)
    assert cfg.layers[0].mixer.rot_dims == 0 and cfg.layers[4].mixer.window == 0
    spec = cfg.to_model_spec()
    assert spec.layers[0].mixer.params["position"] == {"kind": "none"}


@pytest.mark.parametrize("name", sorted(ZEKA))
def test_oracle_whole_equals_its_incremental_form(name):
    """The oracle run on a whole sequence, in two portions and token by token gives the same logits: its states,
    windows and convolution histories are carried the way the equations say."""
    cfg = ZEKA[name]
    W = {n: t.double() for n, t in make_tensors(cfg, 3).items()}
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg["vocab"], (150,), generator=g).tolist()
    whole = P.forward(cfg, W, ids)[0]
    a, _, caches, _ = P.forward(cfg, W, ids[:77])
    b = P.forward(cfg, W, ids[77:], caches, 77)[0]
    assert torch.allclose(torch.cat([a, b]), whole, atol=1e-9, rtol=1e-9)
    logits, _, caches, _ = P.forward(cfg, W, ids[:3])
    rows = [logits]
    for t in range(3, 20):
        logits, _, caches, _ = P.forward(cfg, W, [ids[t]], caches, t)
        rows.append(logits)
    assert torch.allclose(torch.cat(rows), whole[:20], atol=1e-9, rtol=1e-9)


def test_oracle_mechanisms_by_hand():
    """Each oracle function on inputs small enough to work out by hand."""
    F = torch.float64
    # short convolution: taps [1, 10, 100] on 1, 2, 3 with history (7, 8): y_0 = 7 + 80 + 100, y_1 = 8 + 10 + 200, ...
    y, hist = P.short_conv(torch.tensor([[1.0], [2.0], [3.0]], dtype=F), torch.tensor([[1.0, 10.0, 100.0]], dtype=F),
                           torch.tensor([[7.0], [8.0]], dtype=F))
    assert y.flatten().tolist() == [187.0, 218.0, 321.0] and hist.flatten().tolist() == [2.0, 3.0]
    # softmax with a sink: one key of score 0 gets weight 1 / (1 + 1)
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 1, "conv": 1, "scale": 0.0, "mask": {"size": 4}}
    Wm = {"q": torch.eye(2, dtype=F), "k": torch.eye(2, dtype=F), "v": torch.tensor([[1.0, 0.0]], dtype=F),
          "q.conv": torch.ones(2, 1, dtype=F), "k.conv": torch.ones(2, 1, dtype=F), "v.conv": torch.ones(1, 1, dtype=F),
          "g": torch.zeros(1, 2, dtype=F), "o": torch.ones(1, 1, dtype=F)}
    out, _ = P.conv_attention(torch.tensor([[4.0, 0.0]], dtype=F), Wm, m, 1e-6)
    assert abs(float(out) - 4.0 * 0.5 * 0.5) < 1e-12          # value 4, weight 1/2, gate sigmoid(0)
    # routing: groups of two; the group with the single best expert wins although another group's sum is larger
    r = {"experts": 4, "identity": 0, "top": 1, "scale": 3.0, "groups": {"count": 2, "keep": 1}}
    h = torch.tensor([[1.0]], dtype=F)
    idx, wgt, _ = P.route(h, torch.tensor([[0.0], [2.0], [1.5], [1.5]], dtype=F), torch.zeros(4, dtype=F), r)
    s = torch.softmax(torch.tensor([0.0, 2.0, 1.5, 1.5], dtype=F), 0)
    assert idx.tolist() == [[1]] and abs(float(wgt) - 3.0 * float(s[1])) < 1e-12
    # the correction moves the choice, not the weight
    idx, wgt, _ = P.route(h, torch.tensor([[0.0], [2.0], [1.5], [1.5]], dtype=F), torch.tensor([0.0, 0.0, 0.0, 1.0], dtype=F), r)
    assert idx.tolist() == [[3]] and abs(float(wgt) - 3.0 * float(s[3])) < 1e-12
    # retention: two tokens, decay 1/2, no rotation: o_1 = (k_0.q_1 / 2 + k_1.q_1) v
    m = {"heads": 1, "dim": 1, "vdim": 1, "decay": [0.5], "rot": {"base": 10.0, "dims": 0}}
    Wm = {"q": torch.ones(1, 1, dtype=F), "k": torch.ones(1, 1, dtype=F), "v": torch.ones(1, 1, dtype=F),
          "g": torch.ones(1, 1, dtype=F), "o": torch.ones(1, 1, dtype=F)}
    _, S = P.retention(torch.tensor([[1.0], [2.0]], dtype=F), Wm, m, 1e-6)
    assert abs(float(S) - (0.5 * 1.0 + 4.0)) < 1e-12
