"""Nuvilorn without a GPU: the configuration (reading, refusing, writing back, lowering to parts and a
schedule), the checkpoint's tensor names, and the oracle's own invariants."""
import copy

import pytest
import torch

import plain_nuvilorn as P
from nuvilorn_helpers import NUVI, NUVI_A, make_tensors


def test_architecture_is_chosen_by_its_string_key():
    from zlm_b200 import NuvilornConfig
    from zlm_b200.registry import config_from_dict
    cfg = config_from_dict(NUVI_A)
    assert isinstance(cfg, NuvilornConfig)
    assert cfg.to_dict() == NUVI_A
    assert config_from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("name", sorted(NUVI))
def test_lowering_names_parts_and_tensors(name):
    from zlm_b200.parts.model import DecoderModel
    from zlm_b200.registry import config_from_dict
    d = NUVI[name]
    spec = config_from_dict(d).to_model_spec()
    assert [e.cache_of for e in spec.schedule] == [l["mixer"].get("kv_from") for l in d["layers"]]
    specs = DecoderModel(spec).param_specs()
    want = {"embed": (d["vocab"], d["width"]), "embed.norm": (), "final.norm": (), "head": (d["vocab"], d["width"])}
    for i, l in enumerate(d["layers"]):
        m, p = l["mixer"], f"l{i}."
        want[p + "norm1"] = ()
        want[p + "mix.q"] = (m["heads"] * (m["dim"] + m["rot_dim"]), d["width"])
        want[p + "mix.uk"] = (m["heads"] * m["dim"], m["kv_rank"])
        want[p + "mix.uv"] = (m["heads"] * m["vdim"], m["kv_rank"])
        want[p + "mix.o"] = (d["width"], m["heads"] * m["vdim"])
        if "kv_from" not in m:
            want[p + "mix.dkv"] = (m["kv_rank"] + m["rot_dim"], d["width"])
            want[p + "mix.dkv.norm"] = (m["kv_rank"],)
        mlp = l["mlp"]
        if mlp is None:
            continue
        want[p + "norm2"] = ()
        if mlp["kind"] == "dense":
            for n, s in (("gate", (mlp["ff"], d["width"])), ("up", (mlp["ff"], d["width"])), ("down", (d["width"], mlp["ff"]))):
                want[p + "mlp." + n] = s
        else:
            want[p + "mlp.router"] = (mlp["router"]["experts"], d["width"])
            for e in range(mlp["router"]["experts"]):
                want[f"{p}mlp.e{e}.up"] = (mlp["expert"]["ff"], d["width"])
                want[f"{p}mlp.e{e}.down"] = (d["width"], mlp["expert"]["ff"])
            if "shared" in mlp:
                want[p + "mlp.shared.up"] = (mlp["shared"]["ff"], d["width"])
                want[p + "mlp.shared.down"] = (d["width"], mlp["shared"]["ff"])
                want[p + "mlp.shared.sg"] = (1, d["width"])
    assert {n: tuple(s.shape) for n, s in specs.items()} == want


def _bad(change):
    d = copy.deepcopy(NUVI_A)
    change(d)
    return d


@pytest.mark.parametrize("change, word", [
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d["norm"].pop("eps"), "eps"),
    (lambda d: d["layers"][0].update(type="window_attention"), "type"),
    (lambda d: d["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda d: d["layers"][2]["mixer"].update(kv_from=2), "earlier"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=2), "latents of its own"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=1), "differs"),
    (lambda d: d["layers"][1]["mlp"]["router"].update(top=6), "top"),
    (lambda d: d["layers"][1]["mlp"].update(kind="glu"), "kind"),
    (lambda d: d.update(layers=[]), "layers"),
])
def test_refused_configurations(change, word):
    from zlm_b200 import ConfigError
    from zlm_b200.registry import config_from_dict
    with pytest.raises(ConfigError) as e:
        config_from_dict(_bad(change))
    assert word in str(e.value)


def test_oracle_is_causal_and_reads_the_named_layers_latents():
    t = {n: v.double() for n, v in make_tensors(NUVI_A, 1).items()}
    ids = [3, 9, 150, 7, 7, 21, 64, 5]
    full = P.forward(t, NUVI_A, ids)
    assert torch.allclose(P.forward(t, NUVI_A, ids[:5]), full[:5], atol=1e-12)
    # layer 3 reads layer 0's latents: changing layer 1's down-projection norm weight must not reach it
    # except through the stream; changing layer 0's must change what layer 3 attends to
    _, layers = P.forward(t, NUVI_A, ids, return_layers=True)
    t2 = dict(t)
    t2["l0.mix.dkv.norm"] = t["l0.mix.dkv.norm"] * 1.5
    _, layers2 = P.forward(t2, NUVI_A, ids, return_layers=True)
    assert not torch.allclose(layers[0], layers2[0])


def test_oracle_rotation_and_routing_by_hand():
    x = torch.tensor([[1.0, 0.0, 2.0, 0.0, 5.0, 6.0]], dtype=torch.float64)
    out = P.rotate_pairs(x, torch.tensor([2]), base=100.0, dims=4)
    a0, a1 = 2.0, 2.0 * 100.0 ** (-0.5)
    want = [torch.cos(torch.tensor(a0)), torch.sin(torch.tensor(a0)), 2 * torch.cos(torch.tensor(a1)),
            2 * torch.sin(torch.tensor(a1)), 5.0, 6.0]
    assert torch.allclose(out[0], torch.tensor([float(w) for w in want], dtype=torch.float64))
    idx, w = P.route(torch.tensor([[1.0, -1.0]], dtype=torch.float64),
                     torch.tensor([[1.0, 0.0], [0.0, 1.0], [3.0, 0.0]], dtype=torch.float64), 2)
    assert idx.tolist() == [[2, 0]]
    assert torch.allclose(w, torch.sigmoid(torch.tensor([[3.0, 1.0]], dtype=torch.float64)))
    # the weight scales an expert's input: relu^2 makes that the square of the weight on its output
    up, down = torch.eye(2, dtype=torch.float64), torch.eye(2, dtype=torch.float64)
    u = torch.tensor([2.0, -1.0], dtype=torch.float64)
    assert torch.allclose(P.relu2_expert(0.5 * u, up, down), 0.25 * P.relu2_expert(u, up, down))
