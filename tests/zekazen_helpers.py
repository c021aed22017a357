"""Small Zekazen configurations and weights for the tests, and the oracle's inputs.

The configurations differ from each other, and from layer to layer, in every size and option: head counts
(also 1, also more than 16 query heads on one kv head, also kv heads = heads), key and value sizes that differ
both ways and are no multiples of 16, convolutions of 1 to 4 taps, windows below a page, of exactly a page, a
little above it, and none, rotation over a part of a head and over all of it, decays near and far from 1,
routers with and without groups, with and without identity experts, one to four experts per token, a layer
without a feed-forward.

Weights are drawn so that activations are of order one (matrices N(0, 1/in)): attention and routing then
depend visibly on single keys and experts, which N(0, 0.02) would hide."""
from __future__ import annotations

import json
import os
from typing import Dict, List, Sequence

import torch

import plain_zekazen as P


def _ret(heads, dim, vdim, decay, base, dims):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "rot": {"base": base, "dims": dims}}


def _att(heads, kv_heads, dim, vdim, conv, scale, window=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    return m


def _moe(ff, experts, identity, top, scale, count, keep):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "identity": identity, "top": top, "scale": scale,
                       "groups": {"count": count, "keep": keep}}}


def _layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


ZEKA_A = {
    "architecture": "Zekazen", "vocab": 160, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        _layer("retention", _ret(3, 24, 40, [0.9, 0.97, 0.999], 500.0, 16), _moe(32, 6, 2, 2, 2.0, 4, 2)),
        _layer("attention", _att(4, 2, 24, 16, 4, 0.4, 70), _moe(24, 5, 0, 3, 1.0, 1, 1)),
        _layer("attention", _att(3, 3, 8, 40, 2, 0.8, 9), None),
        _layer("retention", _ret(1, 40, 8, [0.98], 10000.0, 40), _moe(16, 3, 1, 1, 0.5, 2, 1)),
        _layer("attention", _att(2, 1, 32, 32, 1, 0.3), _moe(40, 4, 4, 4, 1.25, 2, 2)),
    ],
}
# wider; 18 query heads on one kv head; values wider than 128; keys wider than 128; a window of exactly a page
ZEKA_B = {
    "architecture": "Zekazen", "vocab": 200, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        _layer("attention", _att(18, 1, 16, 16, 3, 0.5, 130), _moe(48, 12, 4, 4, 1.5, 4, 2)),
        _layer("retention", _ret(2, 64, 152, [0.75, 0.9995], 100.0, 32), _moe(24, 8, 0, 2, 1.0, 2, 1)),
        _layer("attention", _att(4, 2, 152, 8, 2, 0.07, 64), None),
    ],
}
ZEKA = {"A": ZEKA_A, "B": ZEKA_B}


def make_tensors(cfg_dict, seed: int) -> Dict[str, torch.Tensor]:
    """fp32 tensors by checkpoint name, every one rounded to bfloat16 values (so that both engine dtypes and
    the oracle compute on the same numbers)."""
    from zlm_b200.parts.model import DecoderModel
    from zlm_b200.registry import config_from_dict
    specs = DecoderModel(config_from_dict(cfg_dict).to_model_spec()).param_specs()
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name in sorted(specs):
        shape = tuple(specs[name].shape)
        if name.endswith(".correction"):
            t = 0.1 * torch.randn(shape, generator=g)
        elif len(shape) == 1:
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        elif name.endswith(".conv"):
            t = torch.randn(shape, generator=g) * 0.7
        else:
            t = torch.randn(shape, generator=g) / shape[1] ** 0.5
            if name.endswith(".router"):
                t = t * 8.0          # decisive routers: few choices hang on a close call
        out[name] = t.to(torch.bfloat16).float()
    return out


def write_model(tmp_path, cfg, tensors, tag: str):
    from zlm_b200.weights import write_safetensors
    folder = os.path.join(str(tmp_path), f"zeka_{tag}")
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), {n: t.to(torch.bfloat16) for n, t in tensors.items()})
    return folder


def make_model(tmp_path, name: str, seed: int = 0):
    """Writes the model to a folder; returns (folder, config mapping, float64 tensors for the oracle)."""
    cfg = ZEKA[name]
    tensors = make_tensors(cfg, seed)
    return write_model(tmp_path, cfg, tensors, f"{name}_{seed}"), cfg, {n: t.double() for n, t in tensors.items()}


# how far a bfloat16 run's choice scores may be from the oracle's: activations rounded to 8 bits of mantissa move
# a router's softmax scores by a few thousandths
CLOSE_CALL = 0.008


class Oracle:
    """The oracle's logits of one sequence, and which positions do not hang on a router's close call (all of them
    in 32-bit).  A bfloat16 run may choose another expert or group where two choice scores nearly tie; it then
    computes another function at that position, and, through windows and states, at later ones.  So the oracle runs
    twice more with every choice score pushed by up to CLOSE_CALL one way and the other; positions whose logits
    move, and positions with a close call of their own, are not compared.  Nor are positions where the design itself
    multiplies a rounding tenfold: a retention head's output is divided by its root mean square, and at the first
    positions it is one or two terms, (q.k) v, whose sign decides everything when q.k is near zero.  They are found by
    one more run on embeddings moved by a bfloat16 rounding (a relative 2^-8): where that moves the logits by 4 % and
    more, no bfloat16 run can be held to the oracle."""

    def __init__(self, tensors, cfg, ids: Sequence[int], dtype: str):
        logits, _, _, margin = P.forward(cfg, tensors, ids)
        self.logits = logits.float()
        self.safe = torch.ones(len(ids), dtype=torch.bool)
        if dtype != "float32":
            self.safe &= margin >= CLOSE_CALL          # the position's own choices; the tilted runs find whom they reach
            for tilt in (CLOSE_CALL, -CLOSE_CALL):
                other = P.forward(cfg, tensors, ids, tilt=tilt)[0]
                self.safe &= (other - logits).norm(dim=-1) <= 0.01 * logits.norm(dim=-1)
            g = torch.Generator().manual_seed(77)
            moved = dict(tensors)
            moved["embed"] = tensors["embed"] * (1.0 + 2.0 ** -8 * (2.0 * torch.rand(tensors["embed"].shape, generator=g,
                                                                                      dtype=torch.float64) - 1.0))
            other = P.forward(cfg, moved, ids)[0]
            self.safe &= (other - logits).norm(dim=-1) <= 0.04 * logits.norm(dim=-1)

    def check(self, got: torch.Tensor, places, dtype: str, what: str = "") -> None:
        places = list(places)
        keep = [i for i, p in enumerate(places) if bool(self.safe[p])]
        assert len(keep) * 10 >= len(places) * 3 or len(places) < 4, f"{what}: too many close calls to test anything"
        if keep:
            assert_rows_close(got.float().cpu().reshape(len(places), -1)[keep], self.logits[[places[i] for i in keep]],
                              dtype, what)


def oracle(tensors, cfg, ids, dtype) -> Oracle:
    return Oracle(tensors, cfg, ids, dtype)


# rows are compared as vectors: |got - want|_2 <= row * |want|_2.  bfloat16: activations are rounded to 8 bits
# of mantissa between kernels while the oracle keeps 64-bit ones; every row has a loose bound and the median
# of many rows a tight one.  A wrong key, expert, state or position shows as tens of per cent (and to four
# digits in the 32-bit runs of the same kernels).  In bfloat16 one row in fifty may pass the loose bound, up to
# OUTLIER_TOL: the design divides small sums by their root mean square (a retention head's output at the first
# positions, where it is one or two terms whose sign a rounding can turn), which multiplies a rounding at single
# positions and nowhere else.
ROW_TOL = {"float32": 2e-4, "bfloat16": 8e-2}
MEDIAN_TOL = {"float32": 1e-4, "bfloat16": 2.5e-2}
OUTLIER_TOL = 0.3


def assert_rows_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = "", tol=None):
    got, want = got.float().cpu(), want.float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    if got.dim() == 1:
        got, want = got[None], want[None]
    rel = (got - want).norm(dim=-1) / want.norm(dim=-1).clamp_min(1e-9)
    outliers = 0 if (dtype == "float32" or tol is not None) else max(1, len(rel) // 50) if len(rel) >= 8 else 0
    tol = tol or ROW_TOL[dtype]
    over = (rel > tol).nonzero().flatten().tolist()
    assert len(over) <= outliers and (not over or float(rel.max()) <= OUTLIER_TOL), (
        f"{what}: row {int(rel.argmax())} differs by {rel.max():.3e} of its norm; rows over {tol}: {over[:12]}")
    if len(rel) >= 8:
        assert float(rel.median()) <= MEDIAN_TOL[dtype], f"{what}: the median row differs by {rel.median():.3e} of its norm"


def prompts(vocab: int, lengths: Sequence[int], seed: int) -> List[List[int]]:
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


def greedy_generate(tensors, cfg, prompt: Sequence[int], n: int) -> List[int]:
    """The oracle's greedy continuation, token by token through its own caches."""
    logits, _, caches, _ = P.forward(cfg, tensors, prompt)
    out, at = [], len(prompt)
    for _ in range(n):
        tok = int(torch.argmax(logits[-1]))
        out.append(tok)
        logits, _, caches, _ = P.forward(cfg, tensors, [tok], caches, at)
        at += 1
    return out
