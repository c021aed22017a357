"""Small Nuvilorn configurations and weights for the tests, and the oracle's inputs.

The configurations differ from each other in every size and option: head count (also 1), plain,
rotated and value sizes that all differ, rotation over a part of the rotated vector, several experts
per token, a layer without a shared expert, a layer without a feed-forward, layers that read an
earlier layer's latents (also not the nearest one), scales that make attention peaked.

Weights are drawn so that activations are of order one (matrices N(0, 1/in)): attention and routing
then depend visibly on single keys and experts, which N(0, 0.02) would hide."""
from __future__ import annotations

import json
import os
from typing import Dict, List, Sequence

import torch

import plain_nuvilorn as P


def _mixer(heads, dim, rot_dim, vdim, kv_rank, scale, base, dims, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
         "rot": {"base": base, "dims": dims}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _moe(ff, experts, top, shared=None):
    d = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


def _layer(mixer, mlp):
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


_MA = dict(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, scale=0.35, base=500.0, dims=8)
_MB = dict(heads=2, dim=8, rot_dim=16, vdim=16, kv_rank=24, scale=0.5, base=10000.0, dims=12)
NUVI_A = {
    "architecture": "Nuvilorn", "vocab": 160, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        _layer(_mixer(**_MA), {"kind": "dense", "ff": 96}),
        _layer(_mixer(**_MB), _moe(32, 5, 2, shared=48)),
        _layer(_mixer(**_MB, kv_from=1), _moe(24, 7, 3)),
        _layer(_mixer(**{**_MA, "heads": 1, "vdim": 8}, kv_from=0), None),
        _layer(_mixer(**{**_MB, "dim": 24, "scale": 0.3}), _moe(16, 4, 4, shared=8)),
    ],
}
# wider, one expert per token, rotation over the whole rotated part, more heads than 16
NUVI_B = {
    "architecture": "Nuvilorn", "vocab": 200, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        _layer(_mixer(18, 16, 16, 8, 72, 0.25, 20000.0, 16), _moe(40, 9, 1, shared=64)),
        _layer(_mixer(18, 16, 16, 8, 72, 0.25, 20000.0, 16, kv_from=0), {"kind": "dense", "ff": 72}),
        _layer(_mixer(4, 32, 32, 32, 136, 0.18, 100.0, 32), _moe(24, 6, 2, shared=16)),
    ],
}
NUVI = {"A": NUVI_A, "B": NUVI_B}


def make_tensors(cfg_dict, seed: int, peaked: bool = True) -> Dict[str, torch.Tensor]:
    """fp32 tensors by checkpoint name, every matrix rounded to bfloat16 values (so that both engine
    dtypes and the oracle compute on the same numbers).  ``peaked`` False halves the queries: a peaked
    softmax multiplies the rounding of bfloat16 queries and latents, which is no fault of a kernel."""
    from zlm_b200.parts.model import DecoderModel
    from zlm_b200.registry import config_from_dict
    specs = DecoderModel(config_from_dict(cfg_dict).to_model_spec()).param_specs()
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name in sorted(specs):
        shape = tuple(specs[name].shape)
        if len(shape) == 0:
            t = 1.0 + 0.1 * torch.randn((), generator=g)
        elif len(shape) == 1:
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / shape[1] ** 0.5
            if name.endswith(".router") or name.endswith(".sg"):
                t = t * 2.0
            if name.endswith(".mix.q") and not peaked:
                t = t * 0.4
        out[name] = t.to(torch.bfloat16).float()
    return out


def make_model(tmp_path, name: str, seed: int = 0, dtype: str = "float32"):
    """Writes the model to a folder; returns (folder, config mapping, float64 tensors for the oracle)."""
    from zlm_b200.weights import write_safetensors
    cfg = NUVI[name]
    tensors = make_tensors(cfg, seed, peaked=dtype == "float32")
    folder = os.path.join(str(tmp_path), f"nuvi_{name}_{seed}")
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), {n: t.to(torch.bfloat16) for n, t in tensors.items()})
    return folder, cfg, {n: t.double() for n, t in tensors.items()}


def oracle_logits(tensors, cfg, ids: Sequence[int]) -> torch.Tensor:
    return P.forward(tensors, cfg, ids).float()


# a router score's distance to the next expert's below which 8 bits of mantissa in the router's input may
# choose another expert (the scores' own rounding is a tenth of it)
CLOSE_CALL = 0.02


def oracle(tensors, cfg, ids: Sequence[int], dtype: str) -> "Oracle":
    margins: List[torch.Tensor] = []
    logits = P.forward(tensors, cfg, ids, margins=margins).float()
    safe = torch.ones(len(ids), dtype=torch.bool)
    if dtype == "bfloat16":
        for m in margins:
            safe &= m >= CLOSE_CALL
    return Oracle(logits, safe)


class Oracle:
    """The oracle's logits of one sequence, and which positions' experts are chosen by a clear margin in
    every routed layer (all of them in 32-bit): a bfloat16 run may choose otherwise at the others, and then
    computes another function there, so they are not compared."""

    def __init__(self, logits: torch.Tensor, safe: torch.Tensor):
        self.logits, self.safe = logits, safe

    def check(self, got: torch.Tensor, places, dtype: str, what: str = "") -> None:
        places = list(places)
        keep = [i for i, p in enumerate(places) if bool(self.safe[p])]
        assert len(keep) * 10 >= len(places) * 7 or len(places) < 4, f"{what}: too many close calls to test anything"
        if keep:
            assert_rows_close(got.float().cpu().reshape(len(places), -1)[keep], self.logits[[places[i] for i in keep]],
                              dtype, what)


# rows are compared as vectors: |got - want|_2 <= row * |want|_2.  bfloat16: activations are rounded to 8 bits
# of mantissa between kernels while the oracle keeps 64-bit ones, and relu^2 experts double a relative error;
# measured on these models the median row differs by 0.4 to 0.9 %, a rare one by 5 %.  So every row has a loose
# bound and the median of many rows a tight one; a wrong key, expert or position shows as tens of per cent
# (and to four digits in the 32-bit runs of the same kernels).
ROW_TOL = {"float32": 2e-4, "bfloat16": 8e-2}
MEDIAN_TOL = {"float32": 1e-4, "bfloat16": 2e-2}


def assert_rows_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = "", tol=None):
    got, want = got.float().cpu(), want.float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    if got.dim() == 1:
        got, want = got[None], want[None]
    rel = (got - want).norm(dim=-1) / want.norm(dim=-1).clamp_min(1e-9)
    tol = tol or ROW_TOL[dtype]
    assert bool((rel <= tol).all()), (f"{what}: row {int(rel.argmax())} differs by {rel.max():.3e} of its norm; "
                                      f"rows over {tol}: {(rel > tol).nonzero().flatten().tolist()[:12]}")
    if len(rel) >= 8:
        assert float(rel.median()) <= MEDIAN_TOL[dtype], f"{what}: the median row differs by {rel.median():.3e} of its norm"


def prompts(vocab: int, lengths: Sequence[int], seed: int) -> List[List[int]]:
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
