"""Plain, slow Nuvilorn forward: whole sequences, no cache, one function per mechanism.

The oracle of the Nuvilorn tests.  It shares no code with the ``zlm_b200`` package: it
takes the configuration as the plain mapping that config.json holds and a dict of tensors
by checkpoint name, and recomputes every position of a sequence from scratch.  Everything
runs in the dtype of the tensors it is given (float64 in the tests).

The design, in this file's notation (h: a layer's input row, W x: a matrix [out, in]
applied to a column):

  stream   x0 = snorm(E[token], g_embed);  x <- x + mix(snorm(x, g1));  x <- x + ff(snorm(x, g2));
           logits = W_head snorm(x, g_final)
  snorm    RMS norm with one gain for the whole row: x * g / sqrt(mean(x^2) + eps)
  mixer    q = W_q h, per head [nope | rope part];  [c_raw | kr_raw] = W_dkv h;
           c = vnorm(c_raw, w_dkv_norm) (gain per coordinate);  kr = rot(kr_raw, position),
           a rotated key slice that every head uses;  k_nope = W_uk c and v = W_uv c per head;
           score(i, j) = (q_nope_i . k_nope_j + rot(q_rope_i) . kr_j) * scale for j <= i, softmax,
           y = W_o [heads' sum_j p_ij v_j].  A layer with ``kv_from`` = j takes c and kr from
           layer j (as that layer made them) and has no W_dkv of its own.
  rot      pairs (2i, 2i + 1), i < dims/2, turned by position * base^(-2i/dims); the
           coordinates from ``dims`` on pass unchanged
  dense ff W_down (silu(W_gate h) * (W_up h))
  moe ff   s = sigmoid(W_router h);  the ``top`` largest s choose the experts;
           y = sum_e expert_e(s_e h) + sigmoid(W_sg h) * shared(h);
           expert(u) = W_down relu(W_up u)^2 (the weight scales the expert's input)
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple

import torch


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def scalar_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose weight is a single number."""
    return rms(x, eps) * gain.reshape(())


def vector_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm with a weight per coordinate."""
    return rms(x, eps) * weight


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [T, ..., D]: neighbouring coordinates (2i, 2i+1), i < dims/2, are turned by the angle
    position * base^(-2i/dims); coordinates dims.. are left alone."""
    T = x.shape[0]
    i = torch.arange(dims // 2, dtype=torch.float64)
    freq = (float(base) ** (-2.0 * i / dims)).to(x.dtype)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]                 # [T, dims/2]
    shape = [T] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def latent_of(h: torch.Tensor, w_dkv: torch.Tensor, w_norm: torch.Tensor, m: Mapping[str, Any], eps: float,
              positions: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """What a latent-attention layer keeps per token: the normed latent c [T, kv_rank] and the
    rotated shared key part [T, rot_dim]."""
    r = int(m["kv_rank"])
    d = h @ w_dkv.t()
    c = vector_norm(d[:, :r], w_norm, eps)
    kr = rotate_pairs(d[:, r:], positions, m["rot"]["base"], int(m["rot"]["dims"]))
    return c, kr


def latent_attention(h: torch.Tensor, t: Mapping[str, torch.Tensor], p: str, m: Mapping[str, Any],
                     positions: torch.Tensor, c: torch.Tensor, kr: torch.Tensor) -> torch.Tensor:
    """The mixer's output for the rows h [T, width], given the latents c and rotated key slices
    kr of the same T positions (its own or another layer's)."""
    T = h.shape[0]
    H, dn, dr, dv, r = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    q = (h @ t[p + "q"].t()).reshape(T, H, dn + dr)
    qn = q[..., :dn]
    qr = rotate_pairs(q[..., dn:], positions, m["rot"]["base"], int(m["rot"]["dims"]))
    kn = (c @ t[p + "uk"].t()).reshape(T, H, dn)
    v = (c @ t[p + "uv"].t()).reshape(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for i in range(T):
        for a in range(H):
            s = (kn[: i + 1, a] @ qn[i, a] + kr[: i + 1] @ qr[i, a]) * float(m["scale"])
            w = torch.softmax(s, dim=0)
            out[i, a] = w @ v[: i + 1, a]
    return out.reshape(T, H * dv) @ t[p + "o"].t()


def dense_ff(h: torch.Tensor, t: Mapping[str, torch.Tensor], p: str) -> torch.Tensor:
    g = h @ t[p + "gate"].t()
    return ((g * torch.sigmoid(g)) * (h @ t[p + "up"].t())) @ t[p + "down"].t()


def relu2_expert(u: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    a = torch.relu(u @ up.t())
    return (a * a) @ down.t()


def route(h: torch.Tensor, w_router: torch.Tensor, top: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """(chosen experts [T, top], their weights [T, top]): the largest sigmoid scores, as they are."""
    s = torch.sigmoid(h @ w_router.t())
    w, idx = torch.topk(s, top, dim=-1)
    return idx, w


def route_margin(h: torch.Tensor, w_router: torch.Tensor, top: int) -> torch.Tensor:
    """[T]: how far the last chosen expert's score lies above the best one not chosen (inf if all are chosen)."""
    s = torch.sigmoid(h @ w_router.t()).sort(dim=-1, descending=True).values
    if top >= s.shape[-1]:
        return torch.full(s.shape[:1], math.inf, dtype=s.dtype)
    return s[:, top - 1] - s[:, top]


def moe_ff(h: torch.Tensor, t: Mapping[str, torch.Tensor], p: str, mlp: Mapping[str, Any],
           margins: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    idx, w = route(h, t[p + "router"], int(mlp["router"]["top"]))
    if margins is not None:
        margins.append(route_margin(h, t[p + "router"], int(mlp["router"]["top"])))
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        for e, we in zip(idx[i].tolist(), w[i]):
            out[i] += relu2_expert(we * h[i], t[f"{p}e{e}.up"], t[f"{p}e{e}.down"])
    if mlp.get("shared"):
        gate = torch.sigmoid(h @ t[p + "shared.sg"].t())                 # [T, 1]
        out = out + gate * relu2_expert(h, t[p + "shared.up"], t[p + "shared.down"])
    return out


def forward(t: Mapping[str, torch.Tensor], cfg: Mapping[str, Any], ids: Sequence[int],
            return_layers: bool = False, margins: Optional[List[torch.Tensor]] = None):
    """Logits [T, vocab] of one whole sequence (and the stream after every layer).  ``margins`` collects,
    per routed layer, every position's ``route_margin``."""
    eps = float(cfg["norm"]["eps"])
    ids = torch.as_tensor(list(ids), dtype=torch.long)
    pos = torch.arange(len(ids))
    x = scalar_norm(t["embed"][ids], t["embed.norm"], eps)
    kept: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
    after: List[torch.Tensor] = []
    for i, layer in enumerate(cfg["layers"]):
        assert layer["type"] == "latent_attention"
        m, p = layer["mixer"], f"l{i}."
        h = scalar_norm(x, t[p + "norm1"], eps)
        if m.get("kv_from") is None:
            kept[i] = latent_of(h, t[p + "mix.dkv"], t[p + "mix.dkv.norm"], m, eps, pos)
            c, kr = kept[i]
        else:
            c, kr = kept[int(m["kv_from"])]
        x = x + latent_attention(h, t, p + "mix.", m, pos, c, kr)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = scalar_norm(x, t[p + "norm2"], eps)
            x = x + (dense_ff(h, t, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(h, t, p + "mlp.", mlp, margins))
        after.append(x)
    logits = scalar_norm(x, t["final.norm"], eps) @ t["head"].t()
    return (logits, torch.stack(after)) if return_layers else logits


def greedy_generate(t, cfg, prompt: Sequence[int], n: int) -> List[int]:
    ids, out = list(prompt), []
    for _ in range(n):
        nxt = int(forward(t, cfg, ids)[-1].argmax())
        out.append(nxt)
        ids.append(nxt)
    return out
