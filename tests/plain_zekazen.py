"""A plain, slow implementation of the Zekazen design in float64 on the CPU: the oracle of the tests.
One function per mechanism, written from the design's equations; it shares no code with the package.

Notation: h [T, width] is a part's input for one sequence whose tokens sit at positions 0 .. T-1;
weights are [out, in] and applied as x @ W.T.

  norm          y = x / sqrt(mean(x^2) + eps) * w
  retention     q, k = rot(W_q h), rot(W_k h) * dim^-1/2;  S_t = d_h S_(t-1) + k_t v_t^T;  o_t = S_t^T q_t;
                out = W_o (unit_norm(o) * silu(W_g h))
  conv attention  q, k, v = conv(W_q h), conv(W_k h), conv(W_v h);  q, k <- unit_norm;  s_ij = q_i . k_j * scale for
                0 <= i - j < window;  p_ij = exp(s_ij) / (1 + sum_j exp(s_ij));  out = W_o (p v * sigmoid(W_g h))
  experts       s = softmax(W_r h);  c = s + correction;  groups of neighbours, the best `keep` by their largest c;
                the `top` largest c inside them;  y = sum_e scale * s_e * expert_e(h), identity experts give h
"""
import math

import torch

F64 = torch.float64


def unit_norm(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return unit_norm(x, eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def rotate_half(x, pos, base, dims):
    """x [T, heads, dim]; the first ``dims`` coordinates of every head are turned, coordinate i with i + dims/2,
    by the angle pos * base^(-2i/dims); the rest pass."""
    if dims == 0:
        return x
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    a = pos.to(F64)[:, None, None] * f[None, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * torch.cos(a) - v * torch.sin(a), v * torch.cos(a) + u * torch.sin(a), x[..., dims:]], -1)


def retention(h, W, m, eps, state=None, start=0):
    """m: heads, dim, vdim, decay (a list per head), rot {base, dims}.  ``state`` [heads, dim, vdim] is what the
    tokens before ``start`` left (None: zeros).  Returns (output [T, width], new state)."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(start, start + T)
    base, dims = (m["rot"]["base"], m["rot"]["dims"]) if m.get("rot") else (1.0, 0)
    q = rotate_half((h @ W["q"].T).view(T, H, D), pos, base, dims)
    k = rotate_half((h @ W["k"].T).view(T, H, D), pos, base, dims) * D ** -0.5
    v = (h @ W["v"].T).view(T, H, V)
    S = torch.zeros(H, D, V, dtype=F64) if state is None else state.clone()
    decay = torch.tensor(m["decay"], dtype=F64)[:, None, None]
    o = torch.zeros(T, H, V, dtype=F64)
    for t in range(T):
        S = decay * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    y = unit_norm(o, eps).reshape(T, H * V) * silu(h @ W["g"].T)
    return y @ W["o"].T, S


def short_conv(u, w, history=None):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] * u_(t - taps + 1 + j); ``history`` [taps-1, C] are the
    values before the first token (None: zeros).  Returns (y, the last taps-1 values)."""
    taps = w.shape[1]
    C = u.shape[1]
    hist = torch.zeros(taps - 1, C, dtype=F64) if history is None else history
    full = torch.cat([hist, u], 0)
    T = u.shape[0]
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + w[:, j][None, :] * full[j:j + T]
    return y, full[full.shape[0] - (taps - 1):]


def conv_attention(h, W, m, eps, cache=None, start=0):
    """m: heads, kv_heads, dim, vdim, conv (taps), scale, mask {size}.  ``cache``: (k [S, G, dim], v [S, G, vdim],
    the three convolutions' histories) of the tokens before ``start``.  Returns (output, new cache)."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"]
    hist = (None, None, None) if cache is None else cache[2]
    q, hq = short_conv(h @ W["q"].T, W["q.conv"], hist[0])
    k, hk = short_conv(h @ W["k"].T, W["k.conv"], hist[1])
    v, hv = short_conv(h @ W["v"].T, W["v.conv"], hist[2])
    q = unit_norm(q.view(T, H, D), eps)
    k = unit_norm(k.view(T, G, D), eps)
    v = v.view(T, G, V)
    if cache is not None:
        k, v = torch.cat([cache[0], k], 0), torch.cat([cache[1], v], 0)
    o = torch.zeros(T, H, V, dtype=F64)
    window = m["mask"]["size"] if m.get("mask") else start + T          # no mask: every earlier token
    for t in range(T):
        i = start + t
        lo = max(0, i - window + 1)
        for hh in range(H):
            g = hh // (H // G)
            s = (k[lo:i + 1, g] @ q[t, hh]) * m["scale"]
            e = torch.exp(s)
            p = e / (1.0 + e.sum())
            o[t, hh] = p @ v[lo:i + 1, g]
    y = o.reshape(T, H * V) * torch.sigmoid(h @ W["g"].T)
    return y @ W["o"].T, (k, v, (hq, hk, hv))


def route(h, w_router, correction, r, tilt=None):
    """r: experts, identity, top, scale, groups {count, keep}.  Returns (indices [T, top], weights [T, top],
    the margin between the last chosen and the first refused choice score, per token).  ``tilt`` [T, n], if given,
    is added to the choice scores (not to the weights): a test's way of asking which outputs hang on close calls."""
    n = r["experts"] + r.get("identity", 0)
    s = torch.softmax(h @ w_router.T, -1)
    c = s + correction[None, :]
    if tilt is not None:
        c = c + tilt
    count, keep = (r["groups"]["count"], r["groups"]["keep"]) if r.get("groups") else (1, 1)
    size = n // count
    best = c.view(-1, count, size).max(-1).values
    kept = torch.zeros_like(best, dtype=torch.bool)
    order = torch.sort(best, dim=-1, descending=True, stable=True).indices[:, :keep]
    kept.scatter_(1, order, True)
    allowed = kept[:, :, None].expand(-1, -1, size).reshape(-1, n)
    c = torch.where(allowed, c, torch.full_like(c, -math.inf))
    srt = torch.sort(c, dim=-1, descending=True, stable=True)
    idx = srt.indices[:, :r["top"]]
    margin = srt.values[:, r["top"] - 1] - (srt.values[:, r["top"]] if n > r["top"] else -math.inf)
    # (the margin between groups matters too: the last kept and the first dropped group)
    gs = torch.sort(best, dim=-1, descending=True).values
    if keep < count:
        margin = torch.minimum(margin, gs[:, keep - 1] - gs[:, keep])
    return idx, torch.gather(s, 1, idx) * r.get("scale", 1.0), margin


def experts(h, W, f, tilt=None):
    """f: expert {ff}, router {...}.  W: router, correction, e<i>.gate / up / down."""
    r = f["router"]
    idx, wgt, margin = route(h, W["router"], W["correction"], r, tilt)
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(r["top"]):
            e = int(idx[t, j])
            if e >= r["experts"]:
                out = h[t]
            else:
                out = (silu(h[t] @ W[f"e{e}.gate"].T) * (h[t] @ W[f"e{e}.up"].T)) @ W[f"e{e}.down"].T
            y[t] = y[t] + wgt[t, j] * out
    return y, margin


def sub(W, prefix):
    return {k[len(prefix):]: v for k, v in W.items() if k.startswith(prefix)}


def forward(config, W, tokens, caches=None, start=0, tilt=0.0):
    """One sequence: the tokens at positions start .. ; ``caches`` is what an earlier call returned.  Returns
    (logits [T, vocab], the stream after every layer [layers, T, width], caches, smallest router margin per token).
    ``tilt``: every router's choice scores are moved by tilt * u, u uniform in [-1, 1] and the same for the same
    (layer, position, expert) whatever the sign and size of tilt."""
    eps = config["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    new, after = [], []
    margin = torch.full((x.shape[0],), math.inf, dtype=F64)
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = rms_norm(x, W[p + "norm1"], eps)
        old = None if caches is None else caches[i]
        if layer["type"] == "retention":
            y, c = retention(h, sub(W, p + "mix."), layer["mixer"], eps, old, start)
        else:
            y, c = conv_attention(h, sub(W, p + "mix."), layer["mixer"], eps, old, start)
        new.append(c)
        x = x + y
        if layer["mlp"] is not None:
            t = None
            if tilt:
                n = layer["mlp"]["router"]["experts"] + layer["mlp"]["router"].get("identity", 0)
                g = torch.Generator().manual_seed(1000 + i)
                u = torch.rand(start + x.shape[0], n, generator=g, dtype=F64) * 2 - 1
                t = tilt * u[start:]
            y, mg = experts(rms_norm(x, W[p + "norm2"], eps), sub(W, p + "mlp."), layer["mlp"], t)
            margin = torch.minimum(margin, mg)
            x = x + y
        after.append(x)
    logits = rms_norm(x, W["final.norm"], eps) @ W["head"].T
    return logits, torch.stack(after), new, margin
