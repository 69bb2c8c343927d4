"""A plain, slow evaluation of the Mogelix decoder: one function per mechanism, float64 on the CPU, whole sequences at
once, recurrences token by token, no cache.  It shares no code with ``dryft_b200`` and takes its sizes and constants
from the same ``config.json`` dictionary the library reads; ``weights`` maps tensor names to tensors.

Notation: ``W`` matrices are ``[out, in]`` and applied as ``x @ W.T``; ``L`` is the number of tokens of the sequence;
positions count from 0.
"""

from __future__ import annotations

import math
from typing import Callable, Dict, List, Mapping, Optional

import torch

F = torch.float64
_ROUND: Optional[torch.dtype] = None      # set by ``forward(..., rounding=...)``: products read and leave values of this type


def rnd(x: torch.Tensor) -> torch.Tensor:
    return x if _ROUND is None else x.to(_ROUND).to(F)


def mm(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``h @ w.T``; with a rounding type set, of the rounded ``h`` and rounded itself (what a 16-bit product does)."""
    return rnd(rnd(h) @ w.T)


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """Every vector along the last dimension divided by its root mean square (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


# ----------------------------------------------------------------------------- rotation
def rotary_frequencies(rot: Mapping) -> torch.Tensor:
    """``f_i = base^(-2i/dims)``, then the wavelength-dependent scaling: short waves kept, long waves slowed by
    ``factor``, the band between them blended linearly in ``original / wavelength``."""
    dims = int(rot["dims"])
    i = torch.arange(dims // 2, dtype=F)
    f = torch.pow(torch.tensor(float(rot["base"]), dtype=F), -2.0 * i / dims)
    sc = rot.get("scaling")
    if sc is None:
        return f
    factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
    out = f.clone()
    for j in range(f.numel()):
        wave = 2.0 * math.pi / float(f[j])
        if wave < orig / high:
            continue
        if wave > orig / low:
            out[j] = f[j] / factor
        else:
            s = (orig / wave - low) / (high - low)
            out[j] = (1.0 - s) * f[j] / factor + s * f[j]
    return out


def rotate(x: torch.Tensor, pos: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """``x [L, heads, dim]``: of the first ``2 * len(freqs)`` dimensions of each head, dimension ``i`` turns together
    with dimension ``i + len(freqs)``; the rest pass unchanged."""
    half = freqs.numel()
    ang = pos.to(F)[:, None] * freqs[None, :]              # [L, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:2 * half]
    out = x.clone()
    out[..., :half] = u * c - v * s
    out[..., half:2 * half] = v * c + u * s
    return out


# ----------------------------------------------------------------------------- attention
def visible(i: int, size: int, pool: int):
    """What the query at position ``i`` sees: the token positions of its window, and the blocks of ``pool`` positions
    that lie wholly before the window."""
    toks = [j for j in range(i + 1) if i - j < size]
    blocks = [b for b in range((i + 1) // pool + 1) if b * pool + pool - 1 <= i - size]
    return toks, blocks


def pooled_window_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, sink: torch.Tensor, scale: float, size: int,
                            pool: int) -> torch.Tensor:
    """``q [L, H, d]``, ``k [L, G, d]``, ``v [L, G, dv]`` as a cache would hold them; ``sink [H]``.  Returns ``[L, H, dv]``."""
    L, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    nb = L // pool
    kb = rnd(k[: nb * pool].reshape(nb, pool, G, -1).mean(1)) if nb else k[:0]
    vb = rnd(v[: nb * pool].reshape(nb, pool, G, -1).mean(1)) if nb else v[:0]
    out = torch.zeros(L, H, v.shape[-1], dtype=F)
    for i in range(L):
        toks, blocks = visible(i, size, pool)
        for h in range(H):
            g = h // rep
            keys = torch.cat([kb[blocks, g], k[toks, g]], 0)
            vals = torch.cat([vb[blocks, g], v[toks, g]], 0)
            s = (keys @ q[i, h]) * scale
            m = torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            out[i, h] = (e[:, None] * vals).sum(0) / (e.sum() + torch.exp(sink[h] - m))
    return out


def attention_keys_values(h: torch.Tensor, p: Mapping, w: Mapping[str, torch.Tensor], pre: str, eps: float):
    """The keys (rotated, then divided by their root mean square) and values layer ``pre`` puts into its cache."""
    L = h.shape[0]
    G, d, dv = int(p["kv_heads"]), int(p["dim"]), int(p["vdim"])
    pos = torch.arange(L)
    k = (mm(h, w[pre + "k"]) + w[pre + "k.b"]).reshape(L, G, d)
    v = rnd(mm(h, w[pre + "v"]) + w[pre + "v.b"]).reshape(L, G, dv)
    k = rnd(rms_unit(rotate(k, pos, rotary_frequencies(p["rot"])), eps))
    return k, v


def attention_mixer(h: torch.Tensor, p: Mapping, w: Mapping[str, torch.Tensor], pre: str, eps: float, kv) -> torch.Tensor:
    """``kv``: the (keys, values) this layer reads -- its own or an earlier layer's."""
    L = h.shape[0]
    H, d = int(p["heads"]), int(p["dim"])
    q = (mm(h, w[pre + "q"]) + w[pre + "q.b"]).reshape(L, H, d)
    q = rnd(rms_unit(rotate(q, torch.arange(L), rotary_frequencies(p["rot"])), eps))
    k, v = kv
    o = pooled_window_attention(q, k, v, w[pre + "sink"], float(p["scale"]), int(p["mask"]["size"]), int(p["mask"]["pool"]))
    return mm(o.reshape(L, -1), w[pre + "o"])


# ----------------------------------------------------------------------------- state-space mixer
def causal_conv(x: torch.Tensor, cw: torch.Tensor, cb: torch.Tensor) -> torch.Tensor:
    """``x [L, C]``; ``cw [C, taps]`` whose last column multiplies the current token; zeros before the start."""
    L, C = x.shape
    taps = cw.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=F), x], 0)
    out = cb.expand(L, C).clone()
    for j in range(taps):
        out = out + pad[j:j + L] * cw[:, j]
    return out


def ssm_scan(x: torch.Tensor, dt: torch.Tensor, a: torch.Tensor, B: torch.Tensor, C: torch.Tensor, D: torch.Tensor) -> torch.Tensor:
    """``x [L, heads, dv]``, ``dt [L, heads]``, ``a [heads]`` (positive: the decay rate), ``B, C [L, groups, N]``, ``D [heads]``.
    ``S_t = exp(-a dt_t) S_(t-1) + dt_t B_t x_t^T``, ``y_t = S_t^T C_t + D x_t``, token by token."""
    L, Hh, dv = x.shape
    Gg, N = B.shape[1], B.shape[2]
    per = Hh // Gg
    y = torch.zeros(L, Hh, dv, dtype=F)
    S = torch.zeros(Hh, N, dv, dtype=F)
    for t in range(L):
        for hh in range(Hh):
            g = hh // per
            S[hh] = torch.exp(-a[hh] * dt[t, hh]) * S[hh] + dt[t, hh] * torch.outer(B[t, g], x[t, hh])
            y[t, hh] = S[hh].T @ C[t, g] + D[hh] * x[t, hh]
    return y


def mamba2_mixer(h: torch.Tensor, p: Mapping, w: Mapping[str, torch.Tensor], pre: str, eps: float) -> torch.Tensor:
    L = h.shape[0]
    Hh, dv, N, Gg = int(p["heads"]), int(p["vdim"]), int(p["state"]), int(p["groups"])
    inner = Hh * dv
    proj = rnd(h) @ w[pre + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * Gg * N], proj[:, 2 * inner + 2 * Gg * N:]
    xbc = silu(causal_conv(xbc, w[pre + "conv"], w[pre + "conv.b"]))
    x = xbc[:, :inner].reshape(L, Hh, dv)
    B = xbc[:, inner:inner + Gg * N].reshape(L, Gg, N)
    C = xbc[:, inner + Gg * N:].reshape(L, Gg, N)
    dt = torch.nn.functional.softplus(dt + w[pre + "dt_bias"], threshold=1e9)
    y = ssm_scan(x, dt, torch.exp(w[pre + "A_log"]), B, C, w[pre + "D"]).reshape(L, inner)
    y = y * silu(z)
    parts = int(p["norm_groups"])
    y = rms_unit(y.reshape(L, parts, inner // parts), eps).reshape(L, inner) * w[pre + "norm"]
    return mm(y, w[pre + "o"])


# ----------------------------------------------------------------------------- feed-forward
def poly_norm(z: torch.Tensor, coef: torch.Tensor, eps: float) -> torch.Tensor:
    """``a N(z) + b N(z^2) + c N(z^3) + e`` with ``N`` the division of a token's vector by its root mean square."""
    return coef[0] * rms_unit(z, eps) + coef[1] * rms_unit(z ** 2, eps) + coef[2] * rms_unit(z ** 3, eps) + coef[3]


def dense_ffn(h: torch.Tensor, w: Mapping[str, torch.Tensor], pre: str, eps: float) -> torch.Tensor:
    return mm(poly_norm(mm(h, w[pre + "up"]), w[pre + "act"], eps), w[pre + "down"])


def relu2_expert(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return mm(torch.relu(mm(h, up)) ** 2, down)


def route(h: torch.Tensor, wr: torch.Tensor, br: torch.Tensor, top: int):
    """Chosen experts ``[L, top]`` and their weights: a softmax over the chosen logits only."""
    z = rnd(h) @ wr.T + br
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, -1)


def moe_ffn(h: torch.Tensor, p: Mapping, w: Mapping[str, torch.Tensor], pre: str) -> torch.Tensor:
    E, top = int(p["router"]["experts"]), int(p["router"]["top"])
    idx, wt = route(h, w[pre + "router"], w[pre + "router.b"], top)
    out = torch.zeros(h.shape[0], w[pre + "e0.down"].shape[0], dtype=F)
    for e in range(E):
        ye = relu2_expert(h, w[pre + f"e{e}.up"], w[pre + f"e{e}.down"])
        gate = (wt * (idx == e)).sum(-1, keepdim=True)
        out = out + gate * ye
    if p.get("shared") is not None:
        ys = relu2_expert(h, w[pre + "shared.up"], w[pre + "shared.down"])
        out = out + torch.sigmoid(mm(h, w[pre + "shared.sg"])) * ys
    return out


# ----------------------------------------------------------------------------- the model
def forward(config: Mapping, weights: Mapping[str, torch.Tensor], tokens: List[int],
            tap: Optional[Callable[[int, torch.Tensor], None]] = None, rounding: Optional[torch.dtype] = None) -> torch.Tensor:
    """Logits ``[L, vocab]`` (float64) of one sequence.  ``tap(i, x)`` is called with the stream after layer ``i``.
    ``rounding=torch.bfloat16`` rounds what enters and leaves every matrix product and what a cache would hold (the
    stream, norms, scores, routers and recurrences stay exact): how far 16-bit arithmetic alone moves the logits."""
    global _ROUND
    _ROUND = rounding
    try:
        return _forward(config, weights, tokens, tap)
    finally:
        _ROUND = None


def _forward(config, weights, tokens, tap):
    w = {k: v.to(F) for k, v in weights.items() if v.is_floating_point()}
    eps = float(config["norm"]["eps"])
    alpha = float(config["postln_alpha"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    kept: Dict[int, tuple] = {}
    for i, layer in enumerate(config["layers"]):
        pre = f"l{i}."
        p = layer["mixer"]
        if layer["type"] == "attention":
            src = p.get("kv_from")
            if src is None:
                kept[i] = attention_keys_values(x, p, w, pre + "mix.", eps)
                src = i
            y = attention_mixer(x, p, w, pre + "mix.", eps, kept[src])
        elif layer["type"] == "mamba2":
            y = mamba2_mixer(x, p, w, pre + "mix.", eps)
        else:
            raise ValueError(layer["type"])
        y = y * torch.sigmoid(mm(x, w[pre + "rg1"]) + w[pre + "rg1.b"])
        x = rms_norm(alpha * x + y, w[pre + "norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            if mlp["kind"] == "dense":
                y = dense_ffn(x, w, pre + "mlp.", eps)
            elif mlp["kind"] == "moe":
                y = moe_ffn(x, mlp, w, pre + "mlp.")
            else:
                raise ValueError(mlp["kind"])
            y = y * torch.sigmoid(mm(x, w[pre + "rg2"]) + w[pre + "rg2.b"])
            x = rms_norm(alpha * x + y, w[pre + "norm2"], eps)
        if tap is not None:
            tap(i, x)
    return rnd(rms_norm(x, w["final.norm"], eps)) @ w["head"].T


def greedy(config: Mapping, weights: Mapping[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    """The best next token, ``n_new`` times, each from a whole evaluation of all tokens so far."""
    ids, out = list(prompt), []
    for _ in range(n_new):
        t = int(torch.argmax(forward(config, weights, ids)[-1]))
        out.append(t)
        ids.append(t)
    return out
