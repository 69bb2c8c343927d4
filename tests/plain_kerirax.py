"""A plain, slow evaluation of the Kerirax decoder: one function per mechanism, float64 on the CPU, whole sequences at
once, the recurrence token by token, no cache.  It shares no code with ``dryft_b200`` and takes its sizes and constants
from the same ``config.json`` dictionary the library reads; ``weights`` maps tensor names to tensors.

Notation: ``W`` matrices are ``[out, in]`` and applied as ``x @ W.T``; ``L`` is the number of tokens of the sequence;
positions count from 0.

The design in short.  One norm per layer, read by the mixer and the feed-forward alike, whose results join the stream
together: ``x <- x + mixer(n) + ff(n)`` with ``n = rmsnorm(x)``.  A stretch of layers runs several times in a row with
the same weights; before every pass the stream is mixed with the embedding's output by a ``[W, 2W]`` matrix and a vector
of the pass is added.  Mixers: attention over low-rank latents with a sink in the softmax; and two mixers side by side
-- grouped-query attention (norm over the whole query / key projection, interleaved rotation with slowed frequencies, a
sigmoid gate per head) and a selective scan with one decay per (channel, state) -- whose results are added with fixed
factors.  Feed-forwards: a gated dense one, and routed experts with sigmoid scores that weight the expert's INPUT.
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


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


# ----------------------------------------------------------------------------- rotation
def rotary_frequencies(rot: Mapping) -> torch.Tensor:
    """``f_i = base^(-2i/dims)``, every one divided by ``scaling.factor`` when there is one."""
    dims = int(rot["dims"])
    f = torch.pow(torch.tensor(float(rot["base"]), dtype=F), -2.0 * torch.arange(dims // 2, dtype=F) / dims)
    sc = rot.get("scaling")
    return f / float(sc["factor"]) if sc is not None else f


def rotate_pairs(v: torch.Tensor, pos: torch.Tensor, rot: Optional[Mapping]) -> torch.Tensor:
    """``v [L, ..., n]``: dims ``2i`` and ``2i + 1`` of the first ``rot.dims`` turn by ``pos * f_i``; the rest stay."""
    if rot is None:
        return v
    dims = int(rot["dims"])
    ang = pos.to(F)[:, None] * rotary_frequencies(rot)[None, :]            # [L, dims/2]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [dims // 2]
    c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out = v.clone()
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# ----------------------------------------------------------------------------- softmax attention, one head at a time
def causal_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                             sink: Optional[float] = None) -> torch.Tensor:
    """``q [L, d]``, ``k [L, d]``, ``v [L, dv]`` of one head: position i sees every j <= i; with a ``sink`` the denominator
    also holds ``exp(sink)`` (no key, no value, not scaled, once)."""
    L = q.shape[0]
    s = (q @ k.T) * scale
    s = s.masked_fill(torch.ones(L, L, dtype=torch.bool).triu(1), -math.inf)
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.clamp(m, min=float(sink))
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(torch.tensor(float(sink), dtype=F) - m)
    return rnd(e / den) @ rnd(v) if _ROUND is not None else (e / den) @ v


# ----------------------------------------------------------------------------- mixer: attention over latents
def latent_attention_mixer(h: torch.Tensor, p: Mapping, w: Mapping[str, torch.Tensor], pre: str, eps: float) -> torch.Tensor:
    L = h.shape[0]
    H, d, r, dv, kr = int(p["heads"]), int(p["dim"]), int(p["rot_dim"]), int(p["vdim"]), int(p["kv_rank"])
    pos = torch.arange(L)
    rot = p.get("rot") if r else None
    cq = rnd(rms_norm(mm(h, w[pre + "dq"]), w[pre + "dq.norm"], eps))
    q = mm(cq, w[pre + "uq"]).view(L, H, d + r)
    down = mm(h, w[pre + "dkv"])
    c = rnd(rms_norm(down[:, :kr], w[pre + "dkv.norm"], eps))
    k_rot = rnd(rotate_pairs(down[:, kr:kr + r], pos, rot))                # one rotated key part for all heads
    k_plain = mm(c, w[pre + "uk"]).view(L, H, d)
    v = mm(c, w[pre + "uv"]).view(L, H, dv)
    q_rot = rotate_pairs(q[:, :, d:], pos, rot)
    out = torch.empty(L, H, dv, dtype=F)
    for hd in range(H):
        qh = torch.cat([q[:, hd, :d], q_rot[:, hd]], dim=-1)
        kh = torch.cat([k_plain[:, hd], k_rot], dim=-1)
        out[:, hd] = causal_softmax_attention(qh, kh, v[:, hd], float(p["scale"]), float(w[pre + "sink"][hd]))
    return mm(out.reshape(L, H * dv), w[pre + "o"])


# ----------------------------------------------------------------------------- mixer: grouped-query attention with a gate
def gated_attention_mixer(h: torch.Tensor, p: Mapping, w: Mapping[str, torch.Tensor], pre: str, eps: float) -> torch.Tensor:
    L = h.shape[0]
    H, G, d, dv = int(p["heads"]), int(p["kv_heads"]), int(p["dim"]), int(p["vdim"])
    pos = torch.arange(L)
    # the norm runs over the whole projection (all heads' rows at once), before the rotation
    q = rms_norm(mm(h, w[pre + "q"]), w[pre + "q.norm"], eps).view(L, H, d)
    k = rms_norm(mm(h, w[pre + "k"]), w[pre + "k.norm"], eps).view(L, G, d)
    v = mm(h, w[pre + "v"]).view(L, G, dv)
    q, k = rotate_pairs(q, pos, p.get("rot")), rnd(rotate_pairs(k, pos, p.get("rot")))
    gate = torch.sigmoid(mm(h, w[pre + "g"]))                              # [L, H]
    out = torch.empty(L, H, dv, dtype=F)
    for hd in range(H):
        g = hd // (H // G)
        out[:, hd] = causal_softmax_attention(q[:, hd], k[:, g], v[:, g], float(p["scale"])) * gate[:, hd:hd + 1]
    return mm(out.reshape(L, H * dv), w[pre + "o"])


# ----------------------------------------------------------------------------- mixer: selective scan
def causal_conv(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """``x [L, C]``, ``weight [C, taps]``: the last column multiplies the current token, zeros before the start."""
    L, taps = x.shape[0], weight.shape[1]
    out = bias.expand(L, -1).clone()
    for j in range(taps):
        back = taps - 1 - j
        if back < L:
            out[back:] += x[:L - back] * weight[:, j]
    return out


def selective_scan_mixer(h: torch.Tensor, p: Mapping, w: Mapping[str, torch.Tensor], pre: str) -> torch.Tensor:
    L = h.shape[0]
    inner, N, R = int(p["inner"]), int(p["state"]), int(p["dt_rank"])
    xz = mm(h, w[pre + "in"])
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(causal_conv(x, w[pre + "conv"], w[pre + "conv.b"]))
    low = mm(x, w[pre + "x"])                                            # [L, R | N | N]
    dt = softplus(low[:, :R] @ w[pre + "dt"].T + w[pre + "dt.b"])           # [L, inner]
    B, C = low[:, R:R + N], low[:, R + N:R + 2 * N]
    A = -torch.exp(w[pre + "A_log"])                                        # [inner, N]
    S = torch.zeros(inner, N, dtype=F)
    y = torch.empty(L, inner, dtype=F)
    for t in range(L):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + w[pre + "D"] * x[t]
    return mm(y * silu(z), w[pre + "o"])


def side_by_side_mixer(h, p, w, pre, eps):
    left = gated_attention_mixer(h, p["left"], w, pre + "left.", eps)
    right = selective_scan_mixer(h, p["right"], w, pre + "right.")
    return float(p["left_scale"]) * left + float(p["right_scale"]) * right


# ----------------------------------------------------------------------------- feed-forwards
def dense_ffn(h: torch.Tensor, w: Mapping[str, torch.Tensor], pre: str) -> torch.Tensor:
    return mm(silu(mm(h, w[pre + "gate"])) * mm(h, w[pre + "up"]), w[pre + "down"])


def router_choice(h: torch.Tensor, mlp: Mapping, w: Mapping[str, torch.Tensor], pre: str):
    """Sigmoid scores; the ``top`` largest name a token's experts (ties to the lower index); the weights are those scores."""
    s = torch.sigmoid(rnd(h) @ w[pre + "router"].T)
    top = int(mlp["router"]["top"])
    vals, idx = torch.sort(s, dim=-1, descending=True, stable=True)
    return idx[:, :top], vals[:, :top]


def expert(h: torch.Tensor, w: Mapping[str, torch.Tensor], pre: str, limit: float) -> torch.Tensor:
    g = torch.clamp(mm(h, w[pre + "gate"]), max=limit)
    u = torch.clamp(mm(h, w[pre + "up"]), min=-limit, max=limit)
    return mm(g * torch.sigmoid(1.702 * g) * (u + 1.0), w[pre + "down"])


def moe_ffn(h: torch.Tensor, mlp: Mapping, w: Mapping[str, torch.Tensor], pre: str) -> torch.Tensor:
    idx, wts = router_choice(h, mlp, w, pre)
    limit = float(mlp["expert"]["limit"]) if mlp["expert"].get("limit") is not None else math.inf
    out = torch.zeros(h.shape[0], w[pre + "e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for k in range(idx.shape[1]):
            e = int(idx[t, k])
            out[t] += expert((wts[t, k] * h[t])[None, :], w, f"{pre}e{e}.", limit)[0]      # the weight scales the input
    return out


# ----------------------------------------------------------------------------- the model
def run_order(config: Mapping) -> List[tuple]:
    """``(layer, pass or None, first of its pass)`` in the order the layers run."""
    n = len(config["layers"])
    loop = config.get("loop")
    if loop is None:
        return [(i, None, False) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, None, False) for i in range(start)]
    for t in range(times):
        order += [(i, t, i == start) for i in range(start, stop)]
    return order + [(i, None, False) for i in range(stop, n)]


def forward(config: Mapping, weights: Mapping[str, torch.Tensor], tokens: List[int],
            tap: Optional[Callable[[int, torch.Tensor], None]] = None, rounding: Optional[torch.dtype] = None) -> torch.Tensor:
    """Logits ``[L, vocab]`` of one sequence.  ``tap(run, x)`` sees the stream after every layer run."""
    global _ROUND
    _ROUND = rounding
    try:
        return _forward(config, weights, tokens, tap)
    finally:
        _ROUND = None


def _forward(config, weights, tokens, tap):
    w = {k: v.to(F) for k, v in weights.items() if v.is_floating_point()}
    eps = float(config["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)] * float((config.get("embedding") or {}).get("scale", 1.0))
    x0 = x
    for run, (i, t, first) in enumerate(run_order(config)):
        layer, pre = config["layers"][i], f"l{i}."
        if first:
            x = mm(torch.cat([x, x0], dim=-1), w["loop.in"]) + w["loop.step"][t]
        n = rms_norm(x, w[pre + "norm1"], eps)
        if layer["type"] == "latent_attention":
            y = latent_attention_mixer(n, layer["mixer"], w, pre + "mix.", eps)
        elif layer["type"] == "parallel":
            y = side_by_side_mixer(n, layer["mixer"], w, pre + "mix.", eps)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp is not None:
            if mlp["kind"] == "dense":
                y = y + dense_ffn(n, w, pre + "mlp.")
            elif mlp["kind"] == "moe":
                y = y + moe_ffn(n, mlp, w, pre + "mlp.")
            else:
                raise ValueError(mlp["kind"])
        x = x + y
        if tap is not None:
            tap(run, x)
    logits = rnd(rms_norm(x, w["final.norm"], eps)) @ w["head"].T
    cap = config.get("logit_softcap")
    return logits if cap is None else float(cap) * torch.tanh(logits / float(cap))


def greedy(config: Mapping, weights: Mapping[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    """The best next token, ``n_new`` times, each from a whole evaluation of all tokens so far."""
    ids, out = list(prompt), []
    for _ in range(n_new):
        t = int(torch.argmax(forward(config, weights, ids)[-1]))
        out.append(t)
        ids.append(t)
    return out
