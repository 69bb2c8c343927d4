"""Small Kerirax models for the tests: configurations of the tests' own, weights drawn here (not by the product's
random-weights code), written as a model folder the engine loads."""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from mogelix_models import FP32_TOL, assert_close  # noqa: F401  (the tests' common yardstick)
from tevovik_models import prompts, row_errors, write_model  # noqa: F401  (shared helpers of the tests)


def pair(heads=4, kv_heads=2, dim=16, vdim=24, rot_dims: Optional[int] = 8, base=500.0, factor: Optional[float] = 3.0, scale=None,
         inner=40, state=6, dt_rank=5, conv=3, left_scale=0.8, right_scale=1.3, mlp="dense") -> dict:
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else 3.0 / math.sqrt(dim)}
    if rot_dims:
        left["rot"] = {"dims": rot_dims, "base": base}
        if factor is not None:
            left["rot"]["scaling"] = {"factor": factor}
    return {"type": "parallel", "mixer": {"left": left, "left_scale": left_scale, "right_scale": right_scale,
                                          "right": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}}, "mlp": _mlp(mlp)}


def latent(heads=3, dim=12, rot_dim=6, vdim=10, q_rank=14, kv_rank=20, base=300.0, scale=None, mlp="moe") -> dict:
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale if scale is not None else 3.0 / math.sqrt(dim + rot_dim)}
    if rot_dim:
        m["rot"] = {"dims": rot_dim, "base": base}
    return {"type": "latent_attention", "mixer": m, "mlp": _mlp(mlp)}


def moe(ff=16, experts=5, top=2, limit: Optional[float] = 1.5) -> dict:
    ex = {"ff": ff}
    if limit is not None:
        ex["limit"] = limit
    return {"kind": "moe", "expert": ex, "router": {"experts": experts, "top": top}}


def _mlp(kind):
    if kind is None or isinstance(kind, dict):
        return kind
    if kind == "dense":
        return {"kind": "dense", "ff": 56}
    if kind == "moe":
        return moe()
    raise ValueError(kind)


def config(layers: List[dict], width=48, vocab=101, eps=1e-5, emb_scale: Optional[float] = 0.7, cap: Optional[float] = 12.0,
           loop: Optional[tuple] = None) -> dict:
    cfg = {"architecture": "Kerirax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if emb_scale is not None:
        cfg["embedding"] = {"scale": emb_scale}
    if cap is not None:
        cfg["logit_softcap"] = cap
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


# Sizes chosen to differ from one another in everything a kernel could take for granted: head sizes that are no multiple of a
# vector or a warp, keys wider and narrower than values, one query head per key head and several, a rotation over part of a
# head, all of it and none, with and without slowed frequencies, states of 1, 5, 40 and 300 numbers, one tap and five, step
# ranks that fit no vector, latents narrower and wider than a warp, no rotated key part, one expert, every expert chosen, no
# clamp, no feed-forward, no squashing of the logits, no embedding factor; a stretch of one layer and of several run once,
# twice and three times, from the first layer and from a later one, up to the last layer and short of it; and one model
# whose sizes take the tensor-core kernels (heads of 64, experts of 32, a width of 256).
CONFIGS: Dict[str, dict] = {
    "pair": config([pair(mlp="dense")]),
    "latent": config([latent(mlp="moe")], cap=None),
    "looped": config([pair(mlp="dense"), latent(mlp=moe(12, 4, 2)), pair(heads=2, kv_heads=1, dim=8, vdim=8, rot_dims=8, factor=None,
                      inner=24, state=9, dt_rank=4, conv=4, mlp="moe"), latent(heads=2, dim=8, rot_dim=4, vdim=16, q_rank=6, kv_rank=40, mlp=None)],
                     width=64, vocab=157, loop=(1, 3, 2)),
    "sizes": config([pair(heads=6, kv_heads=2, dim=10, vdim=20, rot_dims=4, base=37.0, factor=2.5, inner=37, state=5, dt_rank=3, conv=1,
                          left_scale=1.0, right_scale=1.0, mlp=moe(7, 1, 1, None)),
                     latent(heads=3, dim=12, rot_dim=0, vdim=7, q_rank=9, kv_rank=21, mlp="dense"),
                     pair(heads=2, kv_heads=2, dim=24, vdim=8, rot_dims=None, inner=48, state=40, dt_rank=7, conv=5, left_scale=0.3,
                          right_scale=2.0, mlp=moe(9, 3, 3, 0.8)),
                     pair(heads=3, kv_heads=1, dim=12, vdim=12, rot_dims=12, factor=None, inner=5, state=300, dt_rank=1, conv=2, mlp=None),
                     latent(heads=5, dim=6, rot_dim=10, vdim=9, q_rank=40, kv_rank=33, mlp=moe(5, 6, 2, 3.0))],
                    width=40, vocab=131, eps=3e-4, emb_scale=None, loop=(0, 3, 3)),
    "once": config([latent(mlp="dense"), pair(state=1, mlp="moe")], width=56, vocab=77, loop=(1, 2, 1)),
    "tc": config([pair(heads=4, kv_heads=2, dim=64, vdim=64, rot_dims=64, base=10000.0, factor=2.0, inner=128, state=16, dt_rank=16, conv=4,
                       mlp={"kind": "dense", "ff": 128}),
                  latent(heads=4, dim=32, rot_dim=32, vdim=32, q_rank=64, kv_rank=64, mlp=moe(32, 6, 2, 2.5))],
                 width=256, vocab=211, loop=(0, 2, 2)),
}


def draw_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """bfloat16 tensors with spreads that make every stage matter (flat scores and logits hide faults): scores spread over
    several units so that single keys, near and far, carry a row; sinks that take a visible share; decays from a few tokens
    to hundreds; router logits far enough apart that 16-bit rounding rarely flips a choice."""
    g = torch.Generator().manual_seed(seed)
    w = cfg["width"]

    def mat(rows, cols, gain=1.0):
        return (torch.randn(rows, cols, generator=g) * gain / math.sqrt(cols)).to(torch.bfloat16)

    def vec(n, mean, spread):
        return (mean + torch.randn(n, generator=g) * spread).to(torch.bfloat16)

    t = {"embed": torch.randn(cfg["vocab"], w, generator=g).to(torch.bfloat16), "head": mat(cfg["vocab"], w, 3.0),
         "final.norm": vec(w, 1.0, 0.2)}
    if cfg.get("loop") is not None:
        t["loop.in"] = (torch.cat([torch.eye(w), 0.5 * torch.eye(w)], dim=1) + torch.randn(w, 2 * w, generator=g) * 0.4 / math.sqrt(w)).to(torch.bfloat16)
        t["loop.step"] = (torch.randn(cfg["loop"]["times"], w, generator=g) * 0.5).to(torch.bfloat16)
    for i, ly in enumerate(cfg["layers"]):
        m, p = ly["mixer"], f"l{i}."
        t[p + "norm1"] = vec(w, 1.0, 0.2)
        if ly["type"] == "latent_attention":
            H, d, r, dv, qr, kr = m["heads"], m["dim"], m.get("rot_dim", 0), m["vdim"], m["q_rank"], m["kv_rank"]
            t[p + "mix.dq"] = mat(qr, w, 1.5)
            t[p + "mix.dq.norm"] = vec(qr, 1.0, 0.2)
            t[p + "mix.uq"] = mat(H * (d + r), qr, 2.0)
            t[p + "mix.dkv"] = mat(kr + r, w, 1.5)
            t[p + "mix.dkv.norm"] = vec(kr, 1.0, 0.2)
            t[p + "mix.uk"] = mat(H * d, kr, 2.0)
            t[p + "mix.uv"] = mat(H * dv, kr, 1.5)
            t[p + "mix.sink"] = vec(H, 1.0, 1.5)
            t[p + "mix.o"] = mat(w, H * dv, 1.0)
        else:
            a, s = m["left"], m["right"]
            H, G, d, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            t[p + "mix.left.q"] = mat(H * d, w, 2.0)
            t[p + "mix.left.k"] = mat(G * d, w, 2.0)
            t[p + "mix.left.v"] = mat(G * dv, w, 1.5)
            t[p + "mix.left.q.norm"] = vec(H * d, 1.3, 0.4)
            t[p + "mix.left.k.norm"] = vec(G * d, 1.3, 0.4)
            t[p + "mix.left.g"] = mat(H, w, 2.0)
            t[p + "mix.left.o"] = mat(w, H * dv, 1.0)
            inner, N, R, taps = s["inner"], s["state"], s["dt_rank"], s["conv"]
            t[p + "mix.right.in"] = mat(2 * inner, w, 1.5)
            t[p + "mix.right.conv"] = (torch.randn(inner, taps, generator=g) * 0.6).to(torch.bfloat16)
            t[p + "mix.right.conv.b"] = vec(inner, 0.0, 0.2)
            t[p + "mix.right.x"] = mat(R + 2 * N, inner, 1.5)
            t[p + "mix.right.dt"] = mat(inner, R, 1.0)
            t[p + "mix.right.dt.b"] = vec(inner, -2.0, 1.0)
            t[p + "mix.right.A_log"] = (-1.5 + torch.randn(inner, N, generator=g) * 1.5).to(torch.bfloat16)   # memories of a few tokens and of hundreds
            t[p + "mix.right.D"] = vec(inner, 1.0, 0.3)
            t[p + "mix.right.o"] = mat(w, inner, 1.0)
        f = ly["mlp"]
        if f is None:
            continue
        if f["kind"] == "dense":
            t[p + "mlp.gate"] = mat(f["ff"], w, 2.0)
            t[p + "mlp.up"] = mat(f["ff"], w, 2.0)
            t[p + "mlp.down"] = mat(w, f["ff"], 1.0)
        else:
            ff, E = f["expert"]["ff"], f["router"]["experts"]
            t[p + "mlp.router"] = mat(E, w, 4.0)
            for e in range(E):
                t[p + f"mlp.e{e}.gate"] = mat(ff, w, 2.5)      # values on both sides of the clamp
                t[p + f"mlp.e{e}.up"] = mat(ff, w, 2.5)
                t[p + f"mlp.e{e}.down"] = mat(w, ff, 1.0)
    return {k: v.contiguous() for k, v in t.items()}


BF16_TOL = 0.04     # what rounding at every stage does to a typical row of logits of these narrow models (32-bit is the sharp test)
BF16_FAR = 0.2      # ... and to nine rows in ten: rounding flips close calls of the routers


def bf16_limits(cfg: dict, tensors: Dict[str, torch.Tensor], tokens: List[int]):
    """(typical row, nine rows in ten): three times what 16-bit rounding alone does to this model's logits, measured with
    the plain evaluation rounding what enters and leaves its matrix products, and no less than the fixed limits above."""
    import plain_kerirax as P

    e = row_errors(P.forward(cfg, tensors, tokens, rounding=torch.bfloat16), P.forward(cfg, tensors, tokens)).double()
    return max(BF16_TOL, 3.0 * float(e.median())), max(BF16_FAR, 3.0 * float(e.quantile(0.9)))
