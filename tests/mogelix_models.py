"""Small Mogelix models for the tests: configurations of the tests' own, weights drawn here (not by the product's
random-weights code), written as a model folder the engine loads."""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from tevovik_models import prompts, row_errors, write_model  # noqa: F401  (shared helpers of the tests)


def attention(heads=4, kv_heads=2, dim=16, vdim=24, size=20, pool=4, rot_dims: Optional[int] = 8, base=500.0, scaling=None,
              scale=None, kv_from: Optional[int] = None, mlp="dense") -> dict:
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else 2.0 / math.sqrt(dim),
             "mask": {"size": size, "pool": pool},
             "rot": {"dims": rot_dims or dim, "base": base,
                     "scaling": scaling or {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 64}}}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer, "mlp": _mlp(mlp)}


def mamba(heads=4, vdim=12, state=10, groups=2, conv=3, norm_groups=2, mlp="moe") -> dict:
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}, "mlp": _mlp(mlp)}


def _mlp(kind):
    if kind is None or isinstance(kind, dict):
        return kind
    if kind == "dense":
        return {"kind": "dense", "ff": 56}
    if kind == "moe":
        return {"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 5, "top": 2}, "shared": {"ff": 24}}
    raise ValueError(kind)


def moe(ff=16, experts=5, top=2, shared: Optional[int] = 24) -> dict:
    d = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        d["shared"] = {"ff": shared}
    return d


def config(layers: List[dict], width=48, vocab=101, eps=1e-5, alpha=1.7) -> dict:
    return {"architecture": "Mogelix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "postln_alpha": alpha, "layers": layers}


# Sizes chosen to differ from one another in everything a kernel could take for granted: head sizes that are no multiple of a
# vector or a warp, keys wider and narrower than values, one query head per key head and several, a rotation over part of the
# key and all of it, windows below / equal to / above the 64-token page, blocks of one position, blocks longer than the
# window, layers that read an earlier layer's keys with the same window and blocks and with others, one group of B and C and
# several, one convolution tap and five, one norm part and several, no feed-forward, experts without an always-on one, as
# many chosen experts as there are, a single expert.
CONFIGS: Dict[str, dict] = {
    "att": config([attention(mlp="dense")]),
    "att_edges": config([attention(heads=2, kv_heads=2, dim=24, vdim=8, size=64, pool=16, rot_dims=24, mlp=None),
                         attention(heads=6, kv_heads=2, dim=10, vdim=20, size=7, pool=1, rot_dims=4, base=37.0, mlp="dense"),
                         attention(heads=3, kv_heads=1, dim=12, vdim=12, size=97, pool=64, rot_dims=12, mlp=moe(24, 3, 3, None)),
                         attention(heads=2, kv_heads=1, dim=8, vdim=16, size=5, pool=12, rot_dims=2, mlp="dense")],
                        width=40, vocab=131, alpha=1.0),
    "att_shared": config([attention(heads=4, kv_heads=2, dim=16, vdim=16, size=30, pool=8),
                          attention(heads=4, kv_heads=2, dim=16, vdim=16, size=30, pool=8, kv_from=0, mlp="moe"),
                          attention(heads=2, kv_heads=2, dim=16, vdim=16, size=11, pool=3, kv_from=0, scale=0.7, mlp=None),
                          attention(heads=6, kv_heads=2, dim=16, vdim=16, size=70, pool=8, kv_from=0, mlp="dense")],
                         width=64, vocab=89, alpha=2.5),
    "ssm": config([mamba()]),
    "ssm_sizes": config([mamba(heads=3, vdim=7, state=5, groups=1, conv=1, norm_groups=1, mlp=None),
                         mamba(heads=6, vdim=8, state=40, groups=3, conv=5, norm_groups=4, mlp="dense"),
                         mamba(heads=2, vdim=36, state=33, groups=2, conv=2, norm_groups=3, mlp=moe(8, 1, 1, 8)),
                         mamba(heads=2, vdim=3, state=300, groups=1, conv=4, norm_groups=1, mlp=None)],
                        width=40, vocab=77, eps=3e-4, alpha=0.8),
    "mixed": config([attention(mlp="dense"), attention(kv_from=0, mlp="moe"), mamba(), attention(heads=2, kv_heads=1, dim=32, vdim=16,
                     size=33, pool=5, rot_dims=16, mlp="moe"), mamba(heads=2, vdim=16, state=16, groups=1, conv=4, norm_groups=1, mlp=None),
                     attention(heads=2, kv_heads=1, dim=32, vdim=16, size=33, pool=11, rot_dims=16, kv_from=3, mlp=moe(32, 7, 3, 16))],
                    width=64, vocab=157, alpha=2.0),
}


def draw_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """bfloat16 tensors with spreads that make every stage matter (flat logits hide faults)."""
    g = torch.Generator().manual_seed(seed)
    w = cfg["width"]

    def mat(rows, cols, gain=1.0):
        return (torch.randn(rows, cols, generator=g) * gain / math.sqrt(cols)).to(torch.bfloat16)

    def vec(n, mean, spread):
        return (mean + torch.randn(n, generator=g) * spread).to(torch.bfloat16)

    t = {"embed": torch.randn(cfg["vocab"], w, generator=g).to(torch.bfloat16), "head": mat(cfg["vocab"], w, 2.0),
         "final.norm": vec(w, 1.0, 0.2)}
    for i, ly in enumerate(cfg["layers"]):
        m, p = ly["mixer"], f"l{i}."
        t[p + "norm1"] = vec(w, 1.0, 0.2)
        t[p + "rg1"] = mat(w, w, 1.5)
        t[p + "rg1.b"] = vec(w, 0.5, 0.5)
        if ly["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            t[p + "mix.q"] = mat(H * d, w, 2.0)
            t[p + "mix.q.b"] = vec(H * d, 0.0, 0.3)
            if m.get("kv_from") is None:
                t[p + "mix.k"] = mat(G * d, w, 2.0)
                t[p + "mix.k.b"] = vec(G * d, 0.0, 0.3)
                t[p + "mix.v"] = mat(G * dv, w, 1.5)
                t[p + "mix.v.b"] = vec(G * dv, 0.0, 0.3)
            t[p + "mix.sink"] = vec(H, 0.5, 1.0)
            t[p + "mix.o"] = mat(w, H * dv, 1.0)
        else:
            Hh, dv, N, Gg = m["heads"], m["vdim"], m["state"], m["groups"]
            inner, ch = Hh * dv, Hh * dv + 2 * Gg * N
            t[p + "mix.in"] = mat(inner + ch + Hh, w, 1.5)
            t[p + "mix.conv"] = (torch.randn(ch, m["conv"], generator=g) * 0.6).to(torch.bfloat16)
            t[p + "mix.conv.b"] = vec(ch, 0.0, 0.2)
            t[p + "mix.dt_bias"] = vec(Hh, -1.0, 1.0)
            t[p + "mix.A_log"] = vec(Hh, -1.5, 1.0)       # decays from a few tokens to hundreds
            t[p + "mix.D"] = vec(Hh, 1.0, 0.3)
            t[p + "mix.norm"] = vec(inner, 1.0, 0.2)
            t[p + "mix.o"] = mat(w, inner, 1.0)
        f = ly["mlp"]
        if f is None:
            continue
        t[p + "norm2"] = vec(w, 1.0, 0.2)
        t[p + "rg2"] = mat(w, w, 1.5)
        t[p + "rg2.b"] = vec(w, 0.5, 0.5)
        if f["kind"] == "dense":
            t[p + "mlp.up"] = mat(f["ff"], w, 2.0)
            t[p + "mlp.down"] = mat(w, f["ff"], 1.0)
            t[p + "mlp.act"] = torch.tensor([0.9, 0.4, -0.3, 0.1]).to(torch.bfloat16)
        else:
            ff, E = f["expert"]["ff"], f["router"]["experts"]
            t[p + "mlp.router"] = mat(E, w, 3.0)
            t[p + "mlp.router.b"] = vec(E, 0.0, 0.5)
            for e in range(E):
                t[p + f"mlp.e{e}.up"] = mat(ff, w, 2.0)
                t[p + f"mlp.e{e}.down"] = mat(w, ff, 1.0)
            if f.get("shared") is not None:
                t[p + "mlp.shared.up"] = mat(f["shared"]["ff"], w, 2.0)
                t[p + "mlp.shared.down"] = mat(w, f["shared"]["ff"], 1.0)
                t[p + "mlp.shared.sg"] = mat(1, w, 2.0)
    return {k: v.contiguous() for k, v in t.items()}


def bf16_limits(cfg: dict, tensors: Dict[str, torch.Tensor], tokens: List[int]):
    """(typical row, nine rows in ten): three times what 16-bit rounding alone does to this model's logits, measured with
    the plain evaluation rounding what enters and leaves its matrix products, and no less than the fixed limits below."""
    import plain_mogelix as P

    e = row_errors(P.forward(cfg, tensors, tokens, rounding=torch.bfloat16), P.forward(cfg, tensors, tokens)).double()
    return max(BF16_TOL, 3.0 * float(e.median())), max(BF16_FAR, 3.0 * float(e.quantile(0.9)))


FP32_TOL = 5e-5     # sums in another order, device sin / exp, recurrences of hundreds of steps in 32-bit
BF16_TOL = 0.04     # what rounding at every stage does to a typical row of logits of these narrow models (32-bit is the sharp test)
BF16_FAR = 0.2      # ... and to nine rows in ten: rounding flips close calls of the routers, more often the more layers route


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str, limits=None) -> None:
    tol, far = limits or (BF16_TOL, BF16_FAR)
    assert torch.isfinite(got).all(), f"{what}: not finite"
    e = row_errors(got, want)
    if dtype == "float32":
        assert float(e.max()) <= FP32_TOL, f"{what}: row {int(e.argmax())} off by {float(e.max()):.3g}"
    elif e.numel() < 8:
        assert float(e.median()) <= far, f"{what}: median of {e.numel()} rows off by {float(e.median()):.3g}"
    else:
        q90 = float(e.double().quantile(0.9))
        assert float(e.median()) <= tol and q90 <= far, \
            f"{what}: of {e.numel()} rows the median is off by {float(e.median()):.3g}, the ninth decile by {q90:.3g}"
