"""Position encodings a mixer can be given.

``rope``: rotate-half rotary embedding (``engine/dryft_qwen3/model.py:35-41,49-57``):
``inv_freq[j] = 1 / theta^(2j/R)`` for ``j = 0..R/2-1`` from ``arange(0, R, 2)`` int64 -> float32, angle
``pos * inv_freq[j]`` in 32-bit, cos/sin cast to the activation dtype, dims ``j`` and ``j + R/2``
rotated together.  ``R`` (``rotary_dim``) may be smaller than the head size.  The angles and their
cos/sin are evaluated on the device (``csrc/rope_kv.cu``) from the position of each token: inside the
fused kernels for a decode step, and once per step into a table that all layers with the same
``(theta, rotary_dim)`` share for a step of many tokens.  This part owns ``inv_freq``, computed on the
host with exactly the reference's expression so that the 32-bit products ``pos * inv_freq`` agree bit
for bit with a table built the reference's way.

``none``: no position encoding (``rotary_dim = 0``).
"""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from ..ops import kernels as K
from .base import Runtime, StepContext, register_position

TABLE_MIN_TOKENS = 64   # below this every warp evaluates its own angles


def scale_by_wavelength(freq: torch.Tensor, scaling: Mapping) -> torch.Tensor:
    """Rotary frequencies (float64) with long waves slowed: see ``Rope``."""
    import math

    factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    if not (factor > 0 and high > low and orig > 0):
        raise ValueError(f"rope scaling: factor and original must be positive and high above low, got {dict(scaling)}")
    wave = 2.0 * math.pi / freq
    s = ((orig / wave - low) / (high - low)).clamp(0.0, 1.0)
    blended = (1.0 - s) * freq / factor + s * freq
    return torch.where(wave < orig / high, freq, torch.where(wave > orig / low, freq / factor, blended))


@register_position("rope")
class Rope:
    """``params["layout"]``: ``"half"`` (dims ``j`` and ``j + R/2`` turn together; the default) or ``"interleaved"`` (dims
    ``2j`` and ``2j + 1``); the mixers whose kernels take both read ``interleaved``.  ``params["freq"]``: ``"float32"``
    (the reference's expression, evaluated in 32-bit; the default) or ``"rounded_once"`` (``theta^(-2j/R)`` evaluated in
    64-bit and rounded to 32-bit once; what that rounding drops is kept as ``inv_freq_lo`` for kernels that take the pair).
    ``params["scaling"]`` (needs ``freq="rounded_once"``): ``{"factor": s}`` alone divides every frequency by ``s`` (linear
    scaling); otherwise a mapping ``factor, low, high, original`` that slows long waves: with
    the wavelength ``l = 2 pi / f``, ``f`` stays where ``l < original / high``, becomes ``f / factor`` where ``l > original /
    low``, and in between ``(1 - s) f / factor + s f`` with ``s = (original / l - low) / (high - low)``."""

    def __init__(self, params: Mapping, head_dim: int, rt: Runtime):
        self.rotary_dim = int(params.get("rotary_dim", head_dim))
        self.theta = float(params["theta"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2 or self.rotary_dim > head_dim:
            raise ValueError(f"rope: rotary_dim must be even and in (0, head_dim={head_dim}], got {self.rotary_dim}")
        layout = params.get("layout", "half")
        if layout not in ("half", "interleaved"):
            raise ValueError(f"rope: layout must be 'half' or 'interleaved', got {layout!r}")
        self.interleaved = layout == "interleaved"
        r = self.rotary_dim
        self.inv_freq_lo: Optional[torch.Tensor] = None
        if params.get("freq", "float32") == "rounded_once":
            exact = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -torch.arange(0, r, 2, dtype=torch.float64) / r)
            if params.get("scaling") is not None:
                sc = params["scaling"]
                if set(sc) == {"factor"}:      # linear scaling: every frequency divided by the same number
                    if not float(sc["factor"]) > 0:
                        raise ValueError(f"rope scaling: factor must be positive, got {dict(sc)}")
                    exact = exact / float(sc["factor"])
                else:
                    exact = scale_by_wavelength(exact, sc)
            inv_freq = exact.to(torch.float32)
            self.inv_freq_lo = (exact - inv_freq.to(torch.float64)).to(torch.float32).to(rt.device)
        else:
            if params.get("scaling") is not None:
                raise ValueError("rope: frequency scaling is evaluated in 64-bit; ask for freq='rounded_once' with it")
            inv_freq = 1.0 / (self.theta ** (torch.arange(0, r, 2, dtype=torch.int64).to(torch.float32) / r))
        self.inv_freq: Optional[torch.Tensor] = inv_freq.to(rt.device)
        self.dtype = rt.dtype

    def table(self, ctx: StepContext) -> Optional[torch.Tensor]:
        """The step's cos / sin table, made by the first layer that asks and kept in the step's context."""
        if ctx.decode or ctx.n_tokens < TABLE_MIN_TOKENS:
            return None
        key = ("rope_table", self.theta, self.rotary_dim)
        table = ctx.extras.get(key)
        if table is None:
            table = K.rope_table(ctx.tok_pos, self.inv_freq, ctx.n_tokens, self.dtype)
            ctx.extras[key] = table
        return table


@register_position("none")
class NoPosition:
    def __init__(self, params: Mapping, head_dim: int, rt: Runtime):
        self.rotary_dim = 0
        self.inv_freq = None
        self.inv_freq_lo = None
        self.interleaved = False

    def table(self, ctx: StepContext) -> None:
        return None
