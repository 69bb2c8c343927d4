"""RMSNorm: ``w * cast(x32 * rsqrt(mean(x32^2) + eps))`` — the weight multiplies after the cast
back to the activation dtype, and ``(1 + w)`` is not used (``engine/dryft_qwen3/model.py:28-32``;
``kernels/rmsnorm.py:3-6,36-39``).  Its weight is kept in 32-bit on the device (an exact widening of
a bfloat16 tensor) so one kernel serves both precisions.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..ops import kernels as K
from .base import Runtime, TensorInfo, register_norm


@register_norm("rmsnorm")
class RMSNorm:
    """``params["name"]`` is the weight's tensor name behind the prefix (default ``weight``)."""

    @staticmethod
    def tensors(params: Mapping, prefix: str) -> Dict[str, TensorInfo]:
        return {prefix + params.get("name", "weight"): TensorInfo((params["size"],), "vector")}

    def __init__(self, params: Mapping, prefix: str, weights, rt: Runtime):
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.rt = rt
        self.weight = weights.load(prefix + params.get("name", "weight"), "vector")  # float32 [size]

    def rms_params(self):
        """This norm is ``weight * cast(x32 * rsqrt(mean(x32^2) + eps))``: products may fold it into themselves."""
        return self.weight, self.eps

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None) -> torch.Tensor:
        n = n_rows if n_rows is not None else (rows.numel() if rows is not None else x.shape[0])
        out = torch.empty((n, self.size), dtype=x.dtype, device=x.device)
        K.rmsnorm(x, self.weight, self.eps, out, rows=rows)
        return out

    def add_forward(self, x: torch.Tensor, delta: torch.Tensor, rows: Optional[torch.Tensor] = None,
                    n_rows: Optional[int] = None) -> torch.Tensor:
        """``x += delta`` (32-bit sum, rounded once) and the norm of the sum.  With ``rows`` only those
        rows are summed and normed, and ``x`` is left as it is."""
        n = n_rows if n_rows is not None else (rows.numel() if rows is not None else x.shape[0])
        out = torch.empty((n, self.size), dtype=x.dtype, device=x.device)
        K.rmsnorm(x, self.weight, self.eps, out, delta=delta, rows=rows, x_out=None if rows is not None else x)
        return out


@register_norm("rmsnorm_offset")
class OffsetRMSNorm:
    """``x / sqrt(mean(x^2) + eps) * (offset + w)``, all of it in 32-bit and rounded once: the norm whose stored weight is a
    deviation from one (``offset = 1``).  Its input may be a 32-bit stream while the output has the activation type.
    It does not offer ``rms_params`` (its arithmetic is not the one the decode products fold into themselves).
    ``add_into`` is the form a layer with the norm on the sublayer's *output* uses: ``x32 += norm(y)``; ``sum_norm`` the
    form of a layer whose norm follows the sum: ``x32 <- norm(keep * x32 + gate * y)``.
    ``params["name"]`` is the weight's tensor name behind the prefix (default ``weight``)."""

    @staticmethod
    def tensors(params: Mapping, prefix: str) -> Dict[str, TensorInfo]:
        # random weights are drawn around 1 - offset, so that the factor (offset + w) is around 1
        return {prefix + params.get("name", "weight"): TensorInfo((params["size"],), "vector", False, 1.0 - float(params.get("offset", 1.0)))}

    def __init__(self, params: Mapping, prefix: str, weights, rt: Runtime):
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.offset = float(params.get("offset", 1.0))
        self.rt = rt
        self.weight = weights.load(prefix + params.get("name", "weight"), "vector")  # float32 [size]
        self._factor: Optional[torch.Tensor] = None   # offset + weight, formed when ``sum_norm`` first asks

    def plain_params(self):
        """``(factor, eps)``: this norm is ``x / sqrt(mean(x^2) + eps) * factor`` in 32-bit, rounded once -- what a kernel that
        has the row in hand anyway (the sum that forms the stream) may compute on the side."""
        if self._factor is None:
            self._factor = self.weight if self.offset == 0.0 else (self.weight + self.offset)
        return self._factor, self.eps

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None) -> torch.Tensor:
        n = n_rows if n_rows is not None else (rows.numel() if rows is not None else x.shape[0])
        out = torch.empty((n, self.size), dtype=self.rt.dtype, device=x.device)
        K.stream_norm_rows(x, self.weight, self.offset, self.eps, out, rows=rows)
        return out

    def add_forward(self, x: torch.Tensor, delta: torch.Tensor, rows: Optional[torch.Tensor] = None,
                    n_rows: Optional[int] = None) -> torch.Tensor:
        """``x += delta`` (in place, whatever ``rows`` says) and the norm of the sum: the pre-norm arrangement's use."""
        K.residual_add(x, delta)
        return self.forward(x, rows, n_rows)

    def add_into(self, x32: torch.Tensor, y: torch.Tensor, want_h: bool = True, wts: Optional[torch.Tensor] = None,
                 top: int = 0) -> Optional[torch.Tensor]:
        """``x32 += norm(y)`` in place (``y``: a sublayer's output in the activation type; with ``wts [n, top]`` the
        weighted sum of ``top`` rows of ``y`` per row of the stream).  Returns the new stream rounded to the
        activation type (the stream itself in the 32-bit path), or None if ``want_h`` is off."""
        h = None
        if want_h and y.dtype != torch.float32:
            h = torch.empty(x32.shape, dtype=y.dtype, device=x32.device)
        K.stream_norm_add(y, self.weight, self.offset, self.eps, x32, h, wts=wts, top=top)
        return (x32 if y.dtype == torch.float32 else h) if want_h else None

    def sum_norm(self, x32: torch.Tensor, y: torch.Tensor, keep: float, *, gate: Optional[torch.Tensor] = None,
                 gate_bias: Optional[torch.Tensor] = None, wts: Optional[torch.Tensor] = None, top: int = 0,
                 shared: Optional[torch.Tensor] = None, shared_gate: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The norm AFTER the sum: ``x32 <- norm(keep * x32 + g * y)`` in place, ``g = sigmoid(gate + gate_bias)`` element by
        element (1 without gate logits), sum and norm in 32-bit.  With ``wts [n, top]``, ``y`` holds ``top`` rows per row of
        the stream (their weighted sum is formed first); ``shared`` / ``shared_gate``: one more row per token, weighted by
        the sigmoid of its own logit.  Returns the new stream rounded to the activation type (the stream itself in the
        32-bit path)."""
        h = None if y.dtype == torch.float32 else torch.empty(x32.shape, dtype=y.dtype, device=x32.device)
        if self._factor is None:
            self._factor = self.weight if self.offset == 0.0 else (self.weight + self.offset)
        K.gated_postnorm(y, x32, self._factor, keep, self.eps, h, gate=gate, gate_b=gate_bias, wts=wts, top=top, shared=shared,
                         shared_gate=shared_gate)
        return x32 if h is None else h
