"""Arrangements of a mixer, a feed-forward and their norms in one layer.

``prenorm`` (``engine/dryft_qwen3/model.py:151-184``):
    x += delta_in ; h = norm_mixer(x)          (one fused kernel; delta_in is the previous block's
    a  = mixer(h)                               not-yet-added feed-forward output)
    x += a        ; h = norm_ffn(x)            (one fused kernel)
    delta_out = ffn(h)
A layer without a feed-forward stops after the mixer and returns its output as ``delta_out``.
The block returns the stream and ``delta_out``: the add of ``delta_out`` is left to whatever norm comes
next (the next block's, or the final norm), which is how the reference fuses "residual add + next
norm".  With few rows (decode) and parts that offer it, the norms, the adds and the activation are
folded into the matrix products instead (``csrc/gemm_small_m.cu``).
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional, Tuple

import torch

from ..ops import kernels as K
from .base import Residual, Runtime, StepContext, TensorInfo, fused_rms, register_block, register_connection
from .linear import linear, weighted_for


@register_block("prenorm")
class PreNormBlock:
    def __init__(self, norm_mixer, mixer, norm_ffn, ffn):
        self.norm_mixer = norm_mixer
        self.mixer = mixer
        self.norm_ffn = norm_ffn
        self.ffn = ffn

    def _fusable(self, n_rows: int) -> bool:
        m, f = self.mixer, self.ffn
        if f is None:
            return False
        return (hasattr(m, "forward_normed") and hasattr(f, "forward_normed")
                and m.can_fuse(n_rows, self.norm_mixer) and f.can_fuse(n_rows, self.norm_ffn))

    takes_next_norm = True   # forward accepts the norm that will read the stream after this block

    def forward(self, res: Residual, ctx: StepContext, cache, state, owns_cache: bool = True, next_norm=None) -> Residual:
        x = res.x
        if self._fusable(x.shape[0]):
            # few rows: five launches per layer.  Each product normalises / adds / activates on its own
            # and hands the stream's sums of squares (and, where sizes allow, the stream weighted for the
            # next norm) to the next one.
            if res.delta is not None:
                K.residual_add(x, res.delta)
                res = Residual(x)
            ss, parts = res.ss, res.ss_parts
            xw = res.xw if res.xw_norm is self.norm_mixer else None
            ahead_m = getattr(self.mixer, "weighted_ahead", False)
            ahead_f = getattr(self.ffn, "weighted_ahead", False)
            if ss is None:
                ss = torch.empty(K.SS_STRIDE, dtype=torch.float32, device=x.device)
                if ahead_m and weighted_for(self.norm_mixer, x.shape[1], x.shape[1], self.mixer.rt, x.shape[0]):
                    xw = torch.empty_like(x)
                    K.row_sumsq(x, ss, norm_w=fused_rms(self.norm_mixer)[0], xw_out=xw)
                else:
                    K.row_sumsq(x, ss)
                parts = 1
            if ahead_m:
                ss, parts, xw = self.mixer.forward_normed(x, ss, parts, self.norm_mixer, ctx, cache, state, owns_cache,
                                                          xw=xw, next_norm=self.norm_ffn if ahead_f else None)
            else:
                ss, parts = self.mixer.forward_normed(x, ss, parts, self.norm_mixer, ctx, cache, state, owns_cache)
                xw = None
            if ahead_f:
                ss, parts, xw = self.ffn.forward_normed(x, ss, parts, self.norm_ffn, ctx, xw=xw, next_norm=next_norm)
            else:
                ss, parts = self.ffn.forward_normed(x, ss, parts, self.norm_ffn, ctx)
                xw = None
            return Residual(x, None, ss, parts, xw, next_norm if xw is not None else None)
        h = self.norm_mixer.forward(x) if res.delta is None else self.norm_mixer.add_forward(x, res.delta)
        a = self.mixer.forward(h, ctx, cache, state, owns_cache)
        if self.ffn is None:           # a layer without a feed-forward: the mixer's output is what the next norm adds
            return Residual(x, a)
        h = self.norm_ffn.add_forward(x, a)
        return Residual(x, self.ffn.forward(h, ctx))


@register_block("outnorm")
class OutNormBlock:
    """The norm on each sublayer's output only, around a 32-bit stream:

        x += norm_mixer(mixer(h))      h = x rounded to the activation type (the sublayers read the stream itself)
        x += norm_ffn(ffn(h))

    ``res.x`` is float32 in both precisions; each norm-and-add is one kernel that also leaves the rounded stream for
    the next sublayer (``csrc/stream32.cu``).  The norms must offer ``add_into`` (``rmsnorm_offset`` does).  A
    feed-forward that offers ``forward_parts`` (a routed one: ``top`` rows per token and their weights) has its
    weighted sum formed inside that kernel.  A layer without a feed-forward stops after the mixer."""

    def __init__(self, norm_mixer, mixer, norm_ffn, ffn):
        for nm in (norm_mixer, norm_ffn):
            if nm is not None and not hasattr(nm, "add_into"):
                raise ValueError("the 'outnorm' arrangement needs norms that offer add_into (a 32-bit stream)")
        self.norm_mixer = norm_mixer
        self.mixer = mixer
        self.norm_ffn = norm_ffn
        self.ffn = ffn

    def forward(self, res: Residual, ctx: StepContext, cache, state, owns_cache: bool = True) -> Residual:
        x = res.x
        if x.dtype != torch.float32:
            raise ValueError("the 'outnorm' arrangement keeps its stream in float32; the embedding must start one")
        if res.delta is not None:
            x.add_(res.delta)
        act = self.mixer.rt.dtype
        h = res.h if res.h is not None else (x if act == torch.float32 else x.to(act))
        a = self.mixer.forward(h, ctx, cache, state, owns_cache)
        h = self.norm_mixer.add_into(x, a)
        if self.ffn is None:
            return Residual(x, h=h)
        parts = getattr(self.ffn, "forward_parts", None)
        if parts is not None:
            y, wts, top = parts(h, ctx)
            h = self.norm_ffn.add_into(x, y, wts=wts, top=top)
        else:
            h = self.norm_ffn.add_into(x, self.ffn.forward(h, ctx))
        return Residual(x, h=h)


@register_connection("gated_sum")
class GatedSum:
    """How a sublayer's result ``y`` joins a stream whose norm follows the sum: ``keep * x + g * y`` with ``g = sigmoid(W h +
    b)`` element by element, ``h`` being the sublayer's own input.  ``params``: ``size``, ``keep`` (default 1), ``gate`` and
    ``gate_bias`` (tensor names behind the prefix; no ``gate``: ``g = 1`` and no tensors)."""

    @staticmethod
    def tensors(params: Mapping, prefix: str) -> Dict[str, TensorInfo]:
        if not params.get("gate"):
            return {}
        t = {prefix + params["gate"]: TensorInfo((params["size"], params["size"]), "matrix")}
        if params.get("gate_bias"):
            t[prefix + params["gate_bias"]] = TensorInfo((params["size"],), "vector", False, 0.0)
        return t

    def __init__(self, params: Mapping, prefix: str, weights, rt: Runtime):
        self.rt = rt
        self.keep = float(params.get("keep", 1.0))
        self.w = weights.load(prefix + params["gate"], "matrix") if params.get("gate") else None
        self.b = weights.load(prefix + params["gate_bias"], "vector") if self.w is not None and params.get("gate_bias") else None
        self.source = None      # the part whose first product also forms the gate logits (``ride_with``)

    def ride_with(self, part) -> bool:
        """Let ``part``, which reads the same input, form ``W h`` inside its own first product (``part.absorb_rows``): one
        launch less per sublayer.  True if it took the rows; the matrix then lives in the part's fused weight only."""
        if self.w is None or self.source is not None or not hasattr(part, "absorb_rows") or not part.absorb_rows(self.w):
            return False
        self.source, self.w = part, None
        return True

    def logits(self, h: torch.Tensor) -> Optional[torch.Tensor]:
        """``W h`` in the activation type (the bias and the sigmoid belong to the kernel that forms the sum).  When the rows
        ride with a part's product this is a column slice of that product's output: ask AFTER the part has run."""
        if self.source is not None:
            return self.source.side_out
        return linear(h, self.w, self.rt) if self.w is not None else None


@register_block("postnorm")
class PostNormBlock:
    """The norm after the sum, around a 32-bit stream:

        x <- norm_mixer(keep * x + g1 * mixer(h))      h = x rounded to the activation type (the sublayers read the stream itself)
        x <- norm_ffn  (keep * x + g2 * ffn(h))

    ``extra`` holds a ``gated_sum`` connection per sublayer (``gate_mixer``, ``gate_ffn``) that gives ``keep`` and the gate
    ``g``; each sum, gate and norm is one kernel that also leaves the rounded stream for the next sublayer
    (``csrc/rowops.cu``).  The norms must offer ``sum_norm``.  A routed feed-forward (``forward_parts``) has its weighted
    sum, and its always-on expert (``forward_shared``), joined inside that kernel.  A layer without a feed-forward stops
    after the mixer."""

    def __init__(self, norm_mixer, mixer, norm_ffn, ffn, extra: Optional[Mapping] = None):
        extra = extra or {}
        for nm in (norm_mixer, norm_ffn):
            if nm is not None and not hasattr(nm, "sum_norm"):
                raise ValueError("the 'postnorm' arrangement needs norms that offer sum_norm (a 32-bit stream)")
        self.norm_mixer, self.mixer, self.norm_ffn, self.ffn = norm_mixer, mixer, norm_ffn, ffn
        self.gate_mixer, self.gate_ffn = extra.get("gate_mixer"), extra.get("gate_ffn")
        if self.gate_mixer is None or (ffn is not None and self.gate_ffn is None):
            raise ValueError("the 'postnorm' arrangement needs a connection per sublayer (extra parts gate_mixer, gate_ffn)")
        self.extra = dict(extra)
        self.gate_mixer.ride_with(mixer)
        if ffn is not None:
            self.gate_ffn.ride_with(ffn)

    def forward(self, res: Residual, ctx: StepContext, cache, state, owns_cache: bool = True) -> Residual:
        x = res.x
        if x.dtype != torch.float32:
            raise ValueError("the 'postnorm' arrangement keeps its stream in float32; the embedding must start one")
        if res.delta is not None:
            x.add_(res.delta)
        act = self.mixer.rt.dtype
        h = res.h if res.h is not None else (x if act == torch.float32 else x.to(act))
        conn = self.gate_mixer
        a = self.mixer.forward(h, ctx, cache, state, owns_cache)
        h = self.norm_mixer.sum_norm(x, a, conn.keep, gate=conn.logits(h), gate_bias=conn.b)
        if self.ffn is None:
            return Residual(x, h=h)
        conn = self.gate_ffn
        parts = getattr(self.ffn, "forward_parts", None)
        if parts is not None:
            y, wts, top = parts(h, ctx)
            sh = self.ffn.forward_shared(h) if hasattr(self.ffn, "forward_shared") else None
            ys, sg = sh if sh is not None else (None, None)
            h = self.norm_ffn.sum_norm(x, y, conn.keep, gate=conn.logits(h), gate_bias=conn.b, wts=wts, top=top, shared=ys,
                                       shared_gate=sg)
        else:
            y = self.ffn.forward(h, ctx)
            h = self.norm_ffn.sum_norm(x, y, conn.keep, gate=conn.logits(h), gate_bias=conn.b)
        return Residual(x, h=h)


@register_block("parallel")
class ParallelBlock:
    """One norm, read by the mixer and the feed-forward alike, whose results join a 32-bit stream together:

        n = norm_mixer(x) ;  x <- x + mixer(n) + ffn(n)

    ``res.x`` is float32 in both precisions.  The sum is one kernel (``csrc/stream_par.cu``): a mixer that offers
    ``forward_terms`` (two mixers side by side) hands over its results unsummed with their factors, a routed feed-forward
    whose weights are already inside its experts (``sums_plainly``) its ``top`` rows per token; the same kernel leaves the
    stream normed for the layer that runs next when that layer's norm is known (``next_norm``), so a layer is one norm-less
    chain of products and one sum; in a step of few rows the feed-forward runs beside the mixer on a stream of its own
    (``Runtime.run_branches``).  There is no second norm (``norm_ffn`` must be None); a layer without a feed-forward
    adds the mixer's result alone."""

    takes_next_norm = True

    def __init__(self, norm_mixer, mixer, norm_ffn, ffn):
        if norm_ffn is not None:
            raise ValueError("the 'parallel' arrangement has one norm: its feed-forward reads the mixer's normed input")
        self.norm_mixer, self.mixer, self.norm_ffn, self.ffn = norm_mixer, mixer, None, ffn
        K.stream_par_lib()

    @staticmethod
    def _plain(norm):
        """``(factor, eps)`` of a norm that is ``x / sqrt(mean(x^2) + eps) * factor`` in 32-bit, rounded once; else None."""
        get = getattr(norm, "plain_params", None)
        return get() if callable(get) else None

    def forward(self, res: Residual, ctx: StepContext, cache, state, owns_cache: bool = True, next_norm=None) -> Residual:
        x = res.x
        if x.dtype != torch.float32:
            raise ValueError("the 'parallel' arrangement keeps its stream in float32; the embedding must start one")
        if res.delta is not None:
            x.add_(res.delta)
        n = res.hn if (res.hn is not None and res.hn_norm is self.norm_mixer) else self.norm_mixer.forward(x)
        def mix():
            terms = getattr(self.mixer, "forward_terms", None)
            return list(terms(n, ctx, cache, state, owns_cache)) if terms is not None else [(self.mixer.forward(n, ctx, cache, state, owns_cache), 1.0)]

        def feed():
            if getattr(self.ffn, "sums_plainly", False):
                return self.ffn.forward_rows(n, ctx)
            return self.ffn.forward(n, ctx)

        rt = self.mixer.rt
        rows, top = None, 0
        if self.ffn is None:
            terms = mix()
        else:
            # few rows: the feed-forward runs beside the mixer on a stream of its own (both read the same normed rows)
            terms, f = rt.run_branches([mix, feed], first_stream=0) if rt.branches(x.shape[0]) else (mix(), feed())
            if isinstance(f, tuple):
                rows, top = f
            else:
                terms = terms + [(f, 1.0)]
        plain = self._plain(next_norm) if next_norm is not None else None
        hn = None
        if plain is not None:
            hn = torch.empty(x.shape, dtype=self.mixer.rt.dtype, device=x.device)
            K.stream_sum(x, terms, rows=rows, top=top, norm_w=plain[0], eps=plain[1], h=hn)
        else:
            K.stream_sum(x, terms, rows=rows, top=top)
        return Residual(x, hn=hn, hn_norm=next_norm if hn is not None else None)


@register_connection("loop_mix")
class LoopMix:
    """How a stretch of layers that runs several times is entered: ``x <- W [x | x0] + step[t]`` with ``x0`` the embedding's
    output, ``W`` a ``[size, 2 size]`` matrix (the stream's columns first) and ``step`` one vector per pass ``t``.  The two
    32-bit rows are rounded side by side as the product's operand; the product's 32-bit sums, plus the pass's vector,
    are the new stream.  ``params``: ``size``, ``times``, ``matrix`` and ``steps`` (tensor names behind the prefix)."""

    @staticmethod
    def tensors(params: Mapping, prefix: str) -> Dict[str, TensorInfo]:
        size = int(params["size"])
        return {prefix + params.get("matrix", "in"): TensorInfo((size, 2 * size), "matrix"),
                prefix + params.get("steps", "step"): TensorInfo((int(params["times"]), size), "vector", False, 0.0)}

    def __init__(self, params: Mapping, prefix: str, weights, rt: Runtime):
        self.rt = rt
        self.size, self.times = int(params["size"]), int(params["times"])
        self.w = weights.load(prefix + params.get("matrix", "in"), "matrix")
        self.steps = weights.load(prefix + params.get("steps", "step"), "vector").to(torch.float32).contiguous()   # [times, size]
        K.stream_par_lib()

    def enter(self, res: Residual, x0: torch.Tensor, number: int, next_norm=None) -> Residual:
        if not 0 <= number < self.times:
            raise ValueError(f"loop_mix: pass {number} of {self.times}")
        x = res.x
        if x.dtype != torch.float32 or x0 is None or x0.dtype != torch.float32:
            raise ValueError("loop_mix joins 32-bit streams; the embedding must start one")
        if res.delta is not None:
            x.add_(res.delta)
        pair = torch.empty((x.shape[0], 2 * self.size), dtype=self.rt.dtype, device=x.device)
        K.pack_pair(x, x0, pair)
        y = linear(pair, self.w, self.rt, out_dtype=torch.float32)
        plain = ParallelBlock._plain(next_norm) if next_norm is not None else None
        if plain is None:
            K.stream_sum(y, vec=self.steps[number])
            return Residual(y)
        hn = torch.empty(y.shape, dtype=self.rt.dtype, device=y.device)
        K.stream_sum(y, vec=self.steps[number], norm_w=plain[0], eps=plain[1], h=hn)
        return Residual(y, hn=hn, hn_norm=next_norm)
