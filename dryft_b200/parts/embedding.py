"""Token embedding ``x = embed[ids]`` (``engine/dryft_qwen3/model.py:132,226``) and the output head
``logits = h @ W_head.T`` with ``W_head`` the embedding table itself when tied
(``engine/dryft_qwen3/weights.py:47-49``).  Unlike the reference, an untied ``lm_head.weight`` is
served (``weights.py:84-85`` refuses it), and logits leave the product's 32-bit accumulator
unrounded.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..ops import kernels as K
from .base import Residual, Runtime, StepContext, TensorInfo, fused_rms, register_embedding, register_head
from .linear import fusable_rows, linear


@register_embedding("embedding")
class Embedding:
    """``params["name"]``: the table's tensor name behind the prefix (default ``weight``).  ``params["stream32"]``: the rows
    start a 32-bit residual stream (a ``Residual`` whose ``x`` is float32 and whose ``h`` is the rows in the activation type)."""

    @staticmethod
    def tensors(params: Mapping, prefix: str) -> Dict[str, TensorInfo]:
        return {prefix + params.get("name", "weight"): TensorInfo((params["vocab_size"], params["hidden_size"]), "table")}

    def __init__(self, params: Mapping, prefix: str, weights, rt: Runtime):
        self.rt = rt
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.table = weights.load(prefix + params.get("name", "weight"), "table")
        self.stream32 = bool(params.get("stream32", False))
        # raised by the gather for an id outside the table (its row is zeroed, not read); read with the other
        # device flags by ``kernels.check_error_flags``
        self.err = torch.zeros(1, dtype=torch.int32, device=rt.device)
        K.watch_flag(self.err, "a token id outside the embedding table reached the embedding gather (its row was zeroed)")

    def forward(self, tokens: torch.Tensor, n_rows: int):
        out = torch.empty((n_rows, self.hidden), dtype=self.table.dtype, device=self.table.device)
        K.embed(tokens, self.table, out, self.err)
        # a table the checkpoint stores in 32-bit stays 32-bit; its rows are rounded on the way out
        h = out if out.dtype == self.rt.dtype else out.to(self.rt.dtype)
        if self.stream32:
            return Residual(out if out.dtype == torch.float32 else out.to(torch.float32), h=h)
        return h


@register_embedding("sinusoid_embedding")
class SinusoidEmbedding:
    """``x = table[id] * scale + s(p)``: the token's row times a constant, plus a sinusoidal vector of the token's
    position ``p`` in its sequence, ``s[2i] = sin(p * base^(-2i/W))`` and ``s[2i+1] = cos`` of the same angle.  The
    frequencies are evaluated on the host in 64-bit and rounded once; angles, sines and the sum are 32-bit
    (``csrc/stream32.cu``).  It starts a 32-bit residual stream: the result is a ``Residual`` whose ``x`` is float32 and
    whose ``h`` is the same rows in the activation type (the stream itself in the 32-bit path).  ``params["name"]`` is
    the table's tensor name behind the prefix (default ``weight``)."""

    takes_context = True   # forward needs the step's token positions

    @staticmethod
    def tensors(params: Mapping, prefix: str) -> Dict[str, TensorInfo]:
        return {prefix + params.get("name", "weight"): TensorInfo((params["vocab_size"], params["hidden_size"]), "table")}

    def __init__(self, params: Mapping, prefix: str, weights, rt: Runtime):
        self.rt = rt
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.scale = float(params.get("scale", 1.0))
        base = float(params.get("base", 10000.0))
        self.table = weights.load(prefix + params.get("name", "weight"), "table")
        half = (self.hidden + 1) // 2
        freq = torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * torch.arange(half, dtype=torch.float64) / self.hidden)
        self.freq = freq.to(torch.float32).to(rt.device)
        self.err = torch.zeros(1, dtype=torch.int32, device=rt.device)
        K.watch_flag(self.err, "a token id outside the embedding table reached the embedding gather (its row was zeroed)")

    def forward(self, tokens: torch.Tensor, n_rows: int, ctx: StepContext) -> Residual:
        x = torch.empty((n_rows, self.hidden), dtype=torch.float32, device=self.table.device)
        h = None if self.rt.dtype == torch.float32 else torch.empty((n_rows, self.hidden), dtype=self.rt.dtype, device=x.device)
        K.embed_sinusoid(tokens, ctx.tok_pos, self.table, self.freq, self.scale, x, h, self.err)
        return Residual(x, h=x if h is None else h)


@register_head("lm_head")
class LMHead:
    @staticmethod
    def tensors(params: Mapping, prefix: str) -> Dict[str, TensorInfo]:
        return {prefix + params.get("name", "weight"): TensorInfo((params["vocab_size"], params["hidden_size"]), "matrix",
                                                                  optional=bool(params["tied"]))}

    def __init__(self, params: Mapping, prefix: str, weights, rt: Runtime, embedding: Optional[Embedding] = None):
        self.rt = rt
        self.vocab = int(params["vocab_size"])
        self.tied = bool(params["tied"])
        name = prefix + params.get("name", "weight")   # the tensor's name behind the prefix
        if self.tied:
            if embedding is None:
                raise ValueError("a tied output head needs the embedding it is tied to")
            self.weight = embedding.table
            if weights.has(name):
                # present although tied: it has to be the same tensor (weights.py:86-87)
                other = weights.load(name, "matrix")
                if other.shape != self.weight.shape or not torch.equal(other.to(self.weight.dtype), self.weight):
                    raise ValueError(f"{name} is present and differs from the embedding table although the "
                                     "output head is tied to it")
                del other
        else:
            self.weight = weights.load(name, "matrix")
        # ``params["softcap"]``: logits <- cap * tanh(logits / cap), in 32-bit, after the product
        self.softcap = float(params["softcap"]) if params.get("softcap") is not None else None
        if self.softcap is not None:
            if not self.softcap > 0.0:
                raise ValueError(f"lm_head: softcap must be positive, got {self.softcap}")
            K.stream_par_lib()

    def _cap(self, logits: torch.Tensor) -> torch.Tensor:
        if self.softcap is not None:
            K.softcap(logits, self.softcap)
        return logits

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        """32-bit logits ``[rows, vocab]``."""
        return self._cap(linear(h, self.weight, self.rt, out_dtype=torch.float32))

    def can_fuse(self, n_rows: int, norm) -> bool:
        rt = self.rt
        return (rt.fuse_decode and rt.is_bf16 and fusable_rows(n_rows, self.weight.shape[1], rt, normed=True)
                and fused_rms(norm) is not None and self.weight.dtype == torch.bfloat16)

    def forward_normed(self, x: torch.Tensor, ss, ss_parts: int, norm, xw=None) -> torch.Tensor:
        """Logits of every row of ``x`` with the final norm inside the product (decode); ``xw``: ``x``
        weighted by the final norm's weight already."""
        out = torch.empty((x.shape[0], self.vocab), dtype=torch.float32, device=x.device)
        norm_w, eps = fused_rms(norm)
        small = self.rt.small_m_max
        if xw is not None and K.weighted_ahead_supported(x.shape[1]):
            K.fused_product(x, self.weight, out, small_m_max=small, xw_in=xw, norm_w=norm_w, ss_in=ss, ss_parts=ss_parts, eps=eps, pdl=self.rt.pdl)
        else:
            K.fused_product(x, self.weight, out, small_m_max=small, norm_w=norm_w, ss_in=ss, ss_parts=ss_parts, eps=eps, pdl=self.rt.pdl)
        return self._cap(out)


@register_embedding("pair_embedding")
class PairEmbedding:
    """``x = norm(table[id] * scale + pairs[row]) * w``: the token's row times a constant, plus a row of a second table chosen
    by a hash of the token and the one before it in its sequence, ``row = (prev * mul_prev + id * mul_cur) mod buckets``; a
    sequence's first token takes the row behind the buckets (row ``buckets`` of a table of ``buckets + 1`` rows).  The token
    before the first one of a step is per-sequence state (``state_need``): one int32 per slot, stored after every step.
    The sum and the norm are 32-bit, and the result starts a 32-bit residual stream (a ``Residual`` whose ``x`` is float32).
    ``params``: ``scale``; ``pair`` (None, or ``buckets``, ``mul_prev``, ``mul_cur``, ``name``); ``norm`` (None, or ``eps``,
    ``name``); ``name`` (the table's tensor name behind the prefix)."""

    takes_state = True   # forward needs the step's context and the per-sequence state

    @staticmethod
    def tensors(params: Mapping, prefix: str) -> Dict[str, TensorInfo]:
        w = params["hidden_size"]
        t = {prefix + params.get("name", "weight"): TensorInfo((params["vocab_size"], w), "table")}
        pair = params.get("pair")
        if pair:
            t[prefix + pair.get("name", "pairs")] = TensorInfo((int(pair["buckets"]) + 1, w), "table")
        norm = params.get("norm")
        if norm:
            t[prefix + norm.get("name", "norm.weight")] = TensorInfo((w,), "vector")
        return t

    def __init__(self, params: Mapping, prefix: str, weights, rt: Runtime):
        self.rt = rt
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.scale = float(params.get("scale", 1.0))
        self.table = weights.load(prefix + params.get("name", "weight"), "table")
        pair = params.get("pair")
        self.pairs = None
        self.buckets = self.mul_prev = self.mul_cur = 0
        if pair:
            self.buckets, self.mul_prev, self.mul_cur = int(pair["buckets"]), int(pair["mul_prev"]), int(pair["mul_cur"])
            self.pairs = weights.load(prefix + pair.get("name", "pairs"), "table")
            if self.pairs.dtype != self.table.dtype:
                self.pairs = self.pairs.to(self.table.dtype)
        norm = params.get("norm")
        self.norm_w, self.eps = None, 0.0
        if norm:
            self.norm_w, self.eps = weights.load(prefix + norm.get("name", "norm.weight"), "vector"), float(norm["eps"])
        self.err = torch.zeros(1, dtype=torch.int32, device=rt.device)
        K.watch_flag(self.err, "a token id outside the embedding table reached the embedding gather (its row was zeroed)")

    def state_need(self):
        from ..cache.store import StateNeed

        return StateNeed((), torch.int32) if self.pairs is not None else None

    def forward(self, tokens: torch.Tensor, n_rows: int, ctx: StepContext, state: Optional[torch.Tensor]) -> Residual:
        x = torch.empty((n_rows, self.hidden), dtype=torch.float32, device=self.table.device)
        K.embed_pair_norm(tokens, ctx.tok_slot, ctx.tok_pos, self.table, x, scale=self.scale, pair_table=self.pairs,
                          buckets=self.buckets, mul_prev=self.mul_prev, mul_cur=self.mul_cur, prev_state=state,
                          norm_w=self.norm_w, eps=self.eps, err=self.err)
        if self.pairs is not None:
            K.seq_last_token(tokens, ctx.tok_slot, n_rows, state)
        return Residual(x)
