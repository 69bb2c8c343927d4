"""A selective state-space mixer in the state-space duality form: per head a matrix state with one scalar decay per token.

With ``inner = heads * v_dim``, ``N = state`` and ``G = groups``, one product of the mixer's input ``h`` leaves
``[z: inner | x: inner | B: G*N | C: G*N | dt: heads]`` per token.  Then

    x, B, C      a causal convolution per channel over ``taps`` tokens (zeros before a sequence's start; the last column of
                 the stored ``[channels, taps]`` weight multiplies the current token) plus bias, then silu
    dt_t         softplus(dt_t + dt_bias_head), no clamp
    S_t          exp(-exp(A_log_head) dt_t) S_(t-1) + dt_t B_t x_t^T      (N x v_dim per head; head ``i`` reads the B and C
                                                                           of group ``i // (heads / G)``)
    y_t          S_t^T C_t + D_head x_t
    out_t        W_o (norm(y_t * silu(z_t)) * w): the gate first, then an RMS norm over each of ``norm_groups`` equal parts of
                 the ``inner`` values (each part by its own root mean square, ``eps`` inside the root)

The matrix state and the convolution's last ``taps - 1`` inputs are per-sequence state of fixed size (32-bit, zero when a
sequence starts), so a prompt, a piece of one and a single token are the same operation (``csrc/ssm.cu``); a step of many
tokens runs its chunks side by side (each from a zero state, a prefix over the chunks' states, then each from its start state).  The product's
result is kept in 32-bit and everything behind it up to the norm's output runs in 32-bit in both precisions.
``params["names"]`` maps the tensors' roles to their names behind the prefix.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..cache.store import KVNeed, StateNeed
from ..ops import kernels as K
from .base import Runtime, StepContext, TensorInfo, register_mixer
from .linear import linear

_ROLES = {"in": "in_proj.weight", "conv": "conv.weight", "conv_bias": "conv.bias", "dt_bias": "dt_bias", "a_log": "A_log",
          "d": "D", "norm": "norm.weight", "o": "o_proj.weight"}


def _names(params: Mapping, prefix: str) -> Dict[str, str]:
    given = params.get("names") or {}
    return {role: prefix + given.get(role, default) for role, default in _ROLES.items()}


@register_mixer("ssd")
class SSD:
    @staticmethod
    def _sizes(params: Mapping):
        heads, dv, n, g = int(params["num_heads"]), int(params["v_dim"]), int(params["state"]), int(params["groups"])
        inner = heads * dv
        return heads, dv, n, g, inner, inner + 2 * g * n

    @staticmethod
    def tensors(params: Mapping, prefix: str) -> Dict[str, TensorInfo]:
        w, taps = params["hidden_size"], int(params["taps"])
        heads, dv, n, g, inner, ch = SSD._sizes(params)
        nm = _names(params, prefix)
        return {
            nm["in"]: TensorInfo((inner + ch + heads, w), "matrix"),
            nm["conv"]: TensorInfo((ch, taps), "vector", False, 1.0 / taps), nm["conv_bias"]: TensorInfo((ch,), "vector", False, 0.0),
            nm["dt_bias"]: TensorInfo((heads,), "vector", False, 0.0), nm["a_log"]: TensorInfo((heads,), "vector", False, 0.0),
            nm["d"]: TensorInfo((heads,), "vector"), nm["norm"]: TensorInfo((inner,), "vector"),
            nm["o"]: TensorInfo((w, inner), "matrix"),
        }

    def __init__(self, params: Mapping, prefix: str, weights, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.taps = int(params["taps"])
        self.parts = int(params.get("norm_groups", 1))
        self.eps = float(params["eps"])
        self.heads, self.v_dim, self.n_state, self.groups, self.inner, self.channels = self._sizes(params)
        if (self.heads % self.groups or self.inner % self.parts or not 1 <= self.taps <= K.SSM_MAX_TAPS
                or not 1 <= self.n_state <= K.SSM_MAX_STATE):
            raise ValueError(f"ssd: {self.heads} heads in {self.groups} groups, state {self.n_state} (at most {K.SSM_MAX_STATE}), "
                             f"{self.taps} taps (at most {K.SSM_MAX_TAPS}), norm over {self.parts} parts of {self.inner}")
        nm = _names(params, prefix)
        self.w_in = weights.load(nm["in"], "matrix")
        self.w_o = weights.load(nm["o"], "matrix")
        f32 = lambda role: weights.load(nm[role], "vector").to(torch.float32).contiguous()
        self.conv_w, self.conv_b = f32("conv"), f32("conv_bias")
        self.dt_bias, self.a_log, self.d_skip, self.norm_w = f32("dt_bias"), f32("a_log"), f32("d"), f32("norm")
        self.chunked_from = int(params.get("chunked_from", 4 * K.SSM_CHUNK_TOKENS))   # steps of fewer tokens walk them in order
        K.ssm_lib()
        K.rowops_lib()

    def kv_need(self) -> Optional[KVNeed]:
        return None

    def state_need(self):
        need = {"s": StateNeed((self.heads, self.n_state, self.v_dim), torch.float32)}
        if self.taps > 1:
            need["tail"] = StateNeed((self.taps - 1, self.channels), torch.float32)
        return need

    def forward(self, h: torch.Tensor, ctx: StepContext, cache, state, owns_cache: bool = True) -> torch.Tensor:
        n, dev = h.shape[0], h.device
        proj = linear(h, self.w_in, self.rt, out_dtype=torch.float32)     # [n, inner | channels | heads], 32-bit sums kept
        xbc = torch.empty((n, self.channels), dtype=torch.float32, device=dev)
        K.ssm_conv(proj, self.inner, self.conv_w, self.conv_b, ctx.cu_q, ctx.seq_slot, ctx.n_seqs, state.get("tail"), xbc)
        y = torch.empty((n, self.inner), dtype=torch.float32, device=dev)
        K.ssm_scan(xbc, proj, self.inner + self.channels, self.dt_bias, self.a_log, self.d_skip, ctx.cu_q, ctx.seq_slot, ctx.n_seqs,
                   self.heads, self.groups, self.n_state, self.v_dim, state["s"], y,
                   chunked=not ctx.decode and n >= self.chunked_from)
        out = torch.empty((n, self.inner), dtype=h.dtype, device=dev)
        K.gated_group_norm(y, proj[:, :self.inner], self.norm_w, self.parts, self.eps, out)
        return linear(out, self.w_o, self.rt)
