"""A selective state-space mixer whose state is a vector per channel, with one decay per (channel, state).

With ``inner`` channels, ``N = state``, ``R = dt_rank`` and ``h`` the mixer's input:

    [x | z]      = W_in h                                   (``inner`` columns each)
    x            a causal convolution per channel over ``taps`` tokens (zeros before a sequence's start; the last column of
                 the stored ``[inner, taps]`` weight multiplies the current token) plus bias, then silu
    [d | B | C]  = W_x x                                    (``R``, ``N`` and ``N`` columns)
    dt           = softplus(W_dt d + dt_bias)               (one step size per channel)
    S[c, n]     <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n ,   A = -exp(A_log)  ([inner, N])
    y_c          = sum_n S[c, n] C_n + D_c x_c
    out          = W_o (y * silu(z))

The state ``S`` and the convolution's last ``taps - 1`` inputs are per-sequence state of fixed size (32-bit, zero when a
sequence starts), so a prompt, a piece of one and a single token are the same operation; a step of many tokens runs its
chunks side by side (``csrc/selscan.cu``).  The products keep their 32-bit sums, and the convolution, the step sizes, the
decays, the state and the read-out are 32-bit in both precisions; the gated result is rounded once for the output
product.  ``params["names"]`` maps the tensors' roles to their names behind the prefix.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..cache.store import KVNeed, StateNeed
from ..ops import kernels as K
from .base import Runtime, StepContext, TensorInfo, register_mixer
from .linear import linear

_ROLES = {"in": "in_proj.weight", "conv": "conv.weight", "conv_bias": "conv.bias", "x": "x_proj.weight", "dt": "dt_proj.weight",
          "dt_bias": "dt_proj.bias", "a_log": "A_log", "d": "D", "o": "o_proj.weight"}


def _names(params: Mapping, prefix: str) -> Dict[str, str]:
    given = params.get("names") or {}
    return {role: prefix + given.get(role, default) for role, default in _ROLES.items()}


@register_mixer("selective_scan")
class SelectiveScan:
    @staticmethod
    def tensors(params: Mapping, prefix: str) -> Dict[str, TensorInfo]:
        w, inner, n, r, taps = (int(params[k]) for k in ("hidden_size", "inner", "state", "dt_rank", "taps"))
        nm = _names(params, prefix)
        return {
            nm["in"]: TensorInfo((2 * inner, w), "matrix"),
            nm["conv"]: TensorInfo((inner, taps), "vector", False, 1.0 / taps), nm["conv_bias"]: TensorInfo((inner,), "vector", False, 0.0),
            nm["x"]: TensorInfo((r + 2 * n, inner), "matrix"), nm["dt"]: TensorInfo((inner, r), "matrix"),
            nm["dt_bias"]: TensorInfo((inner,), "vector", False, 0.0), nm["a_log"]: TensorInfo((inner, n), "vector", False, 0.0),
            nm["d"]: TensorInfo((inner,), "vector"), nm["o"]: TensorInfo((w, inner), "matrix"),
        }

    def __init__(self, params: Mapping, prefix: str, weights, rt: Runtime):
        self.rt = rt
        self.hidden, self.inner, self.n_state, self.dt_rank, self.taps = (
            int(params[k]) for k in ("hidden_size", "inner", "state", "dt_rank", "taps"))
        if not 1 <= self.taps <= K.SSM_MAX_TAPS or not 1 <= self.n_state <= K.SELSCAN_MAX_STATE:
            raise ValueError(f"selective_scan: state {self.n_state} (at most {K.SELSCAN_MAX_STATE}), {self.taps} taps (at most {K.SSM_MAX_TAPS})")
        nm = _names(params, prefix)
        self.w_in = weights.load(nm["in"], "matrix")
        self.w_x = weights.load(nm["x"], "matrix")
        self.w_dt = weights.load(nm["dt"], "matrix")
        self.w_o = weights.load(nm["o"], "matrix")
        f32 = lambda role: weights.load(nm[role], "vector").to(torch.float32).contiguous()
        self.conv_w, self.conv_b = f32("conv"), f32("conv_bias")
        self.dt_bias, self.a_log, self.d_skip = f32("dt_bias"), f32("a_log"), f32("d")
        self.chunked_from = int(params.get("chunked_from", 4 * K.SELSCAN_CHUNK_TOKENS))   # steps of fewer tokens walk them in order
        K.ssm_lib()
        K.selscan_lib()

    def kv_need(self) -> Optional[KVNeed]:
        return None

    def state_need(self):
        need = {"s": StateNeed((self.inner, self.n_state), torch.float32)}
        if self.taps > 1:
            need["tail"] = StateNeed((self.taps - 1, self.inner), torch.float32)
        return need

    def forward(self, h: torch.Tensor, ctx: StepContext, cache, state, owns_cache: bool = True) -> torch.Tensor:
        n, dev = h.shape[0], h.device
        R, N = self.dt_rank, self.n_state
        proj = linear(h, self.w_in, self.rt, out_dtype=torch.float32)            # [n, x | z], 32-bit sums kept
        xc = torch.empty((n, self.inner), dtype=torch.float32, device=dev)
        xc_act = xc if h.dtype == torch.float32 else torch.empty((n, self.inner), dtype=h.dtype, device=dev)
        K.ssm_conv(proj, 0, self.conv_w, self.conv_b, ctx.cu_q, ctx.seq_slot, ctx.n_seqs, state.get("tail"), xc,
                   out_bf16=None if xc_act is xc else xc_act)
        low = linear(xc_act, self.w_x, self.rt, out_dtype=torch.float32)         # [n, d | B | C]
        d = low[:, :R].contiguous() if h.dtype == torch.float32 else low[:, :R].to(h.dtype)
        dtp = linear(d, self.w_dt, self.rt, out_dtype=torch.float32)             # step sizes before bias and softplus
        out = torch.empty((n, self.inner), dtype=h.dtype, device=dev)
        K.selscan(xc, low, R, R + N, dtp, self.dt_bias, self.a_log, self.d_skip, proj, self.inner, ctx.cu_q, ctx.seq_slot, ctx.n_seqs,
                  state["s"], out, chunked=not ctx.decode and n >= self.chunked_from)
        return linear(out, self.w_o, self.rt)
