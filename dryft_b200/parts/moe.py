"""Mixture-of-experts feed-forward with group-limited top-k routing.

``E`` small experts without biases -- SwiGLU (``down(silu(gate(h)) * up(h))``) or, with ``activation="relu2"``, ungated
(``down(max(up(h), 0)^2)``) -- of which a token uses ``top``.  The router may have a bias on its logits (``router_bias``: a
tensor name), and ``renormalize`` divides the chosen scores by their sum, which is the softmax over the chosen logits only.
An always-on expert of the same form (``shared``: ``{"intermediate_size", "gate"}``) may run for every token beside them; its
output is weighted by ``sigmoid(w_gate . h)``, one number per token, when it has a gate.  Router:
``z = W_router h`` and ``s = softmax(z)`` over all experts in 32-bit; expert ``e`` belongs to group ``e // (E / groups)`` (contiguous and equally
sized), a group is ranked by the maximum of its members' scores, and selection is restricted to the ``keep`` highest-ranked
groups; within them the ``top`` largest scores name the token's experts, each weighted by its own score ``s`` with no
rescaling (or with the scores divided by their sum, ``renormalize``).  The output is the weighted sum of the chosen experts' outputs.

The router's product leaves 32-bit logits (32-bit accumulation over the activations as the layer hands them over); the
choice is ``csrc/moe.cu:moe_route``.  The experts run assignment by assignment for few tokens and in the 32-bit path
(``csrc/moe.cu:moe_rows``: every chosen expert's weights are read once per assignment), and as grouped tensor-core
products over the tokens sorted by expert for prompts in bfloat16 (``csrc/moe_grouped.cu``).  The weighted sum is left
to the caller through ``forward_parts`` (a layer that normalises the sum forms it inside its norm kernel in 32-bit);
``forward`` forms it itself.  ``params["names"]`` maps roles to tensor names behind the prefix.

``score="sigmoid"``: an expert's score is the sigmoid of its own logit (no softmax over the experts).  ``weight_input``: the
chosen expert's weight multiplies its INPUT, ``out = sum_k expert_k(w_k h)``, not its output; since the first products are
linear, the weight is applied to their 32-bit sums, before the activation.  ``activation="clamped"`` (with ``limit``,
``alpha``, ``up_offset``): ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)``, ``down(g * sigmoid(alpha g) * (u +
up_offset))``.
"""

from __future__ import annotations

from typing import Dict, Mapping, Tuple

import torch

from ..ops import kernels as K
from .base import Runtime, StepContext, TensorInfo, register_ffn
from .linear import linear

_ROLES = {"router": "router.weight", "router_bias": "router.bias", "expert": "experts.{}.", "gate": "gate_proj.weight",
          "up": "up_proj.weight", "down": "down_proj.weight", "shared": "shared.", "shared_gate": "shared.gate.weight"}
SHARED_PAD = 8   # the always-on expert's first product carries its gate logit as one more column, padded to this many


def _names(params: Mapping) -> Dict[str, str]:
    given = params.get("names") or {}
    return {role: given.get(role, default) for role, default in _ROLES.items()}


@register_ffn("moe")
class MoE:
    @staticmethod
    def tensors(params: Mapping, prefix: str) -> Dict[str, TensorInfo]:
        w, f, e = params["hidden_size"], params["intermediate_size"], params["experts"]
        nm = _names(params)
        gated = params.get("activation", "swiglu") in ("swiglu", "clamped")
        t = {prefix + nm["router"]: TensorInfo((e, w), "matrix")}
        if params.get("router_bias"):
            t[prefix + nm["router_bias"]] = TensorInfo((e,), "vector", False, 0.0)
        for i in range(e):
            ep = prefix + nm["expert"].format(i)
            if gated:
                t[ep + nm["gate"]] = TensorInfo((f, w), "matrix")
            t[ep + nm["up"]] = TensorInfo((f, w), "matrix")
            t[ep + nm["down"]] = TensorInfo((w, f), "matrix")
        sh = params.get("shared")
        if sh is not None:
            fs, sp = sh["intermediate_size"], prefix + nm["shared"]
            if gated:
                t[sp + nm["gate"]] = TensorInfo((fs, w), "matrix")
            t[sp + nm["up"]] = TensorInfo((fs, w), "matrix")
            t[sp + nm["down"]] = TensorInfo((w, fs), "matrix")
            if sh.get("gate", True):
                t[prefix + nm["shared_gate"]] = TensorInfo((1, w), "matrix")
        return t

    def __init__(self, params: Mapping, prefix: str, weights, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.experts = int(params["experts"])
        self.top = int(params["top"])
        self.groups = int(params.get("groups", 1))
        self.keep = int(params.get("keep", self.groups))
        self.renorm = bool(params.get("renormalize", False))
        if self.experts % self.groups or not 1 <= self.keep <= self.groups or not 1 <= self.top <= self.experts:
            raise ValueError(f"moe: {self.experts} experts, {self.groups} groups, keep {self.keep}, top {self.top} do not go together")
        act = params.get("activation", "swiglu")
        if act not in ("swiglu", "relu2", "clamped"):
            raise ValueError(f"moe: activation must be 'swiglu', 'relu2' or 'clamped', got {act!r}")
        self.gated = act in ("swiglu", "clamped")
        self.score = params.get("score", "softmax")
        if self.score not in ("softmax", "sigmoid"):
            raise ValueError(f"moe: score must be 'softmax' or 'sigmoid', got {self.score!r}")
        # the weight on the expert's input; the clamped activation's constants (a plain gated expert is the clamped one
        # with no limit, alpha 1 and no offset, so both run through the same kernel mode when the weight is on the input)
        self.weight_input = bool(params.get("weight_input", False))
        self.clamped = act == "clamped"
        self.limit = None if params.get("limit") is None else float(params["limit"])
        self.alpha = float(params.get("alpha", 1.0)) if self.clamped else 1.0
        self.up_offset = float(params.get("up_offset", 0.0)) if self.clamped else 0.0
        if not self.clamped:
            self.limit = None
        if self.weight_input and not self.gated:
            raise ValueError("moe: a weight on the expert's input is served for gated experts")
        self.sums_plainly = self.weight_input      # the experts' rows are summed as they are (the weights are inside)
        nm = _names(params)
        # The router's logits are 32-bit sums.  In the bfloat16 path its operands are the bfloat16 activations and the
        # weight as stored (their products are exact in 32-bit), multiplied by the tensor-core products with 32-bit
        # accumulation and a 32-bit result; in the 32-bit path everything is float32.
        self.w_router = weights.load(prefix + nm["router"], "matrix")
        self.router_bias = weights.load(prefix + nm["router_bias"], "vector") if params.get("router_bias") else None
        gu, dn = [], []
        for i in range(self.experts):
            ep = prefix + nm["expert"].format(i)
            gu += [ep + nm["gate"], ep + nm["up"]] if self.gated else [ep + nm["up"]]
            dn.append(ep + nm["down"])
        # [E, 2F, W] (an expert's gate rows, then its up rows; [E, F, W] without a gate) and [E, W, F]
        self.w_gate_up = weights.load_fused(gu, [self.inter] * len(gu), self.hidden).view(
            self.experts, (2 if self.gated else 1) * self.inter, self.hidden)
        self.w_down = weights.load_fused(dn, [self.hidden] * len(dn), self.inter).view(self.experts, self.hidden, self.inter)
        self.use_grouped = (rt.is_bf16 and self.w_gate_up.dtype == torch.bfloat16
                            and K.moe_grouped_supported(self.hidden, self.inter))
        if self.use_grouped:
            K.moe_grouped_lib()
        # the always-on expert: its first product also yields the per-token gate logit (one more row of the weight, padded)
        self.shared_inter = 0
        self.side, self.side_out = None, None      # (first column, columns) of rows that ride with the always-on expert's product
        sh = params.get("shared")
        if sh is not None:
            if self.gated:
                raise ValueError("moe: an always-on expert is served for ungated experts (activation 'relu2') only")
            self.shared_inter = fs = int(sh["intermediate_size"])
            self.shared_gate = bool(sh.get("gate", True))
            sp = prefix + nm["shared"]
            names, rows = [sp + nm["up"]], [fs]
            if self.shared_gate:
                names.append(prefix + nm["shared_gate"])
                rows.append(1)
            w = weights.load_fused(names, rows, self.hidden)
            pad = (-w.shape[0]) % SHARED_PAD
            self.w_shared_up = torch.cat([w, torch.zeros((pad, self.hidden), dtype=w.dtype, device=w.device)]) if pad else w
            self.w_shared_down = weights.load(sp + nm["down"], "matrix")

    GROUPED_MIN_TOKENS = 32   # below this every assignment streams its expert's weights itself
    ROUTE_ROWS_MAX = 16       # up to this many tokens the router's product and choice are one launch ...
    ROUTE_ROWS_MAX_WEIGHTS = 64 * 1024   # ... while one block can stream the router's weight quickly enough (measured: 32 x 1,024
                                         # gains a launch, 64 x 2,048 takes longer than the two launches it replaces)

    def route(self, h: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Chosen experts ``[n, top]`` int32 and their weights ``[n, top]`` float32."""
        n = h.shape[0]
        idx = torch.empty((n, self.top), dtype=torch.int32, device=h.device)
        wts = torch.empty((n, self.top), dtype=torch.float32, device=h.device)
        if (n <= self.ROUTE_ROWS_MAX and self.w_router.dtype == h.dtype and self.w_router.numel() <= self.ROUTE_ROWS_MAX_WEIGHTS
                and K.moe_route_rows_supported(self.hidden, self.experts, self.groups, h.element_size())):
            K.moe_route_rows(h, self.w_router, self.groups, self.keep, self.top, idx, wts, renorm=self.renorm,
                             bias=self.router_bias, score=self.score)   # one launch
            return idx, wts
        logits = linear(h, self.w_router, self.rt, out_dtype=torch.float32)
        K.moe_route(logits, self.groups, self.keep, self.top, idx, wts, renorm=self.renorm, bias=self.router_bias, score=self.score)
        return idx, wts

    def absorb_rows(self, w: torch.Tensor) -> bool:
        """Rows of another product of the same input join the always-on expert's first product (behind up | gate, padded);
        their result is ``side_out`` after every ``forward_shared``."""
        if not self.shared_inter or self.side is not None or w.dim() != 2 or w.shape[1] != self.hidden or w.dtype != self.w_shared_up.dtype:
            return False
        pad = (-w.shape[0]) % SHARED_PAD
        fill = [torch.zeros((pad, self.hidden), dtype=w.dtype, device=w.device)] if pad else []
        self.side = (self.w_shared_up.shape[0], w.shape[0])
        self.w_shared_up = torch.cat([self.w_shared_up, w] + fill)
        return True

    def forward_shared(self, h: torch.Tensor):
        """The always-on expert: ``(ys [n, hidden], gate logits [n, 1] or None)``, or None if there is none.  The caller
        multiplies ``ys`` by ``sigmoid(gate logit)`` and adds it to the routed experts' sum."""
        if not self.shared_inter:
            return None
        z = linear(h, self.w_shared_up, self.rt)
        if self.side is not None:
            self.side_out = z[:, self.side[0]:self.side[0] + self.side[1]]
        act = torch.empty((h.shape[0], self.shared_inter), dtype=h.dtype, device=h.device)
        K.relu2(z[:, :self.shared_inter], act)
        ys = linear(act, self.w_shared_down, self.rt)
        return ys, (z[:, self.shared_inter:self.shared_inter + 1] if self.shared_gate else None)

    def forward_parts(self, h: torch.Tensor, ctx: StepContext) -> Tuple[torch.Tensor, torch.Tensor, int]:
        """``(y [n*top, hidden], wts [n, top], top)``: row ``n*top + k`` is the output of token ``n``'s k-th expert, not yet
        weighted."""
        y, wts = self._experts(h)
        if self.weight_input:      # the weights are inside the experts already: the rows are summed as they are
            wts = torch.ones_like(wts)
        return y, wts, self.top

    def forward_rows(self, h: torch.Tensor, ctx: StepContext) -> Tuple[torch.Tensor, int]:
        """``(y [n*top, hidden], top)`` for experts whose weights are on their input (``sums_plainly``): the caller adds a
        token's ``top`` rows as they are."""
        if not self.sums_plainly:
            raise ValueError("moe: forward_rows is for experts weighted on their input; use forward_parts")
        return self._experts(h)[0], self.top

    def _experts(self, h: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        n = h.shape[0]
        idx, wts = self.route(h)
        y = torch.empty((n * self.top, self.hidden), dtype=h.dtype, device=h.device)
        special = self.weight_input or self.clamped      # the kernel mode with a weight on the input and the clamped activation
        in_w = wts if self.weight_input else (torch.ones_like(wts) if special else None)
        if self.use_grouped and n >= self.GROUPED_MIN_TOKENS:
            K.moe_grouped(h, self.w_gate_up, self.w_down, idx, y, gated=self.gated, in_w=in_w, limit=self.limit, alpha=self.alpha,
                          up_offset=self.up_offset)
        else:
            act = torch.empty((n * self.top, self.inter), dtype=h.dtype, device=h.device)
            if special:
                K.moe_rows(h, self.w_gate_up, idx, act, "gate_up_clamp", in_w=in_w, limit=self.limit, alpha=self.alpha,
                           up_offset=self.up_offset)
            else:
                K.moe_rows(h, self.w_gate_up, idx, act, "gate_up" if self.gated else "up_relu2")
            K.moe_rows(act, self.w_down, idx, y, "down")
        return y, wts

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        y, wts, top = self.forward_parts(h, ctx)
        out = torch.empty((h.shape[0], self.hidden), dtype=h.dtype, device=h.device)
        K.moe_combine(y, wts, out)
        if self.shared_inter:
            raise ValueError("moe: the always-on expert is joined by the layer's arrangement (forward_parts and forward_shared)")
        return out
