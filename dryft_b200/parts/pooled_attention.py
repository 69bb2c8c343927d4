"""Grouped-query attention over a sliding window plus one pooled key and value per block of positions that has left
the window, with a sink in the softmax's denominator.

Per step, with ``h`` the mixer's input:

    q = W_q h (+ b_q), k = W_k h (+ b_k), v = W_v h (+ b_v)           one product (queries only for a run step that reads
                                                                      another step's keys and values)
    q, k: the first ``rotary_dim`` dims of each head rotated by the token's position (position part ``rope``), THEN
          (``unit_norm``) each head divided by its root mean square over ``qk_dim`` (no weight, ``eps`` inside the root)
    k, v -> the cache at the token's position; every token that completes a block of ``pool`` positions leaves the mean
          of the block's cached keys and the mean of its cached values in pooled rows (one row per block)
    the query at position i sees the tokens j with 0 <= i - j < window and the pooled rows of the blocks b with
          b * pool + pool - 1 <= i - window; scores ``(q . k) * scale``; tokens and blocks share one softmax whose
          denominator also holds ``exp(sink_head)`` (``sink``: a number per head without key or value)
    (``head_gate``: head ``h``'s output is multiplied by ``sigmoid(W_g h)_h``, one number per head, ``W_g [heads, hidden]``
          riding in the input product)
    out = W_o (heads concatenated)

``proj_norm``: q and k pass an RMS norm over the WHOLE projection (all heads' rows at once, weights ``q_norm [heads * qk_dim]``
and ``k_norm [kv_heads * qk_dim]``, ``eps`` inside the root) before the rotation.  The rotation's layout is the position
part's (``half``: dims ``i`` and ``i + R/2``; ``interleaved``: dims ``2i`` and ``2i + 1``).

Without a ``window`` every earlier token is seen and there are no pooled rows.  A run step that borrows another's cache uses
its own queries, window, pool, scale and sink over the owner's rows; when it summarises the same blocks as the owner it
reads the owner's pooled rows, else it keeps pooled rows of its own (``CacheEntry.fills_pooled``).
Scores, softmax, sums, angles and the unit norm are 32-bit in both precisions (``csrc/pool_attn.cu``).
``params["names"]`` maps the tensors' roles to their names behind the prefix.
"""

from __future__ import annotations

import math
from typing import Dict, Mapping, Optional

import torch

from ..cache.store import CacheEntry, KVNeed, StateNeed
from ..config.spec import PartSpec
from ..ops import kernels as K
from .base import POSITIONS, Runtime, StepContext, TensorInfo, register_mixer
from .linear import linear

_ROLES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight", "q_bias": "q_proj.bias",
          "k_bias": "k_proj.bias", "v_bias": "v_proj.bias", "sink": "sink", "q_norm": "q_norm.weight", "k_norm": "k_norm.weight",
          "gate": "g_proj.weight"}
NO_WINDOW = 1 << 30   # "every earlier token" as a window size


def _names(params: Mapping, prefix: str) -> Dict[str, str]:
    given = params.get("names") or {}
    return {role: prefix + given.get(role, default) for role, default in _ROLES.items()}


@register_mixer("pooled_window_attention")
class PooledWindowAttention:
    @staticmethod
    def tensors(params: Mapping, prefix: str) -> Dict[str, TensorInfo]:
        w, nh, nkv = params["hidden_size"], params["num_heads"], params["num_kv_heads"]
        d, dv = params["qk_dim"], params["v_dim"]
        nm = _names(params, prefix)
        own, bias = params.get("own_kv", True), params.get("bias", False)
        t = {nm["q"]: TensorInfo((nh * d, w), "matrix"), nm["o"]: TensorInfo((w, nh * dv), "matrix")}
        if own:
            t[nm["k"]] = TensorInfo((nkv * d, w), "matrix")
            t[nm["v"]] = TensorInfo((nkv * dv, w), "matrix")
        if bias:
            t[nm["q_bias"]] = TensorInfo((nh * d,), "vector", False, 0.0)
            if own:
                t[nm["k_bias"]] = TensorInfo((nkv * d,), "vector", False, 0.0)
                t[nm["v_bias"]] = TensorInfo((nkv * dv,), "vector", False, 0.0)
        if params.get("sink", False):
            t[nm["sink"]] = TensorInfo((nh,), "vector", False, 0.0)
        if params.get("proj_norm", False):
            t[nm["q_norm"]] = TensorInfo((nh * d,), "vector")
            if own:
                t[nm["k_norm"]] = TensorInfo((nkv * d,), "vector")
        if params.get("head_gate", False):
            t[nm["gate"]] = TensorInfo((nh, w), "matrix")
        return t

    def __init__(self, params: Mapping, prefix: str, weights, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.n_heads, self.n_kv = int(params["num_heads"]), int(params["num_kv_heads"])
        self.qk_dim, self.v_dim = int(params["qk_dim"]), int(params["v_dim"])
        self.scale = float(params["scale"])
        self.eps = float(params.get("eps", 0.0))
        self.unit_norm = bool(params.get("unit_norm", False))
        win, pool = params.get("window"), params.get("pool")
        self.size = int(win) if win is not None else NO_WINDOW
        self.pool = int(pool) if (pool is not None and win is not None) else 0
        if self.n_heads % self.n_kv or self.size < 1 or self.pool < 0:
            raise ValueError(f"pooled_window_attention: {self.n_heads} heads over {self.n_kv} kv heads, window {win}, pool {pool}")
        self.group = self.n_heads // self.n_kv
        self.own_kv = bool(params.get("own_kv", True))
        self.q_dim, self.o_dim = self.n_heads * self.qk_dim, self.n_heads * self.v_dim
        nm = _names(params, prefix)
        self.head_gate = bool(params.get("head_gate", False))
        names, rows = [nm["q"]], [self.q_dim]
        if self.own_kv:
            names += [nm["k"], nm["v"]]
            rows += [self.n_kv * self.qk_dim, self.n_kv * self.v_dim]
        self.gate_col = sum(rows)
        if self.head_gate:                 # the gate's logits are columns of the input product
            names.append(nm["gate"])
            rows.append(self.n_heads)
        self.w_in = weights.load_fused(names, rows, self.hidden) if len(names) > 1 else weights.load(nm["q"], "matrix")
        self.proj_norm = bool(params.get("proj_norm", False))
        self.q_norm_w = weights.load(nm["q_norm"], "vector") if self.proj_norm else None
        self.k_norm_w = weights.load(nm["k_norm"], "vector") if self.proj_norm and self.own_kv else None
        self.w_o = weights.load(nm["o"], "matrix")
        bias = bool(params.get("bias", False))
        self.q_bias = weights.load(nm["q_bias"], "vector") if bias else None
        self.k_bias = weights.load(nm["k_bias"], "vector") if bias and self.own_kv else None
        self.v_bias = weights.load(nm["v_bias"], "vector") if bias and self.own_kv else None
        self.sink = weights.load(nm["sink"], "vector") if params.get("sink", False) else None
        self.side, self.side_out = None, None      # (first column, columns) of rows that ride with the input product
        pos: PartSpec = params.get("position") or PartSpec("none")
        self.position = POSITIONS.get(pos.kind)(pos.params, self.qk_dim, rt)
        self.interleaved = bool(getattr(self.position, "interleaved", False))
        # the per-token preparation with one block a token takes the norm over whole projections and both rotation layouts
        self.prep_by_token = self.proj_norm or self.interleaved
        if self.prep_by_token and bias:
            raise ValueError("pooled_window_attention: biases do not go with a norm over the whole projection or the interleaved layout")
        if self.head_gate:
            K.latent_attn_lib()            # the per-head gate kernel lives beside the other gated attention
        self.rot = int(getattr(self.position, "rotary_dim", 0) or 0) if getattr(self.position, "inv_freq", None) is not None else 0
        K.pool_attention_lib(self.qk_dim, self.v_dim, self.group)   # build (or find) the kernels of this head shape now
        self.use_prefill_kernel = rt.is_bf16 and K.pool_attention_prefill_supported(self.qk_dim, self.v_dim, self.group)
        if self.use_prefill_kernel:
            K.pool_attention_prefill_lib(self.qk_dim, self.v_dim, self.group)

    def absorb_rows(self, w: torch.Tensor) -> bool:
        """Rows of another product of the same input join the input product (behind q | k | v, from a column that is a
        multiple of 8); their result is ``side_out`` after every ``forward``."""
        if w.dtype != self.w_in.dtype or w.dim() != 2 or w.shape[1] != self.hidden or self.side is not None:
            return False
        pad = (-self.w_in.shape[0]) % 8
        fill = [torch.zeros((pad, self.hidden), dtype=w.dtype, device=w.device)] if pad else []
        self.side = (self.w_in.shape[0] + pad, w.shape[0])
        self.w_in = torch.cat([self.w_in] + fill + [w])
        return True

    def kv_need(self) -> Optional[KVNeed]:
        if self.size >= NO_WINDOW:
            return KVNeed(self.n_kv, self.qk_dim, None, self.v_dim)
        # rows that must stay: the window's, and those of the block that is still to be summarised
        return KVNeed(self.n_kv, self.qk_dim, max(self.size, self.pool), self.v_dim, None, True, self.pool or None)

    def state_need(self) -> Optional[StateNeed]:
        return None

    def _n_splits(self, n_rows: int, max_kv: int) -> int:
        """Keys of a row split over enough blocks to fill the device, a block taking at least 128 keys."""
        keys = min(max(1, max_kv), self.size) + (max(1, max_kv) // self.pool if self.pool else 0)
        want = math.ceil(2 * self.rt.sm_count / max(1, n_rows * self.n_kv))
        return max(1, min(32, want, (keys + 127) // 128))

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: CacheEntry, state, owns_cache: bool = True) -> torch.Tensor:
        if owns_cache != self.own_kv:
            raise ValueError("pooled_window_attention: a layer without key and value projections must read another run step's cache")
        n, dev = h.shape[0], h.device
        proj = linear(h, self.w_in, self.rt)
        if self.side is not None:
            self.side_out = proj[:, self.side[0]:self.side[0] + self.side[1]]
        q = torch.empty((n, self.n_heads, self.qk_dim), dtype=h.dtype, device=dev)
        pos = self.position
        if self.prep_by_token:
            K.pool_attn_prep_tok(proj, self.q_norm_w, self.k_norm_w, self.eps, pos.inv_freq if self.rot else None,
                                 getattr(pos, "inv_freq_lo", None) if self.rot else None, self.rot, self.interleaved, ctx.tok_slot,
                                 ctx.tok_pos, q, cache.k, cache.v, cache.page_table, self.n_heads, self.n_kv,
                                 self.eps if self.unit_norm else -1.0, owns_cache)
        else:
            K.pool_attn_prep(proj, self.q_bias, self.k_bias, self.v_bias, pos.inv_freq if self.rot else None,
                             getattr(pos, "inv_freq_lo", None) if self.rot else None, self.rot, ctx.tok_slot, ctx.tok_pos, q, cache.k,
                             cache.v, cache.page_table, self.n_heads, self.n_kv, self.eps if self.unit_norm else -1.0, owns_cache)
        pooled = None
        if self.pool:
            pc = cache.pooled
            if pc is None:
                raise ValueError("pooled_window_attention: the cache holds no pooled rows for this run step")
            pooled = (pc.k, pc.v, pc.page_table)
            if cache.fills_pooled:
                K.pool_attn_blocks(cache.k, cache.v, cache.page_table, pc.k, pc.v, pc.page_table, ctx.tok_slot, ctx.tok_pos, n,
                                   self.pool, self.group)
        o = torch.empty((n, self.n_heads, self.v_dim), dtype=h.dtype, device=dev)
        if self.use_prefill_kernel and not ctx.decode and ctx.n_tiles > 0 and cache.k.shape[2] == 64:
            K.pool_attn_prefill(q, cache.k, cache.v, cache.page_table, pooled, self.sink, ctx.tile_tok0, ctx.tile_rows, ctx.tok_slot,
                                ctx.tok_pos, o, ctx.n_tiles, self.scale, self.size, self.pool)
        else:
            s = self._n_splits(n, ctx.max_kv)
            part_o = part_ml = None
            if s > 1:
                part_o = torch.empty((n, self.n_heads, s, self.v_dim), dtype=torch.float32, device=dev)
                part_ml = torch.empty((n, self.n_heads, s, 2), dtype=torch.float32, device=dev)
            K.pool_attn_rows(q, cache.k, cache.v, cache.page_table, pooled, self.sink, ctx.tok_slot, ctx.tok_pos, o, self.scale,
                             self.size, self.pool, s, part_o, part_ml)
        o = o.view(n, self.o_dim)
        if self.head_gate:
            K.head_gate_rows(o, proj, self.gate_col, o, self.n_heads, self.v_dim)     # in place: an entry reads only itself
        return linear(o, self.w_o, self.rt)
