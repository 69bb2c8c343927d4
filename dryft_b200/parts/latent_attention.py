"""Attention whose queries, keys and values come from low-rank latents, over a sliding window, with a gate per head.

With ``H`` heads, per head ``d`` unrotated and ``r`` rotated query/key dims, value size ``dv``, latent sizes ``q_rank`` and
``kv_rank``, and ``h`` the mixer's input:

    c_q = rmsnorm(W_dq h) ;  q = W_uq c_q            (head by head: ``d`` unrotated dims, then ``r`` rotated ones)
    [c_raw | k_rot] = W_dkv h ;  c = rmsnorm(c_raw) ;  k_rot rotated at the token's position, one vector for all heads
    per head:  k = W_uk c ,  v = W_uv c ;  score(i, j) = (q_plain . k + q_rot . k_rot) * scale ,  0 <= i - j < window
    o = softmax(score) v ;  o <- o * sigmoid(W_g h)_head  ->  @ W_o.T
    (``sink``: the softmax's denominator of head ``h`` also holds ``exp(sink_h)``, a learned number without key or value)

Only ``[c | k_rot]`` is cached, one row per token for all heads (a keys-only cache group).  The per-head key and value
matrices are folded into the query and the output: ``q_lat = W_uk^T q_plain`` before attention, ``o = W_uv o_lat`` after,
as batched matrix products over the heads (steps of few tokens and the 32-bit path: kernels of this library); attention
itself runs over the cached rows (``csrc/latent_attn.cu``).
A bfloat16 step in which every sequence starts at position 0 (all its keys are its own) makes per-head keys and values
from its latents by one more product and runs the library's tensor-core prompt attention over pages of the step's own;
every other step (a piece that continues a prompt, a single token, everything in 32-bit) runs over the cached latents.
Norms, angles, scores, softmax and the weighted sum are 32-bit in both precisions.  ``W_dq | W_dkv | W_g`` are one
product.  Every size and constant is a parameter; ``params["names"]`` maps the tensors' roles to their names.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..cache.store import CacheEntry, KVNeed, StateNeed
from ..config.spec import PartSpec
from ..ops import kernels as K
from .base import POSITIONS, Runtime, StepContext, TensorInfo, register_mixer
from .linear import linear

_ROLES = {"dq": "q_down.weight", "dq_norm": "q_down.norm", "uq": "q_up.weight", "dkv": "kv_down.weight", "dkv_norm": "kv_down.norm",
          "uk": "k_up.weight", "uv": "v_up.weight", "gate": "g_proj.weight", "o": "o_proj.weight", "sink": "sink"}


def _names(params: Mapping, prefix: str) -> Dict[str, str]:
    given = params.get("names") or {}
    return {role: prefix + given.get(role, default) for role, default in _ROLES.items()}


@register_mixer("latent_attention")
class LatentAttention:
    @staticmethod
    def tensors(params: Mapping, prefix: str) -> Dict[str, TensorInfo]:
        w, h, d, r, dv = params["hidden_size"], params["num_heads"], params["qk_dim"], params["rot_dim"], params["v_dim"]
        qr, kr = params["q_rank"], params["kv_rank"]
        nm = _names(params, prefix)
        t = {nm["dq"]: TensorInfo((qr, w), "matrix"), nm["dq_norm"]: TensorInfo((qr,), "vector"),
             nm["uq"]: TensorInfo((h * (d + r), qr), "matrix"), nm["dkv"]: TensorInfo((kr + r, w), "matrix"),
             nm["dkv_norm"]: TensorInfo((kr,), "vector"), nm["uk"]: TensorInfo((h * d, kr), "matrix"),
             nm["uv"]: TensorInfo((h * dv, kr), "matrix"), nm["o"]: TensorInfo((w, h * dv), "matrix")}
        if params.get("gate", True):
            t[nm["gate"]] = TensorInfo((h, w), "matrix")
        if params.get("sink", False):
            t[nm["sink"]] = TensorInfo((h,), "vector", False, 0.0)
        return t

    def __init__(self, params: Mapping, prefix: str, weights, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.n_heads = int(params["num_heads"])
        self.qk_dim = int(params["qk_dim"])
        self.rot_dim = int(params["rot_dim"])
        self.v_dim = int(params["v_dim"])
        self.q_rank = int(params["q_rank"])
        self.kv_rank = int(params["kv_rank"])
        self.scale = float(params["scale"])
        self.eps = float(params["eps"])
        self.window: Optional[int] = params.get("window")
        self.has_gate = bool(params.get("gate", True))
        if self.kv_rank > 512:
            raise ValueError(f"latent_attention: latents of up to 512 are served, got kv_rank={self.kv_rank}")
        pos: PartSpec = params.get("position") or PartSpec("none")
        self.position = POSITIONS.get(pos.kind)(pos.params, max(self.rot_dim, 2), rt) if self.rot_dim else POSITIONS.get("none")({}, 0, rt)
        if self.position.rotary_dim not in (0, self.rot_dim):
            raise ValueError(f"latent_attention: the rotation covers the whole rotated part ({self.rot_dim} dims), got {self.position.rotary_dim}")
        nm = _names(params, prefix)
        names, rows = [nm["dq"], nm["dkv"]], [self.q_rank, self.kv_rank + self.rot_dim]
        if self.has_gate:
            names.append(nm["gate"])
            rows.append(self.n_heads)
        self.w_in = weights.load_fused(names, rows, self.hidden)    # one product for everything that reads the mixer's input
        self.dkv_off = self.q_rank
        self.gate_col = self.q_rank + self.kv_rank + self.rot_dim
        self.w_uq = weights.load(nm["uq"], "matrix")
        self.w_o = weights.load(nm["o"], "matrix")
        self.dq_norm_w = weights.load(nm["dq_norm"], "vector")
        self.dkv_norm_w = weights.load(nm["dkv_norm"], "vector")
        self.sink = weights.load(nm["sink"], "vector").to(torch.float32).contiguous() if params.get("sink", False) else None
        H, d, dv, kr = self.n_heads, self.qk_dim, self.v_dim, self.kv_rank
        w_uk = weights.load(nm["uk"], "matrix")      # [H*d, kr]
        w_uv = weights.load(nm["uv"], "matrix")      # [H*dv, kr]
        # per head: q_lat = q_plain @ W_uk,h ([d, kr]) and o = o_lat @ W_uv,h^T ([kr, dv]), both with the input index first
        self.w_uk = w_uk.reshape(H, d, kr).contiguous()
        self.w_uv_t = w_uv.reshape(H, dv, kr).transpose(1, 2).contiguous()
        K.latent_attn_lib()
        # prompts whose sequences all start at position 0 (bfloat16): keys and values per head from the step's own latents
        # (one product), then the library's tensor-core prompt attention over pages of the step's own
        hd = d + self.rot_dim
        self.use_prompt_tc = rt.is_bf16 and hd % 16 == 0 and hd <= 256 and dv <= hd and rt.page_size == 64
        self.uses_fresh_steps = self.use_prompt_tc
        if self.use_prompt_tc and self.sink is not None:
            # with a sink the prompt kernel is the one that opens its softmax with it (values padded to the key size)
            self.use_prompt_tc = self.uses_fresh_steps = K.pool_attention_prefill_supported(hd, hd, 1, rt.page_size)
        if self.use_prompt_tc:
            self.w_ukv = torch.cat([w_uk, w_uv], dim=0).contiguous()      # [H*d + H*dv, kr]
            if self.sink is not None:
                K.pool_attention_prefill_lib(hd, hd, 1, rt.page_size)
            else:
                K.attention_prefill_lib(hd, 1, rt.page_size)

    def kv_need(self) -> KVNeed:
        return KVNeed(1, self.kv_rank + self.rot_dim, self.window, values=False)

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: CacheEntry, state, owns_cache: bool = True) -> torch.Tensor:
        if not owns_cache:
            raise ValueError("latent_attention: every layer writes its own latents")
        n, dev, H = h.shape[0], h.device, self.n_heads
        d, r, dv, kr = self.qk_dim, self.rot_dim, self.v_dim, self.kv_rank
        proj = linear(h, self.w_in, self.rt)
        cq = torch.empty((n, self.q_rank), dtype=h.dtype, device=dev)
        lo = getattr(self.position, "inv_freq_lo", None)
        fresh = self.use_prompt_tc and ctx.fresh and not ctx.decode and ctx.n_tiles > 0 and ctx.tile_size <= 64
        c_rows = torch.empty((n, kr), dtype=h.dtype, device=dev) if fresh else None
        K.latent_prep(proj, 0, self.q_rank, self.dq_norm_w, self.dkv_off, kr, r, self.dkv_norm_w, self.eps, self.position.inv_freq,
                      self.position.interleaved, ctx.tok_slot, ctx.tok_pos, cq, cache.k, cache.page_table, inv_freq_lo=lo, c_out=c_rows)
        q = linear(cq, self.w_uq, self.rt).view(n, H, d + r)
        if fresh:
            page, hd = self.rt.page_size, d + r
            kv = linear(c_rows, self.w_ukv, self.rt)                      # [n, H*d | H*dv]
            n_pages = n // page + ctx.n_seqs + 1
            k_s = torch.zeros((n_pages, H, page, hd), dtype=h.dtype, device=dev)
            v_s = torch.zeros((n_pages, H, page, hd), dtype=h.dtype, device=dev)
            table = torch.zeros((cache.page_table.shape[0], (n + page - 1) // page + 1), dtype=torch.int32, device=dev)
            q_full = torch.empty((n, H, hd), dtype=h.dtype, device=dev)
            K.latent_expand_store(q, kv, H * d, proj, self.dkv_off + kr, self.position.inv_freq, self.position.interleaved, ctx.cu_q,
                                  ctx.seq_slot, ctx.n_seqs, ctx.tok_slot, ctx.tok_pos, table, q_full, k_s, v_s, d, r, dv, inv_freq_lo=lo)
            o_pad = torch.empty((n, H * hd), dtype=h.dtype, device=dev)
            if self.sink is not None:
                K.pool_attn_prefill(q_full, k_s, v_s, table, None, self.sink, ctx.tile_tok0, ctx.tile_rows, ctx.tok_slot, ctx.tok_pos,
                                    o_pad.view(n, H, hd), ctx.n_tiles, self.scale, self.window or (1 << 30), 0)
            else:
                K.attn_prefill(q_full, k_s, v_s, table, ctx.tile_tok0, ctx.tile_rows, ctx.tok_slot, ctx.tok_pos, o_pad, ctx.n_tiles,
                               self.scale, self.window)
            out = torch.empty((n, H * dv), dtype=h.dtype, device=dev)
            K.head_gate_rows(o_pad, proj if self.has_gate else None, self.gate_col, out, H, dv)
            return linear(out, self.w_o, self.rt)
        # few tokens, and everything in 32-bit: kernels of this library (sums in a fixed order, the same whether the step is
        # captured in a graph or not); bfloat16 steps of many tokens: one batched library product over the heads
        fits = 4 * (d + 8 * kr) <= 48 * 1024 and 4 * (kr + 8 * dv) <= 48 * 1024     # the kernels' shared memory
        own = fits and (h.dtype == torch.float32 or n <= self.rt.small_m_max)
        if own:
            q_lat = torch.empty((H, n, kr), dtype=torch.float32, device=dev)
            K.latent_fold_q(q, self.w_uk, q_lat, d)
        else:
            q_lat = torch.bmm(q[:, :, :d].transpose(0, 1), self.w_uk, out_dtype=torch.float32)
        o_lat = torch.empty((H, n, kr), dtype=h.dtype, device=dev)
        K.latent_attn_rows(q_lat, q, d, cache.k, cache.page_table, ctx.tok_slot, ctx.tok_pos, self.position.inv_freq,
                           self.position.interleaved, o_lat, kr, r, self.scale, self.window,
                           inv_freq_lo=lo, n_splits=self._n_splits(n, ctx.max_kv), sink=self.sink)
        out = torch.empty((n, H * dv), dtype=h.dtype, device=dev)
        if own:
            K.latent_unfold_o(o_lat, self.w_uv_t, proj if self.has_gate else None, self.gate_col, out)
        else:
            K.head_gate(torch.bmm(o_lat, self.w_uv_t, out_dtype=torch.float32), proj if self.has_gate else None, self.gate_col, out)
        return linear(out, self.w_o, self.rt)

    HEADS_PER_BLOCK, KEYS_PER_TILE = 16, 32     # csrc/latent_attn.cu

    def _n_splits(self, n_rows: int, max_kv: int) -> int:
        """Blocks that share a token's visible keys: enough to fill the device when the step has few tokens, a tile of keys
        per block at least and 32 splits at most.  (A prompt step has a block per token and group of heads already.)"""
        span = max(1, min(max_kv, self.window) if self.window else max_kv)
        tiles = (span + self.KEYS_PER_TILE - 1) // self.KEYS_PER_TILE + 1
        blocks = n_rows * ((self.n_heads + self.HEADS_PER_BLOCK - 1) // self.HEADS_PER_BLOCK)
        return max(1, min(32, tiles, (2 * self.rt.sm_count) // max(1, blocks)))
