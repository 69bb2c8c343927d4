"""Typed configuration of the Kerirax decoder, read from its own ``config.json`` keys.

The design: a 32-bit residual stream; per layer ONE norm whose output both the mixer and the feed-forward read, their
results joining the stream together (``x <- x + mixer(n) + ff(n)``); a stretch of layers that runs several times in a row
with the same weights and a cache or state per pass, entered every time through ``x <- W [x | x0] + step[t]`` (``x0`` the
embedding's output); two kinds of mixer -- attention over low-rank latents with a sink in the softmax's denominator, and
two mixers side by side whose results are added with fixed factors: grouped-query attention (a norm over the whole query /
key projection, interleaved rotation with every frequency divided by a factor, a sigmoid gate per head) and a selective
scan with one decay per (channel, state) behind a short convolution; two kinds of feed-forward -- a gated dense one, and
routed experts with sigmoid scores that weight the expert's input, whose activation is clamped; and logits squashed by
``cap * tanh(. / cap)``.

    architecture        "Kerirax"
    vocab, width, logit_softcap (absent: none)
    embedding.scale     (absent: 1)
    norm.eps
    loop                absent, or start, stop, times: layers start .. stop-1 run ``times`` times in a row
    layers[i].type      "latent_attention" | "parallel"
    layers[i].mixer     latent_attention: heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot.{dims, base}
                        parallel: left.{heads, kv_heads, dim, vdim, scale, rot.{dims, base, scaling.factor}}, left_scale,
                                  right.{inner, state, dt_rank, conv}, right_scale
    layers[i].mlp       null, or kind "dense" with ff, or kind "moe" with expert.{ff, limit}, router.{experts, top}

Tensors: ``embed``, ``loop.in``, ``loop.step``, ``final.norm``, ``head`` and per layer ``l<i>.norm1``, ``l<i>.mix.*``,
``l<i>.mlp.*``.  What the design fixes is a constant below; everything ``config.json`` gives is read from there.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Mapping, Optional, Tuple

from .mogelix import _mapping
from .qwen3 import ConfigError
from .spec import ExtraPart, LayerSpec, ModelSpec, PartSpec, RunStep
from .vobusun import _number, _pos_int

EXPERT_ALPHA = 1.702        # an expert's activation is g * sigmoid(EXPERT_ALPHA * g) * (u + EXPERT_UP_OFFSET)
EXPERT_UP_OFFSET = 1.0
DEFAULT_MAX_POSITIONS = 1 << 20   # the design has no longest sequence; the engine's own limits apply
MIXER_TYPES = ("latent_attention", "parallel")
MLP_KINDS = ("dense", "moe")


def _rot(m: Mapping[str, Any], where: str, limit: int, scaling: bool) -> Optional[Mapping[str, Any]]:
    rot = _mapping(m, "rot", where, optional=True)
    if rot is None:
        return None
    dims, base = _pos_int(rot, "dims", where + ".rot"), _number(rot, "base", where + ".rot")
    if dims % 2 or dims > limit:
        raise ConfigError(f"config.json: {where}.rot.dims must be even and at most {limit}, got {dims}")
    if not base > 0.0:
        raise ConfigError(f"config.json: {where}.rot.base must be positive, got {base!r}")
    sc = _mapping(rot, "scaling", where + ".rot", optional=True)
    if sc is not None:
        if not scaling:
            raise ConfigError(f"config.json: {where}.rot.scaling is not part of this mixer")
        if not _number(sc, "factor", where + ".rot.scaling") > 0.0:
            raise ConfigError(f"config.json: {where}.rot.scaling.factor must be positive")
    return rot


def _check_latent(m: Mapping[str, Any], where: str) -> None:
    for key in ("heads", "dim", "vdim", "q_rank", "kv_rank"):
        _pos_int(m, key, where)
    rot_dim = m.get("rot_dim", 0)
    if isinstance(rot_dim, bool) or not isinstance(rot_dim, int) or rot_dim < 0 or rot_dim % 2:
        raise ConfigError(f"config.json: {where}.rot_dim must be an even integer >= 0, got {rot_dim!r}")
    _number(m, "scale", where)
    rot = _rot(m, where, max(rot_dim, 2), scaling=False)
    if rot_dim and (rot is None or rot["dims"] != rot_dim):
        raise ConfigError(f"config.json: {where}.rot.dims must equal rot_dim ({rot_dim})")


def _check_pair(m: Mapping[str, Any], where: str) -> None:
    left, right = _mapping(m, "left", where), _mapping(m, "right", where)
    lw, rw = where + ".left", where + ".right"
    heads, kv = _pos_int(left, "heads", lw), _pos_int(left, "kv_heads", lw)
    dim = _pos_int(left, "dim", lw)
    _pos_int(left, "vdim", lw)
    if heads % kv:
        raise ConfigError(f"config.json: {lw}.heads ({heads}) must be a multiple of kv_heads ({kv})")
    _number(left, "scale", lw)
    _rot(left, lw, dim, scaling=True)
    for key in ("inner", "state", "dt_rank", "conv"):
        _pos_int(right, key, rw)
    for key in ("left_scale", "right_scale"):
        if key in m:
            _number(m, key, where)


@dataclass(frozen=True)
class KeriraxLayer:
    type: str
    mixer: Mapping[str, Any]                 # the validated mixer sizes, as config.json gives them
    mlp: Optional[Mapping[str, Any]]         # the validated feed-forward description, or None


@dataclass(frozen=True)
class KeriraxConfig:
    vocab: int
    width: int
    norm_eps: float
    embed_scale: float
    softcap: Optional[float]
    loop: Optional[Tuple[int, int, int]]     # (start, stop, times)
    layers: Tuple[KeriraxLayer, ...]
    architecture: str = "Kerirax"

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "KeriraxConfig":
        vocab, width = _pos_int(raw, "vocab", "config"), _pos_int(raw, "width", "config")
        eps = _number(_mapping(raw, "norm", "config"), "eps", "norm")
        if not eps > 0.0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps!r}")
        emb = _mapping(raw, "embedding", "config", optional=True)
        scale = _number(emb, "scale", "embedding") if emb is not None and "scale" in emb else 1.0
        cap = None
        if raw.get("logit_softcap") is not None:
            cap = _number(raw, "logit_softcap", "config")
            if not cap > 0.0:
                raise ConfigError(f"config.json: logit_softcap must be positive, got {cap!r}")
        layers = raw.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: layers must be a non-empty list")
        out: List[KeriraxLayer] = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(layer, Mapping):
                raise ConfigError(f"config.json: {where} must be a mapping")
            kind = layer.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design (known: {', '.join(MIXER_TYPES)})")
            m = _mapping(layer, "mixer", where)
            (_check_latent if kind == "latent_attention" else _check_pair)(m, where + ".mixer")
            mlp = _mapping(layer, "mlp", where, optional=True)
            if mlp is not None:
                lw = where + ".mlp"
                if mlp.get("kind") not in MLP_KINDS:
                    raise ConfigError(f"config.json: {lw}.kind {mlp.get('kind')!r} is not a feed-forward of this design "
                                      f"(known: {', '.join(MLP_KINDS)})")
                if mlp["kind"] == "dense":
                    _pos_int(mlp, "ff", lw)
                else:
                    ex = _mapping(mlp, "expert", lw)
                    _pos_int(ex, "ff", lw + ".expert")
                    if ex.get("limit") is not None and not _number(ex, "limit", lw + ".expert") > 0.0:
                        raise ConfigError(f"config.json: {lw}.expert.limit must be positive")
                    r = _mapping(mlp, "router", lw)
                    experts, top = _pos_int(r, "experts", lw + ".router"), _pos_int(r, "top", lw + ".router")
                    if top > experts:
                        raise ConfigError(f"config.json: {lw}.router.top ({top}) exceeds experts ({experts})")
            out.append(KeriraxLayer(kind, dict(m), dict(mlp) if mlp is not None else None))
        loop = None
        lp = _mapping(raw, "loop", "config", optional=True)
        if lp is not None:
            times = _pos_int(lp, "times", "loop")
            start, stop = lp.get("start"), lp.get("stop")
            for key, v in (("start", start), ("stop", stop)):
                if isinstance(v, bool) or not isinstance(v, int):
                    raise ConfigError(f"config.json: loop.{key} must be an integer, got {v!r}")
            if not 0 <= start < stop <= len(out):
                raise ConfigError(f"config.json: loop.start .. loop.stop must name layers in order, got {start} .. {stop} of {len(out)}")
            loop = (start, stop, times)
        arch = raw.get("architecture") or (raw.get("architectures") or ["Kerirax"])[0]
        return cls(vocab, width, eps, scale, cap, loop, tuple(out), str(arch))

    def to_dict(self) -> dict:
        """The ``config.json`` this configuration is read back from."""
        layers = [{"type": l.type, "mixer": dict(l.mixer), "mlp": dict(l.mlp) if l.mlp is not None else None} for l in self.layers]
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "embedding": {"scale": self.embed_scale}, "layers": layers}
        if self.softcap is not None:
            d["logit_softcap"] = self.softcap
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return d

    # ------------------------------------------------------------------ the run order
    def run_order(self) -> List[Tuple[int, Optional[int]]]:
        """``(layer, pass it opens or None)`` in the order the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        start, stop, times = self.loop
        order: List[Tuple[int, Optional[int]]] = [(i, None) for i in range(start)]
        for t in range(times):
            order += [(i, t if i == start else None) for i in range(start, stop)]
        return order + [(i, None) for i in range(stop, n)]

    # ------------------------------------------------------------------ accounting (benchmarks)
    def _mixer_weights(self, l: KeriraxLayer) -> int:
        w, m = self.width, l.mixer
        if l.type == "latent_attention":
            r = m.get("rot_dim", 0)
            return ((m["q_rank"] + m["kv_rank"] + r) * w + m["heads"] * (m["dim"] + r) * m["q_rank"]
                    + m["heads"] * (m["dim"] + m["vdim"]) * m["kv_rank"] + w * m["heads"] * m["vdim"])
        a, s = m["left"], m["right"]
        n = (a["heads"] * a["dim"] + a["kv_heads"] * (a["dim"] + a["vdim"]) + a["heads"]) * w + w * a["heads"] * a["vdim"]
        n += 2 * s["inner"] * w + (s["dt_rank"] + 2 * s["state"]) * s["inner"] + s["inner"] * s["dt_rank"] + w * s["inner"]
        return n

    def _mlp_weights(self, l: KeriraxLayer, experts_read: Optional[int]) -> int:
        """Feed-forward weights a token passes through (``experts_read=None``: its ``top`` experts) or a step reads."""
        w, f = self.width, l.mlp
        if f is None:
            return 0
        if f["kind"] == "dense":
            return 3 * f["ff"] * w
        r = f["router"]
        return r["experts"] * w + (r["top"] if experts_read is None else min(r["experts"], experts_read)) * 3 * f["expert"]["ff"] * w

    def weight_bytes_per_decode_step(self, itemsize: int, batch: int = 1) -> int:
        """Bytes of weights one decode step of ``batch`` tokens reads at least: every layer run's matrices (a layer that runs
        several times is read every time), the experts the tokens choose, the entry matrix per pass and the output head."""
        total = self.vocab * self.width
        for i, opens in self.run_order():
            l = self.layers[i]
            top = l.mlp["router"]["top"] if l.mlp is not None and l.mlp["kind"] == "moe" else 0
            total += self._mixer_weights(l) + self._mlp_weights(l, batch * top)
            if opens is not None:
                total += 2 * self.width * self.width
        return itemsize * total

    def matmul_flops_per_token(self) -> int:
        """Multiply-add flops of the weight matrices one token passes through, output head excluded."""
        total = 0
        for i, opens in self.run_order():
            l = self.layers[i]
            total += self._mixer_weights(l) + self._mlp_weights(l, None) + (2 * self.width * self.width if opens is not None else 0)
        return 2 * total

    # ------------------------------------------------------------------ the parts of each layer
    def _mixer_spec(self, l: KeriraxLayer) -> PartSpec:
        m, w = l.mixer, self.width

        def rope(rot: Optional[Mapping[str, Any]]) -> Optional[PartSpec]:
            if rot is None:
                return None
            sc = rot.get("scaling")
            return PartSpec("rope", {"theta": float(rot["base"]), "rotary_dim": int(rot["dims"]), "layout": "interleaved",
                                     "freq": "rounded_once", "scaling": {"factor": float(sc["factor"])} if sc else None})

        if l.type == "latent_attention":
            return PartSpec("latent_attention", {
                "hidden_size": w, "num_heads": m["heads"], "qk_dim": m["dim"], "rot_dim": m.get("rot_dim", 0), "v_dim": m["vdim"],
                "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "scale": float(m["scale"]), "eps": self.norm_eps, "window": None,
                "gate": False, "sink": True, "position": rope(m.get("rot")) if m.get("rot_dim", 0) else None,
                "names": {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv",
                          "o": "o", "sink": "sink"}})
        a, s = m["left"], m["right"]
        left = PartSpec("pooled_window_attention", {
            "hidden_size": w, "num_heads": a["heads"], "num_kv_heads": a["kv_heads"], "qk_dim": a["dim"], "v_dim": a["vdim"],
            "scale": float(a["scale"]), "window": None, "pool": None, "eps": self.norm_eps, "own_kv": True, "position": rope(a.get("rot")),
            "sink": False, "bias": False, "unit_norm": False, "proj_norm": True, "head_gate": True,
            "names": {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "gate": "g"}})
        right = PartSpec("selective_scan", {
            "hidden_size": w, "inner": s["inner"], "state": s["state"], "dt_rank": s["dt_rank"], "taps": s["conv"],
            "names": {"in": "in", "conv": "conv", "conv_bias": "conv.b", "x": "x", "dt": "dt", "dt_bias": "dt.b", "a_log": "A_log",
                      "d": "D", "o": "o"}})
        return PartSpec("side_by_side", {"left": left, "right": right, "left_scale": float(m.get("left_scale", 1.0)),
                                         "right_scale": float(m.get("right_scale", 1.0))})

    def _ffn_spec(self, l: KeriraxLayer) -> Optional[PartSpec]:
        f = l.mlp
        if f is None:
            return None
        if f["kind"] == "dense":
            return PartSpec("clamped_glu", {"hidden_size": self.width, "intermediate_size": f["ff"], "limit": None, "alpha": 1.0,
                                            "up_offset": 0.0, "names": {"gate": "gate", "up": "up", "down": "down"}})
        return PartSpec("moe", {
            "hidden_size": self.width, "intermediate_size": f["expert"]["ff"], "experts": f["router"]["experts"],
            "top": f["router"]["top"], "groups": 1, "keep": 1, "renormalize": False, "score": "sigmoid", "weight_input": True,
            "activation": "clamped", "limit": f["expert"].get("limit"), "alpha": EXPERT_ALPHA, "up_offset": EXPERT_UP_OFFSET,
            "names": {"router": "router", "expert": "e{}.", "gate": "gate", "up": "up", "down": "down"}})

    def model_spec(self) -> ModelSpec:
        def norm(name: str) -> PartSpec:
            # the stored weight is the factor itself: an offset of zero
            return PartSpec("rmsnorm_offset", {"size": self.width, "eps": self.norm_eps, "offset": 0.0, "name": name})

        specs = []
        for i, l in enumerate(self.layers):
            specs.append(LayerSpec(
                block="parallel", mixer=self._mixer_spec(l), ffn=self._ffn_spec(l), norm_mixer=norm("norm1"), norm_ffn=None,
                mixer_prefix=f"l{i}.mix.", ffn_prefix=f"l{i}.mlp.", norm_mixer_prefix=f"l{i}.", norm_ffn_prefix=f"l{i}."))
        joints = ()
        if self.loop is not None:
            joints = (ExtraPart("loop", "connection", PartSpec("loop_mix", {"size": self.width, "times": self.loop[2], "matrix": "in",
                                                                            "steps": "step"}), "loop."),)
        spec = ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab,
            hidden_size=self.width,
            max_positions=DEFAULT_MAX_POSITIONS,
            embedding=PartSpec("pair_embedding", {"vocab_size": self.vocab, "hidden_size": self.width, "name": "embed",
                                                  "scale": self.embed_scale, "pair": None, "norm": None}),
            layers=tuple(specs),
            schedule=tuple(RunStep(layer=i, enter=("loop", t) if t is not None else None) for i, t in self.run_order()),
            final_norm=norm("final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied": False, "name": "head",
                                      "softcap": self.softcap}),
            embedding_prefix="",
            final_norm_prefix="",
            head_prefix="",
            joints=joints,
        )
        spec.validate()
        return spec
