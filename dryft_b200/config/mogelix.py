"""Typed configuration of the Mogelix decoder, read from its own ``config.json`` keys.

The design: a 32-bit residual stream whose norm comes AFTER each sum (``x <- norm(alpha x + g * f(x))``, the sublayers read
the stream itself, ``g`` a sigmoid gate per element computed from the sublayer's input); two kinds of mixer -- attention
over a sliding window plus one pooled key and value per block of positions that has left the window, with a sink in the
softmax's denominator, rotary positions whose long waves are slowed, unit-norm queries and keys, and layers that read an
earlier layer's keys and values; and a selective state-space mixer (state-space duality form) behind a short convolution;
and two kinds of feed-forward -- a dense one with a polynomial activation normalised over the token's vector, and routed
experts with a squared-relu activation beside an always-on expert with a gate per token.

    architecture        "Mogelix"
    vocab, width, postln_alpha
    norm.eps
    layers[i].type      "attention" | "mamba2"
    layers[i].mixer     attention: heads, kv_heads, dim, vdim, scale, rot.{dims, base, scaling.{factor, low, high, original}},
                                   mask.{size, pool}, kv_from (the layer whose keys and values this one reads)
                        mamba2: heads, vdim, state, groups, conv, norm_groups
    layers[i].mlp       null, or kind "dense" with ff, or kind "moe" with expert.ff, router.{experts, top}, shared.ff

Tensors: ``embed``, ``final.norm``, ``head`` and per layer ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.rg1`` (+ ``.b``), ``l<i>.rg2``
(+ ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.*``.  What the design fixes is in the parts; everything ``config.json`` gives is read
from there.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple

from .qwen3 import ConfigError
from .spec import ExtraPart, LayerSpec, ModelSpec, PartSpec, RunStep
from .vobusun import _number, _pos_int

DEFAULT_MAX_POSITIONS = 1 << 20   # the design has no longest sequence; the engine's own limits apply
MIXER_TYPES = ("attention", "mamba2")
MLP_KINDS = ("dense", "moe")


def _mapping(d: Mapping[str, Any], key: str, where: str, optional: bool = False) -> Optional[Mapping[str, Any]]:
    v = d.get(key)
    if v is None:
        if optional:
            return None
        raise ConfigError(f"config.json: {where}.{key} is missing")
    if not isinstance(v, Mapping):
        raise ConfigError(f"config.json: {where}.{key} must be a mapping")
    return v


def _check_attention(m: Mapping[str, Any], where: str) -> None:
    heads, kv = _pos_int(m, "heads", where), _pos_int(m, "kv_heads", where)
    dim = _pos_int(m, "dim", where)
    _pos_int(m, "vdim", where)
    if heads % kv:
        raise ConfigError(f"config.json: {where}.heads ({heads}) must be a multiple of kv_heads ({kv})")
    _number(m, "scale", where)
    rot = _mapping(m, "rot", where, optional=True)
    if rot is not None:
        dims, base = _pos_int(rot, "dims", where + ".rot"), _number(rot, "base", where + ".rot")
        if dims % 2 or dims > dim:
            raise ConfigError(f"config.json: {where}.rot.dims must be even and at most dim ({dim}), got {dims}")
        if not base > 0.0:
            raise ConfigError(f"config.json: {where}.rot.base must be positive, got {base!r}")
        sc = _mapping(rot, "scaling", where + ".rot", optional=True)
        if sc is not None:
            f, lo, hi, orig = (_number(sc, k, where + ".rot.scaling") for k in ("factor", "low", "high", "original"))
            if not (f > 0.0 and orig > 0.0 and hi > lo):
                raise ConfigError(f"config.json: {where}.rot.scaling needs factor > 0, original > 0 and high > low")
    mask = _mapping(m, "mask", where, optional=True)
    if mask is not None:
        _pos_int(mask, "size", where + ".mask")
        if mask.get("pool") is not None:
            _pos_int(mask, "pool", where + ".mask")


def _check_mamba2(m: Mapping[str, Any], where: str) -> None:
    heads, groups = _pos_int(m, "heads", where), _pos_int(m, "groups", where)
    inner = heads * _pos_int(m, "vdim", where)
    _pos_int(m, "state", where)
    _pos_int(m, "conv", where)
    parts = _pos_int(m, "norm_groups", where)
    if heads % groups:
        raise ConfigError(f"config.json: {where}.heads ({heads}) must be a multiple of groups ({groups})")
    if inner % parts:
        raise ConfigError(f"config.json: {where}.norm_groups ({parts}) must divide heads * vdim ({inner})")


@dataclass(frozen=True)
class MogelixLayer:
    type: str
    mixer: Mapping[str, Any]                 # the validated mixer sizes, as config.json gives them
    mlp: Optional[Mapping[str, Any]]         # the validated feed-forward description, or None

    @property
    def kv_from(self) -> Optional[int]:
        return self.mixer.get("kv_from") if self.type == "attention" else None


@dataclass(frozen=True)
class MogelixConfig:
    vocab: int
    width: int
    norm_eps: float
    alpha: float
    layers: Tuple[MogelixLayer, ...]
    architecture: str = "Mogelix"

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "MogelixConfig":
        vocab, width = _pos_int(raw, "vocab", "config"), _pos_int(raw, "width", "config")
        eps = _number(_mapping(raw, "norm", "config"), "eps", "norm")
        if not eps > 0.0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps!r}")
        alpha = _number(raw, "postln_alpha", "config") if "postln_alpha" in raw else 1.0
        layers = raw.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: layers must be a non-empty list")
        out: List[MogelixLayer] = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(layer, Mapping):
                raise ConfigError(f"config.json: {where} must be a mapping")
            kind = layer.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design (known: {', '.join(MIXER_TYPES)})")
            m = _mapping(layer, "mixer", where)
            if kind == "attention":
                _check_attention(m, where + ".mixer")
            else:
                _check_mamba2(m, where + ".mixer")
            mlp = _mapping(layer, "mlp", where, optional=True)
            if mlp is not None:
                lw = where + ".mlp"
                if mlp.get("kind") not in MLP_KINDS:
                    raise ConfigError(f"config.json: {lw}.kind {mlp.get('kind')!r} is not a feed-forward of this design "
                                      f"(known: {', '.join(MLP_KINDS)})")
                if mlp["kind"] == "dense":
                    _pos_int(mlp, "ff", lw)
                else:
                    _pos_int(_mapping(mlp, "expert", lw), "ff", lw + ".expert")
                    r = _mapping(mlp, "router", lw)
                    experts, top = _pos_int(r, "experts", lw + ".router"), _pos_int(r, "top", lw + ".router")
                    if top > experts:
                        raise ConfigError(f"config.json: {lw}.router.top ({top}) exceeds experts ({experts})")
                    sh = _mapping(mlp, "shared", lw, optional=True)
                    if sh is not None:
                        _pos_int(sh, "ff", lw + ".shared")
            out.append(MogelixLayer(kind, dict(m), dict(mlp) if mlp is not None else None))
        for i, l in enumerate(out):
            src = l.kv_from
            if src is None:
                continue
            where = f"layers[{i}].mixer.kv_from"
            if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
                raise ConfigError(f"config.json: {where} must name an earlier layer, got {src!r}")
            o = out[src]
            if o.type != "attention" or o.kv_from is not None:
                raise ConfigError(f"config.json: {where} names layers[{src}], which has no keys and values of its own")
            for key in ("kv_heads", "dim", "vdim"):
                if o.mixer[key] != l.mixer[key]:
                    raise ConfigError(f"config.json: {where}: layers[{src}] has another {key} ({o.mixer[key]} against {l.mixer[key]})")
        arch = raw.get("architecture") or (raw.get("architectures") or ["Mogelix"])[0]
        return cls(vocab, width, eps, alpha, tuple(out), str(arch))

    def to_dict(self) -> dict:
        """The ``config.json`` this configuration is read back from."""
        layers = [{"type": l.type, "mixer": dict(l.mixer), "mlp": dict(l.mlp) if l.mlp is not None else None} for l in self.layers]
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "postln_alpha": self.alpha, "layers": layers}

    # ------------------------------------------------------------------ accounting (benchmarks)
    def _mixer_weights(self, l: MogelixLayer) -> int:
        w, m = self.width, l.mixer
        if l.type == "attention":
            n = m["heads"] * m["dim"] * w + w * m["heads"] * m["vdim"]
            if l.kv_from is None:
                n += m["kv_heads"] * (m["dim"] + m["vdim"]) * w
            return n
        inner = m["heads"] * m["vdim"]
        return (2 * inner + 2 * m["groups"] * m["state"] + m["heads"]) * w + w * inner

    def _mlp_weights(self, l: MogelixLayer, experts_read: Optional[int]) -> int:
        """Feed-forward weights a token passes through (``experts_read=None``: its ``top`` experts) or a step reads."""
        w, f = self.width, l.mlp
        if f is None:
            return 0
        if f["kind"] == "dense":
            return 2 * f["ff"] * w
        r = f["router"]
        n = r["experts"] * w + (r["top"] if experts_read is None else min(r["experts"], experts_read)) * 2 * f["expert"]["ff"] * w
        if f.get("shared") is not None:
            n += 2 * f["shared"]["ff"] * w + w
        return n

    def weight_bytes_per_decode_step(self, itemsize: int, batch: int = 1) -> int:
        """Bytes of weights one decode step of ``batch`` tokens reads at least: the projections, both residual gates, the
        experts the tokens choose (at most ``batch * top`` distinct ones per layer) and the output head."""
        total = self.vocab * self.width
        for l in self.layers:
            top = l.mlp["router"]["top"] if l.mlp is not None and l.mlp["kind"] == "moe" else 0
            total += self._mixer_weights(l) + self._mlp_weights(l, batch * top)
            total += self.width * self.width * (2 if l.mlp is not None else 1)
        return itemsize * total

    def matmul_flops_per_token(self) -> int:
        """Multiply-add flops of the weight matrices one token passes through, output head excluded."""
        total = 0
        for l in self.layers:
            total += self._mixer_weights(l) + self._mlp_weights(l, None) + self.width * self.width * (2 if l.mlp is not None else 1)
        return 2 * total

    # ------------------------------------------------------------------ the parts of each layer
    def _mixer_spec(self, l: MogelixLayer) -> PartSpec:
        m, w = l.mixer, self.width
        if l.type == "attention":
            position = None
            rot = m.get("rot")
            if rot is not None:
                position = PartSpec("rope", {"theta": float(rot["base"]), "rotary_dim": int(rot["dims"]), "layout": "half",
                                             "freq": "rounded_once", "scaling": dict(rot["scaling"]) if rot.get("scaling") else None})
            mask = m.get("mask") or {}
            return PartSpec("pooled_window_attention", {
                "hidden_size": w, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "qk_dim": m["dim"], "v_dim": m["vdim"],
                "scale": float(m["scale"]), "window": mask.get("size"), "pool": mask.get("pool"), "eps": self.norm_eps,
                "own_kv": l.kv_from is None, "position": position, "sink": True, "bias": True, "unit_norm": True,
                "names": {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "sink": "sink"}})
        return PartSpec("ssd", {
            "hidden_size": w, "num_heads": m["heads"], "v_dim": m["vdim"], "state": m["state"], "groups": m["groups"],
            "taps": m["conv"], "norm_groups": m["norm_groups"], "eps": self.norm_eps,
            "names": {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "a_log": "A_log", "d": "D",
                      "norm": "norm", "o": "o"}})

    def _ffn_spec(self, l: MogelixLayer) -> Optional[PartSpec]:
        f = l.mlp
        if f is None:
            return None
        if f["kind"] == "dense":
            return PartSpec("polynorm_mlp", {"hidden_size": self.width, "intermediate_size": f["ff"], "eps": self.norm_eps,
                                             "names": {"up": "up", "down": "down", "act": "act"}})
        shared = None
        if f.get("shared") is not None:
            shared = {"intermediate_size": f["shared"]["ff"], "gate": True}
        return PartSpec("moe", {
            "hidden_size": self.width, "intermediate_size": f["expert"]["ff"], "experts": f["router"]["experts"],
            "top": f["router"]["top"], "groups": 1, "keep": 1, "renormalize": True, "activation": "relu2", "router_bias": True,
            "shared": shared,
            "names": {"router": "router", "router_bias": "router.b", "expert": "e{}.", "up": "up", "down": "down",
                      "shared": "shared.", "shared_gate": "shared.sg"}})

    def model_spec(self) -> ModelSpec:
        def norm(name: str) -> PartSpec:
            # the stored weight is the factor itself: an offset of zero
            return PartSpec("rmsnorm_offset", {"size": self.width, "eps": self.norm_eps, "offset": 0.0, "name": name})

        def gate(name: str) -> PartSpec:
            # how a sublayer's result joins the stream: keep * x + sigmoid(W h + b) * result, the norm behind the sum
            return PartSpec("gated_sum", {"size": self.width, "keep": self.alpha, "gate": name, "gate_bias": name + ".b"})

        specs = []
        for i, l in enumerate(self.layers):
            ffn = self._ffn_spec(l)
            extra = [ExtraPart("gate_mixer", "connection", gate("rg1"), f"l{i}.")]
            if ffn is not None:
                extra.append(ExtraPart("gate_ffn", "connection", gate("rg2"), f"l{i}."))
            specs.append(LayerSpec(
                block="postnorm", mixer=self._mixer_spec(l), ffn=ffn, norm_mixer=norm("norm1"),
                norm_ffn=norm("norm2") if ffn is not None else None, mixer_prefix=f"l{i}.mix.", ffn_prefix=f"l{i}.mlp.",
                norm_mixer_prefix=f"l{i}.", norm_ffn_prefix=f"l{i}.", extra=tuple(extra)))
        spec = ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab,
            hidden_size=self.width,
            max_positions=DEFAULT_MAX_POSITIONS,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": self.width, "name": "embed", "stream32": True}),
            layers=tuple(specs),
            schedule=tuple(RunStep(layer=i, cache_from=l.kv_from) for i, l in enumerate(self.layers)),
            final_norm=norm("final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied": False, "name": "head"}),
            embedding_prefix="",
            final_norm_prefix="",
            head_prefix="",
        )
        spec.validate()
        return spec
