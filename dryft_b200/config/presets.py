"""Named ``config.json`` contents: the two tiny test configurations and the three
benchmark shapes.  These are data fed to ``config_from_dict`` exactly as a model
folder's ``config.json`` would be; nothing else in the package refers to them.

The tiny shape follows ``agent/verify.py:36-54`` (2 layers, width 64, 4/2 heads,
head size 16, intermediate 128, vocabulary 256, tied); the second tiny shape differs
from it in every size and option.  The 4B shape is the checkpoint the reference pins
(``engine/dryft_qwen3/config.py:55-70``).
"""

from __future__ import annotations


def _qwen3(**kw) -> dict:
    base = {
        "architectures": ["Qwen3ForCausalLM"],
        "model_type": "qwen3",
        "hidden_act": "silu",
        "attention_bias": False,
        "rope_scaling": None,
        "use_sliding_window": False,
    }
    base.update(kw)
    return base


PRESETS = {
    "tiny-a": _qwen3(
        num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
        intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
        tie_word_embeddings=True, max_position_embeddings=128,
    ),
    "tiny-b": _qwen3(
        num_hidden_layers=3, hidden_size=80, num_attention_heads=6, num_key_value_heads=3, head_dim=32,
        intermediate_size=224, vocab_size=384, rope_theta=1000000.0, rms_norm_eps=1e-5,
        tie_word_embeddings=False, max_position_embeddings=256,
    ),
    "qwen3-4b": _qwen3(
        num_hidden_layers=36, hidden_size=2560, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
        intermediate_size=9728, vocab_size=151936, rope_theta=5000000.0, rms_norm_eps=1e-6,
        tie_word_embeddings=True, max_position_embeddings=8192,
    ),
    "qwen3-8b": _qwen3(
        num_hidden_layers=36, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
        intermediate_size=12288, vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6,
        tie_word_embeddings=False, max_position_embeddings=8192,
    ),
    "qwen3-32b": _qwen3(
        num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, head_dim=128,
        intermediate_size=25600, vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6,
        tie_word_embeddings=False, max_position_embeddings=16384,
    ),
}


def _tevovik(width: int, layers: int, heads: int, kv_heads: int, dim: int, vdim: int, chunk: int, experts: int, ff: int, top: int,
             groups: int, keep: int, vocab: int, share_every: int = 3) -> dict:
    """A Tevovik ``config.json``: every ``share_every``-th layer reads the keys and values of the layer before it."""
    out = []
    for i in range(layers):
        mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5, "diff": 0.4,
                 "mask": {"size": chunk}}
        if share_every and i % share_every == share_every - 1:
            mixer["kv_from"] = i - 1
        out.append({"type": "attention", "mixer": mixer,
                    "mlp": {"kind": "moe", "expert": {"ff": ff},
                            "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}}}})
    return {"architecture": "Tevovik", "vocab": vocab, "width": width, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
            "layers": out}


# Tevovik shapes with layers the size of a real model's, and beside each the dense Qwen3 shape of equal size: the same
# width, layer count, head counts and vocabulary, a head size equal to the value size, and an intermediate size equal
# to the expert size times the experts a token uses (equal weights read and equal flops per token).
PRESETS.update({
    "tevovik-tiny": _tevovik(width=64, layers=3, heads=4, kv_heads=2, dim=16, vdim=32, chunk=48, experts=8, ff=32, top=2,
                             groups=4, keep=2, vocab=256),
    "tevovik-1k": _tevovik(width=1024, layers=8, heads=8, kv_heads=2, dim=64, vdim=128, chunk=1024, experts=32, ff=512, top=4,
                           groups=4, keep=2, vocab=32768),
    "qwen3-1k": _qwen3(
        num_hidden_layers=8, hidden_size=1024, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
        intermediate_size=2048, vocab_size=32768, rope_theta=1000000.0, rms_norm_eps=1e-6,
        tie_word_embeddings=False, max_position_embeddings=8192,
    ),
    "tevovik-2k": _tevovik(width=2048, layers=12, heads=16, kv_heads=4, dim=64, vdim=128, chunk=2048, experts=64, ff=768, top=8,
                           groups=8, keep=4, vocab=65536),
    "qwen3-2k": _qwen3(
        num_hidden_layers=12, hidden_size=2048, num_attention_heads=16, num_key_value_heads=4, head_dim=128,
        intermediate_size=6144, vocab_size=65536, rope_theta=1000000.0, rms_norm_eps=1e-6,
        tie_word_embeddings=False, max_position_embeddings=8192,
    ),
})
EQUAL_SIZE = {"tevovik-1k": "qwen3-1k", "tevovik-2k": "qwen3-2k"}   # a Tevovik shape -> the dense shape of equal size


def _vobusun(width: int, heads: int, head_dim: int, ff: int, vocab: int, repeats: int, window: int, q_rank: int, kv_rank: int,
             rot_dim: int, rec_blocks: int, streams: int = 4) -> dict:
    """A Vobusun ``config.json``: a group of four layers (gated recurrence, two retention layers, latent attention) run
    ``repeats`` times, every run after the first with the first group's weights and a state of its own."""
    decay = [1.0 - 2.0 ** (-4.5 - 6.0 * h / max(1, heads - 1)) for h in range(heads)]   # memories of 20 to 1,400 tokens
    mlp = {"kind": "dense", "ff": ff, "limit": 7.0}
    ret = {"type": "retention", "mlp": mlp,
           "mixer": {"heads": heads, "dim": head_dim, "vdim": head_dim, "decay": decay, "rot": {"dims": head_dim, "base": 500000.0}}}
    group = [
        {"type": "rglru", "mixer": {"width": width, "conv": 4, "blocks": rec_blocks}, "mlp": mlp},
        ret, ret,
        {"type": "latent_attention", "mlp": mlp,
         "mixer": {"heads": heads, "dim": head_dim, "rot_dim": rot_dim, "vdim": head_dim, "q_rank": q_rank, "kv_rank": kv_rank,
                   "scale": (head_dim + rot_dim) ** -0.5, "rot": {"dims": rot_dim, "base": 20000.0}, "mask": {"size": window}}},
    ]
    layers = [dict(l) for l in group]
    for _ in range(repeats - 1):
        layers += [dict(l, weights_of=j) for j, l in enumerate(group)]
    return {"architecture": "Vobusun", "vocab": vocab, "width": width, "embedding": {"scale": width ** 0.5, "bigram": {"buckets": 65521, "mul_prev": 1009, "mul_cur": 31}},
            "norm": {"eps": 1e-5}, "residual_mult": 0.5, "streams": streams, "layers": layers}


# Vobusun shapes with layers the size of a real model's, and beside each the dense Qwen3 shape of equal size (the same width,
# layer count, head count, head size, intermediate size and vocabulary).
PRESETS.update({
    "vobusun-tiny": _vobusun(width=64, heads=2, head_dim=16, ff=96, vocab=256, repeats=2, window=48, q_rank=24, kv_rank=32,
                             rot_dim=8, rec_blocks=4, streams=2),
    "vobusun-1k": _vobusun(width=1024, heads=8, head_dim=128, ff=2048, vocab=32768, repeats=2, window=1024, q_rank=384,
                           kv_rank=256, rot_dim=64, rec_blocks=8),
    "vobusun-2k": _vobusun(width=2048, heads=16, head_dim=128, ff=6144, vocab=65536, repeats=3, window=1024, q_rank=768,
                           kv_rank=512, rot_dim=64, rec_blocks=16),
})
EQUAL_SIZE.update({"vobusun-1k": "qwen3-1k", "vobusun-2k": "qwen3-2k"})


def _mogelix(width: int, layers: int, heads: int, kv_heads: int, dim: int, window: int, pool: int, experts: int, ff: int, top: int,
             vocab: int, ssm_heads: int, ssm_vdim: int, state: int, share_every: int = 3, ssm_every: int = 4) -> dict:
    """A Mogelix ``config.json``: every ``ssm_every``-th layer is a state-space mixer; of the attention layers every
    ``share_every``-th reads the keys and values of the nearest earlier attention layer that has its own.  The first layer's
    feed-forward is dense (the size of the experts a token uses plus the always-on one), the others are routed."""
    rot = {"dims": dim, "base": 500000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}
    out, owner, n_att = [], None, 0
    for i in range(layers):
        mlp = {"kind": "dense", "ff": ff * (top + 1)} if i == 0 else \
            {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}, "shared": {"ff": ff}}
        if ssm_every and i % ssm_every == ssm_every - 1:
            out.append({"type": "mamba2", "mlp": mlp,
                        "mixer": {"heads": ssm_heads, "vdim": ssm_vdim, "state": state, "groups": 1, "conv": 4, "norm_groups": 1}})
            continue
        mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
                 "mask": {"size": window, "pool": pool}, "rot": rot}
        n_att += 1
        if share_every and owner is not None and n_att % share_every == 0:
            mixer["kv_from"] = owner
        else:
            owner = i
        out.append({"type": "attention", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Mogelix", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "postln_alpha": 2.0, "layers": out}


# Mogelix shapes with layers the size of a real model's, and beside each the closest design at equal size: the Tevovik shape
# of the same width, layer count, head counts, expert count and size, experts a token uses and vocabulary (queries and keys
# of 128 against maps of 64 twice; the window equals the chunk).
PRESETS.update({
    "mogelix-tiny": _mogelix(width=64, layers=5, heads=4, kv_heads=2, dim=16, window=40, pool=8, experts=6, ff=32, top=2, vocab=256,
                             ssm_heads=4, ssm_vdim=16, state=16),
    "mogelix-1k": _mogelix(width=1024, layers=8, heads=8, kv_heads=2, dim=128, window=1024, pool=64, experts=32, ff=512, top=4,
                           vocab=32768, ssm_heads=16, ssm_vdim=128, state=128),
    "mogelix-2k": _mogelix(width=2048, layers=12, heads=16, kv_heads=4, dim=128, window=2048, pool=64, experts=64, ff=768, top=8,
                           vocab=65536, ssm_heads=32, ssm_vdim=128, state=128),
})
EQUAL_SIZE.update({"mogelix-1k": "tevovik-1k", "mogelix-2k": "tevovik-2k"})


def _kerirax(width: int, heads: int, kv_heads: int, dim: int, inner: int, state: int, dt_rank: int, q_rank: int, kv_rank: int,
             rot_dim: int, experts: int, ff: int, top: int, vocab: int, stretch: int, times: int, tail: int) -> dict:
    """A Kerirax ``config.json``: a stretch of ``stretch`` layers run ``times`` times, then ``tail`` more layers; every third
    layer is attention over latents, the others two mixers side by side.  The first layer's feed-forward is dense (the size
    of the experts a token uses plus one), the others are routed."""
    rot = {"dims": dim, "base": 500000.0, "scaling": {"factor": 8.0}}
    pair = {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "rot": rot}, "left_scale": 1.0,
            "right": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": 4}, "right_scale": 1.0}
    lat = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": dim, "q_rank": q_rank, "kv_rank": kv_rank,
           "scale": (dim + rot_dim) ** -0.5, "rot": {"dims": rot_dim, "base": 10000.0}}
    out = []
    for i in range(stretch + tail):
        mlp = {"kind": "dense", "ff": ff * (top + 1)} if i == 0 else \
            {"kind": "moe", "expert": {"ff": ff, "limit": 7.0}, "router": {"experts": experts, "top": top}}
        out.append({"type": "latent_attention", "mixer": lat, "mlp": mlp} if i % 3 == 1 else {"type": "parallel", "mixer": pair, "mlp": mlp})
    return {"architecture": "Kerirax", "vocab": vocab, "width": width, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
            "logit_softcap": 50.0, "loop": {"start": 0, "stop": stretch, "times": times}, "layers": out}


# Kerirax shapes with layers the size of a real model's, and beside each the closest design at equal size: the Mogelix shape
# of the same width, number of layer runs (a layer that runs three times counts three times), head counts and size, expert
# count and size, experts a token uses and vocabulary (its state-space layers carry a matrix state per head where the
# selective scan carries a vector per channel).
PRESETS.update({
    "kerirax-tiny": _kerirax(width=64, heads=4, kv_heads=2, dim=16, inner=96, state=8, dt_rank=8, q_rank=24, kv_rank=32, rot_dim=8,
                             experts=6, ff=32, top=2, vocab=256, stretch=2, times=2, tail=1),
    "kerirax-1k": _kerirax(width=1024, heads=8, kv_heads=2, dim=128, inner=2048, state=16, dt_rank=64, q_rank=384, kv_rank=256,
                           rot_dim=64, experts=32, ff=512, top=4, vocab=32768, stretch=2, times=3, tail=2),
    "kerirax-2k": _kerirax(width=2048, heads=16, kv_heads=4, dim=128, inner=4096, state=16, dt_rank=128, q_rank=768, kv_rank=512,
                           rot_dim=64, experts=64, ff=768, top=8, vocab=65536, stretch=3, times=3, tail=3),
})
EQUAL_SIZE.update({"kerirax-1k": "mogelix-1k", "kerirax-2k": "mogelix-2k"})


def preset(name: str) -> dict:
    if name not in PRESETS:
        raise KeyError(f"unknown preset {name!r}; known: " + ", ".join(sorted(PRESETS)))
    return dict(PRESETS[name])
