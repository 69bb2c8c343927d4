"""The Mogelix configuration on the CPU: keys and errors, the spec it yields (parts, tensor names, who reads whose keys),
random model folders read back, and properties of the plain implementation's mechanisms, one by one."""

import copy
import math

import pytest
import torch

import mogelix_models as M
import plain_mogelix as P
from dryft_b200.config import ConfigError, MogelixConfig, config_from_dict, preset
from dryft_b200.weights import expected_tensors

F = torch.float64


def test_every_configuration_is_read_and_round_trips():
    for name, raw in M.CONFIGS.items():
        cfg = config_from_dict(copy.deepcopy(raw))
        assert isinstance(cfg, MogelixConfig)
        assert cfg.to_dict() == raw, name
        spec = cfg.model_spec()
        assert len(spec.schedule) == len(raw["layers"])
        for st, l in zip(spec.schedule, raw["layers"]):
            assert st.cache_from == l["mixer"].get("kv_from"), name


def test_tensor_names_and_shapes_are_the_tests_own_weights():
    for name, raw in M.CONFIGS.items():
        want = {k: tuple(v.shape) for k, v in M.draw_weights(raw, 1).items()}
        exp = expected_tensors(config_from_dict(raw).model_spec())
        got = {k: tuple(v.shape) for k, v in exp.items() if not v.optional or k in want}
        assert got == want, name


def test_presets_parse_and_pair_with_an_equal_size_model():
    from dryft_b200.config.presets import EQUAL_SIZE

    for name in ("mogelix-tiny", "mogelix-1k", "mogelix-2k"):
        cfg = config_from_dict(preset(name))
        kinds = [l.type for l in cfg.layers]
        assert "attention" in kinds and "mamba2" in kinds
        assert any(l.mixer.get("kv_from") is not None for l in cfg.layers)
    assert EQUAL_SIZE["mogelix-1k"] == "tevovik-1k"


@pytest.mark.parametrize("edit, text", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["layers"][0].update(type="retention"), "not a mixer"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][2]["mixer"].update(groups=3), "groups"),
    (lambda c: c["layers"][2]["mixer"].update(norm_groups=7), "norm_groups"),
    (lambda c: c["layers"][1]["mixer"].update(kv_from=1), "earlier"),
    (lambda c: c["layers"][5]["mixer"].update(kv_from=1), "of its own"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=4), "another"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "feed-forward"),
])
def test_a_wrong_configuration_is_refused_by_name(edit, text):
    raw = copy.deepcopy(M.CONFIGS["mixed"])
    edit(raw)
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw).model_spec()
    assert text in str(e.value)


# ----------------------------------------------------------------------------- the plain mechanisms, one by one
def test_rotary_frequencies_keep_short_waves_and_slow_long_ones():
    rot = {"dims": 16, "base": 10000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}
    plain = P.rotary_frequencies({"dims": 16, "base": 10000.0})
    f = P.rotary_frequencies(rot)
    wave = 2 * math.pi / plain
    assert torch.equal(f[wave < 16], plain[wave < 16])
    assert torch.allclose(f[wave > 64], plain[wave > 64] / 8.0)
    mid = (wave >= 16) & (wave <= 64)
    assert mid.any() and bool(((f[mid] < plain[mid]) & (f[mid] > plain[mid] / 8.0)).all())


def test_rotation_turns_pairs_half_apart_and_leaves_the_rest():
    x = torch.randn(5, 2, 12, dtype=F)
    freqs = torch.tensor([0.3, 0.01, 1.1], dtype=F)
    y = P.rotate(x, torch.arange(5), freqs)
    assert torch.equal(y[..., 6:], x[..., 6:]) and torch.equal(y[0], x[0])
    assert torch.allclose(y[..., :6].pow(2).sum(-1), x[..., :6].pow(2).sum(-1))
    a = 3 * 0.01
    assert torch.allclose(y[3, 1, 1], x[3, 1, 1] * math.cos(a) - x[3, 1, 4] * math.sin(a))
    # scores depend on the distance only
    q, k = torch.randn(1, 1, 6, dtype=F), torch.randn(1, 1, 6, dtype=F)
    s = lambda i, j: (P.rotate(q, torch.tensor([i]), freqs) * P.rotate(k, torch.tensor([j]), freqs)).sum()
    assert torch.allclose(s(9, 4), s(105, 100))


def test_window_and_blocks_at_their_edges():
    size, pool = 7, 3
    toks, blocks = P.visible(6, size, pool)
    assert toks == list(range(7)) and blocks == []
    toks, blocks = P.visible(9, size, pool)          # positions 3..9 in the window; block 0 (0..2) lies wholly before it
    assert toks == list(range(3, 10)) and blocks == [0]
    toks, blocks = P.visible(11, size, pool)         # 5..11 seen; block 1 (3..5) is cut by the window: position 3, 4 not seen at all
    assert toks == list(range(5, 12)) and blocks == [0]
    toks, blocks = P.visible(12, size, pool)
    assert toks == list(range(6, 13)) and blocks == [0, 1]
    assert P.visible(39, 5, 12) == (list(range(35, 40)), [0, 1])     # blocks longer than the window: 24..34 unseen
    assert P.visible(40, 5, 12) == (list(range(36, 41)), [0, 1, 2])


def test_a_key_that_stands_out_is_found_in_the_window_in_a_block_and_nowhere_else():
    torch.manual_seed(0)
    L, size, pool = 40, 6, 4
    k = 0.05 * torch.randn(L, 1, 8, dtype=F)
    v = torch.zeros(L, 1, 3, dtype=F)
    q = torch.zeros(L, 1, 8, dtype=F)
    q[:, 0, 0] = 1.0
    k[9, 0, 0], v[9, 0, 1] = 60.0, 1.0               # one key and value that stand out, at position 9 (block 2: 8..11)
    out = P.pooled_window_attention(q, k, v, torch.tensor([-30.0], dtype=F), 1.0, size, pool)[:, 0, 1]
    assert out[8] == 0 and out[9] > 0.99 and out[14] > 0.99            # in the window up to 9 + size - 1
    assert out[15] < 1e-6 and out[16] < 1e-6                            # left the window, its block not yet wholly before it
    assert abs(float(out[17]) - 0.25) < 0.01                            # block 2 seen from 11 + size: the mean of four values
    assert abs(float(out[39]) - 0.25) < 0.01


def test_the_sink_takes_its_share_without_key_or_value():
    q = torch.zeros(1, 2, 4, dtype=F)
    k = torch.zeros(1, 1, 4, dtype=F)
    v = torch.ones(1, 1, 2, dtype=F)
    out = P.pooled_window_attention(q, k, v, torch.tensor([0.0, math.log(3.0)], dtype=F), 5.0, 4, 2)
    assert torch.allclose(out[0, 0], torch.full((2,), 0.5, dtype=F)) and torch.allclose(out[0, 1], torch.full((2,), 0.25, dtype=F))


def test_convolution_reads_zeros_before_the_start_and_its_last_column_is_now():
    x = torch.arange(1.0, 6.0, dtype=F)[:, None]
    cw = torch.tensor([[100.0, 10.0, 1.0]], dtype=F)
    out = P.causal_conv(x, cw, torch.tensor([0.5], dtype=F))[:, 0]
    assert out.tolist() == [1.5, 12.5, 123.5, 234.5, 345.5]


def test_the_scan_decays_per_head_and_reads_its_groups_inputs():
    L, Hh, dv, N = 6, 4, 2, 3
    x, dt = torch.randn(L, Hh, dv, dtype=F), torch.rand(L, Hh, dtype=F)
    B, C = torch.randn(L, 2, N, dtype=F), torch.randn(L, 2, N, dtype=F)
    a, D = torch.tensor([0.1, 1.0, 2.0, 0.5], dtype=F), torch.randn(Hh, dtype=F)
    y = P.ssm_scan(x, dt, a, B, C, D)
    # the closed form: y_t = sum_{s<=t} exp(-a sum_{s<r<=t} dt_r) dt_s (C_t . B_s) x_s + D x_t
    for hh in (0, 3):
        g = hh // 2
        for t in (0, 5):
            want = D[hh] * x[t, hh]
            for s in range(t + 1):
                want = want + torch.exp(-a[hh] * dt[s + 1:t + 1, hh].sum()) * dt[s, hh] * (C[t, g] @ B[s, g]) * x[s, hh]
            assert torch.allclose(y[t, hh], want)


def test_polynorm_and_the_router():
    z = torch.randn(3, 10, dtype=F)
    out = P.poly_norm(z, torch.tensor([0.0, 0.0, 2.0, -1.0], dtype=F), 0.0)
    assert torch.allclose(((out + 1.0) / 2.0).pow(2).mean(-1), torch.ones(3, dtype=F))
    h = torch.randn(4, 6, dtype=F)
    idx, wt = P.route(h, torch.randn(5, 6, dtype=F), torch.tensor([0.0, 0.0, 50.0, 0.0, 0.0], dtype=F), 2)
    assert (idx[:, 0] == 2).all() and torch.allclose(wt.sum(-1), torch.ones(4, dtype=F)) and (wt[:, 0] > 0.99).all()


def test_a_layer_without_keys_reads_the_earlier_layers_rows():
    cfg = M.CONFIGS["att_shared"]
    w = M.draw_weights(cfg, 3)
    toks = M.prompts(cfg, [50], seed=1)[0]
    base = P.forward(cfg, w, toks)
    w2 = dict(w)
    w2["l0.mix.v.b"] = w["l0.mix.v.b"] + 1.0          # the owner's values move: every reader's output moves with them
    taps, taps2 = [], []
    P.forward(cfg, w, toks, lambda i, x: taps.append(x.clone()))
    P.forward(cfg, w2, toks, lambda i, x: taps2.append(x.clone()))
    assert not torch.allclose(taps[0], taps2[0]) and base.shape == (50, cfg["vocab"])
    assert torch.isfinite(base).all()
