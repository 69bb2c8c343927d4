"""The Kerirax configuration on the CPU: keys and errors, the run order of a repeated stretch, the spec and its tensor names
against the tests' own weights, random model folders, and properties of the plain mechanisms one by one (they are the
yardstick of the GPU tests, so they are checked against closed forms here)."""

import math

import pytest
import torch

import kerirax_models as M
import plain_kerirax as P

from dryft_b200.config import ConfigError, KeriraxConfig, config_from_dict
from dryft_b200.weights.expected import expected_tensors


@pytest.mark.parametrize("name", list(M.CONFIGS))
def test_tensor_names_and_shapes_are_those_of_the_tests_own_weights(name):
    cfg = M.CONFIGS[name]
    conf = config_from_dict(cfg)
    assert isinstance(conf, KeriraxConfig)
    want = M.draw_weights(cfg, seed=1)
    got = expected_tensors(conf.model_spec())
    assert set(got) == set(want)
    for k, info in got.items():
        assert tuple(info.shape) == tuple(want[k].shape), k
    again = config_from_dict(conf.to_dict())
    assert again == conf


def test_run_order_of_a_repeated_stretch():
    conf = config_from_dict(M.CONFIGS["looped"])          # layers 1 and 2, twice
    assert conf.run_order() == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    spec = conf.model_spec()
    assert [(s.layer, s.enter) for s in spec.schedule] == [(0, None), (1, ("loop", 0)), (2, None), (1, ("loop", 1)), (2, None), (3, None)]
    assert [j.name for j in spec.joints] == ["loop"]
    assert P.run_order(M.CONFIGS["looped"]) == [(0, None, False), (1, 0, True), (2, 0, False), (1, 1, True), (2, 1, False), (3, None, False)]
    plain = config_from_dict(M.CONFIGS["pair"])
    assert plain.model_spec().joints == () and plain.run_order() == [(0, None)]
    assert config_from_dict(M.CONFIGS["once"]).run_order() == [(0, None), (1, 0)]     # a stretch that runs once is still entered


@pytest.mark.parametrize("change, message", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
    (lambda c: c["layers"][0].update(type="attention"), "type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["right"].pop("dt_rank"), "dt_rank"),
    (lambda c: c["layers"][1]["mixer"].update(rot_dim=4), "rot.dims"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][1]["mlp"].update(kind="glu"), "kind"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(times=0), "times"),
    (lambda c: c.update(logit_softcap=-1.0), "logit_softcap"),
])
def test_errors_name_the_key(change, message):
    import copy

    cfg = copy.deepcopy(M.CONFIGS["looped"])
    change(cfg)
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert message in str(e.value)


def test_random_model_folder_and_accounting(tmp_path):
    import json
    import os

    from dryft_b200.weights import write_random_model

    conf = config_from_dict(M.CONFIGS["looped"])
    d = write_random_model(conf, 3, str(tmp_path / "m"))
    with open(os.path.join(d, "config.json")) as f:
        assert config_from_dict(json.load(f)) == conf
    # a layer that runs twice is read twice, and every pass reads the entry matrix
    once = config_from_dict({**M.CONFIGS["looped"], "loop": {"start": 1, "stop": 3, "times": 1}})
    w = conf.width
    extra = conf.weight_bytes_per_decode_step(2) - once.weight_bytes_per_decode_step(2)
    assert extra == 2 * (conf._mixer_weights(conf.layers[1]) + conf._mlp_weights(conf.layers[1], 2) + conf._mixer_weights(conf.layers[2])
                         + conf._mlp_weights(conf.layers[2], 2) + 2 * w * w)
    assert conf.matmul_flops_per_token() > once.matmul_flops_per_token()


# ----------------------------------------------------------------------------- the plain mechanisms against closed forms
def test_rotation_pairs_neighbours_and_depends_on_distance_only():
    rot = {"dims": 6, "base": 50.0, "scaling": {"factor": 4.0}}
    f = P.rotary_frequencies(rot)
    assert torch.allclose(f, torch.tensor([1.0, 50.0 ** (-1 / 3), 50.0 ** (-2 / 3)], dtype=torch.float64) / 4.0)
    v = torch.zeros(1, 8, dtype=torch.float64)
    v[0, 2] = 1.0                                              # the first of the second pair
    out = P.rotate_pairs(v, torch.tensor([3]), rot)[0]
    a = 3 * float(f[1])
    assert torch.allclose(out, torch.tensor([0, 0, math.cos(a), math.sin(a), 0, 0, 0, 0], dtype=torch.float64))
    q, k = torch.randn(1, 8, dtype=torch.float64), torch.randn(1, 8, dtype=torch.float64)
    dots = [float((P.rotate_pairs(q, torch.tensor([p + 5]), rot) * P.rotate_pairs(k, torch.tensor([p]), rot)).sum()) for p in (0, 9, 400)]
    assert max(dots) - min(dots) < 1e-9
    assert torch.equal(P.rotate_pairs(q, torch.tensor([7]), rot)[0, 6:], q[0, 6:])       # dims behind rot.dims pass unchanged


def test_sink_takes_its_share_and_the_mask_is_causal():
    q = torch.zeros(4, 2, dtype=torch.float64)
    k = torch.zeros(4, 2, dtype=torch.float64)
    v = torch.arange(8, dtype=torch.float64).view(4, 2)
    out = P.causal_softmax_attention(q, k, v, 1.0)            # equal scores: the mean of the visible values
    assert torch.allclose(out[2], v[:3].mean(0))
    out = P.causal_softmax_attention(q, k, v, 1.0, sink=0.0)  # one more unit in the denominator, nothing in the numerator
    assert torch.allclose(out[2], v[:3].sum(0) / 4.0)
    out = P.causal_softmax_attention(q, k, v, 5.0, sink=math.log(3.0))   # the sink is not scaled
    assert torch.allclose(out[0], v[0] / 4.0)


def test_convolution_and_scan_against_their_closed_forms():
    x = torch.arange(1.0, 6.0, dtype=torch.float64)[:, None]
    w = torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64)          # the last column is the current token's
    out = P.causal_conv(x, w, torch.tensor([0.5], dtype=torch.float64))[:, 0]
    assert out.tolist() == [1.5, 12.5, 123.5, 234.5, 345.5]
    # one channel, one state, constant inputs: S_t = a S_(t-1) + b with a = exp(dt A), b = dt x B
    p = {"inner": 1, "state": 1, "dt_rank": 1, "conv": 1}
    one = lambda v: torch.tensor([[v]], dtype=torch.float64)
    wts = {"m.in": torch.tensor([[1.0], [0.0]], dtype=torch.float64), "m.conv": one(1.0), "m.conv.b": torch.zeros(1, dtype=torch.float64),
           "m.x": torch.tensor([[0.0], [0.0], [0.0]], dtype=torch.float64), "m.dt": one(0.0), "m.dt.b": torch.tensor([0.3], dtype=torch.float64),
           "m.A_log": one(math.log(2.0)), "m.D": torch.tensor([0.25], dtype=torch.float64), "m.o": one(1.0)}
    h = torch.full((5, 1), 2.0, dtype=torch.float64)
    y = P.selective_scan_mixer(h, p, wts, "m.")[:, 0]
    xs = 2.0 / (1.0 + math.exp(-2.0))                          # silu of the convolved input
    assert torch.allclose(y, torch.full((5,), 0.25 * xs * 0.0, dtype=torch.float64))      # z = 0: the gate closes the output
    wts["m.in"] = torch.tensor([[1.0], [1.0]], dtype=torch.float64)
    wts["m.x"] = torch.tensor([[0.0], [1.0], [1.0]], dtype=torch.float64)                  # B = C = x
    y = P.selective_scan_mixer(h, p, wts, "m.")[:, 0]
    dt = math.log1p(math.exp(0.3))
    a, b, S, want = math.exp(-2.0 * dt), dt * xs * xs, 0.0, []
    for _ in range(5):
        S = a * S + b
        want.append((S * xs + 0.25 * xs) * xs)                 # silu(z) = silu(2) = xs
    assert torch.allclose(y, torch.tensor(want, dtype=torch.float64))


def test_router_weights_scale_the_input_and_are_not_rescaled():
    torch.manual_seed(0)
    mlp = M.moe(ff=4, experts=3, top=2, limit=0.7)
    W = 6
    w = {"f.router": torch.randn(3, W, dtype=torch.float64)}
    for e in range(3):
        w[f"f.e{e}.gate"], w[f"f.e{e}.up"], w[f"f.e{e}.down"] = (torch.randn(4, W, dtype=torch.float64), torch.randn(4, W, dtype=torch.float64),
                                                                torch.randn(W, 4, dtype=torch.float64))
    h = torch.randn(5, W, dtype=torch.float64)
    idx, wts = P.router_choice(h, mlp, w, "f.")
    s = torch.sigmoid(h @ w["f.router"].T)
    assert torch.equal(idx, s.topk(2).indices) and torch.allclose(wts, s.topk(2).values)
    assert float(wts.sum(-1).min()) != pytest.approx(1.0)
    got = P.moe_ffn(h, mlp, w, "f.")
    t, want = 3, torch.zeros(W, dtype=torch.float64)
    for k in range(2):
        e = int(idx[t, k])
        x = wts[t, k] * h[t]
        g, u = torch.clamp(w[f"f.e{e}.gate"] @ x, max=0.7), torch.clamp(w[f"f.e{e}.up"] @ x, min=-0.7, max=0.7)
        want += w[f"f.e{e}.down"] @ (g * torch.sigmoid(1.702 * g) * (u + 1.0))
    assert torch.allclose(got[t], want)


def test_one_norm_feeds_both_sublayers_and_the_logits_are_squashed():
    cfg = M.CONFIGS["pair"]
    tensors = M.draw_weights(cfg, seed=2)
    toks = M.prompts(cfg, [12], seed=1)[0]
    seen = []
    lg = P.forward(cfg, tensors, toks, lambda i, x: seen.append(x))
    assert len(seen) == 1 and float(lg.abs().max()) < cfg["logit_softcap"]
    w = {k: v.double() for k, v in tensors.items()}
    x = w["embed"][torch.tensor(toks)] * cfg["embedding"]["scale"]
    n = P.rms_norm(x, w["l0.norm1"], cfg["norm"]["eps"])
    want = x + P.side_by_side_mixer(n, cfg["layers"][0]["mixer"], w, "l0.mix.", cfg["norm"]["eps"]) + P.dense_ffn(n, w, "l0.mlp.")
    assert torch.allclose(seen[0], want)
