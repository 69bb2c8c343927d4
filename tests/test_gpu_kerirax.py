"""The Kerirax decoder in the engine against the plain evaluation (``plain_kerirax.py``), in 32-bit (sharp) and in bfloat16:
every mixer alone and mixed, stretches of layers run several times, whole prompts, prompts against token-by-token decoding,
prompts in portions down to two tokens, unequal batches against each request alone, slots, states and pages used again
(poisoned), long decoding across page edges, the first tokens, the stream after every layer run, greedy generation through
``Engine.generate`` / ``generate_many`` (captured graphs and eager), the replay program and the command line as child
processes, configurations drawn at random, sublayers on streams of their own against everything in turn (the same
bits); and the new kernels alone against the plain functions: the selective scan with a
memory of hundreds of tokens (in order and in chunks), the latent attention's sink with one key that outweighs all others,
the norm over whole projections with both rotation layouts, the router's sigmoid scores, the clamp's edges."""

import math

import numpy as np
import pytest
import torch

import kerirax_models as M
import plain_kerirax as P

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
_cache = {}


def model(name, tmp_path_factory):
    if name not in _cache:
        cfg = M.CONFIGS[name]
        tensors = M.draw_weights(cfg, seed=41 + len(name) + ord(name[0]))
        d = M.write_model(cfg, tensors, str(tmp_path_factory.mktemp(f"kerirax_{name}")))
        _cache[name] = (cfg, tensors, d, {})
    return _cache[name]


def plain_logits(entry, tokens):
    cfg, tensors, _, memo = entry
    key = tuple(tokens)
    if key not in memo:
        memo[key] = P.forward(cfg, tensors, list(tokens))
    return memo[key]


def engine(entry, dtype, **kw):
    from dryft_b200.engine.api import Engine, EngineOptions

    opts = dict(dtype=dtype, max_batch=8, max_seq_len=512, max_tokens=2048, cuda_graphs=False)
    opts.update(kw)
    return Engine(entry[2], EngineOptions(**opts))


def limits(entry):
    """The bfloat16 limits of this model, from what rounding alone does to a prompt of its own under the plain evaluation."""
    cfg, tensors, _, memo = entry
    if "limits" not in memo:
        memo["limits"] = M.bf16_limits(cfg, tensors, M.prompts(cfg, [120], seed=77)[0])
    return memo["limits"]


def check(entry, got, want, dtype, what):
    M.assert_close(got, want, dtype, what, limits(entry) if dtype != "float32" else None)


def close_all(entry, pairs, dtype, what):
    if dtype == "float32":
        for got, want, label in pairs:
            check(entry, got, want, dtype, f"{what}: {label}")
    else:   # a single bfloat16 row cannot be judged statistically: the rows of all pairs together
        check(entry, torch.cat([g.detach().float().cpu() for g, _, _ in pairs]), torch.cat([w for _, w, _ in pairs]), dtype, what)


def decode_together(eng, slots, batch, heads):
    """Decode the rest of every request of ``batch`` one token a step; requests end (and give back what they hold) one
    after another.  Returns request index -> list of logits rows."""
    live, step = [b for b in range(len(batch)) if heads[b] < len(batch[b])], 0
    eng.cache.close_sequences([slots[b] for b in range(len(batch)) if b not in live])
    rows = {b: [] for b in live}
    while live:
        got = eng.stepper.step([slots[b] for b in live], [[batch[b][heads[b] + step]] for b in live], [[0]] * len(live))
        for r, b in enumerate(live):
            rows[b].append(got[r:r + 1])
        step += 1
        done = [b for b in live if heads[b] + step >= len(batch[b])]
        eng.cache.close_sequences([slots[b] for b in done])
        live = [b for b in live if b not in done]
    return rows


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(M.CONFIGS))
def test_whole_prompts_decoding_portions_and_batches(tmp_path_factory, name, dtype):
    entry = model(name, tmp_path_factory)
    cfg = entry[0]
    eng = engine(entry, dtype)
    reqs = M.prompts(cfg, [1, 2, 23, 65, 131, 200], seed=3)
    with torch.inference_mode():
        # whole prompts, logits at every place (the first tokens included)
        pairs = []
        for toks in reqs:
            s = eng.cache.open_sequences(1)
            got = eng.stepper.step(s, [toks], [list(range(len(toks)))])
            eng.cache.close_sequences(s)
            pairs.append((got, plain_logits(entry, toks), f"prompt of {len(toks)}"))
        close_all(entry, pairs, dtype, f"{name} whole prompts")
        # a short head at once, the rest token by token (page edges and the convolution's start pass over decoded tokens)
        for toks, head in ((reqs[3], 1), (reqs[4], 40), (reqs[5], 129)):
            s = eng.cache.open_sequences(1)
            rows = [eng.stepper.step(s, [toks[:head]], [[head - 1]])]
            for t in range(head, len(toks)):
                rows.append(eng.stepper.step(s, [[toks[t]]], [[0]]))
            eng.cache.close_sequences(s)
            check(entry, torch.cat(rows), plain_logits(entry, toks)[head - 1:], dtype, f"{name} decoding {len(toks)} from {head}")
        # portions of several sizes, down to two tokens (a convolution's tail shorter than its taps, a state handed on)
        for portion in (2, 7, 64, 97):
            toks = reqs[4]
            s = eng.cache.open_sequences(1)
            rows = []
            for c0 in range(0, len(toks), portion):
                piece = toks[c0:c0 + portion]
                rows.append(eng.stepper.step(s, [piece], [list(range(len(piece)))]))
            eng.cache.close_sequences(s)
            check(entry, torch.cat(rows), plain_logits(entry, toks), dtype, f"{name} portions of {portion}")
        # an unequal batch of prompts (one of a single token), then decoded together; shorter requests end earlier
        batch = [reqs[2], reqs[5], reqs[3], reqs[1], reqs[0] + reqs[2]]
        heads = [max(1, len(t) - 12) for t in batch]
        slots = eng.cache.open_sequences(len(batch))
        got = eng.stepper.step(slots, [t[:h] for t, h in zip(batch, heads)], [list(range(h)) for h in heads])
        at, pairs = 0, []
        for t, h in zip(batch, heads):
            pairs.append((got[at:at + h], plain_logits(entry, t)[:h], f"prompt of {h}"))
            at += h
        close_all(entry, pairs, dtype, f"{name} batched prompts")
        rows = decode_together(eng, slots, batch, heads)
        close_all(entry, [(torch.cat(r), plain_logits(entry, batch[b])[heads[b]:], f"request {b}") for b, r in rows.items()],
                  dtype, f"{name} batched decoding")
    eng.cache.check()


@pytest.mark.parametrize("name", ["looped", "sizes"])
def test_the_stream_after_every_layer_run(tmp_path_factory, name):
    entry = model(name, tmp_path_factory)
    cfg, tensors = entry[0], entry[1]
    eng = engine(entry, "float32")
    toks = M.prompts(cfg, [90], seed=8)[0]
    want = []
    P.forward(cfg, tensors, toks, lambda i, x: want.append(x.clone()))
    got = []
    eng.model.layer_tap = lambda i, block, res: got.append(res.x.double().cpu())
    with torch.inference_mode():
        s = eng.cache.open_sequences(1)
        eng.stepper.step(s, [toks], [[0]])
        eng.cache.close_sequences(s)
    assert len(got) == len(want) == len(P.run_order(cfg)) > len(cfg["layers"])     # a layer that runs again counts again
    for i, (g, w) in enumerate(zip(got, want)):
        assert float((g - w).abs().max()) <= 2e-5 * float(w.abs().max()), f"run {i} (layer {P.run_order(cfg)[i][0]})"


@pytest.mark.parametrize("dtype", DTYPES)
def test_pages_slots_and_states_used_again_hold_nothing_of_their_last_holder(tmp_path_factory, dtype):
    entry = model("looped", tmp_path_factory)
    cfg = entry[0]
    # room for little more than one request: every request reuses the slot, the states and the pages of the one before
    eng = engine(entry, dtype, max_batch=1, max_seq_len=256, max_tokens=256)
    reqs = M.prompts(cfg, [150, 90, 201, 33], seed=5)
    with torch.inference_mode():
        for i, toks in enumerate(reqs):
            s = eng.cache.open_sequences(1)
            head = len(toks) - 9
            rows = [eng.stepper.step(s, [toks[:head]], [list(range(head))])]
            for t in range(head, len(toks)):
                rows.append(eng.stepper.step(s, [[toks[t]]], [[0]]))
            eng.cache.close_sequences(s)
            check(entry, torch.cat(rows), plain_logits(entry, toks), dtype, f"request {i} on a reused slot and pages")
            for g in eng.cache._groups:        # what the freed pages hold must never matter again
                g.k.fill_(float("nan"))
                if g.v is not None:
                    g.v.fill_(float("nan"))
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(tmp_path_factory, dtype):
    entry = model("looped", tmp_path_factory)
    cfg = entry[0]
    eng = engine(entry, dtype, max_batch=2, max_seq_len=512, max_tokens=2048)
    toks = M.prompts(cfg, [330], seed=9)[0]
    with torch.inference_mode():
        s = eng.cache.open_sequences(1)
        rows = [eng.stepper.step(s, [toks[:3]], [[0, 1, 2]])]
        for t in range(3, len(toks)):
            rows.append(eng.stepper.step(s, [[toks[t]]], [[0]]))
        eng.cache.close_sequences(s)
    check(entry, torch.cat(rows), plain_logits(entry, toks), dtype, "330 tokens, nearly all decoded one by one")
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["looped", "tc"])
def test_greedy_generation_through_the_entry_point(tmp_path_factory, name, dtype):
    entry = model(name, tmp_path_factory)
    cfg, tensors = entry[0], entry[1]
    eng = engine(entry, dtype, cuda_graphs=True, max_batch=4)
    prompts = M.prompts(cfg, [5, 19, 40], seed=21)
    n_new = 12
    steps = list(eng.generate(prompts, n_new))
    got = [[st[b] for st in steps] for b in range(len(prompts))]
    many = eng.generate_many(prompts + prompts[:2], n_new)
    assert many[:3] == got and many[3:] == got[:2]
    if dtype == "float32":
        for b, p in enumerate(prompts):
            assert got[b] == P.greedy(cfg, tensors, p, n_new), f"request {b}"
    else:
        # bfloat16 may part ways with the plain tokens at a close call, and the contexts differ from then on.  Teacher-forced
        # instead: under the plain model, fed our tokens, each of our tokens is the best one up to what rounding does
        for b, p in enumerate(prompts):
            lg = plain_logits(entry, list(p) + got[b][:-1])[len(p) - 1:]
            ours = lg.gather(1, torch.tensor(got[b])[:, None])[:, 0]
            lost = (lg.max(dim=-1).values - ours) / lg.std(dim=-1)
            assert float(lost.max()) <= 0.3, f"request {b}: token {int(lost.argmax())} loses {float(lost.max()):.3g} spreads to the plain model's best"
    eager = engine(entry, dtype, cuda_graphs=False, max_batch=4)     # graphs and eager steps choose the same tokens
    assert eager.generate_many(prompts, n_new) == got
    if dtype == "float32":
        chunked = engine(entry, dtype, cuda_graphs=False, max_batch=4, prefill_chunk_tokens=16)
        assert chunked.generate_many(prompts, n_new) == got


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_as_a_child_process(tmp_path_factory, tmp_path, dtype):
    import json
    import os
    import subprocess
    import sys

    import helpers as H

    entry = model("looped", tmp_path_factory)
    cfg = entry[0]
    reqs = M.prompts(cfg, [70, 31, 2], seed=33)
    out = str(tmp_path / "out")
    steps = [{"step": 0, "entries": [{"id": f"r{i}", "tokens": t[:-1] if len(t) > 2 else t[:1], "want": [0, len(t) - 2] if len(t) > 2 else [0]}
                                     for i, t in enumerate(reqs)], "end": []},
             {"step": 1, "entries": [{"id": f"r{i}", "tokens": [t[-1]], "want": [0]} for i, t in enumerate(reqs)], "end": ["r0", "r1", "r2"]},
             {"step": 2, "entries": [{"id": "r0", "tokens": reqs[1], "want": []}], "end": []},
             {"step": 3, "entries": [{"id": "r0", "tokens": [5], "want": [0]}], "end": ["r0"]}]
    proc = subprocess.run([sys.executable, os.path.join(H.ROOT, "bin", "trace_run"), "--model", entry[2], "--dtype", dtype,
                           "--out", out, "--max-tokens", "256"], input="".join(json.dumps(s) + "\n" for s in steps),
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [ln for ln in proc.stdout.splitlines() if ln.startswith("done")] == [f"done {i}" for i in range(4)]
    read = lambda n: torch.from_numpy(np.fromfile(os.path.join(out, f"{n}.f32"), dtype="<f4").reshape(-1, cfg["vocab"]).copy())
    want0 = torch.cat([plain_logits(entry, t)[[0, len(t) - 2] if len(t) > 2 else [0]] for t in reqs])
    check(entry, read(0), want0, dtype, "replayed prompts")
    check(entry, read(1), torch.cat([plain_logits(entry, t)[-1:] for t in reqs]), dtype, "replayed decode step")
    check(entry, read(3), plain_logits(entry, reqs[1] + [5])[-1:], dtype, "a request id used again")


def test_command_line_generates(tmp_path_factory):
    import json
    import subprocess
    import sys

    import helpers as H

    entry = model("looped", tmp_path_factory)
    cfg, tensors = entry[0], entry[1]
    base = [sys.executable, "-m", "dryft_b200", "generate", "--model", entry[2], "--dtype", "float32", "--max-batch", "4",
            "--max-seq-len", "128", "--prompt-ids", "5,17,3,60,9", "--prompt-ids", "7,7,7", "--max-new-tokens", "6"]
    greedy = subprocess.run(base, capture_output=True, text=True, timeout=600, cwd=H.ROOT)
    assert greedy.returncode == 0, greedy.stderr[-2000:]
    rows = [json.loads(ln) for ln in greedy.stdout.splitlines() if ln.startswith("{")]
    assert [r["tokens"] for r in rows] == [P.greedy(cfg, tensors, p, 6) for p in ([5, 17, 3, 60, 9], [7, 7, 7])]


@pytest.mark.parametrize("dtype", DTYPES)
def test_forty_unequal_requests_at_once(tmp_path_factory, dtype):
    """More rows than the few-row products take; requests end one after another."""
    entry = model("looped", tmp_path_factory)
    cfg = entry[0]
    eng = engine(entry, dtype, max_batch=64, max_seq_len=256, max_tokens=8192)
    reqs = M.prompts(cfg, [3 + (7 * i) % 50 for i in range(40)], seed=4)
    with torch.inference_mode():
        slots = eng.cache.open_sequences(len(reqs))
        heads = [max(1, len(r) - 5) for r in reqs]
        got = eng.stepper.step(slots, [r[:h] for r, h in zip(reqs, heads)], [[h - 1] for h in heads])
        pairs = [(got[i:i + 1], plain_logits(entry, reqs[i])[heads[i] - 1:heads[i]], f"prompt {i}") for i in range(len(reqs))]
        rows = decode_together(eng, slots, reqs, heads)
        pairs += [(torch.cat(r), plain_logits(entry, reqs[b])[heads[b]:], f"request {b}") for b, r in rows.items() if r]
    close_all(entry, pairs, dtype, "forty requests")
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_sublayers_on_streams_of_their_own_give_the_same_bits(tmp_path_factory, dtype):
    """Few-row steps run the feed-forward beside the mixer, and the two mixers of a pair beside each other, on side streams
    (parallel branches of a captured step): the logits are the same bits as with everything in turn, eagerly and replayed."""
    entry = model("looped", tmp_path_factory)
    cfg = entry[0]
    reqs = M.prompts(cfg, [70, 31, 2, 9], seed=14)
    rows = {}
    for branch in (16, 0):
        eng = engine(entry, dtype, branch_rows=branch)
        with torch.inference_mode():
            slots = eng.cache.open_sequences(len(reqs))
            got = [eng.stepper.step(slots, reqs, [[len(t) - 1] for t in reqs])]     # four rows wanted of a step of many
            for t in range(20):
                got.append(eng.stepper.step(slots, [[(7 * t + b) % cfg["vocab"]] for b in range(len(reqs))], [[0]] * len(reqs)))
            eng.cache.close_sequences(slots)
            torch.cuda.synchronize()
        rows[branch] = torch.cat(got).cpu()
        toks = engine(entry, dtype, branch_rows=branch, cuda_graphs=True, max_batch=4).generate_many(reqs, 10)
        rows[("tokens", branch)] = toks
    assert torch.equal(rows[16], rows[0])
    assert rows[("tokens", 16)] == rows[("tokens", 0)]
    want = torch.cat([plain_logits(entry, t)[-1:] for t in reqs])
    check(entry, rows[16][:len(reqs)], want, dtype, "prompts before the branched steps")


def _random_config(seed):
    """A configuration drawn at random: layer kinds and order, every size, every constant, where the repeated stretch lies."""
    import random

    r = random.Random(seed)
    even = lambda lo, hi: 2 * r.randint(lo // 2, hi // 2)
    layers = []
    for i in range(r.randint(2, 5)):
        mlp = r.choice([None, "dense", "moe", "moe"])
        if mlp == "dense":
            mlp = {"kind": "dense", "ff": r.randint(5, 70)}
        elif mlp == "moe":
            experts = r.randint(1, 9)
            mlp = M.moe(ff=r.randint(3, 40), experts=experts, top=r.randint(1, experts), limit=r.choice([None, round(r.uniform(0.5, 4.0), 2)]))
        if r.random() < 0.45:
            rot_dim = r.choice([0, even(2, 16)])
            layers.append(M.latent(heads=r.randint(1, 5), dim=r.randint(2, 30), rot_dim=rot_dim, vdim=r.randint(2, 30), q_rank=r.randint(2, 50),
                                   kv_rank=r.randint(2, 70), base=r.choice([37.0, 1000.0, 250000.0]), scale=round(r.uniform(0.2, 1.2), 3), mlp=mlp))
            continue
        kv = r.randint(1, 3)
        dim = r.randint(2, 40)
        layers.append(M.pair(heads=kv * r.randint(1, 4), kv_heads=kv, dim=dim, vdim=r.randint(2, 40), rot_dims=r.choice([None, even(2, dim)]),
                             base=r.choice([37.0, 1000.0, 250000.0]), factor=r.choice([None, round(r.uniform(1.5, 16.0), 2)]),
                             scale=round(r.uniform(0.2, 1.2), 3), inner=r.randint(3, 70), state=r.randint(1, 70), dt_rank=r.randint(1, 20),
                             conv=r.randint(1, 6), left_scale=round(r.uniform(0.3, 2.0), 2), right_scale=round(r.uniform(0.3, 2.0), 2), mlp=mlp))
    loop = None
    if r.random() < 0.75:
        start = r.randint(0, len(layers) - 1)
        loop = (start, r.randint(start + 1, len(layers)), r.randint(1, 3))
    return M.config(layers, width=r.choice([24, 36, 50, 52, 64]), vocab=r.randint(40, 300), eps=r.choice([1e-6, 1e-5, 3e-4]),
                    emb_scale=r.choice([None, round(r.uniform(0.3, 2.0), 2)]), cap=r.choice([None, round(r.uniform(5.0, 40.0), 1)]), loop=loop)


@pytest.mark.parametrize("seed", range(10))
def test_configurations_drawn_at_random(tmp_path, seed):
    cfg = _random_config(seed)
    tensors = M.draw_weights(cfg, seed=100 + seed)
    entry = (cfg, tensors, M.write_model(cfg, tensors, str(tmp_path / "m")), {})
    reqs = M.prompts(cfg, [170, 1, 33], seed=seed)
    for dtype in DTYPES:
        eng = engine(entry, dtype, max_batch=4, max_seq_len=256, max_tokens=1024)
        with torch.inference_mode():
            heads = [max(1, len(t) - 6) for t in reqs]
            slots = eng.cache.open_sequences(len(reqs))
            got = eng.stepper.step(slots, [t[:h] for t, h in zip(reqs, heads)], [list(range(h)) for h in heads])
            at, pairs = 0, []
            for t, h in zip(reqs, heads):
                pairs.append((got[at:at + h], plain_logits(entry, t)[:h], f"prompt of {h}"))
                at += h
            rows = decode_together(eng, slots, reqs, heads)
            pairs += [(torch.cat(v), plain_logits(entry, reqs[b])[heads[b]:], f"request {b} decoded") for b, v in rows.items() if v]
        what = f"random configuration {seed} ({[l['type'] for l in cfg['layers']]}, loop {cfg.get('loop')})"
        if dtype == "float32":
            close_all(entry, pairs, dtype, what)
        else:
            # heads of two or three values and widths of 24 make bfloat16 rounding large in some of these models: the sharp
            # comparison is the 32-bit one; here the typical row must be close and every row finite
            got_all = torch.cat([g.detach().float().cpu() for g, _, _ in pairs])
            assert torch.isfinite(got_all).all(), what
            e = M.row_errors(got_all, torch.cat([w for _, w, _ in pairs]))
            # ... measured against what rounding alone does to the very prompt that is tested (a router's close call in an
            # early layer moves every later row of some of these models)
            limit = M.bf16_limits(cfg, tensors, reqs[0])[0]
            assert float(e.median()) <= limit, f"{what}: median row off by {float(e.median()):.3g} (limit {limit:.3g})"
        eng.cache.check()


# ----------------------------------------------------------------------------- the new kernels alone
@pytest.mark.parametrize("inner, n_state, chunked", [(37, 5, False), (64, 16, True), (5, 300, True), (130, 1, False), (48, 40, True)])
def test_selective_scan_remembers_hundreds_of_tokens(monkeypatch, inner, n_state, chunked):
    """The scan kernel against the recurrence written out in 64-bit: several unequal sequences in one step (one of a single
    token, one that continues from a state), one channel whose decay is so slow that an input 600 tokens back still decides
    its output, in order and cut into chunks of 16 tokens."""
    from dryft_b200.ops import kernels as K

    monkeypatch.setattr(K, "SELSCAN_CHUNK_TOKENS", 16)
    torch.manual_seed(inner + n_state)
    dev = "cuda"
    lens = [700, 1, 45, 130]
    n, R = sum(lens), 3
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32, device=dev)
    slots = torch.tensor([2, 0, 5, 1], dtype=torch.int32, device=dev)
    xc = torch.randn(n, inner, device=dev)
    low = torch.randn(n, R + 2 * n_state + 3, device=dev)
    dtp = torch.randn(n, inner, device=dev) - 1.0
    zrows = torch.randn(n, inner + 7, device=dev)
    dt_bias = torch.randn(inner, device=dev) * 0.5
    a_log = torch.randn(inner, n_state, device=dev) - 1.0
    a_log[0] = -14.0                                          # channel 0 forgets next to nothing ...
    dtp[:, 0] = -2.0
    xc[:, 0] = 0.0
    xc[60, 0] = 50.0                                          # ... of the one input it ever gets
    d_skip = torch.randn(inner, device=dev)
    state = torch.zeros(8, inner, n_state, device=dev)
    state[5] = torch.randn(inner, n_state, device=dev)        # the third sequence goes on from here
    start = state.clone()
    out = torch.empty(n, inner, device=dev)
    K.selscan(xc, low, R, R + n_state, dtp, dt_bias, a_log, d_skip, zrows, 7, cu, slots, len(lens), state, out, chunked=chunked)
    torch.cuda.synchronize()
    f = lambda t: t.double().cpu()
    A = -torch.exp(f(a_log))
    worst = 0.0
    for b, L in enumerate(lens):
        t0 = int(cu[b])
        S = f(start[int(slots[b])]).clone()
        for t in range(t0, t0 + L):
            dt = P.softplus(f(dtp[t]) + f(dt_bias))
            S = torch.exp(dt[:, None] * A) * S + (dt * f(xc[t]))[:, None] * f(low[t, R:R + n_state])[None, :]
            y = S @ f(low[t, R + n_state:R + 2 * n_state]) + f(d_skip) * f(xc[t])
            want = y * P.silu(f(zrows[t, 7:7 + inner]))
            worst = max(worst, float(((f(out[t]) - want).abs() / (1.0 + want.abs())).max()))
        assert float((f(state[int(slots[b])]) - S).abs().max()) <= 1e-4 * (1.0 + float(S.abs().max())), f"state of sequence {b}"
    assert worst <= 2e-4, worst
    assert float(state[3].abs().max()) == 0.0                 # a slot nobody holds is not touched
    # the far input still decides channel 0 at the end of the long sequence
    assert abs(float(state[2, 0].abs().max())) > 1.0


@pytest.mark.parametrize("n_splits", [1, 2, 5])
@pytest.mark.parametrize("far", [0, 63, 64, 300, 698])
def test_latent_attention_sink_and_one_key_that_stands_out(far, n_splits):
    """The latent attention kernel over 700 cached rows (shuffled pages, unused rows poisoned) of which ONE, at ``far``,
    outweighs all others for every later query, with sinks that take a small, an even and nearly the whole share."""
    from dryft_b200.ops import kernels as K

    torch.manual_seed(far)
    dev, page, H, kr, L = "cuda", 64, 3, 24, 700
    c = (0.1 * torch.randn(L, kr)).double()
    c[far, 5] = 30.0
    c[far, 6:] = 2.0                       # what a query that sees it reads back
    q_lat = torch.zeros(H, L, kr, dtype=torch.float64)
    q_lat[:, :, 5] = 1.0
    sink = torch.tensor([-5.0, 30.0, 60.0], dtype=torch.float64)     # the key's score is 30
    want = torch.empty(H, L, kr, dtype=torch.float64)
    for h in range(H):
        want[h] = P.causal_softmax_attention(q_lat[h], c, c, 1.0, float(sink[h]))
    n_pages = 12
    table = torch.randperm(n_pages)[None].to(torch.int32).to(dev)
    rows = torch.full((n_pages, 1, page, kr), float("nan"), device=dev)
    for j in range(L):
        rows[table[0, j // page], 0, j % page] = c[j].float().to(dev)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    got = torch.empty(H, L, kr, device=dev)
    q = torch.zeros(L, H, 4, device=dev)
    K.latent_attn_rows(q_lat.float().to(dev), q, 4, rows, table, i32([0] * L), i32(list(range(L))), None, True, got, kr, 0, 1.0, None,
                       n_splits=n_splits, sink=sink.float().to(dev))
    torch.cuda.synchronize()
    err = (got.double().cpu() - want).abs().amax(dim=(0, 2))
    assert float(err.max()) <= 2e-5, f"position {int(err.argmax())} off by {float(err.max()):.3g}"
    if far < L - 1:
        # the three regimes show in the plain result itself: the key carries the row, shares it evenly, is drowned
        assert float(want[0, L - 1, 7]) > 1.9 and 0.9 < float(want[1, L - 1, 7]) < 1.1 and float(want[2, L - 1, 7]) < 1e-6
        if far > 0:
            assert abs(float(want[0, far - 1, 7])) < 0.5      # and nobody sees it before its time


@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("H, G, d, dv, rot", [(4, 2, 16, 24, 8), (6, 2, 10, 20, 4), (2, 2, 24, 8, 24), (3, 1, 12, 12, 0)])
def test_norm_over_whole_projections_then_rotation(H, G, d, dv, rot, interleaved):
    """The per-token preparation against the plain functions: both norms over all heads at once, then the rotation in either
    layout with slowed frequencies, then the cache write (the page and row of each position)."""
    from dryft_b200.ops import kernels as K

    torch.manual_seed(H * 100 + d)
    dev, page, n = "cuda", 64, 150
    proj = torch.randn(n, H * d + G * d + G * dv + 5, device=dev)
    qw, kw = torch.rand(H * d, device=dev) + 0.5, torch.rand(G * d, device=dev) + 0.5
    eps = 1e-3
    spec = {"dims": rot, "base": 200.0, "scaling": {"factor": 2.5}} if rot else None
    freq = P.rotary_frequencies(spec) if rot else None
    pos = torch.arange(37, 37 + n)
    table = torch.randperm(8)[None].to(torch.int32).to(dev)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    q_out = torch.empty(n, H, d, device=dev)
    k_pages = torch.zeros(8, G, page, d, device=dev)
    v_pages = torch.zeros(8, G, page, dv, device=dev)
    hi = freq.float() if rot else None
    lo = (freq - hi.double()).float().to(dev) if rot else None       # what the 32-bit frequency drops
    K.pool_attn_prep_tok(proj, qw, kw, eps, hi.to(dev) if rot else None, lo, rot, interleaved, i32([0] * n), i32(pos.tolist()),
                         q_out, k_pages, v_pages, table, H, G, -1.0, True)
    torch.cuda.synchronize()
    f = lambda t: t.double().cpu()
    qn = P.rms_norm(f(proj[:, :H * d]), f(qw), eps).view(n, H, d)
    kn = P.rms_norm(f(proj[:, H * d:H * d + G * d]), f(kw), eps).view(n, G, d)
    if rot and interleaved:
        qn, kn = P.rotate_pairs(qn, pos, spec), P.rotate_pairs(kn, pos, spec)
    elif rot:       # dims i and i + rot/2 turn together: the interleaved function applied to the dims brought side by side
        order = [j for i in range(rot // 2) for j in (i, i + rot // 2)]
        back = torch.argsort(torch.tensor(order))
        for t in (qn, kn):
            t[..., :rot] = P.rotate_pairs(t[..., order].contiguous(), pos, spec)[..., back]
    assert float((f(q_out) - qn).abs().max()) <= 3e-5
    for j, p in enumerate(pos.tolist()):
        pg = int(table[0, p // page])
        assert float((f(k_pages[pg, :, p % page]) - kn[j]).abs().max()) <= 3e-5, f"key at position {p}"
        assert torch.equal(v_pages[pg, :, p % page].reshape(-1), proj[j, H * d + G * d:H * d + G * d + G * dv]), f"value at position {p}"


def test_router_scores_and_the_clamp():
    """Sigmoid scores (each expert's own logit, ties to the lower index, weights not rescaled) and the experts' activation
    with its weight on the input: below, at and above the clamp on both sides, in both forms of the expert products."""
    from dryft_b200.ops import kernels as K

    torch.manual_seed(5)
    dev, n, E, top, W, Fd = "cuda", 70, 7, 3, 32, 16
    logits = torch.randn(n, E, device=dev) * 2.0
    logits[0] = 0.25                                           # all equal: the first `top` experts
    idx = torch.empty(n, top, dtype=torch.int32, device=dev)
    wts = torch.empty(n, top, device=dev)
    K.moe_route(logits, 1, 1, top, idx, wts, score="sigmoid")
    s = torch.sigmoid(logits.double().cpu())
    vals, order = torch.sort(s, dim=-1, descending=True, stable=True)
    assert torch.equal(idx.cpu().long(), order[:, :top]) and float((wts.double().cpu() - vals[:, :top]).abs().max()) <= 1e-6
    assert idx[0].tolist() == [0, 1, 2]
    h = torch.randn(n, W, device=dev)
    w_gu = torch.randn(E, 2 * Fd, W, device=dev) * 0.6
    w_d = torch.randn(E, W, Fd, device=dev) * 0.3
    limit, alpha, off = 1.25, 1.702, 1.0
    want = torch.zeros(n * top, W, dtype=torch.float64)
    hits = [0, 0, 0]
    for t in range(n):
        for k in range(top):
            e = int(idx[t, k])
            x = float(wts[t, k]) * h[t].double().cpu()
            g0, u0 = w_gu[e, :Fd].double().cpu() @ x, w_gu[e, Fd:].double().cpu() @ x
            hits[0] += int((g0 > limit).sum()); hits[1] += int((u0 > limit).sum()); hits[2] += int((u0 < -limit).sum())
            g, u = torch.clamp(g0, max=limit), torch.clamp(u0, min=-limit, max=limit)
            want[t * top + k] = w_d[e].double().cpu() @ (g * torch.sigmoid(alpha * g) * (u + off))
    assert min(hits) > 10                                      # the test's inputs reach every edge of the clamp
    act = torch.empty(n * top, Fd, device=dev)
    y = torch.empty(n * top, W, device=dev)
    K.moe_rows(h, w_gu, idx, act, "gate_up_clamp", in_w=wts, limit=limit, alpha=alpha, up_offset=off)
    K.moe_rows(act, w_d, idx, y, "down")
    assert float((y.double().cpu() - want).abs().max()) <= 1e-4
    yb = torch.empty(n * top, W, device=dev, dtype=torch.bfloat16)
    bf = lambda t: t.to(torch.bfloat16)
    K.moe_grouped(bf(h), bf(w_gu), bf(w_d), idx, yb, gated=True, in_w=wts, limit=limit, alpha=alpha, up_offset=off)
    torch.cuda.synchronize()
    err = (yb.double().cpu() - want).abs().max() / want.abs().max()
    assert float(err) <= 0.03, float(err)


def test_stream_sum_and_softcap():
    from dryft_b200.ops import kernels as K

    torch.manual_seed(1)
    dev, n, W, top = "cuda", 9, 50, 3
    x = torch.randn(n, W, device=dev)
    a, b = torch.randn(n, W, device=dev).to(torch.bfloat16), torch.randn(n, W, device=dev).to(torch.bfloat16)
    rows = torch.randn(n * top, W, device=dev).to(torch.bfloat16)
    vec, nw = torch.randn(W, device=dev), torch.rand(W, device=dev) + 0.5
    want = x.double() + 0.8 * a.double() - 1.7 * b.double() + rows.double().view(n, top, W).sum(1) + vec.double()
    h = torch.empty(n, W, device=dev, dtype=torch.bfloat16)
    K.stream_sum(x, [(a, 0.8), (b, -1.7)], rows=rows, top=top, vec=vec, norm_w=nw, eps=1e-5, h=h)
    assert float((x.double() - want).abs().max()) <= 1e-5
    normed = P.rms_norm(want.cpu(), nw.double().cpu(), 1e-5)
    assert float((h.double().cpu() - normed).abs().max()) <= 0.02
    z = torch.randn(4, 33, device=dev) * 40.0
    want = 25.0 * torch.tanh(z.double() / 25.0)
    K.softcap(z, 25.0)
    assert float((z.double() - want).abs().max()) <= 1e-4
