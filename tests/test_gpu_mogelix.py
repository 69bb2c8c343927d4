"""The Mogelix decoder in the engine against the plain evaluation (``plain_mogelix.py``), in 32-bit (sharp) and in bfloat16:
every mixer alone and mixed, whole prompts, prompts against token-by-token decoding, prompts in portions down to two
tokens, unequal batches against each request alone, slots and pages used again (poisoned), long decoding across window,
block and page edges, the first tokens, the stream after every layer, greedy generation through ``Engine.generate`` /
``generate_many`` (captured graphs and eager), the replay program and the command line as child processes; the prompt
attention kernel against the row-wise kernel, both against the plain function with one key that outweighs all others, and the
state-space mixer with many-token steps cut into chunks."""

import math

import numpy as np
import pytest
import torch

import mogelix_models as M
import plain_mogelix as P

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
_cache = {}


def model(name, tmp_path_factory):
    if name not in _cache:
        cfg = M.CONFIGS[name]
        tensors = M.draw_weights(cfg, seed=29 + len(name) + ord(name[0]))
        d = M.write_model(cfg, tensors, str(tmp_path_factory.mktemp(f"mogelix_{name}")))
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
        # a short head at once, the rest token by token (windows, blocks and pages pass over decoded tokens)
        for toks, head in ((reqs[3], 1), (reqs[4], 40), (reqs[5], 129)):
            s = eng.cache.open_sequences(1)
            rows = [eng.stepper.step(s, [toks[:head]], [[head - 1]])]
            for t in range(head, len(toks)):
                rows.append(eng.stepper.step(s, [[toks[t]]], [[0]]))
            eng.cache.close_sequences(s)
            check(entry, torch.cat(rows), plain_logits(entry, toks)[head - 1:], dtype, f"{name} decoding {len(toks)} from {head}")
        # portions of several sizes, down to two tokens (a convolution's tail shorter than its taps, blocks cut by a portion)
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


def test_the_stream_after_every_layer(tmp_path_factory):
    entry = model("mixed", tmp_path_factory)
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
    assert len(got) == len(cfg["layers"])
    for i, (g, w) in enumerate(zip(got, want)):
        assert float((g - w).abs().max()) <= 2e-5 * float(w.abs().max()), f"layer {i} ({cfg['layers'][i]['type']})"


@pytest.mark.parametrize("dtype", DTYPES)
def test_pages_slots_and_states_used_again_hold_nothing_of_their_last_holder(tmp_path_factory, dtype):
    entry = model("mixed", tmp_path_factory)
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
def test_long_decoding_gives_pages_behind_the_window_back(tmp_path_factory, dtype):
    entry = model("att_edges", tmp_path_factory)
    cfg = entry[0]
    eng = engine(entry, dtype, max_batch=2, max_seq_len=512, max_tokens=2048)
    toks = M.prompts(cfg, [330], seed=9)[0]
    with torch.inference_mode():
        s = eng.cache.open_sequences(1)
        rows = [eng.stepper.step(s, [toks[:3]], [[0, 1, 2]])]
        for t in range(3, len(toks)):
            rows.append(eng.stepper.step(s, [[toks[t]]], [[0]]))
        token_pages = [len(g.ledger.held(s[0])) for g in eng.cache._groups]
        eng.cache.close_sequences(s)
    check(entry, torch.cat(rows), plain_logits(entry, toks), dtype, "330 tokens, nearly all decoded one by one")
    # 330 tokens are six pages of 64; no group of token rows keeps more than its window (97 at most) and one page need
    assert max(token_pages) <= 6 and min(token_pages) <= 2, token_pages
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(tmp_path_factory, dtype):
    entry = model("mixed", tmp_path_factory)
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

    entry = model("mixed", tmp_path_factory)
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


def test_command_line_generates_and_samples(tmp_path_factory):
    import json
    import subprocess
    import sys

    import helpers as H

    entry = model("mixed", tmp_path_factory)
    cfg, tensors = entry[0], entry[1]
    base = [sys.executable, "-m", "dryft_b200", "generate", "--model", entry[2], "--dtype", "float32", "--max-batch", "4",
            "--max-seq-len", "128", "--prompt-ids", "5,17,3,60,9", "--prompt-ids", "7,7,7", "--max-new-tokens", "6"]
    run = lambda extra: subprocess.run(base + extra, capture_output=True, text=True, timeout=600, cwd=H.ROOT)
    greedy = run([])
    assert greedy.returncode == 0, greedy.stderr[-2000:]
    rows = [json.loads(ln) for ln in greedy.stdout.splitlines() if ln.startswith("{")]
    assert [r["tokens"] for r in rows] == [P.greedy(cfg, tensors, p, 6) for p in ([5, 17, 3, 60, 9], [7, 7, 7])]
    a, b, c = run(["--temperature", "0.9", "--top-k", "7", "--seed", "3"]), run(["--temperature", "0.9", "--top-k", "7", "--seed", "3"]), \
        run(["--temperature", "0.9", "--top-k", "7", "--seed", "4"])
    assert a.returncode == 0 and a.stdout == b.stdout and a.stdout != c.stdout


@pytest.mark.parametrize("dtype", DTYPES)
def test_forty_unequal_requests_at_once(tmp_path_factory, dtype):
    """More rows than the few-row products take; requests end one after another."""
    entry = model("mixed", tmp_path_factory)
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


def _random_config(seed):
    """A configuration drawn at random: layer kinds and order, every size, every constant, who reads whose keys."""
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
            mlp = M.moe(ff=r.randint(3, 40), experts=experts, top=r.randint(1, experts), shared=r.choice([None, r.randint(2, 40)]))
        if r.random() < 0.35:
            groups = r.randint(1, 3)
            heads = groups * r.randint(1, 3)
            vdim = r.randint(2, 40)
            parts = r.choice([d for d in range(1, heads * vdim + 1) if (heads * vdim) % d == 0 and d <= 8])
            layers.append(M.mamba(heads=heads, vdim=vdim, state=r.randint(1, 70), groups=groups, conv=r.randint(1, 6), norm_groups=parts, mlp=mlp))
            continue
        owners = [j for j, l in enumerate(layers) if l["type"] == "attention" and "kv_from" not in l["mixer"]]
        if owners and r.random() < 0.4:
            j = r.choice(owners)
            o = layers[j]["mixer"]
            layers.append(M.attention(heads=o["kv_heads"] * r.randint(1, 3), kv_heads=o["kv_heads"], dim=o["dim"], vdim=o["vdim"],
                                      size=r.randint(1, 150), pool=r.choice([o["mask"]["pool"], r.randint(1, 40)]), rot_dims=o["rot"]["dims"],
                                      base=o["rot"]["base"], scaling=o["rot"]["scaling"], scale=round(r.uniform(0.2, 1.5), 3), kv_from=j, mlp=mlp))
            continue
        kv = r.randint(1, 3)
        dim = r.randint(2, 40)
        layers.append(M.attention(heads=kv * r.randint(1, 4), kv_heads=kv, dim=dim, vdim=r.randint(2, 40), size=r.randint(1, 150),
                                  pool=r.randint(1, 70), rot_dims=even(2, dim), base=r.choice([37.0, 1000.0, 250000.0]),
                                  scaling={"factor": round(r.uniform(1.5, 16.0), 2), "low": 1.0, "high": round(r.uniform(1.5, 6.0), 2),
                                           "original": r.choice([16, 64, 300])},
                                  scale=round(r.uniform(0.2, 1.5), 3), mlp=mlp))
    return M.config(layers, width=r.choice([24, 36, 50, 52, 64]), vocab=r.randint(40, 300), eps=r.choice([1e-6, 1e-5, 3e-4]),
                    alpha=round(r.uniform(1.0, 3.0), 3))   # below 1 the stream amplifies rounding: a plain 32-bit evaluation is then as far off


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
        what = f"random configuration {seed} ({[l['type'] for l in cfg['layers']]})"
        if dtype == "float32":
            close_all(entry, pairs, dtype, what)
        else:
            # heads of two or three values and widths of 24 make bfloat16 rounding large in some of these models: the sharp
            # comparison is the 32-bit one; here the typical row must be close and every row finite
            got_all = torch.cat([g.detach().float().cpu() for g, _, _ in pairs])
            assert torch.isfinite(got_all).all(), what
            e = M.row_errors(got_all, torch.cat([w for _, w, _ in pairs]))
            assert float(e.median()) <= limits(entry)[0], f"{what}: median row off by {float(e.median()):.3g}"
        eng.cache.check()


@pytest.mark.parametrize("size, pool, d, dv, group", [(20, 4, 32, 16, 2), (64, 16, 16, 48, 1), (130, 64, 64, 64, 4), (7, 1, 16, 16, 3),
                                                       (5, 12, 32, 32, 2), (1, 1, 16, 16, 1), (1000, 8, 16, 32, 2)])
def test_prompt_kernel_against_the_row_kernel(size, pool, d, dv, group):
    """The tensor-core prompt kernel (bfloat16) against the row-wise kernel in 32-bit on the same cache: whole prompts and
    later portions of one, over shuffled pages whose unused rows are poisoned, with scores spread widely so that a key
    wrongly seen or missed at a window's or a block's edge moves whole rows."""
    from dryft_b200.ops import kernels as K

    if not K.pool_attention_prefill_supported(d, dv, group):
        pytest.skip("no prompt kernel for this head shape")
    torch.manual_seed(size * 31 + pool)
    dev, page, n_kv = "cuda", 64, 2
    H = n_kv * group
    seqs = [(0, 200), (37, 181), (0, 1), (128, 330), (63, 66)]              # (first position of this step, length so far)
    max_pages = 8
    n_pages = len(seqs) * max_pages
    perm = torch.randperm(n_pages)
    table = perm.view(len(seqs), max_pages).to(torch.int32).to(dev)
    ptable = torch.randperm(n_pages).view(len(seqs), max_pages).to(torch.int32).to(dev)
    k32 = torch.full((n_pages, n_kv, page, d), float("nan"), device=dev)
    v32 = torch.full((n_pages, n_kv, page, dv), float("nan"), device=dev)
    pk32, pv32 = torch.full_like(k32, float("nan")), torch.full_like(v32, float("nan"))
    slots, poss, t0s, tns = [], [], [], []
    for s, (start, length) in enumerate(seqs):
        kk = torch.randn(length, n_kv, d).to(torch.bfloat16).float().to(dev)
        vv = torch.randn(length, n_kv, dv).to(torch.bfloat16).float().to(dev)
        for j in range(length):
            k32[table[s, j // page], :, j % page] = kk[j]
            v32[table[s, j // page], :, j % page] = vv[j]
        for b in range(length // pool):
            pk32[ptable[s, b // page], :, b % page] = kk[b * pool:(b + 1) * pool].mean(0).to(torch.bfloat16).float()
            pv32[ptable[s, b // page], :, b % page] = vv[b * pool:(b + 1) * pool].mean(0).to(torch.bfloat16).float()
        for q0 in range(start, length, 64):
            t0s.append(len(slots) + q0 - start)
            tns.append(min(64, length - q0))
        slots += [s] * (length - start)
        poss += list(range(start, length))
    n = len(slots)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    tok_slot, tok_pos, tile0, tilen = i32(slots), i32(poss), i32(t0s), i32(tns)
    q32 = torch.randn(n, H, d, device=dev).to(torch.bfloat16).float()
    sink = torch.randn(H, device=dev) * 2.0
    scale = 6.0 / math.sqrt(d)
    want = torch.empty(n, H, dv, device=dev)
    K.pool_attn_rows(q32, k32, v32, table, (pk32, pv32, ptable), sink, tok_slot, tok_pos, want, scale, size, pool)
    got = torch.empty(n, H, dv, device=dev, dtype=torch.bfloat16)
    bf = lambda x: x.to(torch.bfloat16)
    K.pool_attn_prefill(bf(q32), bf(k32), bf(v32), table, (bf(pk32), bf(pv32), ptable), sink, tile0, tilen, tok_slot, tok_pos, got,
                        len(t0s), scale, size, pool)
    torch.cuda.synchronize()
    assert torch.isfinite(want).all() and torch.isfinite(got.float()).all()
    err = (got.float() - want).abs().amax(dim=(1, 2))
    assert float(err.max()) <= 0.03, f"token {int(err.argmax())} (slot {slots[int(err.argmax())]}, position {poss[int(err.argmax())]}) off by {float(err.max()):.3g}"
    # without a sink and without blocks the same kernel is a plain sliding window
    K.pool_attn_rows(q32, k32, v32, table, None, None, tok_slot, tok_pos, want, scale, size, 0)
    K.pool_attn_prefill(bf(q32), bf(k32), bf(v32), table, None, None, tile0, tilen, tok_slot, tok_pos, got, len(t0s), scale, size, 0)
    torch.cuda.synchronize()
    assert float((got.float() - want).abs().max()) <= 0.03


@pytest.mark.parametrize("name", ["ssm_sizes", "mixed"])
def test_many_token_steps_of_the_state_space_mixer_run_in_chunks(tmp_path_factory, monkeypatch, name):
    """Steps of many tokens cut into chunks that run side by side (here chunks of 16 tokens, from steps of 2 tokens on):
    whole prompts, pieces that continue a sequence at odd places, unequal batches with a single-token request, 32-bit."""
    from dryft_b200.ops import kernels as K
    from dryft_b200.parts.ssd import SSD

    monkeypatch.setattr(K, "SSM_CHUNK_TOKENS", 16)
    entry = model(name, tmp_path_factory)
    cfg = entry[0]
    eng = engine(entry, "float32")
    n_ssd = 0
    for blk in eng.model.blocks:
        if isinstance(blk.mixer, SSD):
            blk.mixer.chunked_from = 2
            n_ssd += 1
    assert n_ssd
    reqs = M.prompts(cfg, [200, 131, 1, 47, 16, 33], seed=12)
    n0 = K.launch_count
    with torch.inference_mode():
        for portion in (200, 97, 16, 5):
            toks = reqs[0]
            s = eng.cache.open_sequences(1)
            rows = []
            for c0 in range(0, len(toks), portion):
                piece = toks[c0:c0 + portion]
                rows.append(eng.stepper.step(s, [piece], [list(range(len(piece)))]))
            eng.cache.close_sequences(s)
            check(entry, torch.cat(rows), plain_logits(entry, toks), "float32", f"{name} in chunks, portions of {portion}")
        slots = eng.cache.open_sequences(len(reqs))
        heads = [max(1, len(t) - 3) for t in reqs]
        got = eng.stepper.step(slots, [t[:h] for t, h in zip(reqs, heads)], [list(range(h)) for h in heads])
        at, pairs = 0, []
        for t, h in zip(reqs, heads):
            pairs.append((got[at:at + h], plain_logits(entry, t)[:h], f"prompt of {h}"))
            at += h
        close_all(entry, pairs, "float32", f"{name} in chunks, batched prompts")
        rows = decode_together(eng, slots, reqs, heads)
        close_all(entry, [(torch.cat(r), plain_logits(entry, reqs[b])[heads[b]:], f"request {b}") for b, r in rows.items() if r],
                  "float32", f"{name} decoding behind chunked prompts")
    assert K.launch_count > n0
    eng.cache.check()


@pytest.mark.parametrize("size, pool, far", [(50, 8, 13), (64, 64, 100), (129, 5, 3), (3, 7, 640)])
def test_one_key_that_stands_out_at_every_edge(size, pool, far):
    """Both attention kernels (row-wise in 32-bit, prompts in bfloat16) against the plain function over 700 tokens in which ONE
    key, at position ``far``, outweighs all others for every query: it is seen while in the window, not at all between the
    window and its block's completion, and as a 1 / pool share of its block's row from then on (hundreds of tokens later too)."""
    from dryft_b200.ops import kernels as K

    torch.manual_seed(far)
    dev, page, n_kv, group, d, dv, L = "cuda", 64, 1, 2, 16, 16, 700
    H = n_kv * group
    k = (0.1 * torch.randn(L, n_kv, d)).to(torch.bfloat16).double()
    v = torch.randn(L, n_kv, dv).to(torch.bfloat16).double()
    q = torch.zeros(L, H, d, dtype=torch.float64)
    q[:, :, 3] = 1.0
    k[far, 0, 3] = 40.0                       # its score leads by 40 * scale; in its block's mean by 40 * scale / pool
    v[far, 0] = 7.0
    sink = torch.tensor([-1.0, 2.0], dtype=torch.float64)
    scale = 1.5
    want = P.pooled_window_attention(q, k, v, sink, scale, size, pool)
    n_pages = 12
    table = torch.randperm(n_pages)[None].to(torch.int32).to(dev)
    ptable = torch.randperm(n_pages)[None].to(torch.int32).to(dev)
    k32 = torch.full((n_pages, n_kv, page, d), float("nan"), device=dev)
    v32 = torch.full((n_pages, n_kv, page, dv), float("nan"), device=dev)
    pk32, pv32 = torch.full_like(k32, float("nan")), torch.full_like(v32, float("nan"))
    for j in range(L):
        k32[table[0, j // page], :, j % page] = k[j].float().to(dev)
        v32[table[0, j // page], :, j % page] = v[j].float().to(dev)
    for b in range(L // pool):
        pk32[ptable[0, b // page], :, b % page] = k[b * pool:(b + 1) * pool].mean(0).float().to(dev)
        pv32[ptable[0, b // page], :, b % page] = v[b * pool:(b + 1) * pool].mean(0).float().to(dev)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    tok_slot, tok_pos = i32([0] * L), i32(list(range(L)))
    got = torch.empty(L, H, dv, device=dev)
    for splits in (1, 3):
        po = torch.empty(L, H, splits, dv, device=dev) if splits > 1 else None
        pm = torch.empty(L, H, splits, 2, device=dev) if splits > 1 else None
        K.pool_attn_rows(q.float().to(dev), k32, v32, table, (pk32, pv32, ptable), sink.float().to(dev), tok_slot, tok_pos, got, scale,
                         size, pool, splits, po, pm)
        err = (got.double().cpu() - want).abs().amax(dim=(1, 2))
        assert float(err.max()) <= 2e-5, f"{splits} split(s): position {int(err.argmax())} off by {float(err.max()):.3g}"
    # the plain function itself shows the three regimes (the test's inputs are made for it)
    first_block_seen = (far // pool) * pool + pool - 1 + size
    assert float(want[min(far + size - 1, L - 1), 0, 0]) > 6.0
    if far + size < min(first_block_seen, L):
        assert abs(float(want[far + size, 0, 0])) < 3.0
    if d % 16 == 0 and first_block_seen < L:
        bf = lambda x: x.to(torch.bfloat16)
        t0 = list(range(0, L, 64))
        gotb = torch.empty(L, H, dv, device=dev, dtype=torch.bfloat16)
        K.pool_attn_prefill(bf(q.float().to(dev)), bf(k32), bf(v32), table, (bf(pk32), bf(pv32), ptable), sink.float().to(dev), i32(t0),
                            i32([min(64, L - a) for a in t0]), tok_slot, tok_pos, gotb, len(t0), scale, size, pool)
        errb = (gotb.double().cpu() - want).abs().amax(dim=(1, 2))
        assert float(errb.max()) <= 0.06, f"prompt kernel: position {int(errb.argmax())} off by {float(errb.max()):.3g}"
