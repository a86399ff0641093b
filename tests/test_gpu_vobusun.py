"""The Vobusun decoder in the engine against the plain evaluation (``plain_vobusun.py``), in 32-bit (sharp) and in bfloat16:
every mixer alone and mixed, whole prompts, prompts against token-by-token decoding, prompts in portions down to two
tokens, unequal batches against each request alone, slots and pages used again (poisoned), long decoding across window
and page edges, the first tokens, the stream after every layer, greedy generation through ``Engine.generate`` /
``generate_many`` (captured graphs and eager), the replay program and the command line as child processes."""

import numpy as np
import pytest
import torch

import plain_vobusun as P
import vobusun_models as M

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
_cache = {}


def model(name, tmp_path_factory):
    if name not in _cache:
        cfg = M.CONFIGS[name]
        tensors = M.draw_weights(cfg, seed=17 + len(name) + ord(name[0]))
        d = M.write_model(cfg, tensors, str(tmp_path_factory.mktemp(f"vobusun_{name}")))
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


def close_all(pairs, dtype, what):
    if dtype == "float32":
        for got, want, label in pairs:
            M.assert_close(got, want, dtype, f"{what}: {label}")
    else:   # a single bfloat16 row cannot be judged statistically: the rows of all pairs together
        M.assert_close(torch.cat([g.detach().float().cpu() for g, _, _ in pairs]), torch.cat([w for _, w, _ in pairs]), dtype, what)


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
        close_all(pairs, dtype, f"{name} whole prompts")
        # most of the prompt at once, the rest token by token (across window and page edges)
        for toks in reqs[3:]:
            head = max(1, len(toks) - 70)
            s = eng.cache.open_sequences(1)
            rows = [eng.stepper.step(s, [toks[:head]], [[head - 1]])]
            for t in range(head, len(toks)):
                rows.append(eng.stepper.step(s, [[toks[t]]], [[0]]))
            eng.cache.close_sequences(s)
            M.assert_close(torch.cat(rows), plain_logits(entry, toks)[head - 1:], dtype, f"{name} decoding {len(toks)}")
        # portions of several sizes, down to two tokens (a convolution's tail shorter than its taps among them)
        for portion in (2, 7, 64, 97):
            toks = reqs[4]
            s = eng.cache.open_sequences(1)
            rows = []
            for c0 in range(0, len(toks), portion):
                piece = toks[c0:c0 + portion]
                rows.append(eng.stepper.step(s, [piece], [list(range(len(piece)))]))
            eng.cache.close_sequences(s)
            M.assert_close(torch.cat(rows), plain_logits(entry, toks), dtype, f"{name} portions of {portion}")
        # an unequal batch of prompts (one of a single token), then decoded together; shorter requests end earlier
        batch = [reqs[2], reqs[5], reqs[3], reqs[1]]
        heads = [max(1, len(t) - 12) for t in batch]
        slots = eng.cache.open_sequences(len(batch))
        got = eng.stepper.step(slots, [t[:h] for t, h in zip(batch, heads)], [list(range(h)) for h in heads])
        at, pairs = 0, []
        for t, h in zip(batch, heads):
            pairs.append((got[at:at + h], plain_logits(entry, t)[:h], f"prompt of {h}"))
            at += h
        close_all(pairs, dtype, f"{name} batched prompts")
        live, step = list(range(len(batch))), 0
        collected = {b: [] for b in live}
        while live:
            got = eng.stepper.step([slots[b] for b in live], [[batch[b][heads[b] + step]] for b in live], [[0]] * len(live))
            for r, b in enumerate(live):
                collected[b].append(got[r:r + 1])
            step += 1
            done = [b for b in live if heads[b] + step >= len(batch[b])]
            eng.cache.close_sequences([slots[b] for b in done])
            live = [b for b in live if b not in done]
        close_all([(torch.cat(rows), plain_logits(entry, batch[b])[heads[b]:], f"request {b}") for b, rows in collected.items()],
                  dtype, f"{name} batched decoding")
    eng.cache.check()


def test_the_stream_after_every_layer(tmp_path_factory):
    entry = model("mixed", tmp_path_factory)
    cfg, tensors = entry[0], entry[1]
    eng = engine(entry, "float32")
    toks = M.prompts(cfg, [50], seed=8)[0]
    want = []
    P.forward(cfg, tensors, toks, want)
    got = []
    eng.model.layer_tap = lambda i, block, res: got.append(block.stream_sum(res).double().cpu())
    with torch.inference_mode():
        s = eng.cache.open_sequences(1)
        eng.stepper.step(s, [toks], [[0]])
        eng.cache.close_sequences(s)
    assert len(got) == len(cfg["layers"])
    for i, (g, w) in enumerate(zip(got, want)):
        assert float((g - w).abs().max()) <= 2e-5 * float(w.abs().max()), f"layer {i} ({cfg['layers'][i]['type']})"


@pytest.mark.parametrize("dtype", DTYPES)
def test_pages_and_slots_used_again_hold_nothing_of_their_last_holder(tmp_path_factory, dtype):
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
            M.assert_close(torch.cat(rows), plain_logits(entry, toks), dtype, f"request {i} on a reused slot and pages")
            for g in eng.cache._groups:        # what the freed pages hold must never matter again
                g.k.fill_(float("nan"))
                assert g.v is None             # latents only: no value pages
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_gives_pages_behind_the_window_back(tmp_path_factory, dtype):
    entry = model("lat_page", tmp_path_factory)
    cfg = entry[0]
    eng = engine(entry, dtype, max_batch=2, max_seq_len=512, max_tokens=1024)
    toks = M.prompts(cfg, [300], seed=9)[0]
    with torch.inference_mode():
        s = eng.cache.open_sequences(1)
        rows = [eng.stepper.step(s, [toks[:3]], [[0, 1, 2]])]
        for t in range(3, len(toks)):
            rows.append(eng.stepper.step(s, [[toks[t]]], [[0]]))
        held = sorted(len(g.ledger.held(s[0])) for g in eng.cache._groups)
        assert held == [2, 2, 5], held      # windows of 64 and 97 trim to two pages, the layer without a window keeps all five
        eng.cache.close_sequences(s)
    M.assert_close(torch.cat(rows), plain_logits(entry, toks), dtype, "300 tokens, nearly all decoded one by one")


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
        # bfloat16 may legitimately part ways with the plain tokens at a close call, and the contexts differ from then on.
        # Teacher-forced instead: under the plain model, fed our tokens, each of our tokens is the best one up to what
        # bfloat16 rounding does to logits of this model (a few hundredths of their spread)
        for b, p in enumerate(prompts):
            lg = plain_logits(entry, list(p) + got[b][:-1])[len(p) - 1:]
            ours = lg.gather(1, torch.tensor(got[b])[:, None])[:, 0]
            lost = (lg.max(dim=-1).values - ours) / lg.std(dim=-1)
            assert float(lost.max()) <= 0.25, f"request {b}: token {int(lost.argmax())} loses {float(lost.max()):.3g} spreads to the plain model's best"
    eager = engine(entry, dtype, cuda_graphs=False, max_batch=4)     # graphs and eager steps choose the same tokens
    assert eager.generate_many(prompts, n_new) == got
    chunked = engine(entry, dtype, cuda_graphs=False, max_batch=4, prefill_chunk_tokens=16)
    if dtype == "float32":
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
    M.assert_close(read(0), want0, dtype, "replayed prompts")
    M.assert_close(read(1), torch.cat([plain_logits(entry, t)[-1:] for t in reqs]), dtype, "replayed decode step")
    M.assert_close(read(3), plain_logits(entry, reqs[1] + [5])[-1:], dtype, "a request id used again")


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
        live, step, rows = list(range(len(reqs))), 0, {b: [] for b in range(len(reqs))}
        while live:
            got = eng.stepper.step([slots[b] for b in live], [[reqs[b][heads[b] + step]] for b in live], [[0]] * len(live))
            for i, b in enumerate(live):
                rows[b].append(got[i:i + 1])
            step += 1
            done = [b for b in live if heads[b] + step >= len(reqs[b])]
            eng.cache.close_sequences([slots[b] for b in done])
            live = [b for b in live if b not in done]
        pairs += [(torch.cat(r), plain_logits(entry, reqs[b])[heads[b]:], f"request {b}") for b, r in rows.items() if r]
    close_all(pairs, dtype, "forty requests")
    eng.cache.check()


def _random_config(seed):
    """A configuration drawn at random: layer kinds and order, every size, every constant, which options are absent."""
    import random

    r = random.Random(seed)
    even = lambda lo, hi: 2 * r.randint(lo // 2, hi // 2)
    layers = []
    for _ in range(r.randint(2, 4)):
        kind = r.choice(["retention", "latent", "rglru"])
        ff = r.choice([None, r.randint(6, 50)])
        limit = r.choice([None, round(r.uniform(0.4, 3.0), 3)])
        if kind == "retention":
            heads, dim = r.randint(1, 5), r.randint(2, 36)
            layers.append(M.retention(heads=heads, dim=dim, vdim=r.randint(2, 40), rot_dims=r.choice([None, even(2, dim)]) if dim >= 2 else None,
                                      base=r.choice([37.0, 1000.0, 250000.0]), decay=[round(r.uniform(0.8, 0.9997), 6) for _ in range(heads)],
                                      ff=ff, limit=limit))
        elif kind == "latent":
            rot = r.choice([0, even(2, 16)])
            layers.append(M.latent(heads=r.randint(1, 6), dim=r.randint(3, 30), rot_dim=rot, vdim=r.randint(2, 36), q_rank=r.randint(4, 40),
                                   kv_rank=r.randint(4, 70), window=r.choice([None, r.randint(1, 150)]), base=r.choice([25.0, 5000.0]),
                                   scale=round(r.uniform(0.1, 0.4), 4), ff=ff, limit=limit))
        else:
            blocks = r.randint(1, 4)
            layers.append(M.rglru(width=blocks * r.randint(2, 18), conv=r.randint(1, 5), blocks=blocks, ff=ff, limit=limit))
    for _ in range(r.randint(0, 3)):       # layers that run another layer's weights, anywhere in the order
        j = r.randrange(len(layers))
        if layers[j].get("weights_of") is None:
            layers.append(M.again(layers, j))
    return M.config(layers, width=r.choice([24, 36, 50, 52, 64]), vocab=r.randint(40, 300), emb_scale=round(r.uniform(0.5, 9.0), 3),
                    eps=r.choice([1e-6, 1e-5, 3e-4]), mult=round(r.uniform(0.3, 1.2), 3), streams=r.choice([None, 1, 2, 3, 5]),
                    bigram=r.choice([None, (r.randint(3, 400), r.randint(1, 100000), r.randint(1, 999))]))


@pytest.mark.parametrize("seed", range(10))
def test_configurations_drawn_at_random(tmp_path, seed):
    cfg = _random_config(seed)
    tensors = M.draw_weights(cfg, seed=100 + seed)
    entry = (cfg, tensors, M.write_model(cfg, tensors, str(tmp_path / "m")), {})
    reqs = M.prompts(cfg, [70, 1, 33], seed=seed)
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
            live, step, rows = [b for b in range(len(reqs)) if heads[b] < len(reqs[b])], 0, {b: [] for b in range(len(reqs))}
            eng.cache.close_sequences([slots[b] for b in range(len(reqs)) if b not in live])
            while live:
                out = eng.stepper.step([slots[b] for b in live], [[reqs[b][heads[b] + step]] for b in live], [[0]] * len(live))
                for i, b in enumerate(live):
                    rows[b].append(out[i:i + 1])
                step += 1
                done = [b for b in live if heads[b] + step >= len(reqs[b])]
                eng.cache.close_sequences([slots[b] for b in done])
                live = [b for b in live if b not in done]
            pairs += [(torch.cat(v), plain_logits(entry, reqs[b])[heads[b]:], f"request {b} decoded") for b, v in rows.items() if v]
        what = f"random configuration {seed} ({[l['type'] for l in cfg['layers']]})"
        if dtype == "float32":
            close_all(pairs, dtype, what)
        else:
            # latents of four entries and widths of 24 make bfloat16 rounding large in some of these models: the sharp
            # comparison is the 32-bit one; here the typical row must be close and every row finite
            got_all = torch.cat([g.detach().float().cpu() for g, _, _ in pairs])
            assert torch.isfinite(got_all).all(), what
            e = M.row_errors(got_all, torch.cat([w for _, w, _ in pairs]))
            assert float(e.median()) <= M.BF16_TOL, f"{what}: median row off by {float(e.median()):.3g}"
        eng.cache.check()
