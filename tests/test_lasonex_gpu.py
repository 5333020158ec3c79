"""Lasonex in the engine against the plain implementation (tests/plain_lasonex.py).

Small configurations with weights of their own (tests/lasonex_tiny.py).  The 32-bit engine is
held to 2e-4 of the largest logit against the float64 oracle and, cut against cut, to bitwise
equality (every kernel of that path sums in an order that depends on the token's own place
only); the bfloat16 engine's error, position by position, to a fraction of the logits' spread in
the bulk of the positions.  Every engine runs with the cache's check mode on (pages that go back
are overwritten) and with fewer state slots than requests, so pages and slots are used again.
"""
import copy

import numpy as np
import pytest
import torch

import lasonex_tiny as lt
import plain_lasonex as plain
import replay

pytestmark = pytest.mark.gpu

YARN = (4.0, 64, 8.0, 1.0)
# every size differs from model to model, and some are the degenerate values: one head, heads == kv_heads,
# top == 1, top == experts, one group kept, groups == experts, a window of one, no window, no rotated
# dimensions, all dimensions rotated, key and value widths that are multiples of neither 8 nor 32, a layer
# without feed-forward, a model of one mixer kind only
MODELS = {
    "mix": dict(layers=[(lt.attention(4, 2, 16, 24, window=11, rot=8, scaling=YARN), lt.dense(48, 0.8)),
                        (lt.retention(2, 16, 8, rot=8), lt.moe(6, 2, 24, 1.25, groups=(3, 2))),
                        (lt.attention(4, 2, 16, 24, window=30, rot=16), lt.moe(6, 2, 24, 1.25, groups=(3, 2))),
                        (lt.retention(2, 16, 8, rot=8), None)], vocab=97, width=40, eps=1e-5, scale=3.0, page=8),
    "odd": dict(layers=[(lt.attention(3, 3, 10, 7, window=7, rot=6, base=500.0, diff=0.7), lt.moe(5, 1, 10, 0.5)),
                        (lt.retention(3, 13, 35, rot=12, decay=[0.5, 0.93, 0.999]), lt.dense(30, 2.5)),
                        (lt.attention(1, 1, 24, 40, window=None, rot=0, diff=0.1), None),
                        (lt.retention(1, 24, 6, rot=0, decay=[0.98]), lt.moe(4, 4, 16, 1.0, groups=(4, 4))),
                        (lt.attention(6, 2, 12, 12, window=1, rot=12, scaling=(16.0, 32, 4.0, 0.5)), lt.moe(8, 3, 6, 3.0, groups=(2, 1)))],
                vocab=61, width=36, eps=1e-6, scale=1.0, page=16),
    # sizes that the tensor-core kernels take in bfloat16 (multiples of 16 and 32 throughout, the grouped expert
    # products from 64 prompt tokens on)
    "even": dict(layers=[(lt.attention(4, 2, 32, 64, window=44, rot=32, scaling=(8.0, 128, 16.0, 1.0)), lt.moe(8, 2, 64, 1.25, groups=(4, 2))),
                         (lt.retention(4, 32, 48, rot=16), lt.dense(128, 0.9)),
                         (lt.attention(8, 2, 16, 32, window=70, rot=8), lt.moe(8, 2, 64, 2.0))],
                 vocab=80, width=64, eps=1e-6, scale=8.0, page=16),
}
LENGTHS = {"mix": [1, 2, 9, 23, 40, 77], "odd": [3, 30, 64, 51], "even": [150, 70, 90]}


@pytest.fixture(scope="module")
def made(tmp_path_factory):
    root = tmp_path_factory.mktemp("lasonex")
    out = {}
    for k, (name, m) in enumerate(MODELS.items()):
        raw = lt.config(m["layers"], m["vocab"], m["width"], m["eps"], m["scale"])
        w = lt.weights(raw, seed=5 + k, sharp=3.0)
        rng = np.random.default_rng(40 + k)
        requests = {f"q{i}": rng.integers(0, m["vocab"], size=n).tolist() for i, n in enumerate(LENGTHS[name])}
        want = {rid: plain.forward(raw, w, toks).float() for rid, toks in requests.items()}
        out[name] = dict(raw=raw, weights=w, folder=lt.write(raw, w, root / name), requests=requests, want=want,
                         page=m["page"])
    return out


_engines = {}


def engine(made, name, dtype, max_tokens=None, max_requests=3, graph=False):
    from fastllm_py_b200 import Model

    key = (name, dtype, max_tokens, max_requests, graph)
    if key not in _engines:
        _engines[key] = Model.load(made[name]["folder"], dtype=dtype, page_size=made[name]["page"],
                                   max_tokens=max_tokens or 512, max_requests=max_requests, max_batched_tokens=256,
                                   max_model_len=256, cuda_graph=graph, check_cache=True)
    return _engines[key]


def cuts(requests, live):
    return {"whole": replay.whole(requests), "tail": replay.tail_decode(requests, 12),
            "portions": replay.portions(requests), "small": replay.portions(requests, (2, 3, 2, 5, 2)),
            "mixed": replay.mixed(requests, live=live, seed=3, prefill_sizes=(9, 2, 17, 5), decode_tail=6)}


def worst(got, want):
    return max(float((got[(rid, p)] - want[rid][p]).abs().max()) for (rid, p) in got)


@pytest.mark.parametrize("name", list(MODELS))
def test_every_cut_in_32_bit_equals_the_oracle_and_the_other_cuts(made, name):
    m = made[name]
    top = max(float(v.abs().max()) for v in m["want"].values())
    results = {}
    for cut, steps in cuts(m["requests"], live=3).items():
        pool = replay.peak_tokens(steps, m["page"]) + (0 if cut == "mixed" else m["page"])
        eng = engine(made, name, "float32", pool).engine
        got = replay.run_in_process(eng, steps)
        assert len(got) == sum(len(t) for t in m["requests"].values())
        assert worst(got, m["want"]) <= 2e-4 * max(1.0, top), cut
        results[cut] = got
        assert not eng.cache.live
    for cut, got in results.items():
        for key, row in got.items():
            assert torch.equal(row, results["whole"][key]), (cut, key)
    assert engine(made, name, "float32", replay.peak_tokens(cuts(m["requests"], 3)["mixed"], m["page"])) \
        .engine.cache.pages_poisoned > 0


@pytest.mark.parametrize("name", list(MODELS))
def test_every_cut_in_bfloat16_stays_near_the_oracle(made, name):
    m = made[name]
    spread = float(torch.cat([v.flatten() for v in m["want"].values()]).std())
    for cut, steps in cuts(m["requests"], live=3).items():
        eng = engine(made, name, "bfloat16", replay.peak_tokens(steps, m["page"]) + m["page"]).engine
        got = replay.run_in_process(eng, steps)
        # a rounding error can flip an expert choice or a sharp softmax at single positions (and what follows
        # them through the state), so the bound is on the bulk of the positions, not on the worst one
        errs = np.array([float((got[k] - m["want"][k[0]][k[1]]).pow(2).mean().sqrt()) for k in got])
        assert np.median(errs) <= 0.08 * spread, cut
        assert np.quantile(errs, 0.9) <= 0.3 * spread, cut


def one_layer(mixer, mlp, **kw):
    return lt.config([(mixer, mlp)], **kw)


SINGLE = {
    "attention": one_layer(lt.attention(2, 1, 8, 40, window=6, rot=4), None, width=24, vocab=50),
    "attention_all": one_layer(lt.attention(3, 3, 8, 8, window=None, rot=8, scaling=YARN), None, width=24, vocab=50),
    "attention_wide_key": one_layer(lt.attention(2, 2, 72, 8, window=50, rot=2), None, width=24, vocab=50),
    "attention_wide_value": one_layer(lt.attention(2, 1, 8, 200, window=9, rot=8), None, width=24, vocab=50),
    "retention": one_layer(lt.retention(2, 8, 40, rot=4), None, width=24, vocab=50),
    "retention_wide_key": one_layer(lt.retention(2, 72, 8, rot=72, decay=[0.9, 0.999]), None, width=24, vocab=50),
    "retention_widest_key": one_layer(lt.retention(1, 136, 33, rot=30, decay=[0.97]), None, width=24, vocab=50),
    "dense": one_layer(lt.retention(1, 8, 8, rot=2), lt.dense(36, 0.6), width=24, vocab=50, embed_scale=7.0),
    "routed": one_layer(lt.retention(1, 8, 8, rot=2), lt.moe(8, 3, 12, 0.9, groups=(4, 2)), width=24, vocab=50),
    "routed_free": one_layer(lt.retention(1, 8, 8, rot=2), lt.moe(7, 3, 12, 4.0), width=24, vocab=50),
}


@pytest.mark.parametrize("kind", list(SINGLE))
def test_each_mechanism_alone(tmp_path, kind):
    from fastllm_py_b200 import Model, StepEntry

    raw = SINGLE[kind]
    w = lt.weights(raw, seed=17, sharp=4.0)
    folder = lt.write(raw, w, tmp_path / kind)
    toks = np.random.default_rng(1).integers(0, raw["vocab"], size=45).tolist()
    want = plain.forward(raw, w, toks).float()
    eng = Model.load(folder, dtype="float32", page_size=4, max_tokens=64, max_requests=2, max_batched_tokens=64,
                     max_model_len=64, cuda_graph=False, check_cache=True).engine
    eng.begin("a")
    head = eng.step([StepEntry("a", toks[:20], list(range(20)))]).cpu().clone()
    rest = [eng.step([StepEntry("a", [t], [0])]).cpu().clone() for t in toks[20:]]
    got = torch.cat([head] + rest)
    assert float((got - want).abs().max()) <= 2e-4 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_windows_edges_decide_the_output(tmp_path, dtype):
    """Attention so sharp that single keys decide a row: the oracle with every window one token
    wider or narrower is far from the engine, the oracle itself is not."""
    raw = lt.config([(lt.attention(2, 1, 16, 16, window=9, rot=8), lt.dense(16)),
                     (lt.attention(2, 2, 16, 16, window=17, rot=16), None)], width=32, vocab=40)
    w = lt.weights(raw, seed=3, sharp=8.0)
    folder = lt.write(raw, w, tmp_path / "edges")
    toks = np.random.default_rng(2).integers(0, 40, size=70).tolist()
    want = plain.forward(raw, w, toks).float()
    from fastllm_py_b200 import Model

    eng = Model.load(folder, dtype=dtype, page_size=8, max_tokens=32, max_requests=2, max_batched_tokens=64,
                     max_model_len=128, cuda_graph=False, check_cache=True).engine
    bound = 2e-4 * float(want.abs().max()) if dtype == "float32" else 0.05 * float(want.std())
    for steps in (replay.tail_decode({"a": toks}, 40), replay.portions({"a": toks}, (5, 2, 9, 3))):
        got = replay.run_in_process(eng, steps)       # a pool of 32 tokens: pages behind the window must go back
        if dtype == "float32":
            err = worst(got, {"a": want})
        else:
            err = float(np.median([float((got[k] - want[k[1]]).pow(2).mean().sqrt()) for k in got]))
        assert err <= bound
        for shift in (-1, 1):
            off = copy.deepcopy(raw)
            for layer in off["layers"]:
                layer["mixer"]["mask"]["size"] += shift
            other = plain.forward(off, w, toks).float()
            if dtype == "float32":
                assert float((other - want).abs().max()) > 100 * max(err, 1e-5)
            else:
                assert float(np.median((other - want).pow(2).mean(dim=1).sqrt().numpy()[20:])) > 5 * bound


def test_a_far_key_among_hundreds_stands_out(tmp_path):
    """No window: one early key is made to dominate a late query's first map (its row of the embedding is
    scaled so that query and key align), and the engine's logits there follow the oracle's; without that
    key the oracle is far away."""
    raw = lt.config([(lt.attention(2, 1, 16, 16, window=None, rot=0), None)], width=32, vocab=40)
    w = lt.weights(raw, seed=8, sharp=1.0)
    q1 = w["l0.mix.q"].float()[:16]                                   # head 0, map 1
    w["l0.mix.k"] = w["l0.mix.k"].float().clone()
    w["l0.mix.k"][:16] = q1 * 3.0                                     # keys of map 1 point where queries do
    w["l0.mix.k"] = w["l0.mix.k"].to(torch.bfloat16)
    w["embed"] = w["embed"].float().clone()
    w["embed"][39] *= 6.0                                             # token 39: a loud key and a loud query
    w["embed"] = w["embed"].to(torch.bfloat16)
    folder = lt.write(raw, w, tmp_path / "far")
    rng = np.random.default_rng(5)
    toks = rng.integers(0, 39, size=300).tolist()
    toks[3] = 39
    toks[290] = 39
    want = plain.forward(raw, w, toks).float()
    without = plain.forward(raw, w, toks[:3] + [0] + toks[4:]).float()
    from fastllm_py_b200 import Model

    eng = Model.load(folder, dtype="float32", page_size=16, max_tokens=320, max_requests=1, max_batched_tokens=512,
                     max_model_len=320, cuda_graph=False, check_cache=True).engine
    for steps in (replay.whole({"a": toks}), replay.tail_decode({"a": toks}, 20)):
        got = replay.run_in_process(eng, steps)
        err = worst(got, {"a": want})
        assert err <= 2e-4 * float(want.abs().max())
        assert float((without[290] - want[290]).abs().max()) > 100 * max(err, 1e-5)


def test_a_far_token_reaches_through_the_state(tmp_path):
    """Decays close to one: the first token still moves the last logits, and the engine follows the
    oracle through 150 single-token steps after a short prompt."""
    raw = lt.config([(lt.retention(2, 16, 16, rot=8, decay=[0.999, 0.9999]), lt.dense(16)),
                     (lt.retention(2, 16, 16, rot=16, decay=[0.998, 1.0]), None)], width=24, vocab=40)
    w = lt.weights(raw, seed=9)
    folder = lt.write(raw, w, tmp_path / "far")
    toks = np.random.default_rng(4).integers(0, 40, size=160).tolist()
    want = plain.forward(raw, w, toks).float()
    changed = plain.forward(raw, w, [(toks[0] + 1) % 40] + toks[1:]).float()
    from fastllm_py_b200 import Model

    eng = Model.load(folder, dtype="float32", page_size=16, max_tokens=256, max_requests=2, max_batched_tokens=64,
                     max_model_len=256, cuda_graph=False).engine
    got = replay.run_in_process(eng, replay.tail_decode({"a": toks}, 150))
    err = worst(got, {"a": want})
    assert err <= 2e-4 * float(want.abs().max())
    assert float((changed[-1] - want[-1]).abs().max()) > 100 * max(err, 1e-5)


def test_a_slot_used_again_starts_clean(made):
    """Two requests one after the other in an engine with a single slot equal the same requests in
    fresh engines, bit for bit."""
    m = made["mix"]
    (ra, ta), (rb, tb) = list(m["requests"].items())[3:5]
    eng = engine(made, "mix", "float32", 128, max_requests=1).engine
    first = replay.run_in_process(eng, replay.portions({ra: ta}))
    second = replay.run_in_process(eng, replay.portions({rb: tb}))
    alone = replay.run_in_process(engine(made, "mix", "float32", 512).engine, replay.whole({rb: tb}))
    assert all(torch.equal(second[k], alone[k]) for k in alone)
    assert worst(first, m["want"]) <= 2e-4 * 30.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(made, dtype):
    """Model.generate (scheduler, sampler, captured decode steps) against the oracle's greedy loop;
    where the oracle's two best logits are close the engine may take either."""
    m = made["mix"]
    model = engine(made, "mix", dtype, 512, max_requests=3, graph=True)
    prompts = [m["requests"]["q2"], m["requests"]["q3"], m["requests"]["q1"], m["requests"]["q4"][:20]]
    outs = model.generate(prompts, max_new_tokens=12)
    assert model.generate(prompts, max_new_tokens=12, use_graph=False) == outs          # replayed steps change nothing
    gaps = []                                                    # how far below the oracle's best each token is, in spreads
    for prompt, new in zip(prompts, outs):
        seq = list(prompt)
        for tok in new:
            logits = plain.forward(m["raw"], m["weights"], seq)[-1]
            gaps.append(float(logits.max() - logits[tok]) / float(logits.std()))
            seq.append(tok)
        assert len(new) == 12
    if dtype == "float32":
        assert max(gaps) < 1e-3
    else:
        # a rounding error can flip an expert choice in these narrow models and move single rows: nearly all tokens
        # are the oracle's best or nearly tied with it, none is far from it
        assert sum(g > 0.2 for g in gaps) <= 3 and max(gaps) < 1.0, sorted(gaps)[-5:]


def test_trace_program_on_a_folder(made, tmp_path):
    m = made["odd"]
    steps = replay.mixed(m["requests"], live=2, seed=1, prefill_sizes=(7, 2, 30), decode_tail=3)
    got = replay.run_program(m["folder"], "float32", steps, tmp_path / "out", replay.peak_tokens(steps, 64),
                             m["raw"]["vocab"], extra_args=("--max-requests", "2"))
    top = max(float(v.abs().max()) for v in m["want"].values())
    assert worst(got, m["want"]) <= 2e-4 * max(1.0, top)


def test_command_line_on_a_random_weights_folder(tmp_path):
    """bin/make_model writes a folder from a configuration, bin/generate loads it by its architecture
    string and generates through the scheduler."""
    import json
    import subprocess
    import sys

    raw = lt.config([(lt.retention(2, 16, 16, rot=8), lt.moe(4, 2, 16, groups=(2, 1))),
                     (lt.attention(2, 1, 16, 32, window=20, rot=16), lt.dense(32))], width=32, vocab=64)
    (tmp_path / "config.json").write_text(json.dumps(raw))
    made_ = subprocess.run([sys.executable, str(replay.ROOT / "bin" / "make_model"), str(tmp_path / "config.json"),
                            str(tmp_path / "m"), "--seed", "4", "--std", "0.2"], capture_output=True, text=True)
    assert made_.returncode == 0 and "Lasonex" in made_.stdout, made_.stderr
    run = subprocess.run([sys.executable, str(replay.ROOT / "bin" / "generate"), str(tmp_path / "m"), "-", "9",
                          "bfloat16", "--random-prompt", "30", "--seed", "1"], capture_output=True, text=True)
    assert run.returncode == 0, run.stderr[-2000:]
    lines = run.stdout.strip().splitlines()
    assert "Lasonex: 2L width=32" in lines[0]
    assert len([int(t) for t in lines[1].split(",")]) == 9


# ------------------------------------------------------------------ kernels alone

def test_router_choice_with_groups_follows_the_oracle():
    from fastllm_py_b200.native import ops

    gen = torch.Generator().manual_seed(3)
    for experts, top, groups in ((12, 3, (4, 2)), (20, 4, (5, 3)), (6, 2, (6, 2)), (6, 1, (6, 1)), (8, 8, (2, 2)), (9, 2, None), (40, 5, (5, 2))):
        z = torch.randn(70, experts, generator=gen) * 2.0
        r = {"experts": experts, "top": top}
        if groups:
            r["groups"] = {"count": groups[0], "keep": groups[1]}
        # the oracle's route() takes h and a router matrix: an identity router makes its logits z itself
        want_e, want_w = plain.route(z.double(), torch.eye(experts, dtype=torch.float64), r)
        chosen = torch.empty(70, top, dtype=torch.int32, device="cuda")
        weights = torch.empty(70, top, device="cuda")
        ops.moe_pick(z.cuda(), None, chosen, weights, top, True, True, groups and groups[0], groups and groups[1], 1e-20)
        got_e, got_w = chosen.cpu().long(), weights.cpu().double()
        assert torch.equal(got_e.sort(dim=1).values, want_e.sort(dim=1).values), (experts, top, groups)
        assert torch.allclose(got_w.gather(1, got_e.argsort(dim=1)), want_w.gather(1, want_e.argsort(dim=1)), atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clamped_unit_and_pair_norm_kernels(dtype):
    from fastllm_py_b200.native import ops

    gen = torch.Generator().manual_seed(1)
    gu = (torch.randn(37, 2 * 52, generator=gen) * 2.0).to(dtype).cuda()
    out = torch.empty(37, 52, dtype=dtype, device="cuda")
    ops.glu(gu, out, "clamped_swish", (0.9, 1.702))
    g, u = gu[:, :52].double().clamp(max=0.9), gu[:, 52:].double().clamp(-0.9, 0.9)
    want = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    assert float((out.double() - want).abs().max()) <= tol

    x = torch.randn(19, 44, generator=gen).cuda()
    d1 = torch.randn(19, 44, generator=gen).to(dtype).cuda()
    d2 = torch.randn(19, 44, generator=gen).to(dtype).cuda()
    w1 = (1 + 0.2 * torch.randn(44, generator=gen)).to(torch.bfloat16).cuda()
    w2 = (1 + 0.2 * torch.randn(44, generator=gen)).to(torch.bfloat16).cuda()
    o1, o2 = torch.empty(19, 44, dtype=dtype, device="cuda"), torch.empty(19, 44, dtype=dtype, device="cuda")
    total = x.double() + d1.double() + d2.double()
    normed = total / torch.sqrt((total * total).mean(dim=1, keepdim=True) + 1e-5)
    xs = x.clone()
    ops.norm_pair(xs, d1, d2, w1, w2, o1, o2, 1e-5)
    assert float((xs.double() - total).abs().max()) <= 1e-6
    assert float((o1.double() - normed * w1.double()).abs().max()) <= 4 * tol
    assert float((o2.double() - normed * w2.double()).abs().max()) <= 4 * tol
    rows = torch.tensor([4, 0, 17], dtype=torch.int32, device="cuda")
    xs, few = x.clone(), torch.empty(3, 44, dtype=dtype, device="cuda")
    ops.norm_pair(xs, d1, d2, w1, None, few, None, 1e-5, rows)
    assert torch.equal(xs, x)                                               # gathered rows leave the stream alone
    assert float((few.double() - (normed * w1.double())[rows.cpu().long()]).abs().max()) <= 4 * tol


@pytest.mark.parametrize("dim,vdim,window,heads,kv_heads", [(32, 64, 70, 4, 2), (16, 16, None, 6, 2), (64, 128, 33, 3, 3),
                                                           (48, 80, 81, 8, 1), (128, 128, 90, 2, 1)])
def test_tensor_core_attention_equals_the_cuda_core_one(dim, vdim, window, heads, kv_heads):
    """Scattered pages, a prompt portion behind cached tokens beside single tokens, a standout key just
    inside the window of one query and just outside that of the next."""
    from types import SimpleNamespace

    from fastllm_py_b200.native import ops

    gen = torch.Generator().manual_seed(dim + vdim)
    page = 16
    ctx_lens, q_lens = [37, 150, 0, 201], [100, 1, 70, 1]
    row_w = 2 * dim + vdim
    n_pages = sum(-(-(c + q) // page) for c, q in zip(ctx_lens, q_lens))
    order = torch.randperm(n_pages + 5, generator=gen)[:n_pages].tolist()
    cache = (torch.randn(n_pages + 5, kv_heads, page, row_w, generator=gen) * 0.7).to(torch.bfloat16)
    bt = torch.zeros(4, 16, dtype=torch.int32)
    for r, (c, ql) in enumerate(zip(ctx_lens, q_lens)):
        for i in range(-(-(c + ql) // page)):
            bt[r, i] = order.pop()
    n = sum(q_lens)
    q = (torch.randn(n, heads * 2 * dim, generator=gen) * 0.7).to(torch.bfloat16)
    if window is not None:
        # request 0, row 60 (position 97): the key at the window's edge answers its first map loudly
        edge = 97 - window + 1
        pg, off = int(bt[0, edge // page]), edge % page
        cache[pg, 0, off, :dim] = q[60, :dim].float().mul(4.0).to(torch.bfloat16)
    tok_req = torch.tensor(sum(([r] * ql for r, ql in enumerate(q_lens)), []), dtype=torch.int32)
    positions = torch.tensor(sum((list(range(c, c + ql)) for c, ql in zip(ctx_lens, q_lens)), []), dtype=torch.int32)
    starts = [0]
    for ql in q_lens:
        starts.append(starts[-1] + ql)
    dev = lambda t: t.cuda()
    step = SimpleNamespace(req_start=dev(torch.tensor(starts, dtype=torch.int32)),
                           req_ctx=dev(torch.tensor(ctx_lens, dtype=torch.int32)),
                           req_qlen=dev(torch.tensor(q_lens, dtype=torch.int32)), n_requests=4)
    want = torch.empty(n, heads * vdim, dtype=torch.bfloat16, device="cuda")
    got = torch.empty_like(want)
    args = (heads, kv_heads, dim, vdim, window, dim ** -0.5, 0.37, 1e-5, 0.6, page)
    ops.diff_attention_simt(dev(q), want, dev(cache), dev(bt), dev(tok_req), dev(positions), *args)
    ops.diff_attention_tc(dev(q), got, dev(cache), dev(bt), step, *args)
    torch.cuda.synchronize()
    err = (got.float() - want.float()).abs()
    assert float(err.max()) <= 0.06 and float(err.mean()) <= 0.006, (float(err.max()), float(err.mean()))
    # the single tokens through the split-key kernel, the portions through the tensor-core one
    assert ops.diff_decode_takes(heads, kv_heads, dim, vdim)
    singles = dev(torch.tensor([starts[1], starts[3]], dtype=torch.int32))
    n_splits = (min(window or 202, 202) - 1) // ops.DIFF_SPLIT + 2
    partial = torch.empty(2 * heads * 2 * n_splits * (vdim + 2), device="cuda")
    both = torch.zeros_like(want)
    ops.diff_attention_tc(dev(q), both, dev(cache), dev(bt), step, *args, include_single=False)
    assert float(both[starts[1]].float().abs().max()) == 0.0 and float(both[starts[3]].float().abs().max()) == 0.0
    ops.diff_decode(dev(q), both, dev(cache), dev(bt), dev(tok_req), dev(positions), singles, partial, n_splits,
                    *args)
    torch.cuda.synchronize()
    err = (both.float() - want.float()).abs()
    assert float(err.max()) <= 0.06 and float(err.mean()) <= 0.006, (float(err.max()), float(err.mean()))
    exact = torch.empty_like(want, dtype=torch.float32)
    ops.diff_attention_simt(dev(q).float(), exact, dev(cache).float(), dev(bt), dev(tok_req), dev(positions), *args)
    split32 = exact.clone()
    split32[starts[1]] = 0
    split32[starts[3]] = 0
    ops.diff_decode(dev(q).float(), split32, dev(cache).float(), dev(bt), dev(tok_req), dev(positions), singles, partial,
                    n_splits, *args)
    assert float((split32 - exact).abs().max()) <= 2e-5                    # in 32-bit the split changes the order only
    if window is not None:
        far = want.clone()
        ops.diff_attention_simt(dev(q), far, dev(cache), dev(bt), dev(tok_req), dev(positions),
                                *(args[:4] + (window - 1,) + args[5:]))
        assert float((far[60].float() - want[60].float()).abs().max()) > 0.3         # the edge key decides row 60


def test_clamped_unit_in_the_tensor_core_products_epilogue():
    """The gated tcgen05 product with the clamped swish unit against the product and the unit apart, in its
    one-tile form (a decode-sized step) and its CTA-pair form (a prompt-sized step); limits small enough to bite."""
    from fastllm_py_b200.native import gemm_tc

    torch.manual_seed(6)
    taken = 0
    for m, inter, k, limit in ((48, 1536, 256, 0.7), (2048, 4096, 512, 1.2)):
        a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
        w = (torch.randn(2 * inter, k, device="cuda") * k ** -0.5).to(torch.bfloat16)
        out = torch.zeros(m, inter, device="cuda", dtype=torch.bfloat16)
        if not gemm_tc.gemm_swiglu(a, w, out, "clamped_swish", (limit, 1.702)):
            continue
        taken += 1
        prod = a.float() @ w.float().T
        g, u = prod[:, :inter].clamp(max=limit), prod[:, inter:].clamp(-limit, limit)
        ref = g * torch.sigmoid(1.702 * g) * (u + 1.0)
        assert float((g == limit).float().mean()) > 0.05                  # the limit is reached often
        assert float((out.float() - ref).abs().max()) <= 0.03 * float(ref.abs().max()) + 1e-2, m
    assert taken >= 1


@pytest.mark.parametrize("dim,vdim", [(128, 32), (64, 24), (96, 40), (256, 16), (20, 12)])
def test_retention_scan_shapes_agree_with_a_plain_loop(dim, vdim):
    """A lone prompt spreads a value column over 16 or 32 lanes, a batch (and the 32-bit path, always) over 8:
    all against a float64 loop, a portion continuing from a saved state included."""
    from types import SimpleNamespace

    from fastllm_py_b200.native import ops

    gen = torch.Generator().manual_seed(dim)
    heads, n = 2, 75
    work = (torch.randn(n, 2 * heads * dim + heads * vdim, generator=gen) * 0.5).cuda()
    decay = torch.tensor([0.9, 0.999]).cuda()
    q, k, v = (t.double().cpu() for t in (work[:, :heads * dim], work[:, heads * dim:2 * heads * dim], work[:, 2 * heads * dim:]))
    S = torch.zeros(heads, dim, vdim, dtype=torch.float64)
    want = torch.zeros(n, heads * vdim, dtype=torch.float64)
    for t in range(n):
        for h in range(heads):
            S[h] = float(decay[h]) * S[h] + torch.outer(k[t, h * dim:(h + 1) * dim], v[t, h * vdim:(h + 1) * vdim])
            want[t, h * vdim:(h + 1) * vdim] = S[h].T @ q[t, h * dim:(h + 1) * dim]

    def run(cuts, fixed):
        state = torch.full((3, heads * vdim * dim), 7.0, device="cuda")           # what an earlier request left
        out = torch.zeros(n, heads * vdim, device="cuda")
        at = 0
        for length in cuts:
            step = SimpleNamespace(req_start=torch.tensor([0, length], dtype=torch.int32).cuda(),
                                   req_ctx=torch.tensor([at], dtype=torch.int32).cuda(),
                                   req_qlen=torch.tensor([length], dtype=torch.int32).cuda(),
                                   req_slot=torch.tensor([1], dtype=torch.int32).cuda(), n_requests=1)
            ops.retention_scan(work[at:at + length], out[at:at + length], state, decay, step, heads, dim, vdim, fixed)
            at += length
        return out.cpu().double(), state[1].cpu().double()

    scale = float(want.abs().max())
    whole, s_whole = run([n], False)
    fixed, s_fixed = run([n], True)
    cut, s_cut = run([33, 1, 2, 39], True)
    assert float((whole - want).abs().max()) <= 1e-5 * scale and float((fixed - want).abs().max()) <= 1e-5 * scale
    assert torch.equal(cut, fixed) and torch.equal(s_cut, s_fixed)                 # one order whatever the cut
    assert float((s_whole.view(heads, vdim, dim) - S.transpose(1, 2)).abs().max()) <= 1e-5 * float(S.abs().max())


def test_parallel_block_under_a_norm_of_another_kind(tmp_path):
    """Another design uses the parallel block, the retention mixer and the clamped unit with a norm part of its own that
    knows nothing of a second pending tensor (and a second layer without feed-forward): the residual stream adds both
    sums before it hands the row to that norm."""
    import json
    from dataclasses import dataclass

    from fastllm_py_b200 import Model, StepEntry
    from fastllm_py_b200.config import register_architecture
    from fastllm_py_b200.parts import LayerRun, LayerSpec, ModelPlan, Part, PartSpec, register_part

    @register_part("norm", "toy_rms_plus_one")
    class RmsPlusOne(Part):
        category = "norm"

        def __init__(self, spec, ctx):
            super().__init__(spec, ctx)
            self.size, self.eps = int(spec.params["size"]), float(spec.params["eps"])

        def weight_shapes(self):
            return {"weight": (self.size,)}

        def load(self, tensors):
            self.weight = tensors["weight"].float()

        def apply(self, stream, out, rows=None):
            assert getattr(stream, "extra", None) is None
            x = stream.x
            if stream.pending is not None and rows is None:
                x += stream.pending.float()
                stream.pending = None
            elif stream.pending is not None:
                x = x[rows.long()] + stream.pending[rows.long()].float()
            elif rows is not None:
                x = x[rows.long()]
            out.copy_((x * torch.rsqrt(x.pow(2).mean(dim=1, keepdim=True) + self.eps) * (1.0 + self.weight)).to(out.dtype))

    @dataclass(frozen=True)
    class Toy4Config:
        vocab: int
        width: int

        @classmethod
        def from_hf(cls, raw):
            return cls(raw["vocab"], raw["width"])

        def to_hf(self):
            return {"architectures": ["Toy4ForCausalLM"], "vocab": self.vocab, "width": self.width}

    decay, limit = (0.9, 0.99), 0.8

    def make_plan(cfg, names=None):
        w = cfg.width

        def norm(n):
            return PartSpec("toy_rms_plus_one", dict(size=w, eps=1e-5), {"weight": n})

        def mixer(i):
            return PartSpec("retention", dict(hidden_size=w, heads=2, dim=8, vdim=12, decay=decay, norm_eps=1e-5,
                                              position=PartSpec("rotary", dict(rot_dim=4, theta=100.0, scaling=None, exact=True))),
                            {s: f"l{i}.mix.{s}" for s in ("q", "k", "v", "g", "o")})

        ff = PartSpec("glu", dict(hidden_size=w, intermediate_size=20, activation="clamped_swish", activation_params=(limit, 1.702)),
                      {s: f"l0.mlp.{s}" for s in ("gate", "up", "down")})
        layers = [LayerSpec("parallel", mixer(0), ff, {"mixer": norm("l0.norm1"), "feed_forward": norm("l0.norm2")}),
                  LayerSpec("parallel", mixer(1), None, {"mixer": norm("l1.norm1")})]
        io = dict(vocab_size=cfg.vocab, hidden_size=w)
        return ModelPlan(w, cfg.vocab, 256, PartSpec("table", io, {"weight": "embed"}), layers, [LayerRun(0), LayerRun(1)],
                         norm("final.norm"), PartSpec("linear", io, {"weight": "head"}))

    register_architecture("Toy4ForCausalLM", Toy4Config, make_plan)
    raw = lt.config([(lt.retention(2, 8, 12, rot=4, base=100.0, decay=decay), lt.dense(20, limit)),
                     (lt.retention(2, 8, 12, rot=4, base=100.0, decay=decay), None)], vocab=30, width=24, eps=1e-5)
    w = lt.weights(raw, seed=21)
    folder = tmp_path / "toy4"
    lt.write(raw, w, folder)
    (folder / "config.json").write_text(json.dumps(Toy4Config(30, 24).to_hf()))
    toks = np.random.default_rng(3).integers(0, 30, size=31).tolist()

    def norm(x, weight):
        return plain.rms(x, 1e-5) * (1.0 + weight.double())

    x = w["embed"].double()[toks]
    for i in range(2):
        mix = {s: w[f"l{i}.mix.{s}"].double() for s in ("q", "k", "v", "g", "o")}
        y, _ = plain.retention(norm(x, w[f"l{i}.norm1"]), mix, raw["layers"][i]["mixer"], 1e-5)
        if i == 0:
            y = y + plain.clamped_unit(norm(x, w["l0.norm2"]), *(w[f"l0.mlp.{s}"].double() for s in ("gate", "up", "down")), limit)
        x = x + y
    want = (norm(x, w["final.norm"]) @ w["head"].double().T).float()
    eng = Model.load(folder, dtype="float32", page_size=8, max_tokens=64, max_requests=2, max_batched_tokens=64,
                     max_model_len=64, cuda_graph=False).engine
    eng.begin("a")
    got = torch.cat([eng.step([StepEntry("a", toks[:17], list(range(17)))]).cpu().clone(),
                     eng.step([StepEntry("a", toks[17:], [0, 5, 13])]).cpu().clone()])
    assert float((got - want[list(range(17)) + [17, 22, 30]]).abs().max()) <= 2e-4 * max(1.0, float(want.abs().max()))
