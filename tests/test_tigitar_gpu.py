"""Tigitar in the engine against the plain implementation (tests/plain_tigitar.py).

Small configurations with weights of their own (tests/tigitar_tiny.py).  The 32-bit engine is
held to 2e-4 of the largest logit against the float64 oracle and, cut against cut, to bitwise
equality (every kernel of that path sums in an order that depends on the token's own place
only); the bfloat16 engine's error, position by position, to 0.08 of the logits' spread in the
median and 0.3 of it at the ninth decile (these models are narrow and their softmaxes sharp).  Every engine runs with the
cache's check mode on (pages that go back are overwritten) and with fewer state slots than
requests, so pages and slots are used again.
"""
import numpy as np
import pytest
import torch

import plain_tigitar as plain
import replay
import tigitar_tiny as tt

pytestmark = pytest.mark.gpu

# every size differs from model to model, and some are the degenerate values: one head, heads == kv_heads,
# one tap, top == 1, top == experts, a window of one, no window, a value width that is no multiple of 32,
# a key width that is no multiple of 8, a layer without feed-forward, two readers of one latent cache with
# different windows (the reader's the wider one)
MODELS = {
    "mix": dict(layers=[(tt.delta(4, 2, 16, 8, 4), tt.dense(48)),
                        (tt.latent(2, 16, 8, 16, 24, window=11), tt.moe(6, 2, 24)),
                        (tt.delta(4, 2, 16, 8, 4), tt.moe(6, 2, 24)),
                        (tt.latent(2, 16, 8, 16, 24, window=11, kv_from=1), tt.dense(48)),
                        (tt.delta(4, 2, 16, 8, 4), None)], vocab=97, width=40, eps=1e-5, softcap=12.0, page=8),
    "odd": dict(layers=[(tt.latent(3, 12, 4, 20, 17, window=7, base=500.0), tt.moe(5, 1, 10)),
                        (tt.delta(3, 3, 13, 35, 2), tt.dense(30)),
                        (tt.latent(1, 8, 4, 8, 17, window=19, kv_from=0, base=500.0), None),
                        (tt.delta(1, 1, 24, 6, 1), tt.moe(3, 3, 16)),
                        (tt.latent(2, 16, 6, 12, 9, window=None), tt.dense(20)),
                        (tt.latent(2, 8, 6, 4, 9, window=1, kv_from=4), tt.dense(20))],
                vocab=61, width=36, eps=1e-6, softcap=None, page=16),
    # sizes that the tensor-core kernels take in bfloat16 (latent attention with split keys in decode steps,
    # the per-head products, the grouped expert products from 64 prompt tokens on)
    "even": dict(layers=[(tt.latent(3, 32, 16, 32, 32, window=40), tt.moe(4, 2, 64)),
                         (tt.delta(2, 2, 32, 32, 4), tt.dense(128)),
                         (tt.latent(20, 32, 16, 16, 32, window=70, kv_from=0), tt.moe(4, 2, 64))],
                 vocab=80, width=64, eps=1e-6, softcap=20.0, page=16),
}
LENGTHS = {"mix": [1, 2, 9, 23, 40, 77], "odd": [3, 30, 64, 51], "even": [150, 70, 90]}


@pytest.fixture(scope="module")
def made(tmp_path_factory):
    root = tmp_path_factory.mktemp("tigitar")
    out = {}
    for k, (name, m) in enumerate(MODELS.items()):
        raw = tt.config(m["layers"], m["vocab"], m["width"], m["eps"], m["softcap"])
        w = tt.weights(raw, seed=5 + k, sharp=3.0)
        rng = np.random.default_rng(40 + k)
        requests = {f"q{i}": rng.integers(0, m["vocab"], size=n).tolist() for i, n in enumerate(LENGTHS[name])}
        want = {rid: plain.forward(raw, w, toks).float() for rid, toks in requests.items()}
        out[name] = dict(raw=raw, weights=w, folder=tt.write(raw, w, root / name), requests=requests, want=want,
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
    return tt.config([(mixer, mlp)], **kw)


SINGLE = {
    "delta": one_layer(tt.delta(2, 1, 8, 40, 3), None, width=24, vocab=50),
    "delta_wide_key": one_layer(tt.delta(2, 2, 72, 8, 4), None, width=24, vocab=50),
    "latent": one_layer(tt.latent(2, 8, 4, 8, 12, window=6), None, width=24, vocab=50),
    "latent_all": one_layer(tt.latent(3, 8, 4, 8, 12, window=None), None, width=24, vocab=50),
    "dense": one_layer(tt.delta(1, 1, 8, 8, 2), tt.dense(36), width=24, vocab=50),
    "routed": one_layer(tt.delta(1, 1, 8, 8, 2), tt.moe(7, 3, 12), width=24, vocab=50, softcap=3.0),
}


@pytest.mark.parametrize("kind", list(SINGLE))
def test_each_mechanism_alone(tmp_path, kind):
    from fastllm_py_b200 import Model, StepEntry

    raw = SINGLE[kind]
    w = tt.weights(raw, seed=17, sharp=4.0)
    folder = tt.write(raw, w, tmp_path / kind)
    toks = np.random.default_rng(1).integers(0, raw["vocab"], size=45).tolist()
    want = plain.forward(raw, w, toks).float()
    eng = Model.load(folder, dtype="float32", page_size=4, max_tokens=64, max_requests=2, max_batched_tokens=64,
                     max_model_len=64, cuda_graph=False, check_cache=True).engine
    eng.begin("a")
    head = eng.step([StepEntry("a", toks[:20], list(range(20)))]).cpu().clone()
    rest = [eng.step([StepEntry("a", [t], [0])]).cpu().clone() for t in toks[20:]]
    got = torch.cat([head] + rest)
    assert float((got - want).abs().max()) <= 2e-4 * max(1.0, float(want.abs().max()))


def test_windows_edges_decide_the_output(made, tmp_path):
    """Attention so sharp that single keys decide a row: the oracle with every window one token
    wider or narrower is far from the engine, the oracle itself is not."""
    import copy

    raw = tt.config([(tt.latent(2, 8, 4, 8, 12, window=9), tt.dense(16)),
                     (tt.latent(2, 8, 4, 8, 12, window=17, kv_from=0), None)], width=24, vocab=40)
    w = tt.weights(raw, seed=3, sharp=8.0)
    folder = tt.write(raw, w, tmp_path / "edges")
    toks = np.random.default_rng(2).integers(0, 40, size=70).tolist()
    want = plain.forward(raw, w, toks).float()
    from fastllm_py_b200 import Model

    eng = Model.load(folder, dtype="float32", page_size=8, max_tokens=32, max_requests=2, max_batched_tokens=64,
                     max_model_len=128, cuda_graph=False, check_cache=True).engine
    for steps in (replay.tail_decode({"a": toks}, 40), replay.portions({"a": toks}, (5, 2, 9, 3))):
        got = replay.run_in_process(eng, steps)       # a pool of 32 tokens: pages behind the window must go back
        err = worst(got, {"a": want})
        assert err <= 2e-4 * float(want.abs().max())
        for shift in (-1, 1):
            off = copy.deepcopy(raw)
            for layer in off["layers"]:
                layer["mixer"]["mask"]["size"] += shift
            other = plain.forward(off, w, toks).float()
            assert float((other - want).abs().max()) > 100 * max(err, 1e-5)


def test_a_far_token_reaches_through_the_state(tmp_path):
    """Decays close to one: the first token still moves the last logits, and the engine follows the
    oracle through 150 single-token steps after a short prompt."""
    raw = tt.config([(tt.delta(2, 1, 16, 16, 4), tt.dense(16)), (tt.delta(2, 2, 16, 16, 4), None)], width=24, vocab=40)
    w = tt.weights(raw, seed=9)
    for i in range(2):
        w[f"l{i}.mix.A_log"] = torch.full_like(w[f"l{i}.mix.A_log"], -6.0)
    folder = tt.write(raw, w, tmp_path / "far")
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
    assert worst(first, m["want"]) <= 2e-4 * 12.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(made, dtype):
    """Model.generate (scheduler, sampler, captured decode steps) against the oracle's greedy loop;
    where the oracle's two best logits are close the engine may take either."""
    m = made["mix"]
    model = engine(made, "mix", dtype, 512, max_requests=3, graph=True)
    prompts = [m["requests"]["q2"], m["requests"]["q3"], m["requests"]["q1"], m["requests"]["q4"][:20]]
    outs = model.generate(prompts, max_new_tokens=12)
    margin = 1e-3 if dtype == "float32" else 0.3
    for prompt, new in zip(prompts, outs):
        seq = list(prompt)
        for tok in new:
            logits = plain.forward(m["raw"], m["weights"], seq)[-1]
            best = torch.topk(logits, 2)
            assert tok == int(best.indices[0]) or float(best.values[0] - logits[tok]) < margin
            seq.append(tok)
        assert len(new) == 12


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

    raw = tt.config([(tt.delta(2, 1, 16, 16, 3), tt.moe(4, 2, 16)), (tt.latent(2, 16, 16, 16, 32, window=20), tt.dense(32))],
                    width=32, vocab=64)
    (tmp_path / "config.json").write_text(json.dumps(raw))
    made_ = subprocess.run([sys.executable, str(replay.ROOT / "bin" / "make_model"), str(tmp_path / "config.json"),
                            str(tmp_path / "m"), "--seed", "4", "--std", "0.2"], capture_output=True, text=True)
    assert made_.returncode == 0 and "Tigitar" in made_.stdout, made_.stderr
    run = subprocess.run([sys.executable, str(replay.ROOT / "bin" / "generate"), str(tmp_path / "m"), "-", "9",
                          "bfloat16", "--random-prompt", "30", "--seed", "1"], capture_output=True, text=True)
    assert run.returncode == 0, run.stderr[-2000:]
    lines = run.stdout.strip().splitlines()
    assert "Tigitar: 2L width=32" in lines[0]
    assert len([int(t) for t in lines[1].split(",")]) == 9


# ------------------------------------------------------------------ kernels alone

def test_grouped_expert_products_against_the_per_token_kernels():
    from fastllm_py_b200.native import ops

    torch.manual_seed(8)
    n, width, ff, experts, top = 210, 128, 160, 5, 2
    h = torch.randn(n, width, device="cuda").to(torch.bfloat16)
    gate_up = (torch.randn(experts, 2 * ff, width, device="cuda") * width ** -0.5).to(torch.bfloat16)
    down = (torch.randn(experts, width, ff, device="cuda") * ff ** -0.5).to(torch.bfloat16)
    chosen = torch.stack([torch.randperm(experts, device="cuda")[:top] for _ in range(n)]).to(torch.int32)
    chosen[:40] = torch.tensor([3, 1], dtype=torch.int32)              # one expert with many rows, one with none
    chosen[chosen == 4] = 0
    weights = torch.rand(n, top, device="cuda")
    want = torch.empty(n, width, device="cuda", dtype=torch.bfloat16)
    ops.moe_experts(h, gate_up, down, chosen, weights, torch.empty(n * top, ff, device="cuda"), want, "silu")
    rows = ops.moe_group_rows(n, top, experts)
    assert ops.moe_group_takes(torch.bfloat16, torch.bfloat16, width, ff)
    ints = torch.empty(rows + n * top + rows // 64 + 1, dtype=torch.int32, device="cuda")
    got = torch.empty_like(want)
    ops.moe_experts_grouped(h, gate_up, down, chosen, weights, ints, torch.empty(rows, ff, device="cuda", dtype=torch.bfloat16),
                            torch.empty(rows, width, device="cuda"), got, "silu")
    torch.cuda.synchronize()
    assert float((got.float() - want.float()).abs().max()) <= 0.03 * float(want.float().abs().max())
    assert float((got.float() - want.float()).abs().mean()) <= 3e-3 * float(want.float().abs().max())


def test_norm_add_norm_from_partial_sums():
    from fastllm_py_b200.native import gemm_tc, ops

    torch.manual_seed(9)
    rows, dim, splits = 5, 72, 3
    slabs = torch.randn(splits, rows, dim, device="cuda")
    x = torch.randn(rows, dim, device="cuda")
    wa, wb = (1 + 0.2 * torch.randn(2, dim, device="cuda")).to(torch.bfloat16)
    partial = gemm_tc.Partial(slabs, splits, rows, dim, dim, slabs.device)
    y = torch.empty(rows, dim, device="cuda", dtype=torch.bfloat16)
    partial.reduce_into(y)
    want_x, want = x.clone(), torch.empty(rows, dim, device="cuda", dtype=torch.bfloat16)
    ops.sandwich_norm(want_x, y, wa, 1e-5, wb, 1e-6, want)
    got = torch.empty_like(want)
    ops.sandwich_norm_partial(x, partial, wa, 1e-5, wb, 1e-6, got)
    assert torch.equal(x, want_x) and torch.equal(got, want)

def test_norm_add_norm_kernel():
    from fastllm_py_b200.native import ops

    torch.manual_seed(0)
    for dim, dt in ((40, torch.float32), (1000, torch.bfloat16)):
        x = torch.randn(7, dim, device="cuda")
        y = (3 * torch.randn(7, dim, device="cuda")).to(dt)
        wa, wb = (1 + 0.2 * torch.randn(2, dim, device="cuda")).to(torch.bfloat16)
        out = torch.empty(7, dim, device="cuda", dtype=dt)
        yf = y.float()
        summed = x + yf / torch.sqrt((yf * yf).mean(-1, keepdim=True) + 1e-5) * wa.float()
        ref = summed / torch.sqrt((summed * summed).mean(-1, keepdim=True) + 1e-6) * wb.float()
        rows = torch.tensor([5, 0, 5], dtype=torch.int32, device="cuda")
        picked = torch.empty(3, dim, device="cuda", dtype=dt)
        ops.sandwich_norm(x.clone(), y, wa, 1e-5, wb, 1e-6, picked, rows)
        ops.sandwich_norm(x, y, wa, 1e-5, wb, 1e-6, out)
        tol = 1e-5 if dt == torch.float32 else 2e-2
        assert float((x - summed).abs().max()) <= 1e-5
        assert float((out.float() - ref).abs().max()) <= tol
        assert float((picked.float() - ref[rows.long()]).abs().max()) <= tol


def test_gated_unit_soft_cap_and_batched_product_kernels():
    from fastllm_py_b200.native import ops

    torch.manual_seed(1)
    gu = torch.randn(5, 2 * 37, device="cuda")
    acts = {"silu": torch.nn.functional.silu, "relu": torch.relu,
            "gelu_tanh": lambda z: torch.nn.functional.gelu(z, approximate="tanh")}
    for name, fn in acts.items():
        out = torch.empty(5, 37, device="cuda")
        ops.glu(gu, out, name)
        assert float((out - fn(gu[:, :37]) * gu[:, 37:]).abs().max()) <= 1e-6
    logits = 40 * torch.randn(3, 100, device="cuda")
    ref = 7.5 * torch.tanh(logits / 7.5)
    ops.softcap(logits, 7.5)
    assert float((logits - ref).abs().max()) <= 1e-5
    a = torch.randn(70, 3 * 11, device="cuda")                    # three heads, 9 of each head's 11 columns used
    w = torch.randn(3, 13, 9, device="cuda").to(torch.bfloat16)
    out = torch.zeros(70, 3 * 15, device="cuda")
    ops.gemm_simt_batched(a, 11, w, out, 15)
    for h in range(3):
        ref = a[:, h * 11:h * 11 + 9] @ w[h].float().T
        assert float((out[:, h * 15:h * 15 + 13] - ref).abs().max()) <= 1e-4
        assert float(out[:, h * 15 + 13:(h + 1) * 15].abs().max()) == 0.0
    # the same product on tensor cores: 5 heads of 64 + 16 columns, 150 outputs each, 70 and 3 rows
    for rows in (70, 3):
        a = torch.randn(rows, 5 * 80, device="cuda").to(torch.bfloat16)
        w = torch.randn(5, 150, 64, device="cuda").to(torch.bfloat16)
        for dt in (torch.float32, torch.bfloat16):
            out = torch.zeros(rows, 5 * 152, device="cuda", dtype=dt)
            ops.gemm_batched(a, 80, w, out, 152)
            for h in range(5):
                ref = a[:, h * 80:h * 80 + 64].float() @ w[h].float().T
                assert float((out[:, h * 152:h * 152 + 150].float() - ref).abs().max()) <= (1e-3 if dt == torch.float32 else 0.15)
                assert float(out[:, h * 152 + 150:(h + 1) * 152].abs().max()) == 0.0


def test_router_kernel_choice_weights_and_ties():
    from fastllm_py_b200.native import ops

    torch.manual_seed(2)
    h = torch.randn(50, 24, device="cuda")
    wr = torch.randn(9, 24, device="cuda") * 0.3
    bias = torch.randn(9, device="cuda")
    chosen = torch.empty(50, 4, dtype=torch.int32, device="cuda")
    weights = torch.empty(50, 4, device="cuda")
    z = (h.double() @ wr.double().T).float()
    ops.moe_pick(z, bias, chosen, weights, 4)
    s = torch.sigmoid(z.double())
    ref = torch.topk(s + bias.double(), 4, dim=-1).indices
    assert torch.equal(chosen.long().sort(-1).values, ref.sort(-1).values)
    assert float((weights.double() - s.gather(1, chosen.long())).abs().max()) <= 1e-6
    chosen3 = torch.empty(50, 3, dtype=torch.int32, device="cuda")
    weights3 = torch.empty(50, 3, device="cuda")
    ops.moe_pick(z, None, chosen3, weights3, 3, True, True)           # softmax scores, renormalised
    p = torch.softmax(z.double(), -1)
    top = torch.topk(p, 3, dim=-1)
    assert torch.equal(chosen3.long(), top.indices)
    assert float((weights3.double() - top.values / top.values.sum(-1, keepdim=True)).abs().max()) <= 1e-6
    two, two_w = torch.empty(2, 4, dtype=torch.int32, device="cuda"), torch.empty(2, 4, device="cuda")
    ops.moe_pick(torch.zeros(2, 9, device="cuda"), None, two, two_w, 4)                      # all scores equal
    assert two.tolist() == [[0, 1, 2, 3]] * 2


@pytest.mark.parametrize("rank,rot,heads,window", [(160, 32, 5, 37), (64, 16, 19, None), (256, 32, 16, 100)])
def test_tensor_core_latent_attention_against_the_cuda_core_kernel(rank, rot, heads, window):
    """Scattered pages, prompt portions beside single tokens, windows that end inside a tile of keys; one
    query and key scaled so that a single far key just inside the window carries its row."""
    from fastllm_py_b200.native import ops

    torch.manual_seed(rank)
    page, width, n_pages = 8, rank + rot, 64
    cache = torch.randn(n_pages, page, width, device="cuda").to(torch.bfloat16)
    lens = [(0, 70), (150, 1), (33, 9), (199, 1)]                     # (cached before the step, tokens in it)
    table = torch.randperm(n_pages, device="cuda").to(torch.int32).view(len(lens), -1).contiguous()
    tok_req = torch.tensor([r for r, (_, n) in enumerate(lens) for _ in range(n)], dtype=torch.int32, device="cuda")
    positions = torch.tensor([c + i for c, n in lens for i in range(n)], dtype=torch.int32, device="cuda")
    n = tok_req.numel()
    q = (0.3 * torch.randn(n, heads * width, device="cuda")).to(torch.bfloat16)
    if window is not None:                                                # request 1's token sees position 150 - window + 1 last
        far = 150 - window + 1
        row = cache[table[1, far // page].long(), far % page]
        q[70, :width] = (4.0 * row.float() / row.float().norm()).to(torch.bfloat16)
    want = torch.empty(n, heads * rank, device="cuda")
    got = torch.empty_like(want)
    ops.latent_attention(q, want, cache, table, tok_req, positions, heads, rank, rot, window, 0.2, page)
    ops.latent_attention_tc(q, got, cache, table, tok_req, positions, heads, rank, rot, window, 0.2, page)
    split = torch.empty_like(want)                                    # the same with the keys shared out over blocks
    span = 200 if window is None else min(window, 200)
    parts = torch.empty(n * heads * ((span - 1) // 64 + 2) * (rank + 2), device="cuda")
    ops.latent_attention_tc(q, split, cache, table, tok_req, positions, heads, rank, rot, window, 0.2, page,
                            64, (span - 1) // 64 + 2, parts)
    torch.cuda.synchronize()
    for result in (got, split):
        assert float((result - want).abs().max()) <= 2e-2
        assert float((result - want).abs().mean()) <= 2e-3


def test_gated_product_with_relu_and_gelu_in_its_epilogue():
    """The tensor-core product that applies the gate's activation itself, for the activations beside silu,
    in its one-tile form (a decode-sized step) and its CTA-pair form (a prompt-sized step)."""
    from fastllm_py_b200.native import gemm_tc

    torch.manual_seed(5)
    acts = {"relu": torch.relu, "gelu_tanh": lambda z: torch.nn.functional.gelu(z, approximate="tanh"),
            "silu": torch.nn.functional.silu}
    taken = 0
    for m, inter, k in ((48, 1536, 256), (2048, 4096, 512)):
        a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
        w = (torch.randn(2 * inter, k, device="cuda") * k ** -0.5).to(torch.bfloat16)
        for name, fn in acts.items():
            out = torch.zeros(m, inter, device="cuda", dtype=torch.bfloat16)
            if not gemm_tc.gemm_swiglu(a, w, out, name):
                continue
            taken += 1
            prod = a.float() @ w.float().T
            ref = fn(prod[:, :inter]) * prod[:, inter:]
            assert float((out.float() - ref).abs().max()) <= 0.03 * float(ref.abs().max()) + 1e-2, (m, name)
    assert taken >= 3
