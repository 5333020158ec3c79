"""Lasonex without a GPU: configuration keys, the plan of parts, cache needs, the rotary tables, the
random-weights folder, and the plain implementation's own properties (what the GPU tests lean on)."""
import copy
import json

import numpy as np
import pytest
import torch

import lasonex_tiny as lt
import plain_lasonex as plain
from fastllm_py_b200.architectures.lasonex import make_plan
from fastllm_py_b200.cache.needs import FixedState, PagedKeysValues
from fastllm_py_b200.config import ConfigError, load_config
from fastllm_py_b200.config.lasonex import LasonexConfig
from fastllm_py_b200.parts import BuildContext, Decoder, PartSpec, build_part
from fastllm_py_b200.weights import write_model_folder

YARN = (4.0, 64, 8.0, 1.0)
RAW = lt.config([(lt.attention(4, 2, 16, 24, window=11, rot=8, scaling=YARN), lt.dense(48, 0.8)),
                 (lt.retention(3, 12, 20, rot=6), lt.moe(6, 2, 24, 1.25, groups=(3, 2))),
                 (lt.attention(3, 3, 10, 6, window=None, rot=10, diff=0.7), None),
                 (lt.retention(1, 8, 8, rot=0), lt.moe(4, 4, 8, 2.0))], vocab=97, width=40, embed_scale=5.0)


def decoder(raw, page=8):
    cfg = LasonexConfig.from_hf(raw)
    return cfg, Decoder(make_plan(cfg), BuildContext(torch.device("cpu"), torch.float32, page, 64))


def test_config_reads_back_and_names_every_tensor():
    cfg, dec = decoder(RAW)
    assert cfg.to_hf() == RAW
    assert LasonexConfig.from_hf(json.loads(json.dumps(cfg.to_hf()))) == cfg
    assert dec.expected_tensors() == lt.tensor_shapes(RAW)
    assert "Lasonex" in cfg.summary()
    assert dec.embedding.scale == 5.0


def test_cache_needs_follow_the_layers():
    _, dec = decoder(RAW)
    needs = dec.cache_needs()
    assert needs[0] == PagedKeysValues(2, 32, 24, 11)
    assert needs[1] == FixedState((3 * 20 * 12,), "float32")
    assert needs[2] == PagedKeysValues(3, 20, 6, None)          # no window: nothing may go back
    assert needs[3] == FixedState((64,), "float32")
    assert dec.blocks[3].mixer.position is None                 # no rotated dimensions: no tables


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "conv", "type"),
    (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "rot.dims"),
    (("layers", 0, "mixer", "rot", "dims"), 18, "rot.dims"),
    (("layers", 0, "mixer", "rot", "scaling", "factor"), "big", "factor"),
    (("layers", 1, "mixer", "decay"), [0.5, 0.9], "decay"),
    (("layers", 1, "mlp", "router", "top"), 7, "top"),
    (("layers", 1, "mlp", "router", "groups", "count"), 4, "groups"),
    (("layers", 1, "mlp", "router", "groups", "keep"), 4, "groups"),
    (("layers", 1, "mlp", "kind"), "sparse", "kind"),
    (("layers", 0, "mlp", "limit"), None, "limit"),
    (("width",), "wide", "width"),
])
def test_wrong_values_are_refused_by_name(path, value, word):
    raw = copy.deepcopy(RAW)
    at = raw
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        LasonexConfig.from_hf(raw)


def test_groups_too_small_for_the_choices_are_refused():
    raw = copy.deepcopy(RAW)
    raw["layers"][1]["mlp"]["router"].update(top=5)                  # 2 groups of 2 experts cannot give 5
    with pytest.raises(ConfigError, match="groups"):
        LasonexConfig.from_hf(raw)


def test_a_written_folder_loads_by_its_architecture_string(tmp_path):
    cfg = LasonexConfig.from_hf(RAW)
    folder = write_model_folder(cfg, tmp_path / "m", seed=3)
    arch, again = load_config(folder)
    assert arch.name == "Lasonex" and again == cfg
    from safetensors import safe_open

    with safe_open(str(folder / "model.safetensors"), framework="pt") as f:
        assert {k: tuple(f.get_slice(k).get_shape()) for k in f.keys()} == lt.tensor_shapes(RAW)


@pytest.mark.parametrize("scaling", [None, ("yarn",) + YARN, ("yarn", 6.0, 1024, 16.0, 2.0)])
def test_rotary_tables_follow_the_blend(scaling):
    """The position part's tables against the oracle's own (written apart from it)."""
    spec = PartSpec("rotary", dict(rot_dim=12, theta=700.0, scaling=scaling, exact=True))
    part = build_part("position", spec, BuildContext(torch.device("cpu"), torch.float32, 8, 300))
    cos, sin = part.tables()
    raw = None if scaling is None else dict(zip(("factor", "original", "fast", "slow"), scaling[1:]))
    want_cos, want_sin = plain.rotary_tables(300, 12, 700.0, raw)
    assert np.allclose(cos.numpy(), want_cos.numpy(), atol=1e-6) and np.allclose(sin.numpy(), want_sin.numpy(), atol=1e-6)
    if scaling is not None:                                   # the slow pairs are stretched, the gain is on both tables
        plain_cos, _ = plain.rotary_tables(300, 12, 700.0, None)
        assert float((want_cos - plain_cos).abs().max()) > 0.1
        assert abs(float(want_cos[0, 0]) - (0.1 * np.log(scaling[1]) + 1.0)) < 1e-12


def test_plain_implementation_is_causal_and_its_windows_state_and_groups_matter():
    raw = lt.config([(lt.retention(2, 8, 8, rot=4), lt.moe(6, 2, 8, groups=(3, 1))),
                     (lt.attention(2, 1, 8, 8, window=4, rot=8), lt.dense(16))], width=24, vocab=30)
    w = lt.weights(raw, seed=1, sharp=4.0)
    toks = list(range(3, 23))
    full = plain.forward(raw, w, toks)
    assert torch.allclose(plain.forward(raw, w, toks[:11]), full[:11], atol=1e-12)
    wider = copy.deepcopy(raw)
    wider["layers"][1]["mixer"]["mask"]["size"] = 5
    assert float((plain.forward(wider, w, toks) - full)[6:].abs().max()) > 1e-3
    assert torch.allclose(plain.forward(wider, w, toks)[:4], full[:4], atol=1e-12)      # the first tokens see all either way
    moved = plain.forward(raw, w, [toks[0] + 1] + toks[1:])
    assert float((moved - full)[-1].abs().max()) > 1e-6                                 # the retention state reaches back
    free = copy.deepcopy(raw)
    free["layers"][0]["mlp"]["router"]["groups"]["keep"] = 3
    assert float((plain.forward(free, w, toks) - full).abs().max()) > 1e-3              # the groups limit the choice
    nodiff = copy.deepcopy(raw)
    nodiff["layers"][1]["mixer"]["diff"] = 0.1
    assert float((plain.forward(nodiff, w, toks) - full).abs().max()) > 1e-3


def test_routing_oracle_keeps_to_the_best_groups():
    h = torch.randn(50, 16, dtype=torch.float64, generator=torch.Generator().manual_seed(0))
    router = torch.randn(12, 16, dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    chosen, w = plain.route(h, router, {"experts": 12, "top": 3, "groups": {"count": 4, "keep": 2}})
    s = torch.softmax(h @ router.T, dim=-1)
    best = s.view(50, 4, 3).max(dim=-1).values
    for t in range(50):
        kept = set(best[t].topk(2).indices.tolist())
        assert {e // 3 for e in chosen[t].tolist()} <= kept
    assert torch.allclose(w.sum(dim=-1), torch.ones(50, dtype=torch.float64))
