"""Tigitar without a GPU: configuration keys, the plan of parts, cache needs, the random-weights folder,
and the plain implementation's own properties (what the GPU tests lean on)."""
import copy
import json

import pytest
import torch

import plain_tigitar as plain
import tigitar_tiny as tt
from fastllm_py_b200.architectures.tigitar import make_plan
from fastllm_py_b200.cache.needs import FixedState, PagedRows
from fastllm_py_b200.config import ConfigError, load_config
from fastllm_py_b200.config.tigitar import TigitarConfig
from fastllm_py_b200.parts import BuildContext, Decoder
from fastllm_py_b200.weights import write_model_folder

RAW = tt.config([(tt.delta(4, 2, 16, 8, 3), tt.dense(48)),
                 (tt.latent(2, 16, 8, 16, 24, window=11), tt.moe(6, 2, 24)),
                 (tt.latent(3, 8, 8, 4, 24, window=30, kv_from=1), None),
                 (tt.latent(2, 16, 8, 16, 24, window=None), tt.dense(16)),
                 (tt.latent(2, 16, 8, 16, 24, window=5, kv_from=3), tt.dense(16))], vocab=97, width=40, softcap=9.0)


def decoder(raw, page=8):
    cfg = TigitarConfig.from_hf(raw)
    return cfg, Decoder(make_plan(cfg), BuildContext(torch.device("cpu"), torch.float32, page, 64))


def test_config_reads_back_and_names_every_tensor():
    cfg, dec = decoder(RAW)
    assert cfg.to_hf() == RAW
    assert TigitarConfig.from_hf(json.loads(json.dumps(cfg.to_hf()))) == cfg
    assert dec.expected_tensors() == tt.tensor_shapes(RAW)
    assert "Tigitar" in cfg.summary()


def test_cache_needs_follow_the_layers():
    _, dec = decoder(RAW)
    needs = dec.cache_needs()
    assert needs[0] == FixedState((4 * 8 * 16 + 2 * (2 * 2 * 16 + 4 * 8),), "float32")
    assert needs[1] == PagedRows(32, 30)             # the reader's window is the wider one
    assert needs[3] == PagedRows(32, None)           # the owner sees everything: nothing may go back
    assert set(needs) == {0, 1, 3}
    assert [run.cache for run in dec.order] == [None, None, 1, None, 3]


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "conv", "type"),
    (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 1, "mixer", "rot", "dims"), 6, "rot.dims"),
    (("layers", 1, "mixer", "rot_dim"), 7, "rot"),
    (("layers", 2, "mixer", "kv_from"), 0, "kv_from"),
    (("layers", 2, "mixer", "kv_rank"), 16, "kv_rank"),
    (("layers", 1, "mlp", "router", "top"), 7, "top"),
    (("layers", 1, "mlp", "kind"), "sparse", "kind"),
    (("width",), "wide", "width"),
])
def test_wrong_values_are_refused_by_name(path, value, word):
    raw = copy.deepcopy(RAW)
    at = raw
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        TigitarConfig.from_hf(raw)


def test_a_written_folder_loads_by_its_architecture_string(tmp_path):
    cfg = TigitarConfig.from_hf(RAW)
    folder = write_model_folder(cfg, tmp_path / "m", seed=3)
    arch, again = load_config(folder)
    assert arch.name == "Tigitar" and again == cfg
    from safetensors import safe_open

    with safe_open(str(folder / "model.safetensors"), framework="pt") as f:
        assert {k: tuple(f.get_slice(k).get_shape()) for k in f.keys()} == tt.tensor_shapes(RAW)


def test_plain_implementation_is_causal_and_its_windows_and_state_matter():
    raw = tt.config([(tt.delta(2, 1, 8, 8, 3), tt.moe(4, 2, 8)), (tt.latent(2, 8, 4, 8, 12, window=4), tt.dense(16))],
                    width=24, vocab=30)
    w = tt.weights(raw, seed=1, sharp=4.0)
    toks = list(range(3, 23))
    full = plain.forward(raw, w, toks)
    assert torch.allclose(plain.forward(raw, w, toks[:11]), full[:11], atol=1e-12)
    wider = copy.deepcopy(raw)
    wider["layers"][1]["mixer"]["mask"]["size"] = 5
    assert float((plain.forward(wider, w, toks) - full)[6:].abs().max()) > 1e-3
    assert torch.allclose(plain.forward(wider, w, toks)[:4], full[:4], atol=1e-12)      # the first tokens see all either way
    moved = plain.forward(raw, w, [toks[0] + 1] + toks[1:])
    assert float((moved - full)[-1].abs().max()) > 1e-6                                 # the delta rule's state reaches back
    nocap = dict(raw)
    nocap.pop("logit_softcap")
    assert float(plain.forward(nocap, w, toks).abs().max()) >= float(full.abs().max())
