"""Small Tigitar configurations and weights for the tests.

`config(...)` builds the raw config.json dict from layer descriptions, `weights(raw, seed)`
draws every tensor (bfloat16, like a stored model), `write(raw, tensors, folder)` makes a model
folder.  The spread of each kind of tensor is chosen so that every mechanism matters: decays
between 0.3 and 1, corrections large enough to change an expert choice, norm weights away from 1.
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def delta(heads=4, kv_heads=2, dim=16, vdim=8, conv=4):
    return {"type": "delta", "mixer": {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim}}


def latent(heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=24, window=None, kv_from=None, base=10000.0, scale=None):
    m = {"dim": dim, "heads": heads, "kv_rank": kv_rank, "rot": {"base": base, "dims": rot_dim}, "rot_dim": rot_dim,
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5, "vdim": vdim}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def dense(ff=48):
    return {"ff": ff, "kind": "dense"}


def moe(experts=6, top=2, ff=24):
    return {"expert": {"ff": ff}, "kind": "moe", "router": {"experts": experts, "top": top}}


def config(layers, vocab=97, width=40, eps=1e-5, softcap=12.0):
    """layers: list of (mixer description, mlp description | None)."""
    raw = {"architecture": "Tigitar", "layers": [dict(m, mlp=f) for m, f in layers], "norm": {"eps": eps},
           "vocab": vocab, "width": width}
    if softcap is not None:
        raw["logit_softcap"] = softcap
    return raw


def tensor_shapes(raw) -> dict:
    w = raw["width"]
    out = {"embed": (raw["vocab"], w), "final.norm": (w,), "head": (raw["vocab"], w)}
    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = out[p + "norm1b"] = (w,)
        if layer["type"] == "delta":
            qk, hv = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"]
            for s, rows in (("q", qk), ("k", qk), ("v", hv)):
                out[f"{p}mix.{s}"] = (rows, w)
                out[f"{p}mix.{s}.conv"] = (rows, m["conv"])
            out[p + "mix.b"] = out[p + "mix.a"] = (m["heads"], w)
            out[p + "mix.A_log"] = out[p + "mix.dt_bias"] = (m["heads"],)
            out[p + "mix.norm"] = (m["vdim"],)
            out[p + "mix.g"] = (hv, w)
            out[p + "mix.o"] = (w, hv)
        else:
            h = m["heads"]
            out[p + "mix.q"] = (h * (m["dim"] + m["rot_dim"]), w)
            if "kv_from" not in m:
                out[p + "mix.dkv"] = (m["kv_rank"] + m["rot_dim"], w)
                out[p + "mix.dkv.norm"] = (m["kv_rank"],)
            out[p + "mix.uk"] = (h * m["dim"], m["kv_rank"])
            out[p + "mix.uv"] = (h * m["vdim"], m["kv_rank"])
            out[p + "mix.o"] = (w, h * m["vdim"])
        f = layer["mlp"]
        if f is None:
            continue
        out[p + "norm2"] = out[p + "norm2b"] = (w,)
        if f["kind"] == "dense":
            out[p + "mlp.gate"] = out[p + "mlp.up"] = (f["ff"], w)
            out[p + "mlp.down"] = (w, f["ff"])
        else:
            e_ff = f["expert"]["ff"]
            out[p + "mlp.router"] = (f["router"]["experts"], w)
            out[p + "mlp.correction"] = (f["router"]["experts"],)
            for e in range(f["router"]["experts"]):
                out[f"{p}mlp.e{e}.gate"] = out[f"{p}mlp.e{e}.up"] = (e_ff, w)
                out[f"{p}mlp.e{e}.down"] = (w, e_ff)
    return out


def weights(raw, seed=0, gain=1.0, sharp=1.0) -> dict:
    """`gain` scales all matrices; `sharp` scales query and key-side matrices of the attention
    layers on top (larger: peakier softmax, so single keys decide outputs)."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(raw).items():
        leaf = name.split(".")[-1]
        if name.endswith(".conv"):
            t = torch.randn(shape, generator=gen) * 0.5
        elif leaf in ("norm1", "norm2", "norm1b", "norm2b", "norm") or name == "final.norm":
            t = 1.0 + 0.3 * torch.randn(shape, generator=gen)
        elif leaf == "A_log":
            t = torch.rand(shape, generator=gen) * 2.5 - 3.0
        elif leaf == "dt_bias":
            t = torch.randn(shape, generator=gen)
        elif leaf == "correction":
            t = 0.4 * torch.randn(shape, generator=gen)
        elif name == "embed":
            t = torch.randn(shape, generator=gen)
        else:
            t = torch.randn(shape, generator=gen) * gain * (1.5 / shape[1] ** 0.5)
            if ".mix." in name and leaf in ("dkv", "uk") or (leaf == "q" and name + ".conv" not in tensor_shapes(raw)):
                t = t * sharp
        out[name] = t.to(torch.bfloat16)
    return out


def write(raw, tensors, folder):
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(raw, indent=1))
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder
