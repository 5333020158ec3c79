"""Small Lasonex configurations and weights for the tests.

`config(...)` builds the raw config.json dict from layer descriptions, `weights(raw, seed)` draws
every tensor (bfloat16, like a stored model), `write(raw, tensors, folder)` makes a model folder.
The spread of each kind of tensor is chosen so that every mechanism matters: norm weights away
from 1, the four small vectors of differential attention large enough to move lambda, router rows
large enough that groups and choices differ from token to token.
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def attention(heads=4, kv_heads=2, dim=16, vdim=24, window=11, rot=8, base=10000.0, scaling=None, diff=0.3, scale=None):
    m = {"diff": diff, "dim": dim, "heads": heads, "kv_heads": kv_heads, "rot": {"base": base, "dims": rot},
         "scale": scale if scale is not None else dim ** -0.5, "vdim": vdim}
    if window is not None:
        m["mask"] = {"size": window}
    if scaling is not None:
        factor, original, fast, slow = scaling
        m["rot"]["scaling"] = {"factor": factor, "fast": fast, "original": original, "slow": slow}
    return {"type": "attention", "mixer": m}


def retention(heads=2, dim=16, vdim=8, decay=None, rot=8, base=10000.0):
    if decay is None:
        decay = [1.0 - 2.0 ** (-3 - 1.5 * h) for h in range(heads)]
    return {"type": "retention", "mixer": {"decay": list(decay), "dim": dim, "heads": heads,
                                           "rot": {"base": base, "dims": rot}, "vdim": vdim}}


def dense(ff=48, limit=0.75):
    return {"ff": ff, "kind": "dense", "limit": limit}


def moe(experts=6, top=2, ff=24, limit=1.25, groups=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"expert": {"ff": ff, "limit": limit}, "kind": "moe", "router": router}


def config(layers, vocab=97, width=40, eps=1e-5, embed_scale=3.0):
    """layers: list of (mixer description, mlp description | None)."""
    return {"architecture": "Lasonex", "embedding": {"scale": embed_scale},
            "layers": [dict(m, mlp=f) for m, f in layers], "norm": {"eps": eps}, "vocab": vocab, "width": width}


def tensor_shapes(raw) -> dict:
    w = raw["width"]
    out = {"embed": (raw["vocab"], w), "final.norm": (w,), "head": (raw["vocab"], w)}
    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = (w,)
        if layer["type"] == "attention":
            out[p + "mix.q"] = (m["heads"] * 2 * m["dim"], w)
            out[p + "mix.k"] = (m["kv_heads"] * 2 * m["dim"], w)
            out[p + "mix.v"] = (m["kv_heads"] * m["vdim"], w)
            for s in ("lq1", "lk1", "lq2", "lk2"):
                out[f"{p}mix.{s}"] = (m["dim"],)
            out[p + "mix.o"] = (w, m["heads"] * m["vdim"])
        else:
            out[p + "mix.q"] = out[p + "mix.k"] = (m["heads"] * m["dim"], w)
            out[p + "mix.v"] = out[p + "mix.g"] = (m["heads"] * m["vdim"], w)
            out[p + "mix.o"] = (w, m["heads"] * m["vdim"])
        f = layer["mlp"]
        if f is None:
            continue
        out[p + "norm2"] = (w,)
        if f["kind"] == "dense":
            out[p + "mlp.gate"] = out[p + "mlp.up"] = (f["ff"], w)
            out[p + "mlp.down"] = (w, f["ff"])
        else:
            e_ff = f["expert"]["ff"]
            out[p + "mlp.router"] = (f["router"]["experts"], w)
            for e in range(f["router"]["experts"]):
                out[f"{p}mlp.e{e}.gate"] = out[f"{p}mlp.e{e}.up"] = (e_ff, w)
                out[f"{p}mlp.e{e}.down"] = (w, e_ff)
    return out


def weights(raw, seed=0, gain=1.0, sharp=1.0) -> dict:
    """`gain` scales all matrices; `sharp` scales the query and key matrices of the attention layers on
    top (larger: peakier softmax, so single keys decide outputs)."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    kinds = [layer["type"] for layer in raw["layers"]]
    for name, shape in tensor_shapes(raw).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2") or name == "final.norm":
            t = 1.0 + 0.3 * torch.randn(shape, generator=gen)
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            t = 0.35 * torch.randn(shape, generator=gen)
        elif name == "embed":
            t = torch.randn(shape, generator=gen) * 0.4
        elif leaf == "router":
            t = torch.randn(shape, generator=gen) * 3.0 / shape[1] ** 0.5
        else:
            t = torch.randn(shape, generator=gen) * gain * (1.5 / shape[1] ** 0.5)
            if ".mix." in name and leaf in ("q", "k") and kinds[int(name[1:name.index(".")])] == "attention":
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
