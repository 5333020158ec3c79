"""LasonexConfig: the typed configuration of the Lasonex decoder.

A Lasonex model is a list of parallel layers (mixer and feed-forward read the
same normed input and are added together), each with one of two mixers and an
optional feed-forward.  Its config.json is nested:

    architecture     "Lasonex"
    vocab, width     sizes of the embedding table and the residual stream
    embedding.scale  the factor on the embedding rows
    norm.eps         the epsilon of every RMS norm (the unweighted per-head ones too)
    layers[i]        {"type": "attention" | "retention", "mixer": {...}, "mlp": {...} | null}

    mixer of "attention" (differential attention: two softmax maps per head over the same values):
        heads, kv_heads, dim (per map), vdim, scale, diff, mask {size} (absent: all earlier tokens),
        rot {base, dims, scaling {factor, original, fast, slow} (absent: none)}
    mixer of "retention" (linear attention with a fixed decay per head):
        heads, dim, vdim, decay [heads], rot {base, dims, scaling (absent: none)}
    mlp "dense":  ff, limit
    mlp "moe":    expert {ff, limit}, router {experts, top, groups {count, keep} (absent: no groups)}

Every size and constant above is read here and nowhere else; the parts get them
as parameters from the plan (architectures/lasonex.py).
"""
from __future__ import annotations

from dataclasses import dataclass

from .base import ConfigError, KeyReader


@dataclass(frozen=True)
class RotationConfig:
    base: float
    dims: int
    scaling: tuple | None            # None | ("yarn", factor, original, fast, slow)

    def to_raw(self) -> dict:
        out = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            _, factor, original, fast, slow = self.scaling
            out["scaling"] = {"factor": factor, "fast": fast, "original": original, "slow": slow}
        return out


@dataclass(frozen=True)
class DifferentialAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    window: int | None
    rot: RotationConfig

    def to_raw(self) -> dict:
        out = {"diff": self.diff, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
               "rot": self.rot.to_raw(), "scale": self.scale, "vdim": self.vdim}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        return out


@dataclass(frozen=True)
class RetentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: tuple
    rot: RotationConfig

    def to_raw(self) -> dict:
        return {"decay": list(self.decay), "dim": self.dim, "heads": self.heads, "rot": self.rot.to_raw(),
                "vdim": self.vdim}


@dataclass(frozen=True)
class ClampedFeedForwardConfig:
    ff: int
    limit: float

    def to_raw(self) -> dict:
        return {"ff": self.ff, "kind": "dense", "limit": self.limit}


@dataclass(frozen=True)
class GroupedExpertsConfig:
    experts: int
    top: int
    groups: int | None               # None: every expert can be chosen
    keep: int | None
    ff: int
    limit: float

    def to_raw(self) -> dict:
        router = {"experts": self.experts, "top": self.top}
        if self.groups is not None:
            router["groups"] = {"count": self.groups, "keep": self.keep}
        return {"expert": {"ff": self.ff, "limit": self.limit}, "kind": "moe", "router": router}


@dataclass(frozen=True)
class LasonexLayerConfig:
    type: str                        # "attention" | "retention"
    mixer: object
    mlp: object                      # ClampedFeedForwardConfig | GroupedExpertsConfig | None

    def to_raw(self) -> dict:
        return {"mixer": self.mixer.to_raw(), "mlp": None if self.mlp is None else self.mlp.to_raw(),
                "type": self.type}


def _sub(raw: dict, key: str, where: str) -> dict:
    v = raw.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}.{key} must be an object, got {v!r}")
    return v


def _rotation(raw: dict, where: str, dim: int) -> RotationConfig:
    r = KeyReader(_sub(raw, "rot", where))
    dims = r.integer("dims", minimum=0)
    if dims % 2 or dims > dim:
        raise ConfigError(f"rot.dims {dims} must be even and at most dim {dim}")
    scaling = r.mapping("scaling")
    if scaling is not None:
        s = KeyReader(scaling)
        scaling = ("yarn", s.number("factor"), s.number("original"), s.number("fast"), s.number("slow"))
    return RotationConfig(r.number("base"), dims, scaling)


def _mixer(kind: str, raw: dict, i: int):
    where = f"layers[{i}].mixer"
    r = KeyReader(raw)
    try:
        if kind == "attention":
            heads, kv_heads, dim = r.integer("heads"), r.integer("kv_heads"), r.integer("dim")
            if heads % kv_heads:
                raise ConfigError(f"heads {heads} is not a multiple of kv_heads {kv_heads}")
            mask = r.mapping("mask")
            window = None if mask is None else KeyReader(mask).integer("size")
            return DifferentialAttentionConfig(heads, kv_heads, dim, r.integer("vdim"), r.number("scale"),
                                               r.number("diff", positive=False), window, _rotation(raw, where, dim))
        if kind == "retention":
            heads, dim = r.integer("heads"), r.integer("dim")
            decay = raw.get("decay")
            if not isinstance(decay, list) or len(decay) != heads or \
                    not all(isinstance(d, (int, float)) and not isinstance(d, bool) for d in decay):
                raise ConfigError(f"decay must be a list of {heads} numbers, one per head")
            return RetentionConfig(heads, dim, r.integer("vdim"), tuple(float(d) for d in decay),
                                   _rotation(raw, where, dim))
    except ConfigError as e:
        raise ConfigError(f"{e} (in {where})") from None
    raise ConfigError(f"config.json: layers[{i}].type {kind!r} is not a mixer of this architecture "
                      f"('attention', 'retention')")


def _mlp(raw, i: int):
    if raw is None:
        return None
    where = f"layers[{i}].mlp"
    if not isinstance(raw, dict):
        raise ConfigError(f"config.json: {where} must be an object or null, got {raw!r}")
    kind = raw.get("kind")
    try:
        if kind == "dense":
            r = KeyReader(raw)
            return ClampedFeedForwardConfig(r.integer("ff"), r.number("limit"))
        if kind == "moe":
            router = KeyReader(_sub(raw, "router", where))
            experts, top = router.integer("experts"), router.integer("top")
            if top > experts:
                raise ConfigError(f"router.top {top} exceeds router.experts {experts}")
            groups = router.mapping("groups")
            count = keep = None
            if groups is not None:
                g = KeyReader(groups)
                count, keep = g.integer("count"), g.integer("keep")
                if experts % count or keep > count:
                    raise ConfigError(f"router.groups: {count} groups must divide {experts} experts, and keep "
                                      f"{keep} of them")
                if keep * (experts // count) < top:
                    raise ConfigError(f"router.groups: {keep} groups of {experts // count} experts cannot "
                                      f"give {top} choices")
            expert = KeyReader(_sub(raw, "expert", where))
            return GroupedExpertsConfig(experts, top, count, keep, expert.integer("ff"), expert.number("limit"))
    except ConfigError as e:
        raise ConfigError(f"{e} (in {where})") from None
    raise ConfigError(f"config.json: {where}.kind {kind!r} is not supported ('dense', 'moe')")


@dataclass(frozen=True)
class LasonexConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: tuple

    @classmethod
    def from_hf(cls, raw: dict) -> "LasonexConfig":
        r = KeyReader(raw)
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        layers = []
        for i, lr in enumerate(layers_raw):
            if not isinstance(lr, dict) or not isinstance(lr.get("type"), str):
                raise ConfigError(f"config.json: layers[{i}] must be an object with a 'type'")
            mixer = _mixer(lr["type"], _sub(lr, "mixer", f"layers[{i}]"), i)
            layers.append(LasonexLayerConfig(lr["type"], mixer, _mlp(lr.get("mlp"), i)))
        norm = KeyReader(_sub(raw, "norm", "config"))
        embedding = r.mapping("embedding")
        scale = 1.0 if embedding is None else KeyReader(embedding).number("scale", default=1.0)
        return cls(vocab=r.integer("vocab"), width=r.integer("width"), norm_eps=norm.number("eps"),
                   embedding_scale=scale, layers=tuple(layers))

    def summary(self) -> str:
        """One line for a load message."""
        kinds = [layer.type for layer in self.layers]
        routed = sum(isinstance(layer.mlp, GroupedExpertsConfig) for layer in self.layers)
        return (f"Lasonex: {len(kinds)}L width={self.width} ({kinds.count('attention')} differential attention, "
                f"{kinds.count('retention')} retention; {routed} with routed experts)")

    def to_hf(self) -> dict:
        """The config.json that reads back as this configuration."""
        return {"architecture": "Lasonex", "embedding": {"scale": self.embedding_scale},
                "layers": [layer.to_raw() for layer in self.layers], "norm": {"eps": self.norm_eps},
                "vocab": self.vocab, "width": self.width}
