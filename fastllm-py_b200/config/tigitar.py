"""TigitarConfig: the typed configuration of the Tigitar hybrid decoder.

A Tigitar model is a list of layers, each with one of two mixers and an optional
feed-forward.  Its config.json is nested:

    architecture   "Tigitar"
    vocab, width   sizes of the embedding table and the residual stream
    norm.eps       the epsilon of every RMS norm
    logit_softcap  c: logits become c * tanh(logits / c); absent or null: none
    layers[i]      {"type": "delta" | "latent_attention", "mixer": {...}, "mlp": {...} | null}

    mixer of "delta" (gated delta rule):  heads, kv_heads, dim, vdim, conv (taps)
    mixer of "latent_attention":          heads, dim, rot_dim, vdim, kv_rank, scale,
                                          rot {base, dims}, mask {size} (absent: all earlier tokens),
                                          kv_from (absent: the layer has a latent cache of its own)
    mlp "dense":  ff                      mlp "moe":  expert {ff}, router {experts, top}

Every size and constant above is read here and nowhere else; the parts get them
as parameters from the plan (architectures/tigitar.py).
"""
from __future__ import annotations

from dataclasses import dataclass

from .base import ConfigError, KeyReader


@dataclass(frozen=True)
class DeltaMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    def to_raw(self) -> dict:
        return {"conv": self.conv, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
                "vdim": self.vdim}


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    window: int | None
    kv_from: int | None

    def to_raw(self) -> dict:
        out = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank,
               "rot": {"base": self.rot_base, "dims": self.rot_dim}, "rot_dim": self.rot_dim,
               "scale": self.scale, "vdim": self.vdim}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class DenseFeedForwardConfig:
    ff: int

    def to_raw(self) -> dict:
        return {"ff": self.ff, "kind": "dense"}


@dataclass(frozen=True)
class RoutedFeedForwardConfig:
    experts: int
    top: int
    ff: int

    def to_raw(self) -> dict:
        return {"expert": {"ff": self.ff}, "kind": "moe", "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class TigitarLayerConfig:
    type: str                        # "delta" | "latent_attention"
    mixer: object                    # DeltaMixerConfig | LatentAttentionConfig
    mlp: object                      # DenseFeedForwardConfig | RoutedFeedForwardConfig | None

    def to_raw(self) -> dict:
        return {"mixer": self.mixer.to_raw(), "mlp": None if self.mlp is None else self.mlp.to_raw(),
                "type": self.type}


def _sub(raw: dict, key: str, where: str) -> dict:
    v = raw.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}.{key} must be an object, got {v!r}")
    return v


def _mixer(kind: str, raw: dict, i: int, n_layers: int):
    where = f"layers[{i}].mixer"
    r = KeyReader(raw)
    try:
        if kind == "delta":
            heads, kv_heads = r.integer("heads"), r.integer("kv_heads")
            if heads % kv_heads:
                raise ConfigError(f"heads {heads} is not a multiple of kv_heads {kv_heads}")
            return DeltaMixerConfig(heads, kv_heads, r.integer("dim"), r.integer("vdim"), r.integer("conv"))
        if kind == "latent_attention":
            rot_dim = r.integer("rot_dim")
            rot = KeyReader(_sub(raw, "rot", where))
            if rot.integer("dims") != rot_dim:
                raise ConfigError(f"rot.dims {rot.integer('dims')} differs from rot_dim {rot_dim}")
            if rot_dim % 2:
                raise ConfigError(f"rot_dim {rot_dim} must be even for rotary pairs")
            mask = r.mapping("mask")
            window = None if mask is None else KeyReader(mask).integer("size")
            kv_from = r.integer("kv_from", default=None, minimum=0)
            if kv_from is not None and not kv_from < n_layers:
                raise ConfigError(f"kv_from {kv_from} names no layer")
            return LatentAttentionConfig(r.integer("heads"), r.integer("dim"), rot_dim, r.integer("vdim"),
                                         r.integer("kv_rank"), r.number("scale"), rot.number("base"), window, kv_from)
    except ConfigError as e:
        raise ConfigError(f"{e} (in {where})") from None
    raise ConfigError(f"config.json: layers[{i}].type {kind!r} is not a mixer of this architecture "
                      f"('delta', 'latent_attention')")


def _mlp(raw, i: int):
    if raw is None:
        return None
    where = f"layers[{i}].mlp"
    if not isinstance(raw, dict):
        raise ConfigError(f"config.json: {where} must be an object or null, got {raw!r}")
    kind = raw.get("kind")
    try:
        if kind == "dense":
            return DenseFeedForwardConfig(KeyReader(raw).integer("ff"))
        if kind == "moe":
            router = KeyReader(_sub(raw, "router", where))
            experts, top = router.integer("experts"), router.integer("top")
            if top > experts:
                raise ConfigError(f"router.top {top} exceeds router.experts {experts}")
            return RoutedFeedForwardConfig(experts, top, KeyReader(_sub(raw, "expert", where)).integer("ff"))
    except ConfigError as e:
        raise ConfigError(f"{e} (in {where})") from None
    raise ConfigError(f"config.json: {where}.kind {kind!r} is not supported ('dense', 'moe')")


@dataclass(frozen=True)
class TigitarConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_softcap: float | None
    layers: tuple

    @classmethod
    def from_hf(cls, raw: dict) -> "TigitarConfig":
        r = KeyReader(raw)
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        layers = []
        for i, lr in enumerate(layers_raw):
            if not isinstance(lr, dict) or not isinstance(lr.get("type"), str):
                raise ConfigError(f"config.json: layers[{i}] must be an object with a 'type'")
            mixer = _mixer(lr["type"], _sub(lr, "mixer", f"layers[{i}]"), i, len(layers_raw))
            layers.append(TigitarLayerConfig(lr["type"], mixer, _mlp(lr.get("mlp"), i)))
        for i, layer in enumerate(layers):
            src = getattr(layer.mixer, "kv_from", None)
            if src is None:
                continue
            owner = layers[src].mixer
            if not src < i or not isinstance(owner, LatentAttentionConfig) or owner.kv_from is not None:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from {src} must name an earlier "
                                  f"latent_attention layer that has a cache of its own")
            if (owner.kv_rank, owner.rot_dim, owner.rot_base) != \
                    (layer.mixer.kv_rank, layer.mixer.rot_dim, layer.mixer.rot_base):
                raise ConfigError(f"config.json: layers[{i}] reads the latent cache of layer {src}; their "
                                  f"kv_rank, rot_dim and rot.base must be equal")
        norm = KeyReader(_sub(raw, "norm", "config"))
        return cls(vocab=r.integer("vocab"), width=r.integer("width"), norm_eps=norm.number("eps"),
                   logit_softcap=r.number("logit_softcap", default=None) if raw.get("logit_softcap") is not None
                   else None, layers=tuple(layers))

    def summary(self) -> str:
        """One line for a load message."""
        kinds = [layer.type for layer in self.layers]
        routed = sum(isinstance(layer.mlp, RoutedFeedForwardConfig) for layer in self.layers)
        return (f"Tigitar: {len(kinds)}L width={self.width} ({kinds.count('delta')} delta, "
                f"{kinds.count('latent_attention')} latent attention; {routed} with routed experts)")

    def to_hf(self) -> dict:
        """The config.json that reads back as this configuration."""
        out = {"architecture": "Tigitar", "layers": [layer.to_raw() for layer in self.layers],
               "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        return out
