"""Lasonex as a plan of parts: a decoder of parallel layers whose mixers are differential
attention and retention.

Layer i (tensors `l<i>.*`), mixer and feed-forward both reading the same x:
    x <- x + mixer(norm1(x)) + ff(norm2(x))                      (no second term without an `mlp`)
mixer "attention": differential attention (`mix.{q,k,v,o}`, `mix.{lq1,lk1,lq2,lk2}`): q and k hold two
maps per head, each a sliding-window softmax attention over the same values; the second, times a
number made from the four small vectors, is taken off the first, and each head's result is divided
by its root mean square.  Rotary pairs (i, i + dims/2) on the first `rot.dims` dimensions of every
map, frequencies blended towards longer periods where `rot.scaling` says so.
mixer "retention": linear attention with a fixed decay per head (`mix.{q,k,v,g,o}`): a float matrix
state per head and request, the read-out divided by its root mean square and gated by silu(W_g h).
Feed-forward "dense": `mlp.{gate,up,down}` as a clamped gated unit; "moe": `mlp.router`,
`mlp.e<j>.{gate,up,down}`, softmax scores, the choice limited to the best groups of neighbouring
experts, weights renormalised.  The embedding rows are scaled; then `final.norm` and `head`.
"""
from __future__ import annotations

from ..config.lasonex import (ClampedFeedForwardConfig, DifferentialAttentionConfig, GroupedExpertsConfig,
                              LasonexConfig, RetentionConfig)
from ..config.registry import register_architecture
from ..parts.plan import LayerRun, LayerSpec, ModelPlan, PartSpec

DEFAULT_MAX_POSITIONS = 32768        # config.json gives no limit; the engine's max_model_len overrides this
SWISH_SLOPE = 1.702                  # the design's gate: g * sigmoid(1.702 g)
RENORM_EPS = 1e-20                   # added to the sum of the chosen experts' scores


def make_plan(cfg: LasonexConfig, tensor_names=None) -> ModelPlan:
    width, eps = cfg.width, cfg.norm_eps

    def norm(name):
        return PartSpec("rmsnorm", dict(size=width, eps=eps), {"weight": name})

    def rotation(rot):
        if rot.dims == 0:
            return None
        return PartSpec("rotary", dict(rot_dim=rot.dims, theta=rot.base, scaling=rot.scaling, exact=True))

    layers, order = [], []
    for i, layer in enumerate(cfg.layers):
        base, m = f"l{i}.", layer.mixer
        mx = base + "mix."
        if isinstance(m, DifferentialAttentionConfig):
            mixer = PartSpec("differential_attention",
                             dict(hidden_size=width, heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim,
                                  scale=m.scale, diff=m.diff, window=m.window, norm_eps=eps,
                                  position=rotation(m.rot)),
                             {s: mx + s for s in ("q", "k", "v", "o", "lq1", "lk1", "lq2", "lk2")})
        elif isinstance(m, RetentionConfig):
            mixer = PartSpec("retention",
                             dict(hidden_size=width, heads=m.heads, dim=m.dim, vdim=m.vdim, decay=m.decay,
                                  norm_eps=eps, position=rotation(m.rot)),
                             {s: mx + s for s in ("q", "k", "v", "g", "o")})
        else:
            raise ValueError(f"layer {i}: unknown mixer configuration {m!r}")
        order.append(LayerRun(i))
        norms = {"mixer": norm(base + "norm1")}
        f = layer.mlp
        ff = None
        if f is not None:
            fm = base + "mlp."
            if isinstance(f, ClampedFeedForwardConfig):
                ff = PartSpec("glu", dict(hidden_size=width, intermediate_size=f.ff, activation="clamped_swish",
                                          activation_params=(f.limit, SWISH_SLOPE)),
                              {s: fm + s for s in ("gate", "up", "down")})
            elif isinstance(f, GroupedExpertsConfig):
                tensors = {"router": fm + "router"}
                for e in range(f.experts):
                    tensors.update({f"{s}.{e}": f"{fm}e{e}.{s}" for s in ("gate", "up", "down")})
                ff = PartSpec("routed_experts",
                              dict(hidden_size=width, experts=f.experts, top=f.top, expert_ff=f.ff,
                                   activation="clamped_swish", activation_params=(f.limit, SWISH_SLOPE),
                                   score="softmax", renormalise=True, renormalise_eps=RENORM_EPS, choice_bias=False,
                                   groups=f.groups, keep_groups=f.keep), tensors)
            else:
                raise ValueError(f"layer {i}: unknown feed-forward configuration {f!r}")
            norms["feed_forward"] = norm(base + "norm2")
        layers.append(LayerSpec("parallel", mixer, ff, norms))
    io = dict(vocab_size=cfg.vocab, hidden_size=width)
    return ModelPlan(
        hidden_size=width, vocab_size=cfg.vocab, max_positions=DEFAULT_MAX_POSITIONS,
        embedding=PartSpec("table", dict(io, scale=cfg.embedding_scale), {"weight": "embed"}),
        layers=layers, order=order, final_norm=norm("final.norm"),
        head=PartSpec("linear", io, {"weight": "head"}))


register_architecture("Lasonex", LasonexConfig, make_plan, model_types=("lasonex",))
