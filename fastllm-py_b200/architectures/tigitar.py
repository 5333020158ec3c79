"""Tigitar as a plan of parts: a hybrid decoder of gated-delta-rule layers and
latent-attention layers, each normed on both sides of its sublayers.

Layer i (tensors `l<i>.*`):
    x <- x + norm1b(mixer(norm1(x)));   x <- x + norm2b(ff(norm2(x)))    (no second half without an `mlp`)
mixer "delta": the gated delta rule (`mix.{q,k,v}` with `.conv` taps, `mix.{b,a,A_log,dt_bias,norm,g,o}`);
mixer "latent_attention": `mix.{q,dkv,dkv.norm,uk,uv,o}`, a sliding window, rotary pairs (i, i + dims/2)
on the rotated parts; a layer with `kv_from` has no `mix.dkv` and reads the cache that layer's run wrote.
Feed-forward "dense": `mlp.{gate,up,down}` with relu as the gate's activation; "moe": `mlp.router`,
`mlp.correction`, `mlp.e<j>.{gate,up,down}` with silu, sigmoid scores, the correction added for the choice
only, weights not renormalised.  Then `final.norm`, `head`, and the logits' soft cap.

The latent cache of a layer keeps the widest window among the layers that read it.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.tigitar import (DeltaMixerConfig, DenseFeedForwardConfig, LatentAttentionConfig,
                              RoutedFeedForwardConfig, TigitarConfig)
from ..parts.plan import LayerRun, LayerSpec, ModelPlan, PartSpec

DEFAULT_MAX_POSITIONS = 32768        # config.json gives no limit; the engine's max_model_len overrides this


def make_plan(cfg: TigitarConfig, tensor_names=None) -> ModelPlan:
    width, eps = cfg.width, cfg.norm_eps

    def norm(name, size=width):
        return PartSpec("rmsnorm", dict(size=size, eps=eps), {"weight": name})

    # what each latent cache must keep: the widest window of its readers (None: everything)
    keep = {}
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if isinstance(m, LatentAttentionConfig):
            owner = i if m.kv_from is None else m.kv_from
            if owner not in keep:
                keep[owner] = m.window
            elif keep[owner] is not None:
                keep[owner] = None if m.window is None else max(keep[owner], m.window)

    layers, order, run_of = [], [], {}
    for i, layer in enumerate(cfg.layers):
        base, m = f"l{i}.", layer.mixer
        mx = base + "mix."
        if isinstance(m, DeltaMixerConfig):
            tensors = {s: mx + s for s in ("q", "k", "v", "b", "a", "A_log", "dt_bias", "norm", "g", "o")}
            tensors.update({f"{s}_conv": f"{mx}{s}.conv" for s in ("q", "k", "v")})
            mixer = PartSpec("gated_delta", dict(hidden_size=width, heads=m.heads, kv_heads=m.kv_heads, dim=m.dim,
                                                 vdim=m.vdim, taps=m.conv, norm_eps=eps, unit_eps=1e-6), tensors)
            run = LayerRun(i)
        elif isinstance(m, LatentAttentionConfig):
            shares = m.kv_from is not None
            tensors = {s: mx + s for s in ("q", "uk", "uv", "o")}
            if not shares:
                tensors.update({"dkv": mx + "dkv", "dkv_norm": mx + "dkv.norm"})
            position = PartSpec("rotary", dict(rot_dim=m.rot_dim, theta=m.rot_base, scaling=None, exact=True))
            mixer = PartSpec("latent_attention",
                             dict(hidden_size=width, heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim,
                                  kv_rank=m.kv_rank, scale=m.scale, window=m.window,
                                  keep=keep[m.kv_from if shares else i], norm_eps=eps, position=position,
                                  shares_cache=shares), tensors)
            run = LayerRun(i, cache=run_of[m.kv_from] if shares else None)
        else:
            raise ValueError(f"layer {i}: unknown mixer configuration {m!r}")
        run_of[i] = len(order)
        order.append(run)
        norms = {"mixer_in": norm(base + "norm1"), "mixer_out": norm(base + "norm1b")}
        f = layer.mlp
        ff = None
        if f is not None:
            fm = base + "mlp."
            if isinstance(f, DenseFeedForwardConfig):
                ff = PartSpec("glu", dict(hidden_size=width, intermediate_size=f.ff, activation="relu"),
                              {s: fm + s for s in ("gate", "up", "down")})
            elif isinstance(f, RoutedFeedForwardConfig):
                tensors = {"router": fm + "router", "correction": fm + "correction"}
                for e in range(f.experts):
                    tensors.update({f"{s}.{e}": f"{fm}e{e}.{s}" for s in ("gate", "up", "down")})
                ff = PartSpec("routed_experts", dict(hidden_size=width, experts=f.experts, top=f.top, expert_ff=f.ff,
                                                     activation="silu", score="sigmoid", renormalise=False,
                                                     choice_bias=True), tensors)
            else:
                raise ValueError(f"layer {i}: unknown feed-forward configuration {f!r}")
            norms.update({"ff_in": norm(base + "norm2"), "ff_out": norm(base + "norm2b")})
        layers.append(LayerSpec("sandwich", mixer, ff, norms))
    io = dict(vocab_size=cfg.vocab, hidden_size=width)
    return ModelPlan(
        hidden_size=width, vocab_size=cfg.vocab, max_positions=DEFAULT_MAX_POSITIONS,
        embedding=PartSpec("table", io, {"weight": "embed"}),
        layers=layers, order=order, final_norm=norm("final.norm"),
        head=PartSpec("linear", dict(io, softcap=cfg.logit_softcap), {"weight": "head"}))


register_architecture("Tigitar", TigitarConfig, make_plan, model_types=("tigitar",))
