"""Gated delta rule mixer: linear attention whose memory is one matrix per head.

For a head with state S [dim x vdim] (float, one per request, zero at the start):

    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

The token's read-out sees its own write.  q and k (`kv_heads` x `dim`; value head
h uses q/k head h // (heads / kv_heads)) and v (`heads` x `vdim`) are projections
of the input that pass a causal convolution over the last `taps` tokens per
channel and silu; q and k are then scaled to unit length per head
(x / sqrt(sum x^2 + unit_eps)) and q times `q_scale` (dim^-1/2 unless given).
beta = sigmoid(W_b h) and g = exp(-exp(A_log) * softplus(W_a h + dt_bias)) are
per head.  Each head's o is divided by its root mean square over vdim, times a
weight shared by the heads, times silu(W_g h); W_o maps back to the model width.

One stacked matrix serves q | k | v | gate | b | a.  The request's state row
holds S for every head and, behind it, the last taps - 1 raw inputs of the
convolution; both are float and carried from step to step by the cache
manager's state slots.  Everything after the projection is float.
"""
from __future__ import annotations

import torch

from ..cache.needs import FixedState
from ..native import ops
from .base import Part
from .linear import Linear
from .registry import register_part


@register_part("mixer", "gated_delta")
class GatedDelta(Part):
    """params: hidden_size, heads, kv_heads, dim, vdim, taps, norm_eps, unit_eps (1e-6), q_scale (None: dim^-1/2).
    tensors: q, k, v, q_conv, k_conv, v_conv [channels, taps], b, a [heads, hidden], A_log, dt_bias [heads],
    norm [vdim], g, o."""
    category = "mixer"
    native_libraries = ("delta_rule",)

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.kv_heads = int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim, self.taps = int(p["dim"]), int(p["vdim"]), int(p["taps"])
        self.norm_eps = float(p["norm_eps"])
        self.unit_eps = float(p.get("unit_eps", 1e-6))
        self.q_scale = float(p["q_scale"]) if p.get("q_scale") is not None else self.dim ** -0.5
        if self.heads % self.kv_heads:
            raise ValueError(f"gated_delta: {self.heads} heads are not a multiple of {self.kv_heads} kv heads")
        if self.dim > 256:
            raise ValueError(f"gated_delta: dim {self.dim} is beyond the scan kernel's limit of 256")
        self.qk_cols = self.kv_heads * self.dim
        self.hv = self.heads * self.vdim
        self.channels = 2 * self.qk_cols + self.hv                     # what passes the convolution: q | k | v
        self.proj_cols = self.channels + self.hv + 2 * self.heads      # ... | gate | b | a
        self.work_cols = 2 * self.qk_cols + self.hv + 2 * self.heads + self.hv   # q | k | v | beta | decay | o
        self.state_floats = self.heads * self.vdim * self.dim
        self.proj = self.o = None

    def cache_need(self):
        return FixedState((self.state_floats + (self.taps - 1) * self.channels,), "float32")

    def weight_shapes(self):
        qk, hv, w = self.qk_cols, self.hv, self.hidden
        return {"q": (qk, w), "k": (qk, w), "v": (hv, w), "q_conv": (qk, self.taps), "k_conv": (qk, self.taps),
                "v_conv": (hv, self.taps), "b": (self.heads, w), "a": (self.heads, w), "A_log": (self.heads,),
                "dt_bias": (self.heads,), "norm": (self.vdim,), "g": (hv, w), "o": (w, hv)}

    def load(self, tensors):
        mats = [tensors[s] for s in ("q", "k", "v", "g", "b", "a")]
        small = [tensors[s] for s in ("q_conv", "k_conv", "v_conv", "A_log", "dt_bias")]
        if len({m.dtype for m in mats}) != 1 or len({m.dtype for m in small}) != 1:
            raise ValueError("gated_delta: the projections, and the small tensors, must each be stored in one dtype")
        self.proj = Linear(mats)
        self.conv = torch.cat([tensors["q_conv"], tensors["k_conv"], tensors["v_conv"]], dim=0).contiguous()
        self.a_log = tensors["A_log"].contiguous()
        self.dt_bias = tensors["dt_bias"].contiguous()
        self.norm = tensors["norm"].contiguous()
        self.o = Linear([tensors["o"]])

    def reserve(self, limits):
        for lin in (self.proj, self.o):
            if lin is not None:
                lin.reserve(self.ctx.dtype, limits.max_tokens)

    def forward(self, h, out, step, cache):
        n = h.shape[0]
        dt = self.ctx.dtype
        ws = step.workspace
        proj = ws.rows("delta_proj", n, self.proj_cols, dt)
        self.proj.forward(h, proj)
        work = ws.rows("delta_work", n, self.work_cols, torch.float32)
        ops.delta_prep(proj, self.conv, self.a_log, self.dt_bias, cache.tensor, self.state_floats, step, work,
                       self.heads, self.kv_heads, self.dim, self.vdim, self.taps, self.unit_eps, self.q_scale)
        ops.delta_scan(work, cache.tensor, step, self.heads, self.kv_heads, self.dim, self.vdim)
        y = ws.rows("delta_y", n, self.hv, dt)
        ops.delta_gated_norm(work, self.work_cols - self.hv, proj, self.channels, self.norm, y, self.heads,
                             self.vdim, self.norm_eps)
        return self.o.forward(y, out, defer=True)
