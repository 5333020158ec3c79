"""Retention mixer: linear attention with a fixed decay per head, no softmax and no denominator.

For a head with state S [dim x vdim] (float, one per request, zero at the start):

    S <- decay S + k v^T;   o = S^T q

q, k (`heads` x `dim`) and v (`heads` x `vdim`) are projections of the input; rotary encoding
turns the first `rot_dim` dimensions of q and k, and k is multiplied by `k_scale` (dim^-1/2 unless
given) after the rotation.  Each head's o is divided by its root mean square over vdim (no weight),
the heads are concatenated, multiplied by silu(W_g h) and projected by W_o.

One stacked matrix serves q | k | v | gate.  The request's state row holds S for every head; it is
float and carried from step to step by the cache manager's state slots.  Everything after the
projection is float.
"""
from __future__ import annotations

import torch

from ..cache.needs import FixedState
from ..native import ops
from .base import Part
from .linear import Linear
from .registry import build_part, register_part


@register_part("mixer", "retention")
class Retention(Part):
    """params: hidden_size, heads, dim, vdim, decay (one number per head), norm_eps, k_scale (None: dim^-1/2),
    position (PartSpec | None).  tensors: q, k [heads * dim, hidden], v, g [heads * vdim, hidden],
    o [hidden, heads * vdim]."""
    category = "mixer"
    native_libraries = ("retention",)

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.dim, self.vdim = int(p["heads"]), int(p["dim"]), int(p["vdim"])
        self.norm_eps = float(p["norm_eps"])
        self.k_scale = float(p["k_scale"]) if p.get("k_scale") is not None else self.dim ** -0.5
        decay = [float(d) for d in p["decay"]]
        if len(decay) != self.heads:
            raise ValueError(f"retention: {len(decay)} decays for {self.heads} heads")
        if self.dim > 256:
            raise ValueError(f"retention: dim {self.dim} is beyond the scan kernel's limit of 256")
        self.decay = torch.tensor(decay, dtype=torch.float64).to(torch.float32).to(ctx.device)
        self.position = build_part("position", p["position"], ctx) if p.get("position") else None
        if self.position is not None and self.position.rot_dim > self.dim:
            raise ValueError("retention: the position encoding turns more dimensions than a head has")
        self.qk_cols = 2 * self.heads * self.dim
        self.hv = self.heads * self.vdim
        self.proj_cols = self.qk_cols + 2 * self.hv                     # q | k | v | gate
        self.proj = self.o = None

    def children(self):
        return [self.position] if self.position is not None else []

    def cache_need(self):
        return FixedState((self.heads * self.vdim * self.dim,), "float32")

    def weight_shapes(self):
        w = self.hidden
        return {"q": (self.heads * self.dim, w), "k": (self.heads * self.dim, w), "v": (self.hv, w), "g": (self.hv, w),
                "o": (w, self.hv)}

    def load(self, tensors):
        mats = [tensors[s] for s in ("q", "k", "v", "g")]
        if len({m.dtype for m in mats}) != 1:
            raise ValueError("retention: the projections must be stored in one dtype")
        self.proj = Linear(mats)
        self.o = Linear([tensors["o"]])

    def reserve(self, limits):
        for lin in (self.proj, self.o):
            if lin is not None:
                lin.reserve(self.ctx.dtype, limits.max_tokens)

    def forward(self, h, out, step, cache):
        n = h.shape[0]
        dt = self.ctx.dtype
        ws = step.workspace
        proj = ws.rows("retention_proj", n, self.proj_cols, dt)
        self.proj.forward(h, proj)
        if self.position is not None:
            cos, sin = self.position.tables()
            rot = self.position.rot_dim
        else:
            cos, sin, rot = step.no_rotation, step.no_rotation, 0
        work = ws.rows("retention_qkv", n, self.qk_cols + self.hv, torch.float32)
        ops.retention_prep(proj, work, self.heads, self.dim, self.vdim, rot, cos, sin, step.positions, self.k_scale)
        o = ws.rows("retention_o", n, self.hv, torch.float32)
        ops.retention_scan(work, o, cache.tensor, self.decay, step, self.heads, self.dim, self.vdim,
                           fixed_order=dt == torch.float32)     # the 32-bit path: cuts and batches agree bit for bit
        y = ws.rows("retention_y", n, self.hv, dt)
        ops.retention_gated_norm(o, proj, self.qk_cols + self.hv, y, self.heads, self.vdim, self.norm_eps)
        return self.o.forward(y, out, defer=True)
