"""Differential attention mixer: two softmax maps per head over the same values, one taken off the other.

q = W_q h holds, per query head, two maps of `dim` side by side; k = W_k h likewise per key/value
head; v = W_v h is one value of `vdim` per key/value head (query head h reads key/value head
h // (heads / kv_heads)).  Rotary encoding turns the first `rot_dim` dimensions of every map of q
and k.  With a_m = softmax(q_m . k_m * scale) V over the visible keys (at or before the query,
within `window` if the layer has one):

    o = a_1 - lambda a_2,   lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff     (one number per layer)
    out = o / sqrt(mean(o^2) + norm_eps) * (1 - diff)                           (per head, no weight)

then W_o on the concatenated heads.  One stacked matrix serves q|k|v; the cache keeps per token
and key/value head the two rotated key maps followed by the value
(`cache.needs.PagedKeysValues`).  lambda is formed once at load, in double.  Scores, softmax, the
difference and the norm are float.

In bfloat16, with map and value sizes that are multiples of 16 up to 128, attention runs on the
tensor cores (`csrc/diff_attention_tc.cu`, one build per pair of sizes), and requests that bring a
single token take a kernel that shares each token's keys out over blocks at fixed positions and
reads a cache row once for its group of query heads (how many blocks: decided per step on the
host, `plan_step`); everything else, and the 32-bit path, takes the CUDA-core kernel.
"""
from __future__ import annotations

import math

import torch

from ..cache.needs import PagedKeysValues
from ..native import ops, scratch
from .base import Part
from .linear import Linear
from .registry import build_part, register_part


@register_part("mixer", "differential_attention")
class DifferentialAttention(Part):
    """params: hidden_size, heads, kv_heads, dim (per map), vdim, scale, diff, window (None | int), norm_eps,
    position (PartSpec | None).  tensors: q [heads * 2 dim, hidden], k [kv_heads * 2 dim, hidden],
    v [kv_heads * vdim, hidden], o [hidden, heads * vdim], lq1, lk1, lq2, lk2 [dim]."""
    category = "mixer"
    native_libraries = ("diff_attention",)
    SCRATCH = "differential attention splits"

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.kv_heads = int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.scale, self.diff = float(p["scale"]), float(p["diff"])
        self.window = p.get("window")
        self.norm_eps = float(p["norm_eps"])
        if self.heads % self.kv_heads:
            raise ValueError(f"differential_attention: {self.heads} heads are not a multiple of "
                             f"{self.kv_heads} kv heads")
        if self.vdim > 256 or self.dim > 4096:
            raise ValueError(f"differential_attention: vdim {self.vdim} / dim {self.dim} are beyond the kernels' "
                             f"limits of 256 / 4096")
        self.position = build_part("position", p["position"], ctx) if p.get("position") else None
        if self.position is not None and self.position.rot_dim > self.dim:
            raise ValueError("differential_attention: the position encoding turns more dimensions than a map has")
        self.q_cols = self.heads * 2 * self.dim
        self.cols = self.q_cols + self.kv_heads * (2 * self.dim + self.vdim)
        self.qkv = self.o = None
        self.lam = None

    def children(self):
        return [self.position] if self.position is not None else []

    def cache_need(self):
        return PagedKeysValues(self.kv_heads, 2 * self.dim, self.vdim, self.window)

    def weight_shapes(self):
        w = self.hidden
        shapes = {"q": (self.q_cols, w), "k": (self.kv_heads * 2 * self.dim, w), "v": (self.kv_heads * self.vdim, w),
                  "o": (w, self.heads * self.vdim)}
        shapes.update({s: (self.dim,) for s in ("lq1", "lk1", "lq2", "lk2")})
        return shapes

    def load(self, tensors):
        mats = [tensors["q"], tensors["k"], tensors["v"]]
        if len({m.dtype for m in mats}) != 1:
            raise ValueError("differential_attention: q, k and v matrices must be stored in one dtype")
        self.qkv = Linear(mats)
        self.o = Linear([tensors["o"]])
        lq1, lk1, lq2, lk2 = (tensors[s].double().cpu() for s in ("lq1", "lk1", "lq2", "lk2"))
        self.lam = math.exp(float((lq1 * lk1).sum())) - math.exp(float((lq2 * lk2).sum())) + self.diff

    def _tc(self) -> bool:
        return ops.diff_tc_takes(self.ctx.dtype, self.dim, self.vdim)

    def _splits_keys(self) -> bool:
        """Single tokens go to the split-key kernel (beside the tensor-core one, never in the 32-bit path, whose
        sums keep one order whatever the cut)."""
        if not hasattr(self, "_split_ok"):
            self._split_ok = self._tc() and ops.diff_decode_takes(self.heads, self.kv_heads, self.dim, self.vdim)
        return self._split_ok

    # ---- what the host decides per step: how many blocks share a single token's keys
    @property
    def plan_key(self):
        return ("differential_attention", self.window)

    def _splits(self, longest: int) -> int:
        span = longest if self.window is None else min(self.window, longest)
        return (span - 1) // ops.DIFF_SPLIT + 2

    def plan_step(self, step):
        longest = step.max_seq_len
        if step.for_graph:                                    # a captured step serves many: cover the length rounded up
            longest = -(-longest // 1024) * 1024
        step.plans[self.plan_key] = self._splits(longest) if step.n_decode_tokens else 0

    def graph_key(self, step):
        return step.plans.get(self.plan_key)

    def _partials(self, n_tokens: int, n_splits: int):
        return scratch.get(self.ctx.device, self.SCRATCH, n_tokens * self.heads * 2 * n_splits * (self.vdim + 2))

    def reserve(self, limits):
        for lin in (self.qkv, self.o):
            if lin is not None:
                lin.reserve(self.ctx.dtype, limits.max_tokens)
        if self.ctx.device.type == "cuda" and self._tc():
            from ..native.build import load_library
            load_library(*ops.diff_tc_library(self.dim, self.vdim))        # built now, not inside the first step
            if self._splits_keys():                                        # sized now: nothing grows under a graph
                longest = -(-limits.max_model_len // 1024) * 1024
                self._partials(min(limits.max_tokens, limits.max_requests), self._splits(longest))

    def forward(self, h, out, step, cache):
        n = h.shape[0]
        dt = self.ctx.dtype
        ws = step.workspace
        qkv = ws.rows("diff_qkv", n, self.cols, dt)
        self.qkv.forward(h, qkv)
        if self.position is not None:
            cos, sin = self.position.tables()
            rot = self.position.rot_dim
        else:
            cos, sin, rot = step.no_rotation, step.no_rotation, 0
        ops.diff_prep(qkv, self.heads, self.kv_heads, self.dim, self.vdim, rot, cos, sin, step.positions,
                      cache.slots, cache.tensor, cache.page_size)
        ctx = ws.rows("diff_ctx", n, self.heads * self.vdim, dt)
        if self._tc():
            split = self._splits_keys() and step.n_decode_tokens > 0
            if not split or step.n_decode_tokens < step.n_requests:
                ops.diff_attention_tc(qkv, ctx, cache.tensor, cache.block_table, step, self.heads, self.kv_heads,
                                      self.dim, self.vdim, self.window, self.scale, self.lam, self.norm_eps,
                                      1.0 - self.diff, cache.page_size, include_single=not split)
            if split:
                if self.plan_key not in step.plans:               # a step built by hand, not by the engine
                    self.plan_step(step)
                n_splits = step.plans[self.plan_key]
                ops.diff_decode(qkv, ctx, cache.tensor, cache.block_table, step.tok_req, step.positions,
                                step.decode_tokens, self._partials(step.n_decode_tokens, n_splits), n_splits,
                                self.heads, self.kv_heads, self.dim, self.vdim, self.window, self.scale, self.lam,
                                self.norm_eps, 1.0 - self.diff, cache.page_size)
            return self.o.forward(ctx, out, defer=True)
        ops.diff_attention_simt(qkv, ctx, cache.tensor, cache.block_table, step.tok_req, step.positions, self.heads,
                                self.kv_heads, self.dim, self.vdim, self.window, self.scale, self.lam, self.norm_eps,
                                1.0 - self.diff, cache.page_size)
        return self.o.forward(ctx, out, defer=True)
