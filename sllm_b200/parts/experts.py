"""A mixture of experts as a feed-forward: a sigmoid router that narrows its choice to the best groups of experts, small
two-matrix experts, and optionally one expert every token uses.

    z = W_router x (float32);  s = sigmoid(z);  choice = s + correction
    the experts form ``groups`` equal groups of neighbours; a group's score is the sum of its two largest choice scores;
    only experts of the ``keep`` best groups can be chosen; the ``top`` largest choice scores among them win;
    out = sum over the winners of (s_e * scale) * W_down,e gelu(W_up,e x)   (weights not renormalized)   + shared(x)

All experts' up projections are ONE matrix (expert e's rows at e * ff, the shared expert's after them) and their down
projections one matrix side by side: a token's activation row carries its routing weights (zero for an expert not
chosen), so the second product adds up the weighted experts by itself, in float32, in one order whatever else the batch
holds.  Every expert's product is computed for every token: with E experts of which ``top`` are used that is E/top times
the arithmetic of a sorted, grouped product, and none of its bookkeeping; a decode step reads every expert's matrix
either way once the batch holds a few tokens.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import FEED_FORWARDS, FeedForward, TensorSpec
from .standard import Linear


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    """Parameters: ``hidden_size``, ``experts``, ``top``, ``groups`` and ``keep`` (1 and 1: no narrowing), ``scale``,
    ``expert_ff``, ``shared_ff`` (0: no shared expert).  The activation is the exact (erf) gelu; no biases."""

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        p = params
        self.hidden = int(p["hidden_size"])
        self.E, self.top = int(p["experts"]), int(p["top"])
        self.groups, self.keep = int(p.get("groups", 1)), int(p.get("keep", 1))
        self.scale = float(p["scale"])
        self.ff, self.shared_ff = int(p["expert_ff"]), int(p.get("shared_ff") or 0)
        if self.E % self.groups or not 1 <= self.keep <= self.groups:
            raise ValueError(f"routed_experts: {self.groups} groups (keep {self.keep}) do not fit {self.E} experts")
        if not 1 <= self.top <= self.keep * (self.E // self.groups):
            raise ValueError(f"routed_experts: top={self.top} experts cannot come from {self.keep} groups of {self.E // self.groups}")

    def tensor_specs(self):
        W = self.hidden
        specs = []
        for e in range(self.E):
            specs += [TensorSpec(f"e{e}.up", (self.ff, W)), TensorSpec(f"e{e}.down", (W, self.ff))]
        specs += [TensorSpec("router", (self.E, W)), TensorSpec("correction", (self.E,), role="bias")]
        if self.shared_ff:
            specs += [TensorSpec("shared.up", (self.shared_ff, W)), TensorSpec("shared.down", (W, self.shared_ff))]
        return specs

    def bind(self, fetch):
        names = [f"e{e}" for e in range(self.E)] + (["shared"] if self.shared_ff else [])
        self.up = Linear(self._matrix(torch.cat([fetch(f"{n}.up") for n in names], dim=0)))          # [E ff + shared, W]
        self.down = Linear(self._matrix(torch.cat([fetch(f"{n}.down") for n in names], dim=1)))      # [W, E ff + shared]
        self.router = Linear(self._matrix(fetch("router")))
        self.correction = self._f32(fetch("correction"))

    accepts_residual = True

    def route(self, x):
        """(dense weights [T, E], indices [T, top], weights [T, top]) of the normed rows ``x``."""
        return ops.moe_route(self.router(x, torch.float32), self.correction, self.groups, self.keep, self.top, self.scale)

    def forward(self, x, step, residual=None):
        dense, _, _ = self.route(x)
        act = ops.moe_act(self.up(x, self.dtype), dense, self.ff, self.dtype)        # [T, E ff + shared]
        return self.down.into(act, residual)

    def weight_bytes(self):
        return self.up.nbytes() + self.down.nbytes() + self.router.nbytes() + 4 * self.E


@FEED_FORWARDS.register("gated_experts")
class GatedExperts(FeedForward):
    """A mixture of gated experts behind a router that takes the largest logits:

        z = W_router x (float32);  the ``top`` largest z win;  their weights are the softmax over the winners alone
        expert e:  g = min(W_gate,e x, limit),  u = clamp(W_up,e x, -limit, limit),  W_down,e (g sigmoid(alpha g) (u + 1))
        out = sum over the winners of weight_e * expert_e(x)

    With ``activation`` = ``silu`` an expert is W_down,e (silu(W_gate,e x) * W_up,e x) instead (no limit); ``scale`` (1 unless
    given) multiplies the weights.  The softmax over the winners alone is also what a softmax over ALL experts gives once
    the winners' scores are divided by their sum.

    Parameters: ``hidden_size``, ``experts``, ``top``, ``expert_ff``, ``limit``, ``alpha`` (1.702 unless given), ``activation``
    (``clamped_swish`` unless given), ``scale``; no biases.  As
    in `RoutedExperts`, all experts' gate and up projections are ONE matrix (expert e's rows at 2 e ff, gate and up rows
    alternating in blocks of 8, or all of the expert's gate rows before its up rows where ff is no multiple of 8) and their
    down projections one matrix side by side; a token's activation row carries its routing weights, so the second product
    adds up the weighted experts in float32 in one order whatever the batch holds."""

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        p = params
        self.hidden = int(p["hidden_size"])
        self.E, self.top = int(p["experts"]), int(p["top"])
        self.ff = int(p["expert_ff"])
        self.act = str(p.get("activation", "clamped_swish"))
        if self.act not in ("clamped_swish", "silu"):
            raise ValueError(f"gated_experts: activation {self.act!r}; known: clamped_swish, silu")
        self.limit, self.alpha = float(p.get("limit", 0.0) if self.act == "silu" else p["limit"]), float(p.get("alpha", 1.702))
        self.scale = float(p.get("scale", 1.0))
        self.interleave = 8 if self.ff % 8 == 0 else self.ff
        if not 1 <= self.top <= self.E:
            raise ValueError(f"gated_experts: top={self.top} of {self.E} experts cannot be chosen")

    def tensor_specs(self):
        W = self.hidden
        specs = []
        for e in range(self.E):
            specs += [TensorSpec(f"e{e}.gate", (self.ff, W)), TensorSpec(f"e{e}.up", (self.ff, W)), TensorSpec(f"e{e}.down", (W, self.ff))]
        specs.append(TensorSpec("router", (self.E, W)))
        return specs

    def bind(self, fetch):
        n, W = self.interleave, self.hidden
        rows = []
        for e in range(self.E):
            g, u = fetch(f"e{e}.gate").reshape(self.ff // n, n, W), fetch(f"e{e}.up").reshape(self.ff // n, n, W)
            rows.append(torch.stack([g, u], dim=1).reshape(2 * self.ff, W))
        self.gate_up = Linear(self._matrix(torch.cat(rows, dim=0)))                                          # [2 E ff, W]
        self.down = Linear(self._matrix(torch.cat([fetch(f"e{e}.down") for e in range(self.E)], dim=1)))     # [W, E ff]
        self.router = Linear(self._matrix(fetch("router")))

    accepts_residual = True

    def route(self, x):
        """(dense weights [T, E], indices [T, top], weights [T, top]) of the normed rows ``x``."""
        return ops.moe_route_top_softmax(self.router(x, torch.float32), self.top, self.scale)

    def forward(self, x, step, residual=None):
        dense, _, _ = self.route(x)
        gu = self.gate_up(x, self.dtype)                                                                     # [T, 2 E ff]
        act = ops.gated_clamp_act(gu, self.interleave, self.limit, self.dtype, alpha=self.alpha, dense=dense, ff=self.ff, act=self.act)
        return self.down.into(act, residual)

    def weight_bytes(self):
        return self.gate_up.nbytes() + self.down.nbytes() + self.router.nbytes()
