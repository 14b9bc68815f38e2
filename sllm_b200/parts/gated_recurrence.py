"""An element-wise gated recurrence whose gates read only the current token (a minimal GRU):

    z = sigmoid(W_z x + b_z);   u = W_x x + b_x;   c = u + 1/2 where u >= 0, sigmoid(u) elsewhere
    S_t = (1 - z) S_(t-1) + z c   (element by element);   out = W_o (S_t * silu(W_g x))

The state is one float32 vector per request, zero at a sequence's start, carried in the request's state slot, so a prompt's
portions and single decoded tokens continue one another.  Because nothing but S itself feeds back, a portion's tokens are
walked in parallel runs (`ops.mingru_scan`).
"""

from __future__ import annotations

import torch

from .. import ops
from .base import MIXERS, LayerCache, Mixer, SlotState, StepContext, TensorSpec
from .standard import Linear


@MIXERS.register("mingru")
class MinGRU(Mixer):
    """Parameters: ``hidden_size``, ``width`` (of the recurrence).  z, x and the gate are one matrix whose product stays
    float32 with the two biases in its epilogue: everything that enters the recurrence is float32."""

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        self.hidden = int(params["hidden_size"])
        self.width = int(params["width"])

    def cache_need(self):
        return SlotState((self.width,), "mingru")

    def tensor_specs(self):
        W, C = self.hidden, self.width
        return [TensorSpec("z", (C, W)), TensorSpec("z.b", (C,), role="bias"), TensorSpec("x", (C, W)),
                TensorSpec("x.b", (C,), role="bias"), TensorSpec("g", (C, W)), TensorSpec("o", (W, C))]

    def bind(self, fetch):
        C = self.width
        zb = fetch("z.b").float()
        bias = torch.cat([zb, fetch("x.b").float().to(zb.device), torch.zeros(C, device=zb.device)])
        self.inp = Linear(self._matrix(torch.cat([fetch(n) for n in ("z", "x", "g")], dim=0)), self._f32(bias))
        self.out = Linear(self._matrix(fetch("o")))

    def forward(self, x, step: StepContext, cache: LayerCache, position, write_cache=True, residual=None):
        C = self.width
        proj = self.inp(x, torch.float32)                                              # [T, 3C] float32
        y = ops.mingru_scan(proj, (0, C, 2 * C), cache.states["mingru"], step, C, self.dtype)
        return self.out.into(y, residual)

    accepts_residual = True

    def weight_bytes(self):
        return self.inp.nbytes() + self.out.nbytes()
