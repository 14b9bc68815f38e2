"""Gated linear attention: a recurrent mixer whose float32 matrix state per head decays per key channel.

    S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,        o_t = S_t^T q_t

with q = W_q x * dim^(-1/2), k = W_k x (heads x dim), v = W_v x (heads x vdim) and a decay per key channel from a
low-rank pair of products: alpha = sigmoid(W_a2 (W_a1 x) + b)^(1/tau).  Each head's o over its root mean square times a
gain shared by the heads, times silu(W_g x), then W_o.  The state starts at zero and lives in the request's state slot,
so a prompt's portions and single decoded tokens continue one another.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import MIXERS, LayerCache, Mixer, SlotState, StepContext, TensorSpec
from .standard import Linear


@MIXERS.register("gated_linear_attention")
class GatedLinearAttention(Mixer):
    """Parameters: ``hidden_size``, ``heads``, ``dim``, ``vdim``, ``tau``, ``eps`` (of the output's norm); the decay's
    rank is read from the checkpoint (``decay_rank`` for random weights).  q, k, v and the gate are one matrix, its
    product stays float32, as everything that enters the recurrence does."""

    NAMES = ("q", "k", "v", "g")

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.dim = int(params["dim"])
        self.vdim = int(params["vdim"])
        self.tau = float(params["tau"])
        self.eps = float(params["eps"])
        self.rank = params.get("decay_rank")
        if not ops.delta_rule_supports(self.dim, self.vdim):
            raise ValueError(f"gated_linear_attention: a head of {self.dim} key channels is outside what the recurrence kernel "
                             f"keeps in registers (1..256)")
        if not self.tau > 0:
            raise ValueError(f"gated_linear_attention: tau={self.tau} must be positive")

    def cache_need(self):
        return SlotState((self.heads, self.dim, self.vdim), "gla")

    def tensor_specs(self):
        H, W, R = self.heads, self.hidden, self.rank
        K, V = H * self.dim, H * self.vdim
        default = max(4, min(64, W // 16))
        return [TensorSpec("q", (K, W)), TensorSpec("k", (K, W)), TensorSpec("v", (V, W)), TensorSpec("g", (V, W)),
                TensorSpec("o", (W, V)), TensorSpec("norm", (self.vdim,), role="gain"),
                TensorSpec("a1", (R, W), shape_default=(R or default, W)), TensorSpec("a2", (K, R), shape_default=(K, R or default)),
                TensorSpec("a2.b", (K,), role="bias")]

    def bind(self, fetch):
        H = self.heads
        K, V = H * self.dim, H * self.vdim
        self.rank = int(fetch("a1").shape[0])
        if tuple(fetch("a2").shape) != (K, self.rank):
            raise ValueError(f"gated_linear_attention: a2 {tuple(fetch('a2').shape)} does not fit a1's {self.rank} rows")
        self.inp = Linear(self._matrix(torch.cat([fetch(n) for n in self.NAMES], dim=0)))
        self.offs = (0, K, 2 * K)
        self.off_g = 2 * K + V
        self.a1 = Linear(self._matrix(fetch("a1")))
        self.a2 = Linear(self._matrix(fetch("a2")), self._f32(fetch("a2.b")))
        self.gain = self._f32(fetch("norm").float().repeat(H))
        self.out = Linear(self._matrix(fetch("o")))

    accepts_residual = True

    def mix(self, x, step: StepContext, cache: LayerCache, position=None, write_cache=True):
        proj = self.inp(x, torch.float32)                                            # [T, 2K + 2V] float32
        z = self.a2(self.a1(x, self.dtype), torch.float32)                           # [T, K] decay logits, float32
        o = ops.gated_linear_attention(proj, self.offs, z, cache.states["gla"], step, self.heads, self.dim, self.vdim,
                                       self.dim ** -0.5, self.tau)                   # [T, V] float32
        return ops.delta_out(o, self.gain, proj, self.off_g, self.eps, self.heads, self.vdim, self.dtype, "silu")

    def forward(self, x, step, cache, position, write_cache=True, residual=None):
        return self.out.into(self.mix(x, step, cache, position, write_cache), residual)

    def weight_bytes(self):
        return self.inp.nbytes() + self.a1.nbytes() + self.a2.nbytes() + self.out.nbytes() + 4 * self.gain.numel()


@MIXERS.register("decay_linear_attention")
class DecayLinearAttention(Mixer):
    """Linear attention with ONE fixed decay per head:

        S_t = decay_h S_(t-1) + k_t v_t^T,        o_t = S_t^T q_t,        q, k, v = silu of their projections

    (no other scale).  The heads' outputs together, over their common root mean square, times a gain of ``heads * vdim``
    numbers, times sigmoid(W_g x), then W_o.  Parameters: ``hidden_size``, ``heads``, ``dim``, ``vdim``, ``decay`` (one number
    per head), ``eps`` (of the output's norm).  q, k, v and the gate are one matrix whose product stays float32."""

    NAMES = ("q", "k", "v", "g")

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.dim = int(params["dim"])
        self.vdim = int(params["vdim"])
        self.eps = float(params["eps"])
        decay = [float(d) for d in params["decay"]]
        if len(decay) != self.heads:
            raise ValueError(f"decay_linear_attention: {len(decay)} decays for {self.heads} heads")
        if not ops.delta_rule_supports(self.dim, self.vdim):
            raise ValueError(f"decay_linear_attention: a head of {self.dim} key channels is outside what the recurrence kernel "
                             f"keeps in registers (1..256)")
        self.decay = torch.tensor(decay, dtype=torch.float32).to(self.device)

    def cache_need(self):
        return SlotState((self.heads, self.dim, self.vdim), "lightning")

    def tensor_specs(self):
        H, W = self.heads, self.hidden
        K, V = H * self.dim, H * self.vdim
        return [TensorSpec("q", (K, W)), TensorSpec("k", (K, W)), TensorSpec("v", (V, W)), TensorSpec("g", (V, W)),
                TensorSpec("o", (W, V)), TensorSpec("norm", (V,), role="gain")]

    def bind(self, fetch):
        K, V = self.heads * self.dim, self.heads * self.vdim
        self.inp = Linear(self._matrix(torch.cat([fetch(n) for n in self.NAMES], dim=0)))
        self.offs = (0, K, 2 * K)
        self.off_g = 2 * K + V
        self.gain = self._f32(fetch("norm"))
        self.out = Linear(self._matrix(fetch("o")))

    accepts_residual = True

    def mix(self, x, step: StepContext, cache: LayerCache, position=None, write_cache=True):
        proj = self.inp(x, torch.float32)                                            # [T, 2K + 2V] float32
        o = ops.decay_linear_attention(proj, self.offs, self.decay, cache.states["lightning"], step, self.heads, self.dim, self.vdim)
        # one norm over all heads: the output kernel's "head" is the whole row
        return ops.delta_out(o, self.gain, proj, self.off_g, self.eps, 1, self.heads * self.vdim, self.dtype, "sigmoid")

    def forward(self, x, step, cache, position, write_cache=True, residual=None):
        return self.out.into(self.mix(x, step, cache, position, write_cache), residual)

    def weight_bytes(self):
        return self.inp.nbytes() + self.out.nbytes() + 4 * self.gain.numel() + 4 * self.heads


@MIXERS.register("forget_gate_attention")
class ForgetGateAttention(Mixer):
    """Linear attention whose forget gate also decides what is written (HGRN2):

        S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T,        o_t = S_t^T q_t

    with q = silu(W_q x) (heads x dim), v = W_v x (heads x vdim) and, per head and key channel,
    f = lower + (1 - lower) sigmoid(W_f x + b): there is no key and no other scale.  Each head's o over its root mean
    square times a gain of ``vdim`` numbers shared by the heads, then W_o.  Parameters: ``hidden_size``, ``heads``, ``dim``,
    ``vdim``, ``eps`` (of the output's norm), ``out_scale`` (a factor on the mixer's term, 1 unless given; it rides on the
    gain).  q, the gate's logits and v are one matrix whose product stays float32, as everything that enters the
    recurrence does."""

    NAMES = ("q", "f", "v")

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.dim = int(params["dim"])
        self.vdim = int(params["vdim"])
        self.eps = float(params["eps"])
        self.out_scale = float(params.get("out_scale", 1.0))
        if not ops.delta_rule_supports(self.dim, self.vdim):
            raise ValueError(f"forget_gate_attention: a head of {self.dim} key channels is outside what the recurrence kernel "
                             f"keeps in registers (1..256)")

    def cache_need(self):
        return SlotState((self.heads, self.dim, self.vdim), "forget_gate")

    def tensor_specs(self):
        H, W = self.heads, self.hidden
        K, V = H * self.dim, H * self.vdim
        return [TensorSpec("q", (K, W)), TensorSpec("f", (K, W)), TensorSpec("f.b", (K,), role="bias"),
                TensorSpec("lower", (K,), role="mix"), TensorSpec("v", (V, W)), TensorSpec("norm", (self.vdim,), role="gain"),
                TensorSpec("o", (W, V))]

    def bind(self, fetch):
        K = self.heads * self.dim
        self.inp = Linear(self._matrix(torch.cat([fetch(n) for n in self.NAMES], dim=0)))
        self.offs = (0, K, 2 * K)
        self.f_bias, self.lower = self._f32(fetch("f.b")), self._f32(fetch("lower"))
        self.gain = self._f32(fetch("norm").float().repeat(self.heads) * self.out_scale)
        self.out = Linear(self._matrix(fetch("o")))

    accepts_residual = True

    def adopt_inp(self, linear):
        self.inp = linear              # (a view of a joint matrix)

    def mix(self, x, step: StepContext, cache: LayerCache, position=None, write_cache=True, out=None, out_off=0, proj=None, proj_off=0):
        """``proj`` (float32, with ``proj_off``): the input projection's result where the caller has made it already, as
        columns of a wider product."""
        if proj is None:
            proj = self.inp(x, torch.float32)                                        # [T, 2K + V] float32
        offs = tuple(o + proj_off for o in self.offs)
        o = ops.forget_gate_attention(proj, offs, self.f_bias, self.lower, cache.states["forget_gate"], step, self.heads,
                                      self.dim, self.vdim)                           # [T, V] float32
        return ops.delta_out(o, self.gain, None, 0, self.eps, self.heads, self.vdim, self.dtype, "none", out=out, out_off=out_off)

    def forward(self, x, step, cache, position, write_cache=True, residual=None):
        return self.out.into(self.mix(x, step, cache, position, write_cache), residual)

    def weight_bytes(self):
        return self.inp.nbytes() + self.out.nbytes() + 4 * (self.gain.numel() + 2 * self.f_bias.numel())
