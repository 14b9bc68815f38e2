"""Parts of a "parallel" layer: an RMS norm taken in groups, a sinusoidal position vector added to the
input, a gated feed-forward with biases and a choice of activation, and the block that lets the mixer
and the feed-forward read ONE norm's output and adds both terms to the stream, with an optional token
shift in front of the mixer.  Each takes its sizes and constants as parameters; none names a model.

All arithmetic runs in the kernels behind `sllm_b200.ops`.
"""

from __future__ import annotations

import numpy as np
import torch

from .. import ops
from .base import (BLOCKS, FEED_FORWARDS, NORMS, POSITIONS, SHIFTS, FeedForward, Norm, OwedNorm, Part,
                   PositionEncoding, SlotState, TensorSpec, flatten_needs)
from .standard import Linear


@NORMS.register("group_rmsnorm")
class GroupRMSNorm(Norm):
    """The vector in ``groups`` equal consecutive parts, each divided by its own sqrt(mean(part^2) + eps); the
    whole times a plain gain.  float32 on the float32 stream.  ``groups`` = 1 is the ordinary RMS norm.  The gain
    is the tensor that carries the norm's own name.  ``offset``: the stored tensor is the gain minus this (a gain kept
    around zero has ``offset`` 1); ``gain_scale``: a constant the output is multiplied by as well (a model whose output
    head scales its logits puts the factor here, into its last norm)."""

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        self.size = int(params["size"])
        self.groups = int(params.get("groups", 1))
        self.eps = float(params["eps"])
        self.offset = float(params.get("offset", 0.0))
        self.gain_scale = float(params.get("gain_scale", 1.0))
        if self.groups < 1 or self.size % self.groups:
            raise ValueError(f"group_rmsnorm: {self.groups} groups do not divide {self.size}")
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec("", (self.size,), role="gain" if self.offset == 0.0 else "gain_offset")]

    def bind(self, fetch):
        w = self._f32(fetch(""))
        if self.offset != 0.0:
            w = w + self.offset
        if self.gain_scale != 1.0:
            w = w * self.gain_scale
        self.weight = w.contiguous()

    def complete(self, residual, delta) -> None:
        """Add what a block before has left pending into the stream (nothing to do when its products added their
        terms themselves)."""
        terms = pending_terms(delta)
        if terms:
            ops.add_group_ssq(residual, terms, self.groups, self.eps, want_rinv=False)

    def add_norm(self, residual, delta, out_dtype=None):
        """``out_dtype``: the normed copy's dtype where it is not the compute dtype (a norm whose output enters the float32
        stream itself)."""
        self.complete(residual, delta)
        return ops.group_norm_shift(residual, None, self.weight, out_dtype or self.dtype, groups=self.groups, eps=self.eps)

    def weight_bytes(self):
        return self.size * 4


def pending_terms(delta) -> list:
    """The terms a block before has left to be added: nothing, one tensor (possibly a stack of partial sums), a
    sequence of such, or a norm still owed (whose stream is complete: nothing to add)."""
    if delta is None or isinstance(delta, OwedNorm):
        return []
    if isinstance(delta, (tuple, list)):
        return [d for d in delta if d is not None]
    return [delta]


@POSITIONS.register("sinusoidal")
class Sinusoidal(PositionEncoding):
    """A position vector added to the input: channels come in pairs (sin, cos) of the angle p * f_i, with f_i =
    base^(-2i/width) for pair i of position p.  The frequencies are computed once in float64 and kept in float32; the angle
    is a float32 product.  No table over positions, so no limit on them."""

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        self.width = int(params["width"])
        self.base = float(params.get("base", 10000.0))
        if self.width % 2:
            raise ValueError(f"sinusoidal positions need an even width, got {self.width}")
        f = self.base ** (-2.0 * np.arange(self.width // 2, dtype=np.float64) / self.width)
        self.inv_freq = torch.from_numpy(f.astype(np.float32)).to(self.device)

    def on_embedding(self, residual, step):
        ops.add_sinusoid_(residual, step.positions, self.inv_freq)


@FEED_FORWARDS.register("gated_dense")
class GatedDense(FeedForward):
    """down(act(gate(x)) * up(x)) with a bias on each of the three products (optional as a set) and ``act`` one of
    ``gelu_tanh`` (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))) and ``silu``; or, with ``activation`` =
    ``clamped_swish``, down(g sigmoid(alpha g) (u + 1)) with g = min(gate(x), limit) and u = clamp(up(x), -limit, limit)
    (``limit``; ``alpha``, 1.702 unless given).  gate and up are one matrix whose rows
    (and biases) alternate in blocks of 8, so that a tile of the product holds a gate row and its up row together and the
    activation can be applied where the tile is made (all gate rows first where the size is no multiple of 8)."""

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.act = str(params.get("activation", "gelu_tanh"))
        self.bias = bool(params.get("bias", True))
        self.names = params.get("names", ("gate", "up", "down"))
        self.bias_suffix = params.get("bias_suffix", "b")
        self.interleave = 8 if self.inter % 8 == 0 else self.inter
        if self.act not in ops.ACTIVATIONS and self.act != "clamped_swish":
            raise ValueError(f"gated_dense: activation {self.act!r}; known: {sorted(ops.ACTIVATIONS) + ['clamped_swish']}")
        if self.act == "clamped_swish":
            self.limit, self.alpha = float(params["limit"]), float(params.get("alpha", 1.702))
        self.gate_up = None
        self.down = None

    def tensor_specs(self):
        g, u, d = self.names
        specs = [TensorSpec(g, (self.inter, self.hidden)), TensorSpec(u, (self.inter, self.hidden)),
                 TensorSpec(d, (self.hidden, self.inter))]
        if self.bias:
            b = self.bias_suffix
            specs += [TensorSpec(f"{g}.{b}", (self.inter,), role="bias"), TensorSpec(f"{u}.{b}", (self.inter,), role="bias"),
                      TensorSpec(f"{d}.{b}", (self.hidden,), role="bias")]
        return specs

    def bind(self, fetch):
        g, u, d = self.names
        b = self.bias_suffix
        n = self.interleave

        def alternate(a, c):           # blocks of n rows of a, then of c, in turn
            return torch.stack([a.reshape(self.inter // n, n, *a.shape[1:]), c.reshape(self.inter // n, n, *c.shape[1:])],
                               dim=1).reshape(2 * self.inter, *a.shape[1:])
        gu_b = self._f32(alternate(fetch(f"{g}.{b}").float(), fetch(f"{u}.{b}").float())) if self.bias else None
        self.gate_up = Linear(self._matrix(alternate(fetch(g), fetch(u))), gu_b)
        self.down = Linear(self._matrix(fetch(d)), self._f32(fetch(f"{d}.{b}")) if self.bias else None)

    accepts_residual = True

    def forward(self, x, step, residual=None):
        if self.act == "clamped_swish":
            gu = ops.linear(x, self.gate_up.weight, self.gate_up.bias, self.dtype)                               # [T, 2I]
            act = ops.gated_clamp_act(gu, self.interleave, self.limit, self.dtype, alpha=self.alpha)
        else:
            act = ops.linear_act_mul(x, self.gate_up.weight, self.gate_up.bias, self.interleave, self.dtype, self.act)   # [T, I]
        return self.down.into(act, residual)

    def weight_bytes(self):
        return self.gate_up.nbytes() + self.down.nbytes()


@BLOCKS.register("parallel_shift")
class ParallelShiftBlock:
    """x <- x + (mixer(shift(h)) + ffn(h)) with h = norm(x): one norm, both sublayers read its output.

    The token shift (present when the layer has a ``shift`` tensor role): the mixer reads h + (h' - h) * mix, element
    by element, with h' the previous token's h as the norm gave it (zeros before a sequence's first token).  The
    previous h is per-request state of the layer (a `SlotState` named ``shift`` beside whatever the mixer keeps),
    held in float32.  The feed-forward is optional.

    A term that a product could not add into the stream itself is handed on for the next norm's kernel to add:
    both of them when that norm is a `GroupRMSNorm` (whose kernel takes two), else one, the other being added
    here."""

    ROLES = ("norm", "mixer", "ffn", "shift")

    def __init__(self, parts: dict):
        unknown = set(parts) - set(self.ROLES)
        if unknown or "norm" not in parts or "mixer" not in parts:
            raise ValueError(f"the parallel block arranges norm, mixer and optionally ffn and shift; the layer names {sorted(parts)}")
        self.norm, self.mixer = parts["norm"], parts["mixer"]
        self.ffn, self.shift = parts.get("ffn"), parts.get("shift")
        if not isinstance(self.norm, GroupRMSNorm):
            raise ValueError("the parallel block's norm is a group_rmsnorm (groups=1 for the ordinary one)")

    def cache_need(self):
        needs = flatten_needs(self.mixer.cache_need())
        if self.shift is not None:
            needs.append(SlotState((self.norm.size,), "shift"))
        return tuple(needs) if needs else None

    accepts_next_norm = True

    @property
    def first_norm(self):
        return self.norm

    def forward(self, residual, delta, step, cache, position, write_cache=True, next_norm=None):
        norm = self.norm
        norm.complete(residual, delta)
        kw = dict(groups=norm.groups, eps=norm.eps)
        if self.shift is not None:
            h, hs = ops.group_norm_shift(residual, None, norm.weight, norm.dtype, mix=self.shift.mix,
                                         state=cache.states["shift"], step=step, want_plain=self.ffn is not None, **kw)
        else:
            h = hs = ops.group_norm_shift(residual, None, norm.weight, norm.dtype, **kw)
        kw = {"residual": residual} if getattr(self.mixer, "accepts_residual", False) else {}
        terms = [self.mixer.forward(hs, step, cache, position, write_cache, **kw)]
        if self.ffn is not None:
            kw = {"residual": residual} if getattr(self.ffn, "accepts_residual", False) else {}
            terms.append(self.ffn.forward(h, step, **kw))
        terms = [t for t in terms if t is not None]
        if not terms:
            return None
        if len(terms) == 2 and not isinstance(next_norm, GroupRMSNorm):
            ops.add_group_ssq(residual, terms[:1], 1, 0.0, want_rinv=False)
            terms = terms[1:]
        return terms[0] if len(terms) == 1 else tuple(terms)


@BLOCKS.register("parallel_pair")
class ParallelPairBlock:
    """x <- x + (mixer(norm_a(x)) + ffn(norm_b(x))): two norms of the same x, one for each sublayer, both taken before
    either term is added.  The norms are plain RMS norms (`group_rmsnorm` with one group) of one eps: one kernel takes the
    row's root mean square once and writes both.  The feed-forward (with its norm) is optional.  Whatever factor the
    design puts on the sum is the parts' business (they scale their own terms).  Roles: ``mixer_norm``, ``mixer``,
    ``ffn_norm``, ``ffn``."""

    ROLES = ("mixer_norm", "mixer", "ffn_norm", "ffn")

    def __init__(self, parts: dict):
        if set(parts) != set(self.ROLES) and set(parts) != {"mixer_norm", "mixer"}:
            raise ValueError(f"the two-norm parallel block arranges {self.ROLES} (or mixer_norm and mixer alone); the layer names {sorted(parts)}")
        self.mixer, self.ffn = parts["mixer"], parts.get("ffn")
        self.mixer_norm, self.ffn_norm = parts["mixer_norm"], parts.get("ffn_norm")
        for n in (self.mixer_norm, self.ffn_norm):
            if n is not None and not (isinstance(n, GroupRMSNorm) and n.groups == 1):
                raise ValueError("the two-norm parallel block's norms are group_rmsnorm with one group")
        if self.ffn_norm is not None and self.ffn_norm.eps != self.mixer_norm.eps:
            raise ValueError("the two-norm parallel block's norms share one eps")

    def cache_need(self):
        return self.mixer.cache_need()

    accepts_next_norm = True

    @property
    def first_norm(self):
        return self.mixer_norm

    def forward(self, residual, delta, step, cache, position, write_cache=True, next_norm=None):
        na, nb = self.mixer_norm, self.ffn_norm
        na.complete(residual, delta)
        ha, hb = ops.norm_pair(residual, na.weight, nb.weight if nb is not None else None, na.eps, na.dtype)
        kw = {"residual": residual} if getattr(self.mixer, "accepts_residual", False) else {}
        terms = [self.mixer.forward(ha, step, cache, position, write_cache, **kw)]
        if self.ffn is not None:
            kw = {"residual": residual} if getattr(self.ffn, "accepts_residual", False) else {}
            terms.append(self.ffn.forward(hb, step, **kw))
        terms = [t for t in terms if t is not None]
        if len(terms) == 2 and not isinstance(next_norm, GroupRMSNorm):
            ops.add_group_ssq(residual, terms[:1], 1, 0.0, want_rinv=False)
            terms = terms[1:]
        if not terms:
            return None
        return terms[0] if len(terms) == 1 else tuple(terms)


@SHIFTS.register("token_shift")
class TokenShiftMix(Part):
    """The per-channel blend of a token shift, h + (h_prev - h) * mix: one float32 vector, the tensor that carries
    the part's own name, applied inside the norm's kernel."""

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        self.size = int(params["size"])
        self.mix = None

    def tensor_specs(self):
        return [TensorSpec("", (self.size,), role="mix")]

    def bind(self, fetch):
        self.mix = self._f32(fetch(""))

    def weight_bytes(self):
        return self.size * 4
