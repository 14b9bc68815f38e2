"""A layer that wraps each sublayer in two norms and puts a short convolution in front of it:

    x <- x + post1(mixer(conv1(pre1(x))));   x <- x + post2(ffn(conv2(pre2(x))))

with conv(h) = h + (a causal convolution over time of h, per channel).  The parts: an RMS norm whose gain is ONE number,
the convolution's taps with the last inputs as per-request state, and the block that arranges them.  Each takes its
sizes and constants as parameters; none names a model.

A sublayer's output is normed before it joins the stream, so no product can add into the stream itself; instead one
kernel per sublayer norms the output, adds it, and norms the stream for the next reader (`ops.post_add_norm`), also
across the border between two such layers: a layer's last term is handed to the next layer still pending (`Pending`),
and that layer's first kernel adds it.  Where every request of a step brings one token, the reader's convolution runs in
that kernel too (`ops.post_add_norm_conv`).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops
from .base import BLOCKS, NORMS, SHIFTS, Norm, OwedNorm, Part, SlotState, TensorSpec, flatten_needs


@NORMS.register("scalar_rmsnorm")
class ScalarRMSNorm(Norm):
    """y = x / sqrt(mean(x^2) + eps) * g with one number g for all channels (the tensor that carries the norm's own name,
    of no dimensions).  float32 on the float32 stream.  The kernels take a gain per channel; g is spread at bind time."""

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec("", (), role="gain")]

    def bind(self, fetch):
        g = fetch("").to(torch.float32).reshape(())
        self.weight = torch.full((self.size,), float(g), dtype=torch.float32).to(self.device)

    def add_norm(self, residual, delta):
        if isinstance(delta, Pending):        # (made for another reader: the term joins the stream here)
            return ops.post_add_norm(residual, delta.term, delta.post.weight, delta.post.eps, self.weight, self.eps, self.dtype)
        if delta is not None and not isinstance(delta, OwedNorm):
            ops.add_group_ssq(residual, [delta], 1, self.eps, want_rinv=False)
        return ops.post_add_norm(residual, None, None, 0.0, self.weight, self.eps, self.dtype)

    def weight_bytes(self):
        return 4


@SHIFTS.register("input_conv")
class InputConv(Part):
    """The taps of a causal convolution over time on each channel, ``[size, taps]`` with the current token's tap last (the
    tensor that carries the part's own name).  What reads through it gets h + conv(h); the last ``taps - 1`` inputs of a
    request are state the layer keeps."""

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        self.size = int(params["size"])
        self.taps = int(params["taps"])
        if self.taps < 1:
            raise ValueError(f"input_conv: taps={self.taps} must be at least 1")
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec("", (self.size, self.taps))]

    def bind(self, fetch):
        self.weight = self._f32(fetch(""))

    def state(self, name: str):
        return SlotState((self.size, self.taps - 1), name) if self.taps > 1 else None

    def __call__(self, h, state, step):
        return ops.short_conv_add(h, self.weight, state, step, self.dtype)

    def weight_bytes(self):
        return self.size * self.taps * 4


@dataclass
class Pending:
    """What a sandwich block hands to the next one: the stream still lacks ``post(term)``; the block whose first norm is
    ``norm`` adds it in the kernel that norms the stream for its mixer."""
    term: torch.Tensor
    post: Norm
    norm: Norm


@BLOCKS.register("sandwich")
class SandwichBlock:
    """Roles: ``mixer``, ``mixer_norm``, ``mixer_post`` and optionally ``mixer_conv``; for a feed-forward ``ffn``,
    ``ffn_norm``, ``ffn_post`` and optionally ``ffn_conv``.  The norms are `ScalarRMSNorm`s (anything with ``weight``
    float32 ``[size]`` and ``eps``); the convolutions `InputConv`s.  The mixer and the feed-forward return their term (or a
    stack of partial sums) in float32; nothing is added into the stream before its norm."""

    ROLES = ("mixer", "mixer_norm", "mixer_post", "mixer_conv", "ffn", "ffn_norm", "ffn_post", "ffn_conv")
    fuse_single_token = True      # norm and convolution in one kernel where every request brings one token (False: two, for comparison)

    def __init__(self, parts: dict):
        unknown = set(parts) - set(self.ROLES)
        if unknown or not {"mixer", "mixer_norm", "mixer_post"} <= set(parts):
            raise ValueError(f"the sandwich block arranges {self.ROLES}; the layer names {sorted(parts)}")
        if ("ffn" in parts) != ("ffn_norm" in parts) or ("ffn" in parts) != ("ffn_post" in parts) or \
                ("ffn_conv" in parts and "ffn" not in parts):
            raise ValueError("the sandwich block: a feed-forward comes with both its norms (and maybe its convolution), or not at all")
        g = parts.get
        self.mixer, self.mixer_norm, self.mixer_post, self.mixer_conv = g("mixer"), g("mixer_norm"), g("mixer_post"), g("mixer_conv")
        self.ffn, self.ffn_norm, self.ffn_post, self.ffn_conv = g("ffn"), g("ffn_norm"), g("ffn_post"), g("ffn_conv")
        for n in (self.mixer_norm, self.mixer_post, self.ffn_norm, self.ffn_post):
            if n is not None and not (hasattr(n, "eps") and hasattr(n, "weight")):
                raise ValueError("the sandwich block's norms are RMS norms with a gain per channel (scalar_rmsnorm spreads its one)")
        # the block before may leave its last term to this one's first kernel
        self.mixer_norm.takes_pending = True

    def cache_need(self):
        needs = flatten_needs(self.mixer.cache_need())
        for conv, name in ((self.mixer_conv, "conv_mixer"), (self.ffn_conv, "conv_ffn")):
            st = conv.state(name) if conv is not None else None
            if st is not None:
                needs.append(st)
        return tuple(needs) if needs else None

    accepts_next_norm = True

    @property
    def first_norm(self):
        return self.mixer_norm

    def _finish(self, residual, term, post, next_norm):
        """The sublayer's term, normed, joins the stream; where the next reader is such a block too, its first kernel does it."""
        if getattr(next_norm, "takes_pending", False):
            return Pending(term, post, next_norm)
        ops.post_add_norm(residual, term, post.weight, post.eps, None, 0.0)
        return None

    def _read(self, residual, term, post, norm, conv, cache, name, step):
        """stream += post(term) (if any), then what the sublayer behind ``norm`` reads: conv(norm(stream))."""
        pg, pe = (post.weight, post.eps) if term is not None else (None, 0.0)
        if conv is None:
            return ops.post_add_norm(residual, term, pg, pe, norm.weight, norm.eps, norm.dtype)
        state = cache.states.get(name) if cache is not None else None
        if self.fuse_single_token and residual.shape[0] == step.num_seqs and (state is not None or conv.taps == 1):
            # every request brings one token: one kernel, the normed row never leaves it
            return ops.post_add_norm_conv(residual, term, pg, pe, norm.weight, norm.eps, conv.weight, state, step, conv.dtype)
        return conv(ops.post_add_norm(residual, term, pg, pe, norm.weight, norm.eps, torch.float32), state, step)

    def forward(self, residual, delta, step, cache, position, write_cache=True, next_norm=None):
        norm = self.mixer_norm
        term = post = None
        if isinstance(delta, Pending):
            term, post = delta.term, delta.post
        elif delta is not None and not isinstance(delta, OwedNorm):
            ops.add_group_ssq(residual, [delta], 1, norm.eps, want_rinv=False)
        h = self._read(residual, term, post, norm, self.mixer_conv, cache, "conv_mixer", step)
        term = self.mixer.forward(h, step, cache, position, write_cache)
        if self.ffn is None:
            return self._finish(residual, term, self.mixer_post, next_norm)
        h = self._read(residual, term, self.mixer_post, self.ffn_norm, self.ffn_conv, cache, "conv_ffn", step)
        return self._finish(residual, self.ffn.forward(h, step), self.ffn_post, next_norm)
