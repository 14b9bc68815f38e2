"""Two mixers side by side on one input, and the attention one of them usually is.

`NormedAttention`: grouped-query softmax attention over the paged cache whose query and key heads are RMS-normed (one
gain of the head's size, shared by the heads) before they are rotated; it owns its rotary table (each layer may have
other frequencies, and a two-regime frequency scaling); a query may be restricted to the keys of its own block of
positions; the value size may differ from the key size.

`SideBySide`: both mixers read the same input; the layer's term is the mean of their outputs, each first RMS-normed over
the model width with a gain of its own.

`PooledWindowAttention`: grouped-query softmax attention that sees a window of recent tokens and, beside them, one mean
key and value per block of older tokens; a factor per head on the scores; a sink in the softmax's denominator.

`SideBySideSum`: both mixers read the same input; the layer's term is the plain sum of their terms (each mixer scales
its own).
"""

from __future__ import annotations

import torch

from .. import ops
from ..config.plan import PartSpec
from .base import MIXERS, POSITIONS, LayerCache, Mixer, PagedKV, StepContext, TensorSpec, flatten_needs, join_name
from .standard import Linear

_TABLES: dict = {}       # rotary tables by their parameters: layers with the same frequencies share one


def rotary_for(params: dict, dtype, device):
    sc = params.get("scaling")
    key = (float(params["theta"]), int(params["rotary_dim"]), int(params["max_positions"]),
           tuple(sorted((k, float(v)) for k, v in sc.items())) if sc else None, str(device))
    if key not in _TABLES:
        _TABLES[key] = POSITIONS.build(PartSpec("rotary", dict(params)), dtype=dtype, device=device)
    return _TABLES[key]


@MIXERS.register("normed_attention")
class NormedAttention(Mixer):
    """Parameters: ``hidden_size``, ``heads``, ``kv_heads``, ``dim`` (query/key size of a head), ``vdim`` (value size),
    ``scale`` (of the scores), ``eps`` (of the head norms), ``rotary`` (None, or ``theta``, ``rotary_dim``, optional
    ``scaling``: see `parts.standard.Rotary`), ``block`` (None, or the size of the blocks of positions, counted from 0,
    inside which a query sees the keys at or before it), ``max_positions``.

    The cache's head holds max(dim, vdim) channels (rounded up to a size the tensor-core kernels take, in bfloat16):
    keys and values are stored with zeros beyond their own size, which neither scores nor sums see; the output
    projection's matrix has zero columns there."""

    MAX_HEAD = 256

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        p = params
        self.hidden = int(p["hidden_size"])
        self.nq, self.nkv = int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.scale = float(p["scale"])
        self.eps = float(p["eps"])
        self.block = int(p["block"]) if p.get("block") else None
        self.max_positions = int(p["max_positions"])
        rot = p.get("rotary")
        self.rot_params = dict(rot, max_positions=self.max_positions) if rot else None
        self.rot = int(rot["rotary_dim"]) if rot else 0
        if self.nq % self.nkv:
            raise ValueError(f"normed_attention: {self.nq} query heads are no multiple of {self.nkv} key/value heads")
        if self.rot % 2 or self.rot > self.dim:
            raise ValueError(f"normed_attention: {self.rot} rotated channels must be even and at most dim={self.dim}")
        D = max(self.dim, self.vdim)
        if not 1 <= D <= self.MAX_HEAD:
            raise ValueError(f"normed_attention: a head of {D} channels is outside 1..{self.MAX_HEAD}, the largest the attention kernels take")
        if self.dtype == torch.bfloat16:
            D = next((s for s in (16, 32, 64, 128) if s >= D), D)
        self.D = D
        self.rotary = None

    def cache_need(self):
        return PagedKV(self.nkv, self.D, None)

    def tensor_specs(self):
        W = self.hidden
        return [TensorSpec("q", (self.nq * self.dim, W)), TensorSpec("k", (self.nkv * self.dim, W)),
                TensorSpec("v", (self.nkv * self.vdim, W)), TensorSpec("q.norm", (self.dim,), role="gain"),
                TensorSpec("k.norm", (self.dim,), role="gain"), TensorSpec("o", (W, self.nq * self.vdim))]

    def bind(self, fetch):
        self.qkv = Linear(self._matrix(torch.cat([fetch(n) for n in ("q", "k", "v")], dim=0)))
        self.q_gain, self.k_gain = self._f32(fetch("q.norm")), self._f32(fetch("k.norm"))
        o = fetch("o")
        if self.D != self.vdim:
            wide = torch.zeros((self.hidden, self.nq, self.D), dtype=o.dtype)
            wide[:, :, :self.vdim] = o.reshape(self.hidden, self.nq, self.vdim)
            o = wide.reshape(self.hidden, self.nq * self.D)
        self.out = Linear(self._matrix(o))
        if self.rot_params is not None:
            self.rotary = rotary_for(self.rot_params, self.dtype, self.device)

    accepts_residual = True

    def mix(self, x, step: StepContext, cache: LayerCache, position=None, write_cache=True):
        g = step.groups[cache.group]
        qkv = self.qkv(x, torch.float32)                                             # [T, (nq+nkv) dim + nkv vdim] float32
        q = ops.qk_norm_rope_kv_write(qkv, self.q_gain, self.k_gain, self.eps, step.positions,
                                      self.rotary.table if self.rotary is not None else None, self.rot, self.nq, self.nkv,
                                      self.dim, self.vdim, g.slot_mapping if write_cache else None, cache.k, cache.v, self.dtype)
        return ops.paged_attention(q, cache.k, cache.v, step, cache.group, self.nq, self.nkv, self.D, self.scale, None, self.block)

    def forward(self, x, step, cache, position, write_cache=True, residual=None):
        return self.out.into(self.mix(x, step, cache, position, write_cache), residual)

    def weight_bytes(self):
        return self.qkv.nbytes() + self.out.nbytes() + 8 * self.dim


@MIXERS.register("side_by_side")
class SideBySide(Mixer):
    """Parameters: ``hidden_size``, ``eps``, and ``left`` and ``right``, each ``{"kind": ..., "params": {...}}`` naming a
    registered mixer that offers ``mix(x, step, cache, position, write_cache)`` (its output before the projection) and
    ``out`` (that projection).  Tensors: the mixers' under ``left.`` and ``right.``, and the gains ``left.out`` and
    ``right.out`` of the model's width.  What the two ask of the cache manager is asked together (at most one of them
    pages; state names must differ)."""

    SIDES = ("left", "right")

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        self.hidden = int(params["hidden_size"])
        self.eps = float(params["eps"])
        self.sides = [MIXERS.build(PartSpec(params[s]["kind"], params[s]["params"]), **kw) for s in self.SIDES]
        for s, m in zip(self.SIDES, self.sides):
            if not hasattr(m, "mix"):
                raise ValueError(f"side_by_side: the {s} mixer ({params[s]['kind']}) does not offer its output before the projection")

    def cache_need(self):
        needs = []
        for m in self.sides:
            needs.extend(flatten_needs(m.cache_need()))
        return tuple(needs) if needs else None

    def tensor_specs(self):
        specs = []
        for s, m in zip(self.SIDES, self.sides):
            specs.extend(t.prefixed(s) for t in m.tensor_specs())
        specs += [TensorSpec(f"{s}.out", (self.hidden,), role="gain") for s in self.SIDES]
        return specs

    def bind(self, fetch):
        for s, m in zip(self.SIDES, self.sides):
            m.bind(lambda rel, _s=s: fetch(f"{_s}.{rel}"))
        self.gains = [self._f32(fetch(f"{s}.out")) for s in self.SIDES]

    accepts_residual = True

    def forward(self, x, step, cache, position, write_cache=True, residual=None):
        a, b = (m.out(m.mix(x, step, cache, position, write_cache), torch.float32) for m in self.sides)    # [T, W] float32 each
        if residual is None:
            residual = torch.zeros_like(a)
            ops.norm_mean_add_(residual, a, self.gains[0], b, self.gains[1], self.eps)
            return residual
        ops.norm_mean_add_(residual, a, self.gains[0], b, self.gains[1], self.eps)
        return None

    def weight_bytes(self):
        return sum(m.weight_bytes() for m in self.sides) + 8 * self.hidden


@MIXERS.register("pooled_window_attention")
class PooledWindowAttention(Mixer):
    """Grouped-query softmax attention over a window of recent tokens and pooled blocks of older ones.

    q = W_q x, k = W_k x, v = W_v x (no biases); q and k rotated over their first ``rotary_dim`` channels; the score of
    query head h is (q . k) ``scale`` temp_h, temp a stored number per head.  The query at position i sees the keys j with
    0 <= i - j < ``window`` and one key and value for every block of ``pool`` positions (counted from 0) that lies wholly
    before the window: the means of the block's keys, as the cache holds them, and of its values.  Tokens that have left
    the window and whose block is not complete before it are not seen.  One softmax over both kinds, whose denominator
    also holds exp(``sink``) (0: one is added).  ``window`` None: plain causal attention, no blocks.

    Parameters: ``hidden_size``, ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``window``, ``pool``, ``sink`` (None:
    no such term), ``rotary`` (None, or ``theta``, ``rotary_dim``, optional ``scaling``: see `parts.standard.Rotary`),
    ``out_scale`` (a factor on the mixer's term, 1 unless given; it rides on the attention's output), ``max_positions``.

    Two paged caches: the tokens' keys and values (``kv``; pages older than max(window, pool) positions go back to the pool,
    since a block's means are taken when its last token arrives) and the blocks' means (``pooled``; one entry per ``pool``
    tokens, kept for good).  The cache's head holds max(dim, vdim) channels, zeros beyond a key's or a value's own size."""

    MAX_HEAD = 256

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        p = params
        self.hidden = int(p["hidden_size"])
        self.nq, self.nkv = int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.scale = float(p["scale"])
        self.window = int(p["window"]) if p.get("window") else None
        self.pool = int(p["pool"]) if (self.window and p.get("pool")) else None
        self.sink_value = None if p.get("sink") is None else float(p["sink"])
        self.out_scale = float(p.get("out_scale", 1.0))
        self.max_positions = int(p["max_positions"])
        rot = p.get("rotary")
        self.rot_params = dict(rot, max_positions=self.max_positions) if rot else None
        self.rot = int(rot["rotary_dim"]) if rot else 0
        if self.nq % self.nkv:
            raise ValueError(f"pooled_window_attention: {self.nq} query heads are no multiple of {self.nkv} key/value heads")
        if self.rot % 2 or self.rot > self.dim:
            raise ValueError(f"pooled_window_attention: {self.rot} rotated channels must be even and at most dim={self.dim}")
        D = max(self.dim, self.vdim)
        if not 1 <= D <= self.MAX_HEAD:
            raise ValueError(f"pooled_window_attention: a head of {D} channels is outside 1..{self.MAX_HEAD}, the largest the attention kernels take")
        if self.dtype == torch.bfloat16:
            D = next((s for s in (16, 32, 64, 128) if s >= D), D)
        self.D = D
        self.rotary = None

    def cache_need(self):
        keep = max(self.window, self.pool or 0) if self.window else None
        needs = [PagedKV(self.nkv, self.D, keep)]
        if self.pool:
            needs.append(PagedKV(self.nkv, self.D, None, stride=self.pool, name="pooled"))
        return tuple(needs)

    def tensor_specs(self):
        W = self.hidden
        return [TensorSpec("q", (self.nq * self.dim, W)), TensorSpec("k", (self.nkv * self.dim, W)),
                TensorSpec("v", (self.nkv * self.vdim, W)), TensorSpec("temp", (self.nq,), role="gain"),
                TensorSpec("o", (W, self.nq * self.vdim))]

    def bind(self, fetch):
        self.qkv = Linear(self._matrix(torch.cat([fetch(n) for n in ("q", "k", "v")], dim=0)))
        self.temp = self._f32(fetch("temp"))
        self.sink = torch.full((self.nq,), self.sink_value, dtype=torch.float32, device=self.device) if self.sink_value is not None else None
        self.out = Linear(self._matrix(fetch("o")))
        if self.rot_params is not None:
            self.rotary = rotary_for(self.rot_params, self.dtype, self.device)

    accepts_residual = True

    def adopt_inp(self, linear):
        self.qkv = linear              # (a view of a joint matrix)

    @property
    def inp(self):
        """The input projection, for a container that runs several mixers' projections as one product."""
        return self.qkv

    def mix(self, x, step: StepContext, cache: LayerCache, position=None, write_cache=True, out=None, out_off=0, proj=None, proj_off=0):
        """``proj`` (float32, with ``proj_off``): the input projection's result where the caller has made it already, as
        columns of a wider product."""
        g = step.groups[cache.group]
        qkv = self.qkv(x, torch.float32) if proj is None else proj                   # [T, (nq+nkv) dim + nkv vdim] float32
        # rotation, the head's factor on its scores (carried by the query) and the cache write in one kernel
        q = ops.qk_norm_rope_kv_write(qkv, None, None, 0.0, step.positions, self.rotary.table if self.rotary is not None else None,
                                      self.rot, self.nq, self.nkv, self.dim, self.vdim, g.slot_mapping if write_cache else None,
                                      cache.k, cache.v, self.dtype, q_mul=self.temp, col_off=proj_off)
        pooled = cache.paged.get("pooled") if self.pool else None
        if pooled is not None and write_cache:
            ops.pool_kv_write(cache.k, cache.v, step, cache.group, pooled.k, pooled.v, pooled.group, self.pool)
        return ops.pooled_attention(q, cache.k, cache.v, pooled.k if pooled else None, pooled.v if pooled else None, step, cache.group,
                                    pooled.group if pooled else None, self.nq, self.nkv, self.vdim, self.scale, self.window,
                                    self.pool, self.sink, self.out_scale, out=out, out_off=out_off)

    def forward(self, x, step, cache, position, write_cache=True, residual=None):
        return self.out.into(self.mix(x, step, cache, position, write_cache), residual)

    def weight_bytes(self):
        return self.qkv.nbytes() + self.out.nbytes() + 4 * self.nq


@MIXERS.register("side_by_side_sum")
class SideBySideSum(Mixer):
    """Parameters: ``hidden_size`` and ``left`` and ``right``, each ``{"kind": ..., "params": {...}}`` naming a registered
    mixer that offers ``mix(x, step, cache, position, write_cache, out=, out_off=)`` (its output before the projection, in
    the compute dtype, written to columns ``out_off ..`` of ``out``), ``mix_width`` (how many columns that is) and ``out``
    (that projection).  The layer's term is left's plus right's; a factor on either is that mixer's own
    parameter.  The two projections are ONE product: [W_o,left | W_o,right] over the two outputs side by side.  Tensors:
    the mixers' under ``left.`` and ``right.``.  What the two ask of the cache manager is asked together.  Where both
    mixers offer their input projection (``inp``) and take its result from outside (``mix(..., proj=, proj_off=)``), those
    two are ONE product as well, kept in float32."""

    SIDES = ("left", "right")

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        self.hidden = int(params["hidden_size"])
        self.sides = [MIXERS.build(PartSpec(params[s]["kind"], params[s]["params"]), **kw) for s in self.SIDES]
        for s, m in zip(self.SIDES, self.sides):
            if not hasattr(m, "mix"):
                raise ValueError(f"side_by_side_sum: the {s} mixer ({params[s]['kind']}) does not offer its output before the projection")

    def cache_need(self):
        needs = []
        for m in self.sides:
            needs.extend(flatten_needs(m.cache_need()))
        return tuple(needs) if needs else None

    def tensor_specs(self):
        specs = []
        for s, m in zip(self.SIDES, self.sides):
            specs.extend(t.prefixed(s) for t in m.tensor_specs())
        return specs

    def bind(self, fetch):
        for s, m in zip(self.SIDES, self.sides):
            m.bind(lambda rel, _s=s: fetch(join_name(_s, rel)))
        self.widths = [m.out.weight.shape[1] for m in self.sides]
        self.out = Linear(torch.cat([m.out.weight for m in self.sides], dim=1).contiguous())
        for m, lo in zip(self.sides, (0, self.widths[0])):
            m.out = Linear(self.out.weight[:, lo:lo + m.out.weight.shape[1]])          # (a view: the joint matrix holds it)
        self.inp = None
        if all(getattr(m, "inp", None) is not None and m.inp.bias is None for m in self.sides):
            self.in_widths = [m.inp.weight.shape[0] for m in self.sides]
            self.inp = Linear(torch.cat([m.inp.weight for m in self.sides], dim=0).contiguous())
            for m, lo in zip(self.sides, (0, self.in_widths[0])):
                m.adopt_inp(Linear(self.inp.weight[lo:lo + m.inp.weight.shape[0]]))

    accepts_residual = True

    def forward(self, x, step, cache, position, write_cache=True, residual=None):
        both = torch.empty((x.shape[0], sum(self.widths)), dtype=self.dtype, device=x.device)
        if self.inp is not None:
            proj = self.inp(x, torch.float32)                        # both mixers' projections of the one input
            self.sides[0].mix(x, step, cache, position, write_cache, out=both, out_off=0, proj=proj, proj_off=0)
            self.sides[1].mix(x, step, cache, position, write_cache, out=both, out_off=self.widths[0], proj=proj, proj_off=self.in_widths[0])
        else:
            self.sides[0].mix(x, step, cache, position, write_cache, out=both, out_off=0)
            self.sides[1].mix(x, step, cache, position, write_cache, out=both, out_off=self.widths[0])
        return self.out.into(both, residual)

    def weight_bytes(self):
        return sum(m.weight_bytes() for m in self.sides)
