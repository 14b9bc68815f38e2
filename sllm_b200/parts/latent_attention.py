"""Latent attention: keys and values of every head are up-projections of one small vector per token, and only that
vector is cached.

    q = W_q x  [heads, dim];   c = rmsnorm(W_dkv x) * gain  [rank]  (the latent, cached);
    k_h = W_uk,h c,  v_h = W_uv,h c;   score = (q_h . k_h) * scale;   causal softmax;
    head h's output times sigmoid(W_g x)_h;   W_o on the concatenated heads.

No positions enter (unless a rotated key part is asked for, see the class).  The score of a query against a key is computed in the latent space: q_h . (W_uk,h c) =
(W_uk,h^T q_h) . c, so each head's query is carried through its key up-projection once per token, the attention
kernels read the cached latents as ONE shared key-and-value head of size ``rank`` (the cache holds each latent
once: `PagedKV(values=False)`), and each head's weighted sum of latents goes through its value up-projection
afterwards.  Nothing per head is ever stored per cached token.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import MIXERS, LayerCache, Mixer, PagedKV, StepContext, TensorSpec
from .standard import Linear


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """Parameters: ``hidden_size``, ``heads``, ``dim`` (query/key size of a head), ``vdim`` (value size), ``kv_rank``,
    ``scale``, ``eps`` (of the latent's norm), ``gate`` (a sigmoid gate on the output: true or ``"head"`` one number per head,
    ``"element"`` one per output channel, false none; default true).  q, the down-projection and the gate are one matrix;
    its product stays float32 (the latent's norm is float32).

    Optional: ``rot_dim`` > 0 gives every query head ``rot_dim`` more channels, laid out behind its ``dim`` unrotated ones,
    and the down-projection ``rot_dim`` more rows behind the latent's: ONE rotated key part per token that all heads share,
    not normed.  Both are rotated by position (``rotary``: ``theta``, ``rotary_dim`` <= rot_dim, ``max_positions``); the
    score is the sum of both dot products.  The cache then holds [latent | rotated key part] per token as one key-and-value
    head (its value is read from the latent's columns only), a query is [its carried form | its rotated part].
    ``sink`` true: a learned number per head (``sink``) whose exponential joins the softmax's denominator.
    ``shared_kv`` true: the layer has no down-projection of its own and reads the cache another run wrote."""

    MAX_RANK = 640      # the CUDA-core attention kernel's largest head (its second instance; the tensor-core forms end at 128)

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.dim = int(params["dim"])
        self.vdim = int(params["vdim"])
        self.rank = int(params["kv_rank"])
        self.scale = float(params["scale"])
        self.eps = float(params["eps"])
        gate = params.get("gate", True)
        self.gate = {True: "head", False: None, None: None}.get(gate, gate)
        if self.gate not in (None, "head", "element"):
            raise ValueError(f"latent_attention: gate={gate!r}; one of true, false, 'head', 'element'")
        self.rot_dim = int(params.get("rot_dim") or 0)
        self.has_sink = bool(params.get("sink", False))
        self.shared_kv = bool(params.get("shared_kv", False))
        rot = params.get("rotary") if self.rot_dim else None
        self.rot_params = dict(rot) if rot else None
        self.rot = int(rot["rotary_dim"]) if rot else 0
        if self.rot % 2 or self.rot > self.rot_dim:
            raise ValueError(f"latent_attention: {self.rot} rotated channels must be even and at most rot_dim={self.rot_dim}")
        D = self.rank + self.rot_dim
        if not 1 <= D <= self.MAX_RANK:
            raise ValueError(f"latent_attention: kv_rank={self.rank} (+ rot_dim={self.rot_dim}) is outside 1..{self.MAX_RANK}, the "
                             f"largest head the attention kernels take")
        if self.rot_dim and self.dtype == torch.bfloat16:
            D = next((s for s in (16, 32, 64, 128) if s >= D), D)       # a size the tensor-core forms take; zeros beyond
        self.D = D
        self.rotary = None
        self.sink = None

    def cache_need(self):
        return PagedKV(1, self.D, None, values=False)

    def tensor_specs(self):
        H, W, r = self.heads, self.hidden, self.rank
        specs = [TensorSpec("q", (H * (self.dim + self.rot_dim), W))]
        if not self.shared_kv:
            specs += [TensorSpec("dkv", (r + self.rot_dim, W)), TensorSpec("dkv.norm", (r,), role="gain")]
        specs += [TensorSpec("uk", (H * self.dim, r)), TensorSpec("uv", (H * self.vdim, r))]
        if self.has_sink:
            specs.append(TensorSpec("sink", (H,), role="bias"))
        if self.gate:
            specs.append(TensorSpec("g", (H if self.gate == "head" else H * self.vdim, W)))
        specs.append(TensorSpec("o", (W, H * self.vdim)))
        return specs

    def bind(self, fetch):
        H, r = self.heads, self.rank
        names = ["q"] + ([] if self.shared_kv else ["dkv"]) + (["g"] if self.gate else [])
        self.inp = Linear(self._matrix(torch.cat([fetch(n) for n in names], dim=0)))
        self.qdim = self.dim + self.rot_dim
        self.off_c = H * self.qdim
        self.off_g = self.off_c + (0 if self.shared_kv else r + self.rot_dim)
        self.c_gain = None if self.shared_kv else self._f32(fetch("dkv.norm"))
        # [H, rank, dim]: carries a head's query into the latent space;  [H, vdim, rank]: a head's latent sum out of it
        self.uk_t = self._matrix(fetch("uk").reshape(H, self.dim, r).transpose(1, 2))
        self.uv = self._matrix(fetch("uv").reshape(H, self.vdim, r))
        self.out = Linear(self._matrix(fetch("o")))
        if self.has_sink:
            self.sink = self._f32(fetch("sink"))
        if self.rot_params is not None:
            from .side_by_side import rotary_for
            self.rotary = rotary_for(self.rot_params, self.dtype, self.device)

    accepts_residual = True

    def forward(self, x, step: StepContext, cache: LayerCache, position, write_cache=True, residual=None):
        g = step.groups[cache.group]
        table = self.rotary.table if self.rotary is not None else None
        proj = self.inp(x, torch.float32)                                           # [T, H*(dim+rot_dim) (+ rank+rot_dim) (+ gate)] float32
        if write_cache and not self.shared_kv:
            if self.rot_dim:
                ops.latent_rope_write(proj, self.off_c, self.rank, self.rot_dim, self.rot, self.c_gain, self.eps, step.positions,
                                      table, g.slot_mapping, cache.k)
            else:
                ops.latent_write(proj, self.off_c, self.rank, self.c_gain, self.eps, g.slot_mapping, cache.k)
        # [T, H*D] queries: a head's unrotated part carried into the latent space, its rotated part behind it
        ql = ops.head_linear(proj, 0, self.uk_t, self.dtype, xstride=self.qdim, ostride=self.D)
        if self.D > self.rank:
            ops.rope_cols_(ql, self.rank, self.D, proj, self.dim, self.qdim, self.rot_dim, self.rot, step.positions, table, self.heads)
        al = ops.paged_attention(ql, cache.k, cache.v, step, cache.group, self.heads, 1, self.D, self.scale, None, sink=self.sink)
        y = ops.head_linear(al, 0, self.uv, self.dtype, gate=proj if self.gate else None, goff=self.off_g,
                            gate_elem=self.gate == "element", xstride=self.D)      # [T, H*vdim]
        return self.out.into(y, residual)

    def weight_bytes(self):
        n = self.inp.nbytes() + self.out.nbytes() + 4 * self.rank + (4 * self.heads if self.has_sink else 0)
        return n + (self.uk_t.numel() + self.uv.numel()) * self.uk_t.element_size()
