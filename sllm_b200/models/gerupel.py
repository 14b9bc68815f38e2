"""Gerupel: typed configuration and model plan.

A decoder-only model whose embedding passes a norm before it enters the stream and whose output head is the embedding
table.  A layer adds both its terms at once, x <- x + m (mixer(norm1(x)) + ff(norm2(x))) with one factor m for the whole
model.  The mixer (``parallel``) is two mixers side by side on one input, summed with a factor each: grouped-query softmax
attention (part of each head rotated by position with a frequency scaling in three regimes of the wavelength, a stored
factor per head on the scores, a window of recent tokens plus one mean key and value per block of older tokens, one added
to the softmax's denominator) next to a linear attention whose forget gate also writes (HGRN2).  The feed-forward
(optional) is a mixture of gated experts behind a softmax router whose chosen scores are renormalized and scaled.  A range
of layers may run several times in a row with the same weights (``loop``): every pass has a cache and state of its own,
takes the embedding output in again (passes after the first) and a stored vector per pass.

This file is all that names the architecture: it reads config.json's keys (``architecture``, ``vocab``, ``width``,
``residual_mult``, ``norm.eps``, ``loop.{start, stop, times}`` and ``layers[i].{type, mixer, mlp}``), turns them into part
specifications, and registers itself.  Tensor names: ``embed``, ``embed.norm``, ``final.norm``, ``loop.step`` and under
``l<i>``: ``norm1``, ``norm2``, ``mix.left.*``, ``mix.right.*``, ``mlp.*``.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from ..config.errors import ConfigError
from ..config.fields import get_float, get_int, get_str
from ..config.plan import LayerSpec, ModelPlan, PartEntry, PartSpec, RunEntry
from ..config.registry import Architecture, register_architecture

NAME = "Gerupel"
MIXER_TYPES = ("parallel",)
MAX_POSITIONS = 1 << 17      # the design itself has no limit; this is the engine's (block tables and rotary tables are sized for it)


def _section(raw: dict, key: str, where: str = "config.json") -> dict:
    v = raw.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: key {key!r} must be an object")
    return v


def _check_mixer(i: int, m: dict) -> None:
    where = f"config.json: layers[{i}].mixer"
    left, right = _section(m, "left", where), _section(m, "right", where)
    get_float(m, "left_scale", positive=False), get_float(m, "right_scale", positive=False)
    for k in ("heads", "kv_heads", "dim", "vdim"):
        get_int(left, k)
    for k in ("heads", "dim", "vdim"):
        get_int(right, k)
    get_float(left, "scale")
    if left["heads"] % left["kv_heads"]:
        raise ConfigError(f"{where}.left: heads={left['heads']} is no multiple of kv_heads={left['kv_heads']}")
    if left.get("mask") is not None:                     # (no mask: every earlier position is seen, no pooled blocks)
        mask = _section(left, "mask", where + ".left")
        get_int(mask, "size")
        if mask.get("pool") is not None:
            get_int(mask, "pool")
    if left.get("rot") is not None:                      # (no rot: queries and keys are not rotated)
        rot = _section(left, "rot", where + ".left")
        get_float(rot, "base")
        if get_int(rot, "dims", minimum=2) % 2 or rot["dims"] > left["dim"]:
            raise ConfigError(f"{where}.left.rot.dims={rot['dims']} must be even and at most dim={left['dim']}")
        sc = rot.get("scaling")
        if sc is not None:
            if not isinstance(sc, dict):
                raise ConfigError(f"{where}.left.rot.scaling must be an object or null")
            for k in ("factor", "low", "high", "original"):
                get_float(sc, k)


def _check_mlp(i: int, mlp: dict) -> None:
    where = f"config.json: layers[{i}].mlp"
    if get_str(mlp, "kind") != "moe":
        raise ConfigError(f"{where}.kind={mlp['kind']!r}; this design has 'moe'")
    get_int(_section(mlp, "expert", where), "ff")
    r = _section(mlp, "router", where)
    E, top = get_int(r, "experts"), get_int(r, "top")
    get_float(r, "scale", positive=False)
    if top > E:
        raise ConfigError(f"{where}.router: top={top} of {E} experts cannot be chosen")


@dataclass(frozen=True)
class LayerConfig:
    type: str
    mixer: dict
    mlp: dict | None


@dataclass(frozen=True)
class GerupelConfig:
    vocab: int
    width: int
    residual_mult: float
    norm_eps: float
    layers: tuple = field(default_factory=tuple)
    loop: tuple | None = None        # (start, stop, times)
    architecture: str = NAME

    @classmethod
    def from_dict(cls, raw: dict) -> "GerupelConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: key 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(layers_raw):
            if not isinstance(entry, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            typ = get_str(entry, "type")
            if typ not in MIXER_TYPES:
                raise ConfigError(f"config.json: layers[{i}].type={typ!r}; this design has {MIXER_TYPES}")
            mixer = dict(_section(entry, "mixer", f"config.json: layers[{i}]"))
            _check_mixer(i, mixer)
            mlp = entry.get("mlp")
            if mlp is not None:
                mlp = dict(_section(entry, "mlp", f"config.json: layers[{i}]"))
                _check_mlp(i, mlp)
            layers.append(LayerConfig(typ, mixer, mlp))
        loop = None
        if raw.get("loop") is not None:
            lp = _section(raw, "loop")
            start, stop, times = get_int(lp, "start", minimum=0), get_int(lp, "stop", minimum=0), get_int(lp, "times")
            if not start <= stop <= len(layers):
                raise ConfigError(f"config.json: loop {start}..{stop} lies outside the model's {len(layers)} layers")
            if stop > start:                     # (an empty range repeats nothing)
                loop = (start, stop, times)
        return cls(vocab=get_int(raw, "vocab"), width=get_int(raw, "width"),
                   residual_mult=get_float(raw, "residual_mult", 1.0, positive=False),
                   norm_eps=get_float(_section(raw, "norm"), "eps"), layers=tuple(layers), loop=loop)

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "residual_mult": self.residual_mult,
             "norm": {"eps": self.norm_eps},
             "layers": [{"type": l.type, "mixer": dict(l.mixer), "mlp": dict(l.mlp) if l.mlp is not None else None}
                        for l in self.layers]}
        if self.loop is not None:
            d["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        return d


def _mixer_spec(cfg: GerupelConfig, l: LayerConfig) -> PartSpec:
    m, W, eps, mult = l.mixer, cfg.width, cfg.norm_eps, cfg.residual_mult
    left, right = m["left"], m["right"]
    rot, mask = left.get("rot"), left.get("mask")
    # the layer's factor on its terms and each side's own ride on the sides' outputs
    attention = {"hidden_size": W, "heads": left["heads"], "kv_heads": left["kv_heads"], "dim": left["dim"], "vdim": left["vdim"],
                 "scale": left["scale"], "window": mask["size"] if mask else None, "pool": mask.get("pool") if mask else None,
                 "sink": 0.0, "out_scale": mult * m["left_scale"], "max_positions": MAX_POSITIONS,
                 "rotary": {"theta": rot["base"], "rotary_dim": rot["dims"], "scaling": rot.get("scaling")} if rot else None}
    recurrent = {"hidden_size": W, "heads": right["heads"], "dim": right["dim"], "vdim": right["vdim"], "eps": eps,
                 "out_scale": mult * m["right_scale"]}
    return PartSpec("side_by_side_sum", {"hidden_size": W, "left": {"kind": "pooled_window_attention", "params": attention},
                                         "right": {"kind": "forget_gate_attention", "params": recurrent}})


def _ffn_spec(cfg: GerupelConfig, mlp: dict) -> PartSpec:
    r = mlp["router"]
    return PartSpec("gated_experts", {"hidden_size": cfg.width, "experts": r["experts"], "top": r["top"],
                                      "scale": cfg.residual_mult * r["scale"], "expert_ff": mlp["expert"]["ff"],
                                      "activation": "silu"})


def run_list(cfg: GerupelConfig) -> tuple:
    L = len(cfg.layers)
    if cfg.loop is None:
        return tuple(RunEntry(i) for i in range(L))
    start, stop, times = cfg.loop
    runs = [RunEntry(i) for i in range(start)]
    for t in range(times):
        runs += [RunEntry(i, reentry=t if i == start else None) for i in range(start, stop)]
    runs += [RunEntry(i) for i in range(stop, L)]
    return tuple(runs)


def plan(cfg: GerupelConfig) -> ModelPlan:
    norm = PartSpec("group_rmsnorm", {"size": cfg.width, "groups": 1, "eps": cfg.norm_eps})
    layers = []
    for i, l in enumerate(cfg.layers):
        parts = {"mixer_norm": PartEntry("norm", norm, "norm1"), "mixer": PartEntry("mixer", _mixer_spec(cfg, l), "mix")}
        if l.mlp is not None:
            parts["ffn_norm"] = PartEntry("norm", norm, "norm2")
            parts["ffn"] = PartEntry("feed_forward", _ffn_spec(cfg, l.mlp), "mlp")
        layers.append(LayerSpec(prefix=f"l{i}", parts=parts, block="parallel_pair"))
    p = ModelPlan(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        embedding_name="embed", layers=tuple(layers), run_list=run_list(cfg),
        final_norm=norm, final_norm_name="final.norm", head_name=None, position=None,
        embedding_norm=norm, embedding_norm_name="embed.norm",
        pass_vectors_name="loop.step" if cfg.loop is not None else None, passes=cfg.loop[2] if cfg.loop is not None else 0,
        ignored_names=tuple(f"l{i}.norm2" for i, l in enumerate(cfg.layers) if l.mlp is None))
    p.validate()
    return p


def config_from_recipe(t: dict) -> dict:
    """A recipe's inline geometry carries config.json's own keys (``vocab``, ``width``, ``residual_mult``, ``norm``,
    ``layers``, optionally ``loop``); a missing one raises KeyError naming it."""
    cfg = {k: t[k] for k in ("vocab", "width", "norm", "layers")}
    cfg["residual_mult"] = t.get("residual_mult", 1.0)
    if t.get("loop") is not None:
        cfg["loop"] = t["loop"]
    cfg["architecture"] = NAME
    return cfg


register_architecture(Architecture(name=NAME, config_cls=GerupelConfig, plan=plan, aliases=("gerupel",),
                                   config_from_recipe=config_from_recipe), replace=True)
