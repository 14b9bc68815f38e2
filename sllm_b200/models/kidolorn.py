"""Kidolorn: typed configuration and model plan.

A decoder-only model whose layers put a norm before AND after each sublayer, x <- x + post(mixer(pre(x))), then the same
around the feed-forward; every norm's gain is one number.  What a sublayer reads first passes a short causal convolution
that is added to its own input.  A layer's mixer is linear attention with a fixed decay per head (``lightning``), an
element-wise gated recurrence (``mingru``), or softmax attention over a small cached latent with one rotated key part
shared by the heads and a sink in the denominator (``latent_attention``; with ``kv_from`` it reads the cache of an
earlier layer).  The feed-forward (optional) is a clamped gated unit, dense with biases or a mixture of experts whose
router takes the largest logits.  The model's norm and an output head of its own follow.

This file is all that names the architecture: it reads config.json's keys (``architecture``, ``vocab``, ``width``,
``norm.eps``, ``canon.taps`` and ``layers[i].{type, mixer, mlp}``), turns them into part specifications, and registers
itself.  Tensor names: ``embed``, ``head``, ``final.norm``, and under ``l<i>``: ``norm1``, ``norm1b``, ``norm2``, ``norm2b``,
``canon1``, ``canon2``, ``mix.*``, ``mlp.*``.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from ..config.errors import ConfigError
from ..config.fields import get_float, get_int, get_str
from ..config.plan import LayerSpec, ModelPlan, PartEntry, PartSpec, RunEntry
from ..config.registry import Architecture, register_architecture

NAME = "Kidolorn"
MIXER_TYPES = ("lightning", "mingru", "latent_attention")
MAX_POSITIONS = 1 << 17      # the design itself has no limit; this is the engine's (block tables and rotary tables are sized for it)
SWISH_ALPHA = 1.702          # the gated unit's g * sigmoid(1.702 g): fixed by the design


def _section(raw: dict, key: str, where: str = "config.json") -> dict:
    v = raw.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: key {key!r} must be an object")
    return v


def _check_mixer(i: int, typ: str, m: dict, layers: list) -> None:
    where = f"config.json: layers[{i}].mixer"
    if typ == "mingru":
        get_int(m, "width")
        return
    for k in ("heads", "dim", "vdim"):
        get_int(m, k)
    if typ == "lightning":
        d = m.get("decay")
        if not isinstance(d, list) or len(d) != m["heads"] or any(isinstance(x, bool) or not isinstance(x, (int, float)) for x in d):
            raise ConfigError(f"{where}.decay must list one number per head ({m['heads']})")
        return
    get_int(m, "kv_rank"), get_int(m, "rot_dim", minimum=0), get_float(m, "scale")
    if m["rot_dim"]:
        rot = _section(m, "rot", where)
        get_float(rot, "base")
        if get_int(rot, "dims", minimum=2) % 2 or rot["dims"] > m["rot_dim"]:
            raise ConfigError(f"{where}.rot.dims={rot['dims']} must be even and at most rot_dim={m['rot_dim']}")
    src = m.get("kv_from")
    if src is not None:
        if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
            raise ConfigError(f"{where}.kv_from={src!r} must name an earlier layer")
        other = layers[src]
        if other.type != "latent_attention" or other.mixer.get("kv_from") is not None:
            raise ConfigError(f"{where}.kv_from={src}: that layer has no down-projection of its own")
        for k in ("kv_rank", "rot_dim", "rot"):
            if other.mixer.get(k) != m.get(k):
                raise ConfigError(f"{where}.kv_from={src}: {k} differs ({other.mixer.get(k)!r} there, {m.get(k)!r} here)")


def _check_mlp(i: int, mlp: dict) -> None:
    where = f"config.json: layers[{i}].mlp"
    kind = get_str(mlp, "kind")
    if kind == "dense":
        get_int(mlp, "ff"), get_float(mlp, "limit")
    elif kind == "moe":
        e = _section(mlp, "expert", where)
        get_int(e, "ff"), get_float(e, "limit")
        r = _section(mlp, "router", where)
        if get_int(r, "top") > get_int(r, "experts"):
            raise ConfigError(f"{where}.router: top={r['top']} of {r['experts']} experts cannot be chosen")
    else:
        raise ConfigError(f"{where}.kind={kind!r}; this design has 'dense' and 'moe'")


@dataclass(frozen=True)
class LayerConfig:
    type: str
    mixer: dict
    mlp: dict | None


@dataclass(frozen=True)
class KidolornConfig:
    vocab: int
    width: int
    norm_eps: float
    taps: int | None = None          # of the convolution in front of every sublayer (None: no convolution)
    layers: tuple = field(default_factory=tuple)
    architecture: str = NAME

    @classmethod
    def from_dict(cls, raw: dict) -> "KidolornConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: key 'layers' must be a non-empty list")
        layers: list = []
        for i, entry in enumerate(layers_raw):
            if not isinstance(entry, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            typ = get_str(entry, "type")
            if typ not in MIXER_TYPES:
                raise ConfigError(f"config.json: layers[{i}].type={typ!r}; this design has {MIXER_TYPES}")
            mixer = dict(_section(entry, "mixer", f"config.json: layers[{i}]"))
            _check_mixer(i, typ, mixer, layers)
            mlp = entry.get("mlp")
            if mlp is not None:
                mlp = dict(_section(entry, "mlp", f"config.json: layers[{i}]"))
                _check_mlp(i, mlp)
            layers.append(LayerConfig(typ, mixer, mlp))
        taps = get_int(_section(raw, "canon"), "taps") if raw.get("canon") is not None else None
        return cls(vocab=get_int(raw, "vocab"), width=get_int(raw, "width"), norm_eps=get_float(_section(raw, "norm"), "eps"),
                   taps=taps, layers=tuple(layers))

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "layers": [{"type": l.type, "mixer": dict(l.mixer), "mlp": dict(l.mlp) if l.mlp is not None else None}
                        for l in self.layers]}
        if self.taps is not None:
            d["canon"] = {"taps": self.taps}
        return d


def _mixer_spec(cfg: KidolornConfig, l: LayerConfig) -> PartSpec:
    m, W, eps = l.mixer, cfg.width, cfg.norm_eps
    if l.type == "mingru":
        return PartSpec("mingru", {"hidden_size": W, "width": m["width"]})
    if l.type == "lightning":
        return PartSpec("decay_linear_attention", {"hidden_size": W, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
                                                   "decay": tuple(float(d) for d in m["decay"]), "eps": eps})
    rot = m.get("rot") if m["rot_dim"] else None
    return PartSpec("latent_attention", {
        "hidden_size": W, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"], "kv_rank": m["kv_rank"], "scale": m["scale"],
        "eps": eps, "gate": "element", "sink": True, "rot_dim": m["rot_dim"], "shared_kv": m.get("kv_from") is not None,
        "rotary": {"theta": rot["base"], "rotary_dim": rot["dims"], "max_positions": MAX_POSITIONS} if rot else None})


def _ffn_spec(cfg: KidolornConfig, mlp: dict) -> PartSpec:
    if mlp["kind"] == "dense":
        return PartSpec("gated_dense", {"hidden_size": cfg.width, "intermediate_size": mlp["ff"], "activation": "clamped_swish",
                                        "limit": mlp["limit"], "alpha": SWISH_ALPHA, "bias": True})
    r = mlp["router"]
    return PartSpec("gated_experts", {"hidden_size": cfg.width, "experts": r["experts"], "top": r["top"],
                                      "expert_ff": mlp["expert"]["ff"], "limit": mlp["expert"]["limit"], "alpha": SWISH_ALPHA})


def plan(cfg: KidolornConfig) -> ModelPlan:
    norm = PartSpec("scalar_rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps})
    conv = PartSpec("input_conv", {"size": cfg.width, "taps": cfg.taps}) if cfg.taps is not None else None
    layers, runs = [], []
    for i, l in enumerate(cfg.layers):
        parts = {"mixer_norm": PartEntry("norm", norm, "norm1"), "mixer": PartEntry("mixer", _mixer_spec(cfg, l), "mix"),
                 "mixer_post": PartEntry("norm", norm, "norm1b")}
        if conv is not None:
            parts["mixer_conv"] = PartEntry("shift", conv, "canon1")
        if l.mlp is not None:
            parts.update(ffn_norm=PartEntry("norm", norm, "norm2"), ffn=PartEntry("feed_forward", _ffn_spec(cfg, l.mlp), "mlp"),
                         ffn_post=PartEntry("norm", norm, "norm2b"))
            if conv is not None:
                parts["ffn_conv"] = PartEntry("shift", conv, "canon2")
        layers.append(LayerSpec(prefix=f"l{i}", parts=parts, block="sandwich"))
        # a layer that reads another layer's latents borrows that run's pages (and writes none)
        runs.append(RunEntry(i, cache_from=l.mixer.get("kv_from") if l.type == "latent_attention" else None))
    p = ModelPlan(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        embedding_name="embed", layers=tuple(layers), run_list=tuple(runs),
        final_norm=norm, final_norm_name="final.norm", head_name="head", position=None)
    p.validate()
    return p


def config_from_recipe(t: dict) -> dict:
    """A recipe's inline geometry carries config.json's own keys (``vocab``, ``width``, ``norm``, ``canon``, ``layers``); a
    missing one raises KeyError naming it."""
    cfg = {k: t[k] for k in ("vocab", "width", "norm", "layers")}
    if t.get("canon") is not None:
        cfg["canon"] = t["canon"]
    cfg["architecture"] = NAME
    return cfg


register_architecture(Architecture(name=NAME, config_cls=KidolornConfig, plan=plan, aliases=("kidolorn",),
                                   config_from_recipe=config_from_recipe), replace=True)
