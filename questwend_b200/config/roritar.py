"""Configuration of the Roritar design: a decoder whose layers are listed one by one, each a recurrent block around a
real-gated linear recurrent unit or attention over a sliding window plus pooled blocks of what lies before it, with a
dense feed-forward or none; a norm in front of and behind every sublayer; a run of layers may be looped.

config.json:  ``architecture`` (the design's name), ``vocab``, ``width``, ``norm.eps``, ``layers``: a list of
``{"type": "rglru" | "attention", "mixer": {sizes}, "mlp": {"kind": "dense", "ff": n} | null}``, and optionally
``loop`` {start, stop, times} (layers start .. stop-1 run ``times`` times in a row with the same weights, each pass with
a cache and state of its own), ``logit_scale`` and ``logit_softcap``.  Every size and constant that can differ between
two models of the design is read from there.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from ..kernels.limits import conv_taps_refusal, pool_attention_refusal
from .base import ConfigError, ConfigReader, ModelConfig

ARCHITECTURE = "Roritar"
MIXER_TYPES = ("rglru", "attention")
ROTATION_LAYOUTS = ("halves", "interleaved")


def _sub(r: ConfigReader, key: str, optional: bool = False):
    m = r.mapping(key, None) if optional else r.mapping(key)
    return None if m is None else ConfigReader(m, f"{r.where}: '{key}'")


def _refuse(where: str, refusal):
    if refusal:
        raise ConfigError(f"{where}: {refusal}")


def _read_mixer(kind: str, r: ConfigReader) -> dict:
    w = r.where
    if kind == "rglru":
        m = {k: r.integer(k, minimum=1) for k in ("blocks", "conv", "width")}
        if m["width"] % m["blocks"]:
            raise ConfigError(f"{w}: key 'width' ({m['width']}) must be a multiple of 'blocks' ({m['blocks']})")
        _refuse(f"{w}: key 'conv'", conv_taps_refusal(m["conv"]))
        return m
    m = {k: r.integer(k, minimum=1) for k in ("dim", "heads", "kv_heads", "vdim")}
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"{w}: key 'heads' ({m['heads']}) must be a multiple of 'kv_heads' ({m['kv_heads']})")
    if m["vdim"] % 2:
        raise ConfigError(f"{w}: key 'vdim' ({m['vdim']}) must be even: values are turned in pairs")
    m["scale"] = r.number("scale", positive=True)
    mask = _sub(r, "mask", optional=True)
    m["mask"] = None
    if mask is not None:
        m["mask"] = {"size": mask.integer("size", minimum=1), "pool": mask.integer("pool", 0, minimum=0)}
    rot = _sub(r, "rot")
    m["rot"] = {"base": rot.number("base", positive=True), "dims": rot.integer("dims", minimum=0)}
    if rot.has("layout"):
        m["rot"]["layout"] = rot.string("layout")
        if m["rot"]["layout"] not in ROTATION_LAYOUTS:
            raise ConfigError(f"{rot.where}: key 'layout' must be one of {', '.join(ROTATION_LAYOUTS)}, got {m['rot']['layout']!r}")
    if m["rot"]["dims"] % 2 or m["rot"]["dims"] > m["dim"]:
        raise ConfigError(f"{rot.where}: key 'dims' ({m['rot']['dims']}) must be even and at most 'dim' ({m['dim']})")
    if not m["rot"]["base"] > 1:
        raise ConfigError(f"{rot.where}: key 'base' must be > 1, got {m['rot']['base']}")
    _refuse(f"{w}: keys 'dim' and 'vdim'", pool_attention_refusal(m["dim"], m["vdim"]))
    return m


def _read_mlp(r: ConfigReader | None):
    if r is None:
        return None
    kind = r.string("kind")
    if kind != "dense":
        raise ConfigError(f"{r.where}: key 'kind' must be 'dense', got {kind!r}")
    return {"kind": "dense", "ff": r.integer("ff", minimum=1)}


@dataclass(frozen=True)
class RoritarConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    layers: tuple = field(default_factory=tuple)     # dicts: {"type", "mixer": {...}, "mlp": {...} | None}
    loop: tuple | None = None                        # (start, stop, times)
    logit_scale: float = 1.0
    logit_softcap: float = 0.0

    architecture = ARCHITECTURE

    @classmethod
    def from_reader(cls, r: ConfigReader) -> "RoritarConfig":
        vocab = r.integer("vocab", minimum=1)
        width = r.integer("width", minimum=1)
        eps = _sub(r, "norm").number("eps", positive=True)
        r.read_keys.add("layers")
        raw = r.data.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError(f"{r.where}: key 'layers' must be a list with at least one layer")
        layers = []
        for i, entry in enumerate(raw):
            lr = ConfigReader(entry, f"{r.where}: layers[{i}]")
            kind = lr.string("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"{lr.where}: key 'type' must be one of {', '.join(MIXER_TYPES)}, got {kind!r}")
            layers.append({"type": kind, "mixer": _read_mixer(kind, _sub(lr, "mixer")), "mlp": _read_mlp(_sub(lr, "mlp", optional=True))})
        loop = None
        lp = _sub(r, "loop", optional=True)
        if lp is not None:
            loop = (lp.integer("start", minimum=0), lp.integer("stop", minimum=0), lp.integer("times", minimum=1))
            if not loop[0] <= loop[1] <= len(layers):
                raise ConfigError(f"{lp.where}: layers {loop[0]} .. {loop[1]} - 1 do not lie within the {len(layers)} layers")
        scale = r.number("logit_scale", 1.0, positive=True)
        cap = r.number("logit_softcap", 0.0)
        if cap < 0:
            raise ConfigError(f"{r.where}: key 'logit_softcap' must be >= 0, got {cap}")
        return cls(vocab=vocab, width=width, norm_eps=eps, layers=tuple(layers), loop=loop, logit_scale=scale, logit_softcap=cap)

    def schedule(self) -> list[int]:
        """The layers in the order they run: the looped run repeated, the rest once."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))

    def to_dict(self) -> dict:
        import copy
        out = {"architecture": ARCHITECTURE, "layers": copy.deepcopy(list(self.layers)), "norm": {"eps": self.norm_eps},
               "vocab": self.vocab, "width": self.width, "logit_scale": self.logit_scale, "logit_softcap": self.logit_softcap}
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return out
