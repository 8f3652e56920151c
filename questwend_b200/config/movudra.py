"""Configuration of the Movudra design: a decoder whose layers are listed one by one, each with one of three
mixers (a Mamba-2 state-space layer, a gated delta rule with a decay per key channel, attention through a latent
with a sliding window and a sink) and a dense or routed feed-forward, or none.

config.json:  ``architecture`` (the design's name), ``vocab``, ``width``, ``norm.eps``, and ``layers``: a list of
``{"type": <mixer>, "mixer": {sizes}, "mlp": {..} | null}``.  Every size and constant that can differ between two
models of the design is read from there; the tensors' shapes follow from them.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from ..kernels.limits import conv_taps_refusal, latent_refusal, moe_refusal, state_matrix_refusal
from .base import ConfigError, ConfigReader, ModelConfig

ARCHITECTURE = "Movudra"
MIXER_TYPES = ("mamba2", "channel_delta", "latent_attention")
LOW_RANKS = {"decay_rank": "a1", "gate_rank": "g1"}     # the delta rule's low ranks: key -> the tensor whose rows they are
DEFAULT_LOW_RANK = 16                                   # for a configuration that names none and has no weights at hand


def _sub(r: ConfigReader, key: str, optional: bool = False):
    m = r.mapping(key, None) if optional else r.mapping(key)
    return None if m is None else ConfigReader(m, f"{r.where}: '{key}'")


def _refuse(where: str, refusal):
    if refusal:
        raise ConfigError(f"{where}: {refusal}")


def _read_mixer(kind: str, r: ConfigReader) -> dict:
    w = r.where
    if kind == "mamba2":
        m = {k: r.integer(k, minimum=1) for k in ("conv", "groups", "heads", "norm_groups", "state", "vdim")}
        if m["heads"] % m["groups"]:
            raise ConfigError(f"{w}: key 'heads' ({m['heads']}) must be a multiple of 'groups' ({m['groups']})")
        if (m["heads"] * m["vdim"]) % m["norm_groups"]:
            raise ConfigError(f"{w}: 'heads' x 'vdim' ({m['heads'] * m['vdim']}) must be a multiple of 'norm_groups' ({m['norm_groups']})")
        _refuse(f"{w}: key 'conv'", conv_taps_refusal(m["conv"]))
        _refuse(f"{w}: keys 'state' and 'vdim'", state_matrix_refusal(m["state"], m["vdim"]))
        return m
    if kind == "channel_delta":
        m = {k: r.integer(k, minimum=1) for k in ("conv", "dim", "heads", "kv_heads", "vdim")}
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"{w}: key 'heads' ({m['heads']}) must be a multiple of 'kv_heads' ({m['kv_heads']})")
        for k in LOW_RANKS:                      # not in a config.json as published: the tensors' shapes give them
            if r.has(k):
                m[k] = r.integer(k, minimum=1)
        _refuse(f"{w}: key 'conv'", conv_taps_refusal(m["conv"]))
        _refuse(f"{w}: keys 'dim' and 'vdim'", state_matrix_refusal(m["dim"], m["vdim"]))
        return m
    m = {k: r.integer(k, minimum=1) for k in ("dim", "heads", "kv_rank", "q_rank", "vdim")}
    m["rot_dim"] = r.integer("rot_dim", minimum=2)
    m["scale"] = r.number("scale", positive=True)
    mask = _sub(r, "mask", optional=True)
    m["mask"] = None if mask is None else {"size": mask.integer("size", minimum=1)}
    rot = _sub(r, "rot")
    m["rot"] = {"base": rot.number("base", positive=True), "dims": rot.integer("dims", minimum=2)}
    if m["rot"]["dims"] % 2 or m["rot"]["dims"] > m["rot_dim"]:
        raise ConfigError(f"{rot.where}: key 'dims' ({m['rot']['dims']}) must be even and at most 'rot_dim' ({m['rot_dim']})")
    if not m["rot"]["base"] > 1:
        raise ConfigError(f"{rot.where}: key 'base' must be > 1, got {m['rot']['base']}")
    sc = _sub(rot, "scaling", optional=True)
    if sc is not None:
        m["rot"]["scaling"] = {"factor": sc.number("factor", positive=True), "fast": sc.number("fast", positive=True),
                               "original": sc.number("original", positive=True), "slow": sc.number("slow", positive=True)}
    _refuse(f"{w}: keys 'kv_rank' and 'rot_dim'", latent_refusal(m["kv_rank"], m["rot_dim"]))
    return m


def _read_mlp(r: ConfigReader | None):
    if r is None:
        return None
    kind = r.string("kind")
    if kind == "dense":
        return {"kind": "dense", "ff": r.integer("ff", minimum=1)}
    if kind == "moe":
        router = _sub(r, "router")
        out = {"kind": "moe", "expert": {"ff": _sub(r, "expert").integer("ff", minimum=1)},
               "router": {"experts": router.integer("experts", minimum=1), "top": router.integer("top", minimum=1)}}
        _refuse(f"{router.where}: keys 'experts' and 'top'", moe_refusal(out["router"]["experts"], out["router"]["top"]))
        return out
    raise ConfigError(f"{r.where}: key 'kind' must be 'dense' or 'moe', got {kind!r}")


@dataclass(frozen=True)
class MovudraConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    layers: tuple = field(default_factory=tuple)     # dicts: {"type", "mixer": {...}, "mlp": {...} | None}

    architecture = ARCHITECTURE

    @classmethod
    def from_reader(cls, r: ConfigReader) -> "MovudraConfig":
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
        return cls(vocab=vocab, width=width, norm_eps=eps, layers=tuple(layers))

    def with_tensor_shapes(self, shapes) -> "MovudraConfig":
        """The delta rule's low ranks (decay and gate projections) are the row counts of ``l<i>.mix.a1`` / ``.g1``."""
        import copy
        import dataclasses
        layers = copy.deepcopy(list(self.layers))
        for i, layer in enumerate(layers):
            if layer["type"] == "channel_delta":
                for key, tensor in LOW_RANKS.items():
                    name = f"l{i}.mix.{tensor}"
                    if key not in layer["mixer"] and name in shapes and len(shapes[name]) == 2:
                        layer["mixer"][key] = int(shapes[name][0])
        return dataclasses.replace(self, layers=tuple(layers))

    def to_dict(self) -> dict:
        import copy
        return {"architecture": ARCHITECTURE, "layers": copy.deepcopy(list(self.layers)), "norm": {"eps": self.norm_eps},
                "vocab": self.vocab, "width": self.width}
