"""Roritar: configuration -> plan.

Every layer is ``h += norm1b(mixer(norm1(h))); h += norm2b(feed_forward(norm2(h)))`` with layer norms (a weight, no
bias); the mixer is a recurrent block around a real-gated linear recurrent unit or attention over a sliding window and
pooled blocks, chosen layer by layer; the feed-forward is dense with the xIELU activation, or absent.  A run of layers
may be looped: the schedule names those layers several times, each run with a cache and state of its own.  The output
head is the embedding table; its logits are scaled and soft-capped.  Tensors: ``embed``, ``l<i>.norm1``, ``.norm1b``,
``.norm2``, ``.norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.roritar import ARCHITECTURE, RoritarConfig
from ..engine.plan import LayerSpec, ModelPlan, Run
from ..parts.base import PartSpec

RGLRU_SHARPNESS = 8.0       # log a = -8 r softplus(lam): fixed by the design


def _mixer(kind: str, m: dict, width: int, eps: float):
    """(mixer spec, position spec(s) or None)."""
    if kind == "rglru":
        return PartSpec("rglru", {"hidden_size": width, "width": m["width"], "blocks": m["blocks"], "conv": m["conv"],
                                  "sharpness": RGLRU_SHARPNESS}), None
    rot, mask = m["rot"], m.get("mask")
    spec = PartSpec("window_pool_attention",
                    {"hidden_size": width, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                     "value_dim": m["vdim"], "qk_norm": True, "norm_eps": eps, "scale": m["scale"],
                     "window": mask["size"] if mask else 0, "pool": mask["pool"] if mask else 0,
                     "rotate_values": True, "layout": rot.get("layout", "halves")})
    keys = PartSpec("rotary_neox", {"theta": rot["base"], "rotary_dim": rot["dims"]}) if rot["dims"] else None
    values = PartSpec("rotary_neox", {"theta": rot["base"], "rotary_dim": m["vdim"]})
    return spec, (keys, values)


def _feed_forward(mlp, width: int):
    if mlp is None:
        return None
    return PartSpec("plain_mlp", {"hidden_size": width, "intermediate_size": mlp["ff"], "activation": "xielu", "biases": False})


def roritar_plan(cfg: RoritarConfig) -> ModelPlan:
    D, eps = cfg.width, cfg.norm_eps
    norm = PartSpec("layer", {"dim": D, "eps": eps})
    layers = []
    for i, layer in enumerate(cfg.layers):
        mixer, position = _mixer(layer["type"], layer["mixer"], D, eps)
        layers.append(LayerSpec(block=PartSpec("sandwich_norm", {"mixer_norm": "norm1", "mixer_post_norm": "norm1b",
                                                                 "ffn_norm": "norm2", "ffn_post_norm": "norm2b",
                                                                 "mixer_prefix": "mix", "ffn_prefix": "mlp"}, prefix=f"l{i}."),
                                mixer=mixer, feed_forward=_feed_forward(layer["mlp"], D), norm=norm, position=position))
    return ModelPlan(
        architecture=ARCHITECTURE, hidden_size=D, vocab_size=cfg.vocab,
        embedding=PartSpec("token", {"vocab_size": cfg.vocab, "hidden_size": D, "name": "embed"}),
        layers=layers, schedule=[Run(i) for i in cfg.schedule()],
        final_norm=PartSpec("layer", {"dim": D, "eps": eps, "name": "final.norm"}),
        head=PartSpec("linear", {"vocab_size": cfg.vocab, "hidden_size": D, "tied": True, "name": "head", "tied_to": "embed",
                                 "scale": cfg.logit_scale, "softcap": cfg.logit_softcap}),
        stop_token_ids=(), max_position=None)


register_architecture(ARCHITECTURE, RoritarConfig, roritar_plan, replace=True)
