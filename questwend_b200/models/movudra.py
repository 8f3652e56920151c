"""Movudra: configuration -> plan.

Every layer is ``h += norm1(mixer(h)); h += norm2(feed_forward(h))`` (the norms on the sublayers' outputs; a layer
may have no feed-forward), with the mixer and the feed-forward chosen layer by layer; one epsilon for every norm; a
final norm and an untied output head.  Tensors: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``final.norm``, ``head``.  The low ranks of the delta rule's decay and gate projections are not in a
published config.json: the configuration takes them from the tensors' shapes (``MovudraConfig.with_tensor_shapes``),
and a configuration without them and without weights (random weights) gets ``DEFAULT_LOW_RANK``.
"""
from __future__ import annotations

from ..config.movudra import ARCHITECTURE, DEFAULT_LOW_RANK, MovudraConfig
from ..config.registry import register_architecture
from ..engine.plan import LayerSpec, ModelPlan, Run
from ..parts.base import PartSpec

def _mixer(kind: str, m: dict, width: int, eps: float):
    """(mixer spec, position spec or None)."""
    if kind == "mamba2":
        return PartSpec("mamba2", {"hidden_size": width, "heads": m["heads"], "vdim": m["vdim"], "state": m["state"],
                                   "groups": m["groups"], "norm_groups": m["norm_groups"], "conv": m["conv"],
                                   "norm_eps": eps}), None
    if kind == "channel_delta":
        return PartSpec("gated_delta_channelwise",
                        {"hidden_size": width, "heads": m["heads"], "key_heads": m["kv_heads"], "key_dim": m["dim"],
                         "vdim": m["vdim"], "conv": m["conv"], "decay_rank": m.get("decay_rank", DEFAULT_LOW_RANK),
                         "gate_rank": m.get("gate_rank", DEFAULT_LOW_RANK),
                         "norm_eps": eps, "unit_eps": 1e-6}), None
    rot = m["rot"]
    position = {"theta": rot["base"], "rotary_dim": rot["dims"]}
    if rot.get("scaling"):
        position.update({k: rot["scaling"][k] for k in ("factor", "original", "fast", "slow")})
    return (PartSpec("latent_attention",
                     {"hidden_size": width, "heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"],
                      "kv_rank": m["kv_rank"], "q_rank": m["q_rank"], "scale": m["scale"],
                      "window": m["mask"]["size"] if m.get("mask") else 0, "sink": True, "norm_eps": eps}),
            PartSpec("rotary_pairs", position))


def _feed_forward(mlp, width: int):
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("biased_mlp", {"hidden_size": width, "intermediate_size": mlp["ff"], "activation": "relu2"})
    return PartSpec("routed_experts", {"hidden_size": width, "expert_size": mlp["expert"]["ff"],
                                       "experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
                                       "renormalize": False})


def movudra_plan(cfg: MovudraConfig) -> ModelPlan:
    D, eps = cfg.width, cfg.norm_eps
    norm = PartSpec("rms", {"dim": D, "eps": eps})
    layers = []
    for i, layer in enumerate(cfg.layers):
        mixer, position = _mixer(layer["type"], layer["mixer"], D, eps)
        layers.append(LayerSpec(block=PartSpec("output_norm", {"mixer_norm": "norm1", "ffn_norm": "norm2",
                                                               "mixer_prefix": "mix", "ffn_prefix": "mlp"}, prefix=f"l{i}."),
                                mixer=mixer, feed_forward=_feed_forward(layer["mlp"], D), norm=norm, position=position))
    return ModelPlan(
        architecture=ARCHITECTURE, hidden_size=D, vocab_size=cfg.vocab,
        embedding=PartSpec("token", {"vocab_size": cfg.vocab, "hidden_size": D, "name": "embed"}),
        layers=layers, schedule=[Run(i) for i in range(len(layers))],
        final_norm=PartSpec("rms", {"dim": D, "eps": eps, "name": "final.norm"}),
        head=PartSpec("linear", {"vocab_size": cfg.vocab, "hidden_size": D, "tied": False, "name": "head", "tied_to": "embed"}),
        stop_token_ids=(), max_position=None)


register_architecture(ARCHITECTURE, MovudraConfig, movudra_plan, replace=True)
