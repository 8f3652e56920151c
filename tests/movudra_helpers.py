"""Shared by the Movudra tests: small configurations of their own, weights drawn so that every mechanism matters
(O(1) activations, decays from fast to almost none, sinks that weigh in, biases that are not zero), model folders."""
from __future__ import annotations

import json
import os

import numpy as np
import torch

import plain_movudra as pmv


def delta(heads=3, kv_heads=3, dim=16, vdim=24, conv=4):
    return {"type": "channel_delta", "mixer": {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim}}


def mamba(heads=6, vdim=16, state=24, groups=3, norm_groups=2, conv=3):
    return {"type": "mamba2", "mixer": {"conv": conv, "groups": groups, "heads": heads, "norm_groups": norm_groups,
                                        "state": state, "vdim": vdim}}


def latent(heads=3, dim=24, rot_dim=8, vdim=20, kv_rank=40, q_rank=48, window=5, dims=None, scaling=True, base=10000.0,
           scale=0.3):
    rot = {"base": base, "dims": dims or rot_dim}
    if scaling:
        rot["scaling"] = {"factor": 8.0, "fast": 16.0, "original": 64, "slow": 2.0}
    m = {"dim": dim, "heads": heads, "kv_rank": kv_rank, "q_rank": q_rank, "rot": rot, "rot_dim": rot_dim, "scale": scale,
         "vdim": vdim}
    if window:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m}


def dense(ff=96):
    return {"kind": "dense", "ff": ff}


def moe(ff=40, experts=6, top=3):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def config(layers, width=64, vocab=96, eps=1e-5):
    """layers: (mixer entry, mlp entry or None) pairs."""
    return {"architecture": "Movudra", "layers": [{**mix, "mlp": mlp} for mix, mlp in layers], "norm": {"eps": eps},
            "vocab": vocab, "width": width}


# One of everything, sizes that share no value with one another where they could be confused: 3 and 6 heads, key heads
# fewer than heads, groups that are not 1, a window that ends inside the first page, a layer without a feed-forward.
MIXED = config([(delta(heads=6, kv_heads=3), dense()), (latent(), moe()), (mamba(), None),
                (latent(heads=5, dim=16, rot_dim=12, dims=8, vdim=16, kv_rank=24, q_rank=20, window=70, scaling=False), moe(top=1)),
                (delta(heads=2, kv_heads=1, dim=40, vdim=16, conv=2), moe(ff=24, experts=3, top=2)),
                (mamba(heads=2, vdim=40, state=16, groups=1, norm_groups=1, conv=1), dense(ff=40))], width=64, vocab=96)
# sizes that happen to be equal or 1: one head, one group, one expert of one, a window of one token, two taps
ONES = config([(delta(heads=1, kv_heads=1, dim=16, vdim=16, conv=2), moe(ff=16, experts=1, top=1)),
               (latent(heads=1, dim=16, rot_dim=2, vdim=16, kv_rank=16, q_rank=16, window=1), dense(ff=16)),
               (mamba(heads=1, vdim=16, state=16, groups=1, norm_groups=1, conv=2), None),
               (latent(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=8, q_rank=8, window=0, scaling=False), None)],
              width=16, vocab=32, eps=1e-6)


def draw_weights(cfgd, seed=0, slow_decay=False):
    """float64 arrays by tensor name, every value a bfloat16 number, for the tensors that the library's plan lists."""
    import questwend_b200  # noqa: F401
    from questwend_b200.config.registry import config_from_dict, get_architecture
    cfg = config_from_dict(cfgd)
    rng = np.random.default_rng(seed)
    out = {}
    for spec in get_architecture(cfg.architecture).plan(cfg).manifest():
        name, shape = spec.name, tuple(spec.shape)
        last = name.rsplit(".", 1)[-1]
        if name.endswith((".norm1", ".norm2", "final.norm", ".mix.norm", ".dq.norm", ".dkv.norm")):
            v = 1.0 + 0.3 * rng.standard_normal(shape)
        elif name.endswith(".conv"):
            v = 0.6 * rng.standard_normal(shape)
        elif name.endswith(".b") and len(shape) == 1:                    # conv.b, up.b, down.b
            v = 0.4 * rng.standard_normal(shape)
        elif last == "A_log":
            v = rng.uniform(-9.0, -6.0, shape) if slow_decay else rng.uniform(-4.0, 1.0, shape)
        elif last == "dt_bias":
            v = rng.standard_normal(shape)
        elif last == "D":
            v = 1.0 + 0.5 * rng.standard_normal(shape)
        elif last == "sink":
            v = 1.5 * rng.standard_normal(shape) + 1.0
        elif name == "embed":
            v = rng.standard_normal(shape)
        elif last == "router":
            v = 4.0 * rng.standard_normal(shape) / np.sqrt(shape[1])
        else:                                                            # a matrix [out, in]
            v = 1.3 * rng.standard_normal(shape) / np.sqrt(shape[1])
        out[name] = pmv.round_bf16(v)
    return out


def write_folder(path, cfgd, w):
    from questwend_b200.weights import write_safetensors
    os.makedirs(path, exist_ok=True)
    write_safetensors(os.path.join(path, "model.safetensors"),
                      {k: torch.from_numpy(np.asarray(v, dtype=np.float32)).to(torch.bfloat16) for k, v in w.items()})
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfgd, f)
    return str(path)


def row_err(got, ref):
    """Largest difference of any row, relative to the largest logit."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    return float(np.abs(got - ref).max() / np.abs(ref).max())
