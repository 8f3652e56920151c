"""Shared by the Roritar tests: small configurations of their own, weights drawn so that every mechanism matters
(O(1) activations, decays from fast to almost none, sharp attention, biases that are not zero), model folders."""
from __future__ import annotations

import json
import os

import numpy as np
import torch

import plain_roritar as pr


def rglru(width=48, blocks=3, conv=4):
    return {"type": "rglru", "mixer": {"blocks": blocks, "conv": conv, "width": width}}


def attention(heads=4, kv_heads=2, dim=24, vdim=16, size=20, pool=5, dims=8, base=10000.0, scale=0.3, layout=None):
    rot = {"base": base, "dims": dims}
    if layout:
        rot["layout"] = layout
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "rot": rot, "scale": scale, "vdim": vdim}
    if size:
        m["mask"] = {"size": size, "pool": pool}
    return {"type": "attention", "mixer": m}


def dense(ff=96):
    return {"kind": "dense", "ff": ff}


def config(layers, width=64, vocab=96, eps=1e-5, loop=None, logit_scale=1.5, logit_softcap=9.0):
    """layers: (mixer entry, mlp entry or None) pairs."""
    out = {"architecture": "Roritar", "layers": [{**mix, "mlp": mlp} for mix, mlp in layers], "norm": {"eps": eps},
           "vocab": vocab, "width": width}
    if loop:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    if logit_scale is not None:
        out["logit_scale"] = logit_scale
    if logit_softcap is not None:
        out["logit_softcap"] = logit_softcap
    return out


# Sizes that share no value where they could be confused: key/value heads fewer than heads, keys larger than values and
# the other way round, a block size that does not divide the page of 64, a window that ends inside the first page and
# one that crosses pages, a looped run that starts after the first layer, a layer without a feed-forward.
MIXED = config([(attention(heads=4, kv_heads=2, dim=24, vdim=16, size=20, pool=5, dims=8), dense()),
                (rglru(width=48, blocks=3, conv=4), dense(ff=40)),
                (attention(heads=3, kv_heads=3, dim=16, vdim=40, size=70, pool=12, dims=16, base=500.0), None),
                (rglru(width=80, blocks=5, conv=2), dense(ff=72)),
                (attention(heads=6, kv_heads=1, dim=8, vdim=8, size=7, pool=7, dims=2, scale=0.6), dense(ff=24))],
               width=64, vocab=96, loop=(1, 4, 3))
# values that happen to be equal or 1: one head, one block, one tap, blocks of one token, a window of one token, no
# rotation of keys, a loop of one pass, no cap on the logits
ONES = config([(rglru(width=16, blocks=1, conv=1), None),
               (attention(heads=1, kv_heads=1, dim=16, vdim=16, size=1, pool=1, dims=0), dense(ff=16)),
               (attention(heads=2, kv_heads=2, dim=8, vdim=8, size=0, pool=0, dims=8), None),
               (rglru(width=16, blocks=16, conv=2), dense(ff=16))],
              width=16, vocab=37, eps=1e-6, loop=(0, 2, 1), logit_scale=None, logit_softcap=None)


def draw_weights(cfgd, seed=0, slow_decay=False, sharp=1.0):
    """float64 arrays by tensor name, every value a bfloat16 number, from the configuration alone.  ``sharp`` scales the
    q and k norm weights: a sharper softmax shows a key that is seen or not seen."""
    rng = np.random.default_rng(seed)
    D, V = cfgd["width"], cfgd["vocab"]
    w = {}

    def matrix(*shape):
        return 1.3 * rng.standard_normal(shape) / np.sqrt(shape[-1])

    def norm_weight(n):
        return 1.0 + 0.3 * rng.standard_normal(n)

    w["embed"] = rng.standard_normal((V, D))
    w["final.norm"] = norm_weight(D)
    for i, layer in enumerate(cfgd["layers"]):
        px, m = f"l{i}.", layer["mixer"]
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if layer["mlp"] else ()):
            w[px + n] = norm_weight(D)
        if layer["type"] == "rglru":
            W, nb = m["width"], m["blocks"]
            w[px + "mix.y"], w[px + "mix.x"], w[px + "mix.o"] = matrix(W, D), matrix(W, D), matrix(D, W)
            w[px + "mix.y.b"], w[px + "mix.x.b"] = 0.4 * rng.standard_normal(W), 0.4 * rng.standard_normal(W)
            w[px + "mix.conv"], w[px + "mix.conv.b"] = 0.6 * rng.standard_normal((W, m["conv"])), 0.4 * rng.standard_normal(W)
            for g in ("ra", "ri"):
                w[px + f"mix.{g}"] = 2.0 * matrix(nb, W // nb, W // nb)
                w[px + f"mix.{g}.b"] = 0.5 * rng.standard_normal((nb, W // nb))
            # softplus(lam) from ~0.001 to ~1: decays from almost none to fast
            w[px + "mix.lam"] = rng.uniform(-9.0, -6.0, W) if slow_decay else rng.uniform(-6.0, 1.0, W)
        else:
            H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[px + "mix.q"], w[px + "mix.k"], w[px + "mix.v"] = matrix(H * dim, D), matrix(G * dim, D), matrix(G * vdim, D)
            w[px + "mix.o"] = matrix(D, H * vdim)
            w[px + "mix.q.norm"], w[px + "mix.k.norm"] = sharp * norm_weight(dim), sharp * norm_weight(dim)
        if layer["mlp"]:
            ff = layer["mlp"]["ff"]
            w[px + "mlp.up"], w[px + "mlp.down"] = matrix(ff, D), matrix(D, ff)
            w[px + "mlp.act"] = rng.standard_normal(2)
    return {k: pr.round_bf16(v) for k, v in w.items()}


def write_folder(path, cfgd, w):
    from questwend_b200.weights import write_safetensors
    os.makedirs(path, exist_ok=True)
    write_safetensors(os.path.join(path, "model.safetensors"),
                      {k: torch.from_numpy(np.asarray(v, dtype=np.float32)).to(torch.bfloat16) for k, v in w.items()})
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfgd, f)
    return str(path)
