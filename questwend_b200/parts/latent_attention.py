"""Attention through a latent: per token the cache holds one row, a normed low-rank latent c and one rotated key part
shared by all heads, instead of keys and values per head.  A head's unrotated key is W_uk c and its value W_uv c, so
the score q . (W_uk c) is formed as (W_uk^T q) . c and the output as W_uv (sum_j p_j c_j): every head attends over the
same cached rows, and keys and values per head are never made.  Causal, with an optional sliding window and an
optional learned sink per head in the softmax's denominator.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..kernels.limits import latent_refusal
from ..weights.manifest import MATRIX, NORM_WEIGHT, VECTOR, TensorSpec
from .base import KVSpec, Mixer
from .linear import _check_true_fp32, kernel_modules as linear_modules, linear
from .registry import register_mixer


PROMPT_KERNEL_MIN_TOKENS = 17      # whole prompts of at least this many tokens (the longest of the step) take the
                                   # tensor-core kernel; shorter ones are scored against the latents like single tokens


class LatentAttention(Mixer):
    """params: hidden_size, heads, dim (unrotated query/key size per head), rot_dim (rotated size), vdim, kv_rank,
    q_rank, scale, window (0: none), sink (bool), norm_eps, names (optional overrides).

    c_q = RMSnorm(W_dq h); q = W_uq c_q, head by head [dim | rot_dim].  W_dkv h = [kv_rank latent, RMS-normed ->
    c | rot_dim rotated key part].  The position encoding turns neighbouring pairs of the rotated parts of q and k.
    score = (q_plain . W_uk c + q_rot . k_rot) * scale; softmax over the visible keys (and the sink); value W_uv c."""

    NAMES = {"q_down": "dq", "q_norm": "dq.norm", "q_up": "uq", "kv_down": "dkv", "kv_norm": "dkv.norm", "k_up": "uk",
             "v_up": "uv", "sink": "sink", "out": "o"}

    def __init__(self, spec, runtime, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.heads = int(p["hidden_size"]), int(p["heads"])
        self.dim, self.rot_dim, self.vdim = int(p["dim"]), int(p["rot_dim"]), int(p["vdim"])
        self.kv_rank, self.q_rank = int(p["kv_rank"]), int(p["q_rank"])
        self.scale = float(p["scale"])
        self.window = int(p.get("window", 0) or 0)
        self.has_sink = bool(p.get("sink", False))
        self.eps = float(p["norm_eps"])
        self.names = {**self.NAMES, **dict(p.get("names", {}))}
        self.position = position
        rotated = getattr(position, "rotary_dim", 0) if position is not None else 0
        if rotated > self.rot_dim:
            raise ValueError(f"latent attention '{self.prefix}': the rotation covers {rotated} values, the rotated part has {self.rot_dim}")
        refusal = latent_refusal(self.kv_rank, self.rot_dim)
        if refusal:
            raise ValueError(f"latent attention '{self.prefix}': {refusal}")

    def tensors(self):
        n, px, D, H = self.names, self.prefix, self.hidden, self.heads
        out = [TensorSpec(px + n["q_down"], (self.q_rank, D), MATRIX),
               TensorSpec(px + n["q_norm"], (self.q_rank,), VECTOR, NORM_WEIGHT),
               TensorSpec(px + n["q_up"], (H * (self.dim + self.rot_dim), self.q_rank), MATRIX),
               TensorSpec(px + n["kv_down"], (self.kv_rank + self.rot_dim, D), MATRIX),
               TensorSpec(px + n["kv_norm"], (self.kv_rank,), VECTOR, NORM_WEIGHT),
               TensorSpec(px + n["k_up"], (H * self.dim, self.kv_rank), MATRIX),
               TensorSpec(px + n["v_up"], (H * self.vdim, self.kv_rank), MATRIX),
               TensorSpec(px + n["out"], (D, H * self.vdim), MATRIX)]
        if self.has_sink:
            out.append(TensorSpec(px + n["sink"], (H,), VECTOR))
        return out

    def bind(self, weights):
        n, px, H = self.names, self.prefix, self.heads
        self.w_q_down, self.w_q_up, self.w_kv_down, self.w_out = (weights[px + n[k]] for k in ("q_down", "q_up", "kv_down", "out"))
        self.q_norm_w = weights[px + n["q_norm"]].to(torch.float32).contiguous()
        self.kv_norm_w = weights[px + n["kv_norm"]].to(torch.float32).contiguous()
        self.w_k_up_flat, self.w_v_up_flat = weights[px + n["k_up"]], weights[px + n["v_up"]]
        self.w_k_up = weights[px + n["k_up"]].view(H, self.dim, self.kv_rank)                    # q_plain @ this: W_uk^T q
        self.w_v_up_t = weights[px + n["v_up"]].view(H, self.vdim, self.kv_rank).transpose(1, 2)   # latent @ this: W_uv c
        self.sink = weights[px + n["sink"]].to(torch.float32).contiguous() if self.has_sink else None

    def kernel_modules(self):
        mods = ["attention_latent", "elementwise", "rope_kv", *linear_modules(self.runtime.dtype)]
        if ops.latent_prefill_fits(self.runtime.dtype, self.dim, self.rot_dim, self.vdim, self.kv_rank):
            mods.append("attention_latent_mma")
        return tuple(mods)

    def kv_spec(self):
        return KVSpec(1, self.kv_rank + self.rot_dim, self.window, values=False)

    def _per_head(self, a, b):
        """Batched over heads: a [H, T, n] @ b [H, n, m] -> float32 [H, T, m] (a library product, 32-bit sums)."""
        if a.dtype == torch.bfloat16:
            return torch.bmm(a, b, out_dtype=torch.float32)
        _check_true_fp32()
        return torch.bmm(a, b)

    def forward(self, x, ctx, cache):
        dtype, H, T = self.runtime.dtype, self.heads, x.shape[0]
        cq = ops.rmsnorm(linear(x, self.w_q_down), self.q_norm_w, self.eps, dtype)
        q = linear(cq, self.w_q_up)
        dkv = linear(x, self.w_kv_down)
        cos = sin = None
        if self.position is not None:
            cos, sin = self.position.prepare(ctx)
        table = ctx.page_tables[cache.group_id]
        if (ctx.all_start and ctx.max_new >= PROMPT_KERNEL_MIN_TOKENS
                and ops.latent_prefill_fits(dtype, self.dim, self.rot_dim, self.vdim, self.kv_rank)):
            # whole prompts: keys and values per head from the prompt's own latents (two library products with bfloat16
            # results), then the usual attention on the tensor cores
            q_heads, rows = ops.latent_prep(q, dkv, self.kv_norm_w, cos, sin, ctx, table, cache.k_pool, H, self.dim,
                                            self.rot_dim, self.kv_rank, self.eps, store=cache.writable, whole_heads=True)
            c = rows[:, :self.kv_rank]
            att = ops.latent_prefill(q_heads, torch.mm(c, self.w_k_up_flat.t()), rows, torch.mm(c, self.w_v_up_flat.t()), ctx,
                                     self.sink, self.scale, self.window, H, self.dim, self.rot_dim, self.vdim)
            return linear(att, self.w_out)
        q_plain, q_rot = ops.latent_prep(q, dkv, self.kv_norm_w, cos, sin, ctx, table, cache.k_pool, H, self.dim,
                                         self.rot_dim, self.kv_rank, self.eps, store=cache.writable)
        q_abs = self._per_head(q_plain, self.w_k_up)
        latent = ops.latent_attention(q_abs, q_rot, cache.k_pool, table, ctx, self.sink, self.scale, self.window)
        values = self._per_head(latent, self.w_v_up_t)                                             # [H, T, vdim]
        att = torch.empty((T, H, self.vdim), dtype=dtype, device=x.device)
        att.copy_(values.permute(1, 0, 2))
        return linear(att.view(T, H * self.vdim), self.w_out)


register_mixer("latent_attention", LatentAttention)
