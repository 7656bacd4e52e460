"""Gated linear attention (kind "gla"): a [head_dim, v_dim] state per head with a decay per key channel.

    q = W_q h / sqrt(head_dim),  k = W_k h,  v = W_v h,  a = sigmoid(W_2 (W_1 h) + b) ** (1 / tau)
    S_t = diag(a_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t
    y = W_o (RMSNorm_head(o) * norm * silu(W_g h))

One product makes q, k, v, the gate and the decay's inner vector; the second small product hands 32-bit numbers to
the recurrence kernel, where the bias, the logarithm of the sigmoid, the division by tau and the exponential are
32-bit, as are the state, the unit norm and the gate.  A sequence's state is one 32-bit record in the cache's state
group, zero when the sequence starts; a step of many tokens leaves the record that the same tokens leave one by one.
"""

from __future__ import annotations

import torch

from ..cache.cache import StateRequest
from .registry import register_part


class GatedLinearAttention:
    @staticmethod
    def weight_shapes(spec):
        h, kd, vd = spec.hidden_size, spec.num_heads * spec.head_dim, spec.num_heads * spec.v_dim
        return {"q": (kd, h), "k": (kd, h), "v": (vd, h), "g": (vd, h), "o": (h, vd), "norm": (spec.v_dim,),
                "a1": (spec.decay_rank, h), "a2": (kd, spec.decay_rank), "a2_bias": (kd,)}

    def __init__(self, spec, weights, runtime):
        if not spec.tau > 0:
            raise ValueError(f"tau must be positive, got {spec.tau}")
        self.spec = spec
        self.ops = runtime.ops
        self.kd, self.vd = spec.num_heads * spec.head_dim, spec.num_heads * spec.v_dim
        self.w_in = self.ops.prepare_matrix(torch.cat([weights[n] for n in ("q", "k", "v", "g", "a1")], dim=0))
        self.w_a2 = self.ops.prepare_matrix(weights["a2"])
        self.w_o = self.ops.prepare_matrix(weights["o"])
        self.bias = weights["a2_bias"].float().contiguous()
        self.norm = weights["norm"].float().contiguous()

    def cache_request(self):
        s = self.spec
        return StateRequest(shape=(s.num_heads * s.head_dim * s.v_dim,), dtype="float32")

    def prepare(self, cache) -> None:
        pass

    def forward(self, ctx, h, layer_cache):
        s, ops, kd, vd = self.spec, self.ops, self.kd, self.vd
        p = ops.linear(h, self.w_in)
        q, k, v, g = p[:, :kd], p[:, kd:2 * kd], p[:, 2 * kd:2 * kd + vd], p[:, 2 * kd + vd:2 * kd + 2 * vd]
        low = p[:, 2 * kd + 2 * vd:].contiguous()     # the products read contiguous rows; this one is decay_rank wide
        z = ops.linear(low, self.w_a2, out_float32=True)
        y = ops.gla_scan(ctx, q, k, v, g, z, self.bias, self.norm, float(s.norm_eps), float(s.tau), float(s.head_dim) ** -0.5,
                         layer_cache.state, s.num_heads, s.head_dim, s.v_dim)
        return ops.linear(y, self.w_o)


register_part("mixer", "gla", GatedLinearAttention)
