"""Linear recurrence with a matrix state per head and a data-dependent decay (kind "wkv").

With n the token's input and n' the previous token's (zeros before a sequence's first token), each of the five
projections reads its own blend n + (n' - n) * mu.  Per head, with S [key channel, value channel]:

    out_t = (S + (u * k_t) v_t^T)^T r_t            S <- decay_t[:, None] * S + k_t v_t^T
    decay_t = exp(-exp(w2 tanh(w1 blend_w) + w0))

and the head's output is divided by its root mean square, scaled, gated by silu(g) and projected.

The state of a sequence is one 32-bit record in the cache's state group: the heads' matrices, then the last
token's input.  It is zero when a sequence starts, and a step of many tokens leaves the same record as the same
tokens one by one: the recurrence kernel walks a sequence's rows in order from the record and writes it back.
"""

from __future__ import annotations

import torch

from ..cache.cache import StateRequest
from .registry import register_part

MIXES = ("r", "k", "v", "g", "w")


class WKV:
    @staticmethod
    def weight_shapes(spec):
        h, inner = spec.hidden_size, spec.num_heads * spec.head_dim
        shapes = {"mu_" + m: (h,) for m in MIXES}
        shapes.update({"r": (inner, h), "k": (inner, h), "v": (inner, h), "g": (inner, h),
                       "w1": (spec.decay_rank, h), "w2": (inner, spec.decay_rank), "w0": (inner,),
                       "u": (spec.num_heads, spec.head_dim), "norm": (inner,), "o": (h, inner)})
        return shapes

    def __init__(self, spec, weights, runtime):
        self.spec = spec
        self.ops = runtime.ops
        self.inner = spec.num_heads * spec.head_dim
        self.mu = torch.stack([weights["mu_" + m] for m in MIXES]).contiguous()
        self.w_in = [self.ops.prepare_matrix(weights[m]) for m in ("r", "k", "v", "g")]
        self.w1 = self.ops.prepare_matrix(weights["w1"])
        self.w2 = self.ops.prepare_matrix(weights["w2"])
        self.w_o = self.ops.prepare_matrix(weights["o"])
        # what enters the recurrence beside the projections is 32-bit
        self.w0 = weights["w0"].float().contiguous()
        self.u = weights["u"].float().reshape(-1).contiguous()
        self.norm = weights["norm"].float().contiguous()
        self.eps = float(spec.norm_eps)
        self.state_floats = spec.num_heads * spec.head_dim * spec.head_dim

    def cache_request(self):
        return StateRequest(shape=(self.state_floats + self.spec.hidden_size,), dtype="float32")

    def prepare(self, cache) -> None:
        pass

    def forward(self, ctx, h, layer_cache):
        ops, s = self.ops, self.spec
        state = layer_cache.state                                   # [slots + 1, matrices | last input]
        blends = ops.token_shift(ctx, h, state, self.state_floats, self.mu)          # [5, rows, hidden]
        r, k, v, g = (ops.linear(blends[i], w) for i, w in enumerate(self.w_in))
        low = ops.tanh(ops.linear(blends[4], self.w1))
        decay_pre = ops.linear(low, self.w2, out_float32=True)      # 32-bit from here on: it goes through two exponentials
        y = ops.wkv_scan(ctx, r, k, v, g, decay_pre, self.w0, self.u, self.norm, self.eps, h, state, s.num_heads,
                         s.head_dim, self.state_floats)
        return ops.linear(y, self.w_o)


register_part("mixer", "wkv", WKV)
