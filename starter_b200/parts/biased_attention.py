"""Causal grouped-query attention with options on the score and the mask (kind "biased_attention").

Beside the plain part (kind "attention": per-head norm of q and k, rotary positions, a window) this one takes keys
and values of different widths and, each only when its spec names it: a unit norm of every head's value before it
is cached, a learned number per query head on the scaled score, a penalty slope_h * (i - j) on the distance of
query i and key j, and a mask that shows a query only the keys of its own block of ``chunk`` positions (blocks
counted from the sequence's start, wherever a prompt was cut).  Positions enter through the penalty and the mask
only; nothing is rotated.

A chunked or windowed layer asks the cache for a ring of pages: a query never looks back further than one chunk
(or window), so older pages are written over.
"""

from __future__ import annotations

import torch

from ..cache.cache import KVRequest
from .registry import register_part


class BiasedAttention:
    @staticmethod
    def weight_shapes(spec):
        H, G, D, V, h = spec.num_heads, spec.num_kv_heads, spec.head_dim, spec.v_dim, spec.hidden_size
        shapes = {"q": (H * D, h), "k": (G * D, h), "v": (G * V, h), "o": (h, H * V)}
        if spec.head_temperature:
            shapes["temp"] = (H,)
        return shapes

    def __init__(self, spec, weights, runtime):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} query heads cannot share {spec.num_kv_heads} key/value heads evenly")
        for name in ("chunk", "window"):
            value = getattr(spec, name)
            if value is not None and value < 1:
                raise ValueError(f"{name} must be a positive number of positions, got {value}")
        self.spec = spec
        self.ops = runtime.ops
        self.w_qkv = self.ops.prepare_matrix(torch.cat([weights["q"], weights["k"], weights["v"]], dim=0))
        self.w_o = self.ops.prepare_matrix(weights["o"])
        self.temp = weights["temp"].float().contiguous() if spec.head_temperature else None
        self.slopes = None
        if spec.slope_log2 is not None:
            H = spec.num_heads
            self.slopes = torch.tensor([2.0 ** (-float(spec.slope_log2) * (i + 1) / H) for i in range(H)],
                                       dtype=torch.float32, device=runtime.device)
        self.scale = float(spec.scale)

    def _reach(self):
        """How far back a query may look, in positions (None: to the sequence's start)."""
        reach = [r for r in (self.spec.chunk, self.spec.window) if r is not None]
        return min(reach) if reach else None

    def cache_request(self):
        s = self.spec
        return KVRequest(num_kv_heads=s.num_kv_heads, head_dim=s.head_dim, window=self._reach(), v_dim=s.v_dim)

    def prepare(self, cache) -> None:
        pass

    def forward(self, ctx, h, layer_cache):
        s, ops = self.spec, self.ops
        H, G, D, V = s.num_heads, s.num_kv_heads, s.head_dim, s.v_dim
        rows = h.shape[0]
        qkv = ops.linear(h, self.w_qkv)
        ops.kv_store(ctx, qkv[:, H * D:(H + G) * D], qkv[:, (H + G) * D:], layer_cache, s.value_norm_eps)
        q = qkv[:, :H * D].view(rows, H, D)
        a = ops.flex_attention(ctx, q, layer_cache, self.scale, v_dim=V, head_scale=self.temp, slopes=self.slopes,
                               chunk=s.chunk, window=s.window)
        return ops.linear(a, self.w_o)


register_part("mixer", "biased_attention", BiasedAttention)
