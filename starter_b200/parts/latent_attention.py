"""Causal attention through low-rank latents (kind "latent_attention").

What is cached per token is one row [latent | rotated part] of kv_rank + rot_dim columns, shared by all heads; a
head's plain key W_uk[h] c and its value W_uv[h] c are never formed for cached tokens.  Instead the head's query is
carried into the latent's space and the head's output is taken there:

    q'[h] = W_uk[h]^T q_plain[h]                       score = (q'[h] . c + q_rot[h] . k_rot) * scale
    o'[h] = sum_j weight_j c_j                         o[h]  = W_uv[h] o'[h]

which is the same sum in another order: every head then reads the one cached row per key, in prompts and in decoding
alike, and a prompt may come in any number of pieces.  The softmax may hold a sink: one more term exp(s_h) in the
denominator, with no key and no value.

A step that is ONE sequence's first (nothing cached before it: a whole prompt, or a prompt's first portion) may also
take the narrow form: the step's own keys [W_uk[h] c | k_rot] and values W_uv[h] c are formed once, laid into pages of
a scratch cache that the part keeps, and attended there with heads of head_dim + rot_dim and v_dim columns instead of
kv_rank + rot_dim and kv_rank: a third of the arithmetic per (query, key) pair at usual sizes.  The step's rows go
into the real cache all the same, for the steps that follow.

Steps: one product for both down-projections; one kernel that norms the query latent, norms the key/value latent,
rotates the shared part and writes the cache row; the query's up-projection; its rotated part and, per head, its
plain part times W_uk[h] into [rows, heads, kv_rank + rot_dim]; attention over the cached rows with the row's first
kv_rank columns as values; per head times W_uv[h]; the output projection.
"""

from __future__ import annotations

import dataclasses
from types import SimpleNamespace

import torch

from ..cache.cache import PAGE, KVGroup, KVRequest, LayerCache
from .registry import build_part, register_part

NARROW_MIN_ROWS = 64   # a first step of fewer rows stays on the one path that serves every step


class LatentAttention:
    @staticmethod
    def weight_shapes(spec):
        h, H, D, R, V = spec.hidden_size, spec.num_heads, spec.head_dim, spec.rot_dim, spec.v_dim
        shapes = {"dq": (spec.q_rank, h), "dq_norm": (spec.q_rank,), "uq": (H * (D + R), spec.q_rank),
                  "dkv": (spec.kv_rank + R, h), "dkv_norm": (spec.kv_rank,), "uk": (H * D, spec.kv_rank),
                  "uv": (H * V, spec.kv_rank), "o": (h, H * V)}
        if spec.sink:
            shapes["sink"] = (H,)
        return shapes

    def __init__(self, spec, weights, runtime):
        self.spec = spec
        self.ops = runtime.ops
        H, D, R, V = spec.num_heads, spec.head_dim, spec.rot_dim, spec.v_dim
        if spec.position is not None and spec.position.rotary_dim > R:
            raise ValueError(f"the rotated part has {R} columns, the position encoding wants {spec.position.rotary_dim}")
        self.position = build_part("position", spec.position, {}, runtime) if spec.position is not None else None
        if self.position is not None and not hasattr(self.position, "frequencies"):
            raise ValueError("latent attention rotates with a position part that offers 32-bit ``frequencies``")
        self.w_down = self.ops.prepare_matrix(torch.cat([weights["dq"], weights["dkv"]], dim=0))
        self.w_uq = self.ops.prepare_matrix(weights["uq"])
        self.w_o = self.ops.prepare_matrix(weights["o"])
        # per head [kv_rank, head_dim]: the matrix that carries a plain query into the latent's space
        self.w_absorb = weights["uk"].view(H, D, spec.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = weights["uv"].view(H, V, spec.kv_rank).contiguous()
        self.w_uk_rows = self.ops.prepare_matrix(weights["uk"])      # [heads * head_dim, kv_rank]: the narrow form's keys
        self.w_uv_rows = self.ops.prepare_matrix(weights["uv"])
        self._scratch = None                                         # (scratch cache of the narrow form, its batch description)
        self.q_norm = weights["dq_norm"]
        self.kv_norm = weights["dkv_norm"]
        self.sink = weights["sink"].float().contiguous() if spec.sink else None
        self.scale = float(spec.scale)
        self.eps = float(spec.norm_eps)

    def cache_request(self):
        return KVRequest(num_kv_heads=1, head_dim=self.spec.kv_rank + self.spec.rot_dim, window=None, v_dim=0)

    def prepare(self, cache) -> None:
        if self.position is not None:
            self.position.prepare(cache.max_seq_tokens)

    def _scratch_cache(self, ctx, rows):
        """Pages for ``rows`` tokens of one sequence with a key and a value per head, page j of the sequence = page j,
        and the step described as that sequence starting at position 0."""
        s = self.spec
        pages = -(-rows // PAGE)
        if self._scratch is None or self._scratch[0].group.pool_pages < pages:
            group = KVGroup(KVRequest(s.num_heads, s.head_dim + s.rot_dim, None, s.v_dim), [0], 1, pages, pages, rows,
                            ctx.runtime.dtype, ctx.runtime.device)
            group.table[0] = torch.arange(pages, dtype=torch.int32, device=group.table.device)
            zeros = torch.zeros(2, dtype=torch.int32, device=group.table.device)
            self._scratch = (LayerCache(group, 0), zeros)
        layer, zeros = self._scratch
        alone = dataclasses.replace(ctx, cache=SimpleNamespace(null_slot=1), seq_slot=zeros[:1], lengths=zeros, scratch={})
        return layer, alone

    def _narrow(self, ctx, cq, kept, rows, freqs, rot):
        s, ops = self.spec, self.ops
        H, D, R, V, rank = s.num_heads, s.head_dim, s.rot_dim, s.v_dim, s.kv_rank
        q = ops.linear(cq, self.w_uq).view(rows, H, D + R)
        ops.rotate_pairs(ctx, q[:, :, D:], q[:, :, D:], freqs, rot)          # in place: a pair is read and written by one thread
        latent = kept[:, :rank].contiguous()
        keys = torch.empty((rows, H, D + R), dtype=q.dtype, device=q.device)
        keys[:, :, :D] = ops.linear(latent, self.w_uk_rows).view(rows, H, D)
        keys[:, :, D:] = kept[:, None, rank:]
        values = ops.linear(latent, self.w_uv_rows)
        layer, alone = self._scratch_cache(ctx, rows)
        ops.kv_store(alone, keys.view(rows, H * (D + R)), values, layer)
        o = ops.flex_attention(alone, q, layer, self.scale, v_dim=V, sink=self.sink)
        return ops.linear(o, self.w_o)

    def forward(self, ctx, h, layer_cache):
        s, ops = self.spec, self.ops
        H, D, R, rank = s.num_heads, s.head_dim, s.rot_dim, s.kv_rank
        rows = h.shape[0]
        freqs = self.position.frequencies if self.position is not None else None
        rot = self.position.rotary_dim if self.position is not None else 0
        down = ops.linear(h, self.w_down)
        if ctx.n_seqs == 1 and ctx.kv_bound == rows and rows >= NARROW_MIN_ROWS:   # one sequence's first step
            cq, kept = ops.latent_prepare(ctx, down, layer_cache, s.q_rank, rank, R, self.q_norm, self.kv_norm, self.eps, freqs,
                                          rot, rows_too=True)
            return self._narrow(ctx, cq, kept, rows, freqs, rot)
        cq = ops.latent_prepare(ctx, down, layer_cache, s.q_rank, rank, R, self.q_norm, self.kv_norm, self.eps, freqs, rot)
        q = ops.linear(cq, self.w_uq).view(rows, H, D + R)
        q_latent = torch.empty((rows, H, rank + R), dtype=q.dtype, device=q.device)
        ops.linear_heads(q[:, :, :D], self.w_absorb, q_latent[:, :, :rank])
        ops.rotate_pairs(ctx, q[:, :, D:], q_latent[:, :, rank:], freqs, rot)
        o_latent = ops.flex_attention(ctx, q_latent, layer_cache, self.scale, v_dim=rank, values_in_keys=True, sink=self.sink)
        o = torch.empty((rows, H, s.v_dim), dtype=q.dtype, device=q.device)
        ops.linear_heads(o_latent.view(rows, H, rank), self.w_uv, o)
        return ops.linear(o.view(rows, H * s.v_dim), self.w_o)


register_part("mixer", "latent_attention", LatentAttention)
