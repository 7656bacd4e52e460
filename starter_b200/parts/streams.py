"""A residual kept in several 32-bit copies ("streams"), and the layer over it (kinds "stream_rmsnorm", "streams").

With X_1 .. X_S the streams (all equal to the embedding output at the start), a branch reads

    n = RMSNorm(sum_s in[s] X_s) * weight

and its output y comes back to all streams at once, from the old ones:

    X'_t = sum_s mix[s, t] X_s + mult * out[t] * y.

The return is not taken when the branch ends: it waits on the stream (``StreamResidual.pending``) and is taken by the
kernel of the next read, which also blends and norms, so a layer costs one row kernel per branch.  The sum of the
streams before the final norm is a read with in = 1.  With ``streams`` 0 there is one plain residual, x += mult y.
"""

from __future__ import annotations

import torch

from .registry import build_part, register_part


class StreamRMSNorm:
    @staticmethod
    def weight_shapes(spec):
        shapes = {"weight": (spec.size,)}
        if spec.streams:
            shapes.update({"in": (spec.streams,), "out": (spec.streams,), "mix": (spec.streams, spec.streams)})
        return shapes

    def __init__(self, spec, weights, runtime):
        self.size, self.eps, self.streams = spec.size, float(spec.eps), max(int(spec.streams), 1)
        self.weight = weights["weight"]
        self.ops, self.dtype = runtime.ops, runtime.dtype
        S, dev = self.streams, runtime.device
        if spec.streams:
            self.read_w = weights["in"].float().contiguous()
            self.mix = weights["mix"].float().contiguous()
            self.out = (weights["out"].float() * float(spec.mult)).contiguous()     # mult * out[t], 32-bit
        else:
            self.read_w = torch.ones(S, dtype=torch.float32, device=dev)
            self.mix = torch.ones(S, S, dtype=torch.float32, device=dev)
            self.out = torch.full((S,), float(spec.mult), dtype=torch.float32, device=dev)

    def read(self, stream):
        """The branch's input; takes the waiting return of the branch before first."""
        return stream.read(self.ops, self.read_w, self.weight, self.eps, self.dtype)

    def write(self, stream, y) -> None:
        stream.push_return(y, self.mix, self.out)


class StreamBlock:
    """Kind "streams": the mixer, then the feed-forward when there is one, each through its own stream norm."""

    @staticmethod
    def sub_parts(spec):
        parts = (("mixer_norm", "norm", spec.mixer_norm), ("mixer", "mixer", spec.mixer))
        if spec.ff is not None:
            parts += (("ff_norm", "norm", spec.ff_norm), ("ff", "ff", spec.ff))
        return parts

    def __init__(self, spec, weights, runtime):
        self.ff = None
        for name, category, sub in self.sub_parts(spec):
            setattr(self, name, build_part(category, sub, weights[name], runtime))

    def cache_request(self):
        return self.mixer.cache_request()

    def prepare(self, cache) -> None:
        self.mixer.prepare(cache)
        if self.ff is not None:
            self.ff.prepare(cache)

    def forward(self, ctx, stream, layer_cache) -> None:
        self.mixer_norm.write(stream, self.mixer.forward(ctx, self.mixer_norm.read(stream), layer_cache))
        if self.ff is not None:
            self.ff_norm.write(stream, self.ff.forward(ctx, self.ff_norm.read(stream)))


register_part("norm", "stream_rmsnorm", StreamRMSNorm)
register_part("block", "streams", StreamBlock)
