"""What a forward pass hands to every part: the run's kernels and the step's batch.

The reference passes ``pos[B]`` and fixed shapes (B, T) to its kernels
(engine/kernels/rope.py:43, engine/kernels/attention.py:41); here a step is a
ragged batch, described once on the device and read by every kernel:

* ``seq_slot[B]``: the cache slot of each sequence of the step;
* ``cu_q[B+1]``: first row of each sequence among the step's rows;
* ``row_seq[M]``: the sequence of each row;
* ``lengths[slot]``: tokens the sequence held before this step, so that row r of
  sequence b stands at position ``lengths[seq_slot[b]] + r - cu_q[b]``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Sequence

import torch


@dataclass
class Runtime:
    """Dtype, device and kernels of a run.  ``ops`` is the loaded CUDA extension's call table."""

    dtype: torch.dtype
    device: torch.device
    ops: Any

    @property
    def is_bf16(self) -> bool:
        return self.dtype == torch.bfloat16


@dataclass
class StepContext:
    runtime: Runtime
    cache: Any
    n_seqs: int
    n_rows: int
    max_q_len: int          # host-side bound on a sequence's rows in this step
    kv_bound: int           # host-side bound on any sequence's length after this step
    seq_slot: torch.Tensor  # int32 [n_seqs]
    cu_q: torch.Tensor      # int32 [n_seqs + 1]
    row_seq: torch.Tensor   # int32 [n_rows]
    lengths: torch.Tensor   # int32 [n_slots + 1], the cache's
    status: torch.Tensor    # int32 [1], kernels raise bits here instead of faulting
    scratch: Dict[str, Any] = field(default_factory=dict)
    uneven: bool = False    # host-side hint: the longest sequence is several times the mean (see lengths_uneven)

    @property
    def ops(self):
        return self.runtime.ops

    @property
    def is_decode(self) -> bool:
        return self.max_q_len == 1


def lengths_uneven(lengths: Sequence[int], page: int = 64) -> bool:
    """Whether a batch's sequences are of very unequal length: the longest holds more than three times the mean
    number of cache pages.  Kernels that hand each sequence's keys to a block of its own then wait for the longest
    one, and one that shares all pages out evenly is the better choice (the call table decides)."""
    if len(lengths) < 2:
        return False
    pages = [int(n) // page + 1 for n in lengths]
    return max(pages) * len(pages) > 3 * sum(pages)


class ResidualStream:
    """The residual x [rows, hidden] and a branch output not yet added to it.

    The sum x + pending is taken in 32-bit inside the kernel that also norms it
    (the reference's add_rms_norm, engine/kernels/add_rmsnorm.py:16-29), so a
    branch's output meets the residual in the same pass that feeds the next branch.
    A branch whose last product can add to x itself is given the stream as the
    place to add to (``ops.linear(..., add_to=stream)``) and pushes nothing.
    """

    def __init__(self, x: torch.Tensor):
        self.x = x
        self.pending = None
        self.stats = None   # left by a product that added its result to x itself: what a norm folded into the next product reads

    def normed(self, norm) -> torch.Tensor:
        if self.pending is None:
            return norm.forward(self.x)
        delta, self.pending = self.pending, None
        self.stats = None   # x changes here
        if isinstance(delta, tuple):   # a layer whose branches run side by side left more than one output
            return norm.add_forward(self.x, *delta)
        return norm.add_forward(self.x, delta)

    def push(self, branch_output: torch.Tensor, *more: torch.Tensor) -> None:
        """Leave a branch's output to be added by the next norm; several outputs (branches that read the same
        normed rows) wait together and need a norm whose ``add_forward`` takes them all."""
        if self.pending is not None:
            raise RuntimeError("a branch output is already waiting to be added to the residual")
        self.pending = (branch_output, *more) if more else branch_output

    def at_rows(self, ops, rows: torch.Tensor) -> "ResidualStream":
        """The stream of the given rows only (what the output head needs): x and whatever waits, gathered."""
        out = ResidualStream(ops.gather_rows(self.x, rows))
        if self.pending is not None:
            deltas = self.pending if isinstance(self.pending, tuple) else (self.pending,)
            out.push(*(ops.gather_rows(d, rows) for d in deltas))
        return out


_ONES: Dict[Any, torch.Tensor] = {}


class StreamResidual:
    """A residual kept in ``streams`` 32-bit copies side by side, x [rows, streams * hidden].  A branch's output y
    returns as X'_t = sum_s mix[s, t] X_s + out[t] * y; the return waits here (``pending`` = (y, mix, out)) and is
    taken by the kernel of the next read, which blends the streams with the reader's weights and norms the blend."""

    def __init__(self, x: torch.Tensor, streams: int):
        self.x = x
        self.streams = int(streams)
        self.pending = None

    def read(self, ops, read_w, weight, eps, dtype) -> torch.Tensor:
        pending, self.pending = self.pending, None
        return ops.stream_norm(self.x, self.streams, pending, read_w, weight, eps, dtype)

    def push_return(self, y, mix, out) -> None:
        if self.pending is not None:
            raise RuntimeError("a branch output is already waiting to return to the streams")
        self.pending = (y, mix, out)

    def normed(self, norm) -> torch.Tensor:
        """The norm of the sum of the streams (what the output head reads)."""
        key = (self.x.device, self.streams)
        ones = _ONES.get(key)
        if ones is None:   # kept: a step makes no tensor it does not need
            ones = _ONES[key] = torch.ones(self.streams, dtype=torch.float32, device=self.x.device)
        return self.read(norm.ops, ones, norm.weight, norm.eps, norm.dtype)

    def at_rows(self, ops, rows: torch.Tensor) -> "StreamResidual":
        out = StreamResidual(ops.gather_rows(self.x, rows), self.streams)
        if self.pending is not None:
            y, mix, o = self.pending
            out.push_return(ops.gather_rows(y, rows), mix, o)
        return out
