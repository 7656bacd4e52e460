"""Small Nazulorn configurations for the tests, and the plain implementation's logits for them.

The configurations differ from one another in every size and option: one, three and four streams and a plain
residual; fewer key/value heads than query heads, as many, and a single head; maps that turn in part, in full, with
and without stretched frequencies, and not at all; windows of 7, 20 and one page, and none; state heads whose key and
value widths differ, below and above what one block of the recurrence kernel holds; experts with and without identity
outputs and a shared expert, one to four choices; a layer without feed-forward; layers in different orders.
"""

from __future__ import annotations

import copy

import torch

from plain import nazulorn_plain as plain
from starter_b200.config import config_from_dict
from starter_b200.weights import write_model_folder


def _attention(heads, kv_heads, dim, vdim, window=None, dims=None, base=10000.0, scaling=None, diff=0.5):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5, "diff": diff}
    if window is not None:
        m["mask"] = {"size": window}
    if dims is not None:
        m["rot"] = {"base": base, "dims": dims}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "attention", "mixer": m}


def _gla(heads, dim, vdim, tau, rank):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank}}


def _moe(experts, identity, top, scale, ff, limit, shared=None):
    mlp = {"kind": "moe", "router": {"experts": experts, "identity": identity, "top": top, "scale": scale},
           "expert": {"ff": ff, "limit": limit}}
    if shared is not None:
        mlp["shared"] = {"ff": shared[0], "limit": shared[1]}
    return mlp


def _with(entry, mlp):
    entry = copy.deepcopy(entry)
    entry["mlp"] = copy.deepcopy(mlp)
    return entry


def _model(vocab, width, eps, layers, streams=None, mult=1.0, embed=1.0, logit=1.0):
    raw = {"architecture": "Nazulorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embed},
           "residual_mult": mult, "logit_scale": logit, "layers": layers}
    if streams is not None:
        raw["streams"] = streams
    return raw


_A_MOE = _moe(5, 2, 3, 1.7, 40, 0.8, shared=(56, 1.2))
_B_MOE = _moe(4, 0, 1, 1.0, 72, 2.0)
_C_MOE = _moe(2, 3, 4, 0.9, 24, 0.5, shared=(16, 3.0))

CASES = {
    # three streams; maps that turn in part with stretched frequencies, and in full without; windows of 20 and 7; a state
    # head of 24 x 40; a last layer without feed-forward
    "A": _model(211, 96, 1e-5, [
        _with(_attention(6, 2, 16, 24, window=20, dims=8, base=500.0, scaling=(8.0, 16, 4.0, 1.0), diff=0.3), _A_MOE),
        _with(_gla(2, 24, 40, 8.0, 8), _A_MOE),
        _with(_attention(4, 4, 8, 16, window=7, dims=8), _A_MOE),
        _with(_gla(3, 16, 16, 3.0, 5), None)], streams=3, mult=0.4, embed=0.7, logit=1.5),
    # sizes the tensor-core kernels take (maps of 32 and 64 columns, values of 64 and 128, a window of one page), four
    # streams, one chosen expert and no identity outputs, state heads of 64 x 64 and 32 x 128
    "B": _model(300, 128, 1e-6, [
        _with(_gla(2, 64, 64, 16.0, 16), _B_MOE),
        _with(_attention(8, 2, 32, 64, window=64, dims=32, base=2e5, scaling=(6.0, 256, 16.0, 2.0), diff=0.45), _B_MOE),
        _with(_attention(2, 1, 64, 128, window=100, dims=32, diff=0.2), _moe(3, 1, 2, 1.9, 80, 1.1, shared=(96, 0.9))),
        _with(_gla(1, 32, 128, 4.0, 8), _B_MOE)], streams=4, mult=0.3, embed=0.5, logit=2.0),
    # a plain residual (no streams), single heads, widths that are no multiples of 8, no window, nothing turned, a state
    # head of 40 x 72, more choices than real experts
    "C": _model(97, 40, 1e-4, [
        _with(_gla(1, 40, 72, 2.0, 3), _C_MOE),
        _with(_attention(1, 1, 20, 12, diff=0.8), _C_MOE),
        _with(_attention(3, 1, 6, 10, window=33, dims=2), _C_MOE)], mult=0.6),
    # one stream with learned weights
    "D": _model(64, 32, 1e-5, [_with(_gla(2, 8, 8, 1.0, 4), _moe(2, 1, 2, 1.0, 16, 1.0)),
                                _with(_attention(2, 2, 8, 8, window=5, dims=4), None)], streams=1, mult=1.0, embed=2.0),
}
SEEDS = {"A": 15, "B": 16, "C": 17, "D": 18}


def config(name):
    return config_from_dict(copy.deepcopy(CASES[name]))


def write_folder(name, folder, dtype=torch.bfloat16, shards=1):
    return write_model_folder(config(name), SEEDS[name], folder, dtype=dtype, shards=shards)


def plain_logits(folder, seqs):
    cfg, tensors = plain.read_folder(folder)
    return [plain.forward(cfg, tensors, s) for s in seqs]
