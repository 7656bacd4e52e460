"""Small Kudazen configurations for the tests, and the plain implementation's logits for them.

The configurations differ from one another in every size and option: key and value widths that differ, fewer
key/value heads than query heads, one, three and four norm groups, chunk sizes that are and are not multiples of the
cache's page, head sizes that are not multiples of 32 or 8, a layer without feed-forward, layers that run with
another layer's weights (each with a cache or state of its own).
"""

from __future__ import annotations

import copy

import torch

from plain import kudazen_plain as plain
from starter_b200.config import config_from_dict
from starter_b200.weights import write_model_folder


def _latent(heads, dim, rot, vdim, q_rank, kv_rank, base=10000.0, dims=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                      "scale": (dim + rot) ** -0.5, "rot": {"base": base, "dims": dims or rot}}}


def _wkv(heads, dim, rank):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank}}


def _attention(heads, kv_heads, dim, vdim, chunk):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                           "scale": dim ** -0.5, "mask": {"size": chunk}}}


def _with(entry, ff=None, limit=2.0, weights_of=None):
    entry = copy.deepcopy(entry)
    entry["mlp"] = {"kind": "dense", "ff": ff, "limit": limit} if ff else None
    if weights_of is not None:
        entry["weights_of"] = weights_of
    return entry


def _model(vocab, width, groups, eps, layers):
    return {"architecture": "Kudazen", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups}, "layers": layers}


_A_LATENT, _A_WKV, _A_ATT = _latent(3, 24, 8, 40, 48, 56), _wkv(2, 24, 8), _attention(6, 2, 16, 24, 20)
_B_ATT, _B_LATENT, _B_WKV = _attention(4, 4, 32, 32, 64), _latent(2, 32, 16, 32, 32, 64, base=500.0), _wkv(4, 32, 16)
_C_LATENT, _C_WKV, _C_ATT = _latent(1, 20, 4, 12, 44, 36), _wkv(1, 40, 5), _attention(2, 1, 8, 72, 7)

CASES = {
    # every mixer, two of them run twice on shared weights, one layer without feed-forward, three norm groups
    "A": _model(211, 96, 3, 1e-5, [_with(_A_LATENT, ff=72), _with(_A_WKV, ff=136, limit=1.0), _with(_A_ATT, ff=80),
                                   _with(_A_WKV, ff=136, limit=1.0, weights_of=1), _with(_A_ATT, ff=80, weights_of=2),
                                   _with(_latent(2, 16, 8, 16, 24, 32, dims=4))]),   # half of the rotated part turns
    # sizes the tensor-core kernels take (head sizes 32 and 64, chunk = one page), one norm group, another layer order
    "B": _model(300, 128, 1, 1e-6, [_with(_B_ATT, ff=200), _with(_B_LATENT, ff=200), _with(_B_WKV, ff=200),
                                    _with(_B_LATENT, ff=200, weights_of=1), _with(_B_ATT, ff=200, weights_of=0)]),
    # single heads, widths that are no multiples of 8, a chunk of 7 positions, four groups
    "C": _model(97, 40, 4, 1e-4, [_with(_C_WKV, ff=24, limit=0.5), _with(_C_ATT, ff=24), _with(_C_LATENT, ff=52, limit=3.0)]),
}
SEEDS = {"A": 5, "B": 6, "C": 7}


def config(name):
    return config_from_dict(copy.deepcopy(CASES[name]))


def write_folder(name, folder, dtype=torch.bfloat16, shards=1):
    return write_model_folder(config(name), SEEDS[name], folder, dtype=dtype, shards=shards)


def plain_logits(folder, seqs, dtype):
    cfg, tensors = plain.read_folder(folder)
    return [plain.forward(cfg, tensors, s, dtype) for s in seqs]
