"""Plain, slow Nazulorn forward pass: whole sequences, no cache, one function per mechanism.

The oracle of the Nazulorn tests.  It shares no code with the package under test: it reads a model folder through
the ``safetensors`` library, walks a sequence token by token where the design is recurrent, builds every attention
as a dense [T, T] table and runs every expert of a token in a Python loop.

A Nazulorn model keeps ``streams`` copies X_1 .. X_S of the residual.  A sublayer (mixer or feed-forward) reads the
blend u = sum_s a_s X_s through an RMS norm, and its output y comes back as X'_t = sum_s M[s, t] X_s + m c_t y.
Mixers: two-map ("differential") sliding-window attention with partly rotated heads, and gated linear attention with
a matrix state per head.  The feed-forward is a mixture of experts with identity experts and a shared expert.

Everything here is 32-bit.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch
from safetensors import safe_open

SWISH_ALPHA = 1.702


def read_folder(folder):
    """config.json as a dict and every tensor of the folder's *.safetensors files (floats widened to float32)."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    tensors = {}
    for path in sorted(folder.glob("*.safetensors")):
        with safe_open(str(path), framework="pt", device="cpu") as f:
            for name in f.keys():
                t = f.get_tensor(name)
                tensors[name] = t.to(torch.float32) if t.is_floating_point() else t
    return cfg, tensors


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return unit_rms(x, eps) * weight


# ---- positions ---------------------------------------------------------------------------


def rotary_frequencies(rot):
    """(f [dims / 2], magnitude) of a ``rot`` entry {base, dims, scaling or nothing}.  With scaling {factor, original,
    fast, slow}: the pair index at which a wavelength of ``original / t`` positions sits is
    d(t) = dims ln(original / (2 pi t)) / (2 ln base); pairs below d(fast) keep their frequency, pairs above d(slow) are
    slowed by ``factor``, a linear ramp in between; cosines and sines grow by 0.1 ln(factor) + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f.to(torch.float32), 1.0

    def pair_at(t):
        return dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_at(sc["fast"])), 0)
    hi = min(math.ceil(pair_at(sc["slow"])), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    f = f / sc["factor"] * ramp + f * (1.0 - ramp)
    return f.to(torch.float32), 0.1 * math.log(sc["factor"]) + 1.0


def rotate_half(t, positions, rot):
    """t [T, n, D]: the first rot.dims columns of every head turn, column i paired with column i + dims/2."""
    if not rot:
        return t
    dims = int(rot["dims"])
    f, mag = rotary_frequencies(rot)
    angle = positions.to(torch.float32)[:, None] * f[None, :]                  # 32-bit
    c, s = (torch.cos(angle) * mag)[:, None, :], (torch.sin(angle) * mag)[:, None, :]
    a, b = t[..., :dims // 2], t[..., dims // 2:dims]
    return torch.cat([a * c - b * s, b * c + a * s, t[..., dims:]], dim=-1)


# ---- mixers ------------------------------------------------------------------------------


def window_mask(T: int, size):
    """[T, T] True where key j is visible to query i: 0 <= i - j < size (no size: every earlier key)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if size:
        seen &= (i - j) < int(size)
    return seen


def differential_attention(h, w, m, eps, positions=None):
    """h [T, width]; w: the mixer's tensors by short name; m: the mixer's config entry."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = torch.arange(T) if positions is None else positions
    q = (h @ w["q"].T).reshape(T, H, 2, D)
    k = (h @ w["k"].T).reshape(T, G, 2, D)
    v = (h @ w["v"].T).reshape(T, G, V)
    rot = m.get("rot")
    q = rotate_half(q.reshape(T, H * 2, D), positions, rot).reshape(T, H, 2, D)
    k = rotate_half(k.reshape(T, G * 2, D), positions, rot).reshape(T, G, 2, D)
    seen = window_mask(T, (m.get("mask") or {}).get("size"))
    lam = math.exp(float((w["lq1"] * w["lk1"]).sum())) - math.exp(float((w["lq2"] * w["lk2"]).sum())) + m["diff"]
    out = torch.zeros(T, H, V)
    for head in range(H):
        g = head // (H // G)
        maps = []
        for which in range(2):
            score = (q[:, head, which] @ k[:, g, which].T) * m["scale"]
            score = score.masked_fill(~seen, float("-inf"))
            maps.append(torch.softmax(score, dim=-1) @ v[:, g])
        o = maps[0] - lam * maps[1]
        out[:, head] = unit_rms(o, eps) * (1.0 - m["diff"])
    return out.reshape(T, H * V) @ w["o"].T


def gated_linear_attention(h, w, m, eps, state=None):
    """Token by token: S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T q_t.  Returns (output [T, width], final state
    [heads, dim, vdim])."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ w["k"].T).reshape(T, H, D)
    v = (h @ w["v"].T).reshape(T, H, V)
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / m["tau"]).reshape(T, H, D)
    gate = torch.nn.functional.silu(h @ w["g"].T)
    S = torch.zeros(H, D, V) if state is None else state.clone()
    o = torch.zeros(T, H, V)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = unit_rms(o, eps) * w["norm"]
    return (o.reshape(T, H * V) * gate) @ w["o"].T, S


# ---- feed-forward ------------------------------------------------------------------------


def clamped_expert(h, gate, up, down, limit):
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(SWISH_ALPHA * g) * (u + 1.0)) @ down.T


def route(h, router, correction, r):
    """(chosen [T, top], weights [T, top]) over experts + identity outputs."""
    s = torch.softmax(h @ router.T, dim=-1)
    chosen = torch.topk(s + correction, int(r["top"]), dim=-1).indices
    picked = torch.gather(s, 1, chosen)
    return chosen, picked / (picked.sum(dim=-1, keepdim=True) + 1e-20) * r.get("scale", 1.0)


def expert_mixture(h, w, mlp, choice=None):
    """h [T, width]; w: the feed-forward's tensors by short name ('e3.gate', 'router', 'shared.up', ...).  ``choice``:
    (chosen, weights) to use instead of the router's own."""
    r = mlp["router"]
    E, limit = int(r["experts"]), (mlp.get("expert") or {}).get("limit")
    chosen, weights = route(h, w["router"], w["correction"], r) if choice is None else choice
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t].tolist(), weights[t]):
            if e >= E:                        # an identity expert hands its input back
                out[t] += wt * h[t]
            else:
                out[t] += wt * clamped_expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], limit)[0]
    if mlp.get("shared"):
        out = out + clamped_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"], mlp["shared"]["limit"])
    return out


# ---- streams and the model ---------------------------------------------------------------


def stream_read(X, a):
    """X [S, T, width], a [S] -> the blend a sublayer reads."""
    return torch.einsum("s,stw->tw", a, X)


def stream_write(X, M, c, y, m):
    """All streams at once from the old ones: X'_t = sum_s M[s, t] X_s + m c_t y."""
    return torch.einsum("st,sjw->tjw", M, X) + m * c[:, None, None] * y[None]


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, tokens, return_layers=False):
    """tokens: a list of ids -> logits [T, vocab] (and the sum of the streams after every layer)."""
    eps, m = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = tensors["embed"][tokens] * cfg["embedding"]["scale"]
    S = int(cfg.get("streams") or 0)
    X = x[None].repeat(max(S, 1), 1, 1)
    seen = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        branches = [("1", "mix.", layer)]
        if layer.get("mlp") is not None:
            branches.append(("2", "mlp.", layer))
        for q, part, _ in branches:
            if S:
                u = stream_read(X, tensors[p + f"hc{q}.in"])
            else:
                u = X[0]
            n = rms_norm(u, tensors[p + "norm" + q], eps)
            w = sub(tensors, p + part)
            if part == "mlp.":
                y = expert_mixture(n, w, layer["mlp"])
            elif layer["type"] == "attention":
                y = differential_attention(n, w, layer["mixer"], eps)
            elif layer["type"] == "gla":
                y = gated_linear_attention(n, w, layer["mixer"], eps)[0]
            else:
                raise ValueError(layer["type"])
            if S:
                X = stream_write(X, tensors[p + f"hc{q}.mix"], tensors[p + f"hc{q}.out"], y, m)
            else:
                X = X + m * y
        seen.append(X.sum(dim=0))
    x = X.sum(dim=0)
    logits = (rms_norm(x, tensors["final.norm"], eps) @ tensors["head"].T) * cfg.get("logit_scale", 1.0)
    return (logits, torch.stack(seen)) if return_layers else logits


def generate(cfg, tensors, prompts, n_new):
    """Greedy continuation of every prompt by ``n_new`` tokens: the whole sequence is run again for every token."""
    out = []
    for prompt in prompts:
        seq, new = list(prompt), []
        for _ in range(n_new):
            tok = int(forward(cfg, tensors, seq)[-1].argmax())
            new.append(tok)
            seq.append(tok)
        out.append(new)
    return out
