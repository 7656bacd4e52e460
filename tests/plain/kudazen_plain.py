"""Plain, slow Kudazen forward pass: whole sequences, no cache, one function per mechanism.

The oracle of the Kudazen tests.  It shares no code with the package under
test: it reads the model folder through the ``safetensors`` library, walks a
sequence token by token where the design is recurrent, and builds every
attention as a dense [T, T] table.

A Kudazen model is a stack of parallel layers.  With n = grouped RMS norm of
the residual x, a layer does x <- x + (mixer(n) + feed_forward(n)).  Three
mixers exist: attention through a low-rank latent with a sink in the softmax,
a linear recurrence with a matrix state per head and data-dependent decay, and
grouped-query attention inside fixed chunks with a distance penalty.

Two numeric modes: ``"float32"`` rounds nothing; ``"bfloat16"`` rounds the
results of the matrix products and the activations between them to bfloat16,
as a bfloat16 engine may, while norms, scores, softmax weights, angles, the
recurrence and the residual stay in 32-bit.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch
from safetensors import safe_open


def rounder(mode: str):
    if mode == "float32":
        return lambda t: t
    if mode == "bfloat16":
        return lambda t: t.to(torch.bfloat16).to(torch.float32)
    raise ValueError(mode)


def read_folder(folder):
    """config.json as a dict and every tensor of the folder's *.safetensors files, widened to float32."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    tensors = {}
    for path in sorted(folder.glob("*.safetensors")):
        with safe_open(str(path), framework="pt", device="cpu") as f:
            for name in f.keys():
                tensors[name] = f.get_tensor(name).to(torch.float32)
    return cfg, tensors


def owner_of(cfg, i: int) -> int:
    """The layer whose tensors layer i runs with (itself unless it names another)."""
    seen = set()
    while "weights_of" in cfg["layers"][i] and cfg["layers"][i]["weights_of"] is not None:
        if i in seen:
            raise ValueError("weights_of forms a loop")
        seen.add(i)
        i = cfg["layers"][i]["weights_of"]
    return i


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def grouped_rms_norm(x, weight, groups: int, eps: float):
    """The last axis in ``groups`` equal consecutive parts, each brought to unit RMS on its own; then times weight."""
    T, W = x.shape
    parts = x.reshape(T, groups, W // groups)
    return unit_rms(parts, eps).reshape(T, W) * weight


def rotate_pairs(t, positions, base: float, dims: int):
    """Rotary encoding of the first ``dims`` columns of t [T, heads, D], neighbours (2i, 2i+1) forming a pair that
    turns by the angle position * base^(-2i/dims); later columns pass."""
    i = torch.arange(dims // 2, dtype=torch.float32)
    freq = torch.tensor(base, dtype=torch.float32) ** (-2.0 * i / dims)
    angle = positions.to(torch.float32)[:, None] * freq[None, :]          # [T, dims/2], 32-bit
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = t[..., 0:dims:2], t[..., 1:dims:2]
    out = t.clone()
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def latent_attention(h, w, m, eps, rnd):
    """Attention whose queries, keys and values come out of low-rank latents.

    ``w``: the mixer's tensors by short name.  Per head the query is [dim plain | rot_dim rotated]; the key is the
    head's up-projection of the key/value latent beside ONE rotated part that all heads share; the value is the
    head's other up-projection of the same latent.  The softmax has one more term exp(sink_h) in its denominator,
    with no value behind it.
    """
    T = h.shape[0]
    H, D, R, V, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rnd(unit_rms(rnd(h @ w["dq"].T), eps) * w["dq.norm"])
    q = rnd(cq @ w["uq"].T).reshape(T, H, D + R)
    down = rnd(h @ w["dkv"].T)
    latent = rnd(unit_rms(down[:, :rank], eps) * w["dkv.norm"])
    shared = down[:, rank:rank + R].reshape(T, 1, R)
    q_plain, q_rot = q[..., :D], rnd(rotate_pairs(q[..., D:], pos, m["rot"]["base"], m["rot"]["dims"]))
    k_rot = rnd(rotate_pairs(shared, pos, m["rot"]["base"], m["rot"]["dims"]))
    k_plain = rnd(latent @ w["uk"].T).reshape(T, H, D)
    value = rnd(latent @ w["uv"].T).reshape(T, H, V)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot[:, 0])) * m["scale"]
    causal = pos[None, :] <= pos[:, None]
    scores = scores.masked_fill(~causal[None], -math.inf)
    sink = w["sink"].reshape(H, 1, 1)
    top = torch.maximum(scores.max(dim=-1, keepdim=True).values, sink)
    e = torch.exp(scores - top)
    weights = e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink - top))
    out = rnd(torch.einsum("hij,jhv->ihv", weights, value)).reshape(T, H * V)
    return rnd(out @ w["o"].T)


def wkv_mixer(h, w, m, eps, rnd):
    """Linear recurrence with a [dim, dim] state per head, walked token by token.

    Every projection reads its own blend of the token's input and the previous token's (zeros before the first).
    S is the state, indexed [key channel, value channel]:
        out_t = (S + (u * k_t) v_t^T)^T r_t        S <- decay_t[:, None] * S + k_t v_t^T
    with decay_t = exp(-exp(w2 tanh(w1 blend_w) + w0)) per key channel.  Each head's output is brought to unit
    RMS, scaled by a learned vector, gated by silu(g) and projected.
    """
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)

    def blend(name):
        return rnd(h + (before - h) * w["mu." + name])

    r = rnd(blend("r") @ w["r"].T).reshape(T, H, D)
    k = rnd(blend("k") @ w["k"].T).reshape(T, H, D)
    v = rnd(blend("v") @ w["v"].T).reshape(T, H, D)
    g = rnd(blend("g") @ w["g"].T)
    gate = rnd(g * torch.sigmoid(g))
    low = rnd(torch.tanh(rnd(blend("w") @ w["w1"].T)))
    decay = torch.exp(-torch.exp((low @ w["w2"].T) + w["w0"])).reshape(T, H, D)
    u = w["u"].reshape(H, D)
    state = torch.zeros(H, D, D)
    outs = []
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]                         # [H, key, value]
        outs.append(torch.einsum("hk,hkv->hv", r[t], state + u[:, :, None] * kv))
        state = decay[t][:, :, None] * state + kv
    out = unit_rms(torch.stack(outs), eps).reshape(T, H * D)
    out = rnd(rnd(out * w["norm"]) * gate)
    return rnd(out @ w["o"].T)


def chunked_attention(h, w, m, eps, rnd):
    """Grouped-query attention without rotation.  Values are brought to unit RMS per head.  The score of query i
    and key j is (q.k) * scale * temp_h - slope_h * (i - j), slope_h = 2^(-8 (h + 1) / heads); j is visible to i
    when j <= i and both lie in the same block of ``mask.size`` positions counted from the sequence's start."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size = m["mask"]["size"]
    q = rnd(h @ w["q"].T).reshape(T, H, D)
    k = rnd(h @ w["k"].T).reshape(T, G, D).repeat_interleave(H // G, dim=1)
    v = rnd(unit_rms(rnd(h @ w["v"].T).reshape(T, G, V), eps)).repeat_interleave(H // G, dim=1)
    pos = torch.arange(T)
    gap = (pos[:, None] - pos[None, :]).to(torch.float32)
    slopes = torch.tensor([2.0 ** (-8.0 * (i + 1) / H) for i in range(H)], dtype=torch.float32)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"] * w["temp"].reshape(H, 1, 1) - slopes.reshape(H, 1, 1) * gap[None]
    seen = (pos[None, :] <= pos[:, None]) & ((pos[None, :] // size) == (pos[:, None] // size))
    weights = torch.softmax(scores.masked_fill(~seen[None], -math.inf), dim=-1)
    out = rnd(torch.einsum("hij,jhv->ihv", weights, v)).reshape(T, H * V)
    return rnd(out @ w["o"].T)


def feed_forward(h, w, f, rnd):
    """down(g * sigmoid(1.702 g) * (u + 1)) with g = min(gate(h), limit) and u = clamp(up(h), -limit, limit)."""
    limit = f["limit"]
    g = torch.clamp(rnd(h @ w["gate"].T), max=limit)
    u = torch.clamp(rnd(h @ w["up"].T), min=-limit, max=limit)
    return rnd(rnd(g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w["down"].T)


MIXERS = {"latent_attention": latent_attention, "wkv": wkv_mixer, "attention": chunked_attention}


def _sub(tensors, prefix):
    return {name[len(prefix):]: t for name, t in tensors.items() if name.startswith(prefix)}


def forward(cfg, tensors, tokens, mode: str = "float32", trace=None):
    """Logits [T, vocab] of one sequence.  ``trace``: a list that receives the residual after every layer."""
    rnd = rounder(mode)
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    x = tensors["embed"][torch.as_tensor(tokens, dtype=torch.long)].clone()
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{owner_of(cfg, i)}."
        n = rnd(grouped_rms_norm(x, tensors[p + "norm1"], groups, eps))
        branch = MIXERS[layer["type"]](n, _sub(tensors, p + "mix."), layer["mixer"], eps, rnd)
        if layer.get("mlp") is not None:
            branch = branch + feed_forward(n, _sub(tensors, p + "mlp."), layer["mlp"], rnd)
        x = x + branch
        if trace is not None:
            trace.append(x.clone())
    n = rnd(grouped_rms_norm(x, tensors["final.norm"], groups, eps))
    return n @ tensors["embed"].T


def generate(cfg, tensors, prompts, max_new_tokens: int, mode: str = "float32"):
    """Greedy continuation of every prompt, each forward pass over the whole sequence so far."""
    outs = []
    for prompt in prompts:
        seq, new = list(prompt), []
        for _ in range(max_new_tokens):
            tok = int(forward(cfg, tensors, seq, mode)[-1].argmax())
            new.append(tok)
            seq.append(tok)
        outs.append(new)
    return outs


def attend(q, k, v, scale, temp=None, slopes=None, chunk=None, sink=None, first_position=0):
    """Dense attention of queries q [Tq, H, Kd] at positions first_position.. over keys k [T, G, Kd] and values
    v [T, G, Vd] at positions 0..T-1 (T = first_position + Tq), every option of the two attention mixers at once:
    score = q.k * scale * temp_h - slopes_h * (i - j); j visible when j <= i and, with ``chunk``, in i's block;
    ``sink`` adds exp(sink_h) to the denominator."""
    Tq, H, _ = q.shape
    T, G, _ = k.shape
    kk, vv = k.repeat_interleave(H // G, dim=1), v.repeat_interleave(H // G, dim=1)
    i = torch.arange(first_position, first_position + Tq)[:, None]
    j = torch.arange(T)[None, :]
    scores = torch.einsum("ihd,jhd->hij", q, kk) * scale
    if temp is not None:
        scores = scores * temp.reshape(H, 1, 1)
    if slopes is not None:
        scores = scores - slopes.reshape(H, 1, 1) * (i - j).to(torch.float32)[None]
    seen = j <= i
    if chunk is not None:
        seen = seen & ((i // chunk) == (j // chunk))
    scores = scores.masked_fill(~seen[None], -math.inf)
    top = scores.max(dim=-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, sink.reshape(H, 1, 1))
    e = torch.exp(scores - top)
    total = e.sum(dim=-1, keepdim=True)
    if sink is not None:
        total = total + torch.exp(sink.reshape(H, 1, 1) - top)
    return torch.einsum("hij,jhv->ihv", e / total, vv)
