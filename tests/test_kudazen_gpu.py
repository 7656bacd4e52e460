"""Kudazen on the GPU against the plain implementation: every mechanism alone, then whole models in every way of
cutting the work, keys at the edges of chunks and pages, a far key among hundreds, the sink, long decoding, and greedy
generation through the entry point."""

import math

import pytest
import torch

import kudazen_cases as cases
from conftest import random_tokens
from helpers import assert_close, make_session, run_ragged_batches, run_tail_by_one, run_whole
from plain import kudazen_plain as plain
from starter_b200.cache import Cache
from starter_b200.config import (BiasedAttentionSpec, GatedMLPSpec, GroupedNormSpec, LatentAttentionSpec, PairRopeSpec, WKVSpec)
from starter_b200.engine import Engine
from starter_b200.engine.context import Runtime, StepContext
from starter_b200.parts import build_part

pytestmark = pytest.mark.gpu
MODES = ["float32", "bfloat16"]
REL = {"float32": 3e-5, "bfloat16": 2.5e-2}


def runtime(mode):
    from starter_b200.csrc.ops import get_ops
    return Runtime(dtype=getattr(torch, mode), device=torch.device("cuda"), ops=get_ops(verbose=False))


def rand(shape, seed, scale=1.0, mean=0.0):
    g = torch.Generator().manual_seed(seed)
    return (mean + torch.randn(shape, generator=g) * scale).to(torch.bfloat16).float()   # bfloat16 numbers, so both modes read the same


def close(got, want, mode, what, rel=None):
    rel = rel or REL[mode]
    scale = float(want.abs().max())
    err = float((got.float().cpu() - want).abs().max())
    assert err <= rel * scale, f"{what}: {err:.3g} > {rel * scale:.3g}"


def context(rt, cache, slots, q_lens):
    for s, n in zip(slots, q_lens):
        cache.reserve(s, cache.lengths_host[s] + n)
    cache.flush()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    row_seq = [b for b, n in enumerate(q_lens) for _ in range(n)]
    return StepContext(runtime=rt, cache=cache, n_seqs=len(slots), n_rows=cu[-1], max_q_len=max(q_lens),
                       kv_bound=max(cache.lengths_host[s] + n for s, n in zip(slots, q_lens)), seq_slot=i32(slots), cu_q=i32(cu),
                       row_seq=i32(row_seq), lengths=cache.lengths, status=torch.zeros(1, dtype=torch.int32, device="cuda"))


def run_mixer(rt, part, h, cuts, max_step_tokens=1024):
    """The mixer over one sequence whose rows h come in pieces of the given sizes; rows of all pieces, in order."""
    cache = Cache([part.cache_request()], n_slots=2, max_tokens=64 * 12, dtype=rt.dtype, device="cuda", max_step_tokens=max_step_tokens)
    part.prepare(cache)
    cache.alloc()                      # the sequence under test sits in the second slot
    slot = cache.alloc()
    outs, at = [], 0
    pieces = [min(cache.step_limit, n - lo) for n in cuts for lo in range(0, n, cache.step_limit)]   # as the step function cuts
    for n in pieces:
        ctx = context(rt, cache, [slot], [n])
        outs.append(part.forward(ctx, h[at:at + n].to(rt.dtype).cuda().contiguous(), cache.layers[0]))
        rt.ops.advance_lengths(ctx)
        cache.advance_host(slot, n)
        assert int(ctx.status.item()) == 0
        at += n
    return torch.cat(outs)


def cuttings(n):
    """Whole; a tail token by token; portions of two; two unequal portions; every token alone."""
    return [[n], [n - 9] + [1] * 9, [2] * (n // 2) + [1] * (n % 2), [n // 3, n - n // 3], [1] * n]


# ---- row-wise kernels --------------------------------------------------------------------------------------

@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("groups, width", [(1, 96), (3, 96), (4, 1032), (2, 2560)])
def test_grouped_norm_with_residual_sum(mode, groups, width):
    rt = runtime(mode)
    w = rand((width,), 1, 0.1, 1.0)
    part = build_part("norm", GroupedNormSpec(size=width, eps=2e-5, groups=groups), {"weight": w.to(rt.dtype).cuda()}, rt)
    x, d1, d2 = rand((7, width), 2, 3.0), rand((7, width), 3), rand((7, width), 4)
    x = x + 1e-4 * rand((7, width), 5)                # a 32-bit residual is no bfloat16 number
    close(part.forward(x.cuda()), plain.grouped_rms_norm(x, w, groups, 2e-5), mode, "norm")
    xx = x.clone().cuda()
    y = part.add_forward(xx, d1.to(rt.dtype).cuda(), d2.to(rt.dtype).cuda())
    assert xx.dtype == torch.float32 and y.dtype == rt.dtype
    close(xx, x + (d1 + d2), mode, "residual sum stays 32-bit", rel=1e-6)
    close(y, plain.grouped_rms_norm(x + d1 + d2, w, groups, 2e-5), mode, "norm after the sum")
    y1 = part.add_forward(xx, d1.to(rt.dtype).cuda())
    close(y1, plain.grouped_rms_norm(x + d1 + d2 + d1, w, groups, 2e-5), mode, "one delta")


@pytest.mark.parametrize("mode", MODES)
def test_feed_forward_with_clamps(mode):
    rt, rnd = runtime(mode), plain.rounder(mode)
    spec = GatedMLPSpec(hidden_size=72, intermediate_size=200, activation="clamped_swish", limit=0.75, alpha=1.702)
    w = {"gate": rand((200, 72), 4, 0.2), "up": rand((200, 72), 5, 0.2), "down": rand((72, 200), 6, 0.1)}
    part = build_part("ff", spec, {k: v.to(rt.dtype).cuda() for k, v in w.items()}, rt)
    for rows in (3, 16, 40):      # few rows: the activation sits in the decode product's epilogue (bfloat16)
        h = rand((rows, 72), 7)
        gate = h @ w["gate"].T
        assert float(gate.max()) > 0.75 and float((h @ w["up"].T).min()) < -0.75       # the clamps bite
        close(part.forward(None, h.to(rt.dtype).cuda()), plain.feed_forward(h, w, {"limit": 0.75}, rnd), mode, f"{rows} rows")


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("rows", [5, 16, 37, 200])      # a warp per column; tiles of 64 rows; the library's batched product (bfloat16)
def test_product_per_head_on_views(mode, rows):
    rt = runtime(mode)
    a, w = rand((rows, 3, 24 + 8), 1), rand((3, 56, 24), 2, 0.2)
    out = torch.full((rows, 3, 56 + 8), 7.0, dtype=rt.dtype, device="cuda")
    rt.ops.linear_heads(a.to(rt.dtype).cuda()[:, :, :24], w.to(rt.dtype).cuda(), out[:, :, :56])
    close(out[:, :, :56], torch.einsum("rhk,hnk->rhn", a[:, :, :24], w), mode, "per-head product")
    assert bool((out[:, :, 56:] == 7.0).all())


# ---- each mixer alone ----------------------------------------------------------------------------------------

def latent_weights(s, seed):
    H, D, R, V = s.num_heads, s.head_dim, s.rot_dim, s.v_dim
    sh = {"dq": (s.q_rank, s.hidden_size), "uq": (H * (D + R), s.q_rank), "dkv": (s.kv_rank + R, s.hidden_size),
          "uk": (H * D, s.kv_rank), "uv": (H * V, s.kv_rank), "o": (s.hidden_size, H * V)}
    w = {k: rand(v, seed + i, v[1] ** -0.5) for i, (k, v) in enumerate(sh.items())}
    w["dq_norm"], w["dkv_norm"] = rand((s.q_rank,), seed + 10, 0.1, 1.0), rand((s.kv_rank,), seed + 11, 0.1, 1.0)
    w["sink"] = rand((H,), seed + 12, 1.0)
    return w


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("sizes", [(3, 24, 8, 40, 48, 56), (4, 64, 16, 64, 96, 128), (1, 20, 4, 12, 44, 36), (16, 128, 64, 128, 160, 512),
                                   (32, 64, 32, 64, 64, 256)])
def test_latent_attention_alone(mode, sizes):
    rt, rnd = runtime(mode), plain.rounder(mode)
    H, D, R, V, qr, kr = sizes
    s = LatentAttentionSpec(hidden_size=80, num_heads=H, head_dim=D, rot_dim=R, v_dim=V, q_rank=qr, kv_rank=kr, scale=(D + R) ** -0.5,
                            norm_eps=1e-5, position=PairRopeSpec(theta=300.0, rotary_dim=R), sink=True)
    w = latent_weights(s, 20)
    part = build_part("mixer", s, {k: v.to(rt.dtype).cuda() for k, v in w.items()}, rt)
    n = 150
    h = rand((n, 80), 3)
    m = {"heads": H, "dim": D, "rot_dim": R, "vdim": V, "kv_rank": kr, "scale": s.scale, "rot": {"base": 300.0, "dims": R}}
    names = {"dq_norm": "dq.norm", "dkv_norm": "dkv.norm"}
    want = plain.latent_attention(h, {names.get(k, k): v for k, v in w.items()}, m, 1e-5, rnd)
    for cuts in cuttings(n):
        close(run_mixer(rt, part, h, cuts), want, mode, f"latent attention, pieces {cuts[:3]}..")


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("H, D, rank", [(2, 24, 8), (4, 32, 16), (1, 40, 5), (2, 64, 32), (1, 128, 16), (1, 160, 8)])
def test_wkv_alone(mode, H, D, rank):
    rt, rnd = runtime(mode), plain.rounder(mode)
    width, inner = 72, H * D
    s = WKVSpec(hidden_size=width, num_heads=H, head_dim=D, decay_rank=rank, norm_eps=1e-5)
    w = {m: rand((inner, width), 30 + i, width ** -0.5) for i, m in enumerate(("r", "k", "v", "g"))}
    w.update({"mu_" + m: rand((width,), 40 + i, 0.2, 0.5) for i, m in enumerate(("r", "k", "v", "g", "w"))})
    w.update(w1=rand((rank, width), 50, width ** -0.5), w2=rand((inner, rank), 51, rank ** -0.5), w0=rand((inner,), 52, 1.0, -1.0),
             u=rand((H, D), 53, 0.3, 0.3), norm=rand((inner,), 54, 0.1, 1.0), o=rand((width, inner), 55, inner ** -0.5))
    part = build_part("mixer", s, {k: v.to(rt.dtype).cuda() for k, v in w.items()}, rt)
    n = 75
    h = rand((n, width), 5)
    want = plain.wkv_mixer(h, {k.replace("mu_", "mu."): v for k, v in w.items()}, {"heads": H, "dim": D}, 1e-5, rnd)
    for cuts in cuttings(n):
        close(run_mixer(rt, part, h, cuts), want, mode, f"wkv, pieces {cuts[:3]}..")


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("H, G, D, V, chunk", [(6, 2, 16, 24, 20), (4, 4, 32, 32, 64), (2, 1, 8, 72, 7), (8, 2, 64, 64, 128)])
def test_biased_attention_alone(mode, H, G, D, V, chunk):
    rt, rnd = runtime(mode), plain.rounder(mode)
    width = 64
    s = BiasedAttentionSpec(hidden_size=width, num_heads=H, num_kv_heads=G, head_dim=D, v_dim=V, scale=D ** -0.5,
                            value_norm_eps=1e-5, head_temperature=True, slope_log2=8.0, chunk=chunk)
    w = {"q": rand((H * D, width), 60, width ** -0.5), "k": rand((G * D, width), 61, width ** -0.5),
         "v": rand((G * V, width), 62, width ** -0.5), "o": rand((width, H * V), 63, (H * V) ** -0.5), "temp": rand((H,), 64, 0.5, 1.5)}
    part = build_part("mixer", s, {k: v.to(rt.dtype).cuda() for k, v in w.items()}, rt)
    n = 200
    h = rand((n, width), 6)
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": s.scale, "mask": {"size": chunk}}
    want = plain.chunked_attention(h, w, m, 1e-5, rnd)
    for cuts in cuttings(n):
        close(run_mixer(rt, part, h, cuts, max_step_tokens=70), want, mode, f"biased attention, pieces {cuts[:3]}..")


# ---- keys at edges, far keys, the sink: inputs made so that one score stands out ---------------------------------

def fill_and_attend(rt, request, k, v, q, first, **options):
    """Keys k [T, G, Kd] (and values v) stored for one sequence, then queries q [Tq, H, Kd] at positions first..:
    in one step when first == 0, else the first ``first`` tokens are stored by an earlier step."""
    cache = Cache([request], n_slots=1, max_tokens=64 * 10, dtype=rt.dtype, device="cuda", max_step_tokens=256)
    slot = cache.alloc()
    T, G = k.shape[0], k.shape[1]
    dev = lambda t: t.to(rt.dtype).cuda().contiguous()
    out = None
    for lo, hi in ((0, first), (first, T)):
        if hi == lo:
            continue
        ctx = context(rt, cache, [slot], [hi - lo])
        if v is None:
            cache.layers[0].k[cache.layers[0].group.table[slot, torch.arange(lo, hi, device="cuda") // 64].long(), 0,
                              torch.arange(lo, hi, device="cuda") % 64] = dev(k[lo:hi, 0])
        else:
            rt.ops.kv_store(ctx, dev(k[lo:hi].reshape(hi - lo, -1)), dev(v[lo:hi].reshape(hi - lo, -1)), cache.layers[0])
        if lo == first:
            out = rt.ops.flex_attention(ctx, dev(q), cache.layers[0], **options)
        rt.ops.advance_lengths(ctx)
        cache.advance_host(slot, hi - lo)
    return out.float().cpu()


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("chunk", [48, 64, 100])
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("D, V", [(32, 16), (64, 64)])        # the warp-per-row kernel; the tensor-core kernel (bfloat16)
def test_keys_just_inside_and_just_outside_a_chunk(mode, chunk, decode, D, V):
    """Every key is nearly orthogonal to the query but two: the first key of the query's chunk (visible) and the key
    before it (hidden).  Each carries a value of its own, so a mask that is one position off changes the output wholly."""
    from starter_b200.cache import KVRequest
    rt = runtime(mode)
    T, H, G = 3 * chunk + 4, 4, 2
    k, v = rand((T, G, D), 1, 0.05), rand((T, G, V), 2, 0.1)
    q = rand((T, H, D), 3, 0.05)
    for i in (chunk * 2 + 3, T - 1):                       # queries three positions into their chunk
        edge = (i // chunk) * chunk
        q[i, :, 0] = 8.0
        k[edge, :, 0], k[edge - 1, :, 0] = 10.0, 12.0      # the hidden one would win if it were seen
        v[edge], v[edge - 1] = 1.0, -1.0
    first = T - 1 if decode else 0
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)])
    temp = torch.tensor([1.0, 0.5, 2.0, 1.5])
    got = fill_and_attend(rt, KVRequest(G, D, window=chunk, v_dim=V), k, v, q[first:], first, scale=D ** -0.5, v_dim=V,
                          head_scale=temp.cuda(), slopes=slopes.cuda(), chunk=chunk)
    want = plain.attend(q[first:], k, v, D ** -0.5, temp, slopes, chunk, first_position=first).reshape(T - first, H * V)
    close(got, want, mode, "chunk edges")
    assert float(want[-1].min()) > 0.5                     # the visible edge key dominates the last query


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("H, Kd, Vd", [(3, 40, 32), (16, 80, 64), (32, 144, 128)])   # the warp-per-row kernel; the tensor-core kernel
def test_far_key_and_sink_through_the_latent_cache(mode, decode, H, Kd, Vd):
    """One key 400 positions back (in the cache's first page) matches the last query; all others do not.  With a low
    sink the output is that key's row; with a high sink the same weights are shared with a term that has no value."""
    from starter_b200.cache import KVRequest
    rt = runtime(mode)
    T = 420
    k = rand((T, 1, Kd), 1, 0.05)
    q = rand((T, H, Kd), 2, 0.05)
    k[7, 0, 5], q[T - 1, :, 5] = 12.0, 12.0
    k[7, 0, :4] = torch.tensor([1.0, -2.0, 3.0, -4.0])
    first = T - 1 if decode else 0
    for sink in (torch.full((H,), -30.0), torch.tensor([2.0, 14.4, 20.0] + [0.0] * (H - 3))):
        got = fill_and_attend(rt, KVRequest(1, Kd, v_dim=0), k, None, q[first:], first, scale=0.1, v_dim=Vd, values_in_keys=True,
                              sink=sink.cuda())
        want = plain.attend(q[first:], k, k[:, :, :Vd], 0.1, sink=sink, first_position=first).reshape(T - first, H * Vd)
        close(got, want, mode, f"far key, sink {sink.tolist()}")
    low = plain.attend(q[-1:], k, k[:, :, :Vd], 0.1, sink=torch.full((H,), -30.0), first_position=T - 1)[0]
    assert float((low[:, :4] - k[7, 0, :4]).abs().max()) < 0.05       # the far key is what the last query reads
    assert float(want[-1].reshape(H, Vd)[2, :4].abs().max()) < 0.1 * 4   # a sink of 20 against a score of 14.4 takes nearly all the weight


def test_both_tensor_core_kernels_serve_prompts(monkeypatch):
    """The same prompt through the kernel for prompts (64 rows per block) and, with that one switched off, through the
    16-row kernel: both within rounding of the plain formula, for the latent cache and for chunked keys with a penalty."""
    from starter_b200.cache import KVRequest
    rt = runtime("bfloat16")
    T, H, G, D, V = 300, 8, 2, 64, 128
    k, v, q = rand((T, G, D), 1, 0.5), rand((T, G, V), 2, 0.5), rand((T, H, D), 3, 0.5)
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)])
    temp = rand((H,), 4, 0.3, 1.0)
    want = plain.attend(q, k, v, D ** -0.5, temp, slopes, 96).reshape(T, H * V)
    kl, ql = rand((T, 1, 144), 5, 0.4), rand((T, 16, 144), 6, 0.4)
    sink = rand((16,), 7, 1.0)
    want_latent = plain.attend(ql, kl, kl[:, :, :128], 0.1, sink=sink).reshape(T, 16 * 128)
    for rows in (32, 1 << 30):
        monkeypatch.setattr(rt.ops, "FLEX_PROMPT_MIN_ROWS", rows)
        got = fill_and_attend(rt, KVRequest(G, D, window=96, v_dim=V), k, v, q, 0, scale=D ** -0.5, v_dim=V, head_scale=temp.cuda(),
                              slopes=slopes.cuda(), chunk=96)
        close(got, want, "bfloat16", f"chunked, prompt kernel from {rows} rows")
        got = fill_and_attend(rt, KVRequest(1, 144, v_dim=0), kl, None, ql, 0, scale=0.1, v_dim=128, values_in_keys=True, sink=sink.cuda())
        close(got, want_latent, "bfloat16", f"latent, prompt kernel from {rows} rows")


# ---- whole models ------------------------------------------------------------------------------------------

@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name in cases.CASES:
        out[name, "bfloat16"] = cases.write_folder(name, tmp_path_factory.mktemp(f"kudazen_{name}"))
        out[name, "float32"] = cases.write_folder(name, tmp_path_factory.mktemp(f"kudazen_{name}_wide"), dtype=torch.float32, shards=2)
    return out


@pytest.mark.parametrize("dtype", MODES)
@pytest.mark.parametrize("name", list(cases.CASES))
def test_every_cutting_matches_plain(folders, name, dtype):
    folder = folders[name, dtype]
    seqs = random_tokens(cases.CASES[name]["vocab"], (5, 150, 77, 1, 64, 65, 33, 2), seed=11)
    ref = cases.plain_logits(folder, seqs, dtype)
    sess = make_session(folder, dtype, max_tokens=64 * 12, max_seqs=4, max_step_tokens=48, max_rows=100)
    assert_close(run_whole(sess, seqs), ref, dtype, "alone and whole")
    assert_close(run_whole(sess, seqs[:3], together=True), ref[:3], dtype, "one ragged step")
    assert_close(run_tail_by_one(sess, seqs), ref, dtype, "tail one by one")
    assert_close(run_ragged_batches(sess, seqs, batch_size=3, poison=True), ref, dtype, "ragged batches, freed pages poisoned")
    assert_close(run_whole(sess, seqs[:2]), ref[:2], dtype, "whole again, in poisoned slots")
    assert sess.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", MODES)
def test_batch_against_each_alone_and_long_decoding(folders, dtype):
    """Unequal requests in one batch give what each gives alone (to rounding), through 150 decoded tokens that cross
    pages and many chunks."""
    folder = folders["B", dtype]
    seqs = random_tokens(300, (170, 152, 230), seed=12)
    sess = make_session(folder, dtype, max_tokens=64 * 16, max_seqs=4)
    alone = run_tail_by_one(sess, seqs, tail=150)
    together = run_ragged_batches(sess, seqs, batch_size=3, prefix_fraction=0.1)
    assert_close(together, alone, dtype, "batch against alone")
    assert_close(alone, cases.plain_logits(folder, seqs, dtype), dtype, "long decoding")


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", MODES)
def test_greedy_generation_through_the_entry_point(folders, dtype, graphs):
    folder = folders["A", dtype]
    cfg, tensors = plain.read_folder(folder)
    prompts = random_tokens(211, (3, 30, 1, 70), seed=13)
    want = plain.generate(cfg, tensors, prompts, 10, dtype)
    engine = Engine(folder, dtype=dtype, max_batch=4, max_context=128, use_graphs=graphs)
    got = engine.generate_all(prompts, 10)
    for b, (g_seq, w_seq) in enumerate(zip(got, want)):
        seq = list(prompts[b])
        for tok, ref_tok in zip(g_seq, w_seq):
            if tok != ref_tok:      # a near-tie may flip: the chosen token must be close to the maximum, and the rest follows it
                logits = plain.forward(cfg, tensors, seq, dtype)[-1]
                assert float(logits.max() - logits[tok]) <= (1e-4 if dtype == "float32" else 3e-2) * float(logits.abs().max())
                break
            seq.append(tok)
    assert engine.session.cache.slots.n_held == 0


def test_replay_of_a_trace_through_the_command(folders, tmp_path):
    """bin/trace_run on a Kudazen folder: requests alone and whole, a batch of unequal requests that is then decoded
    together (the shorter ones end earlier), logits only where they are wanted."""
    import json
    import subprocess
    import sys
    from pathlib import Path
    import numpy as np
    root = Path(__file__).resolve().parent.parent
    folder, vocab = folders["A", "bfloat16"], 211
    seqs = random_tokens(vocab, (70, 9, 131), seed=14)
    ref = cases.plain_logits(folder, seqs, "bfloat16")
    steps = [{"step": i, "entries": [{"id": f"w{i}", "tokens": s, "want": [0, len(s) - 1]}], "end": [f"w{i}"]} for i, s in enumerate(seqs)]
    cut = [len(s) - 6 for s in seqs]
    cut[1] = 1
    steps.append({"step": 3, "entries": [{"id": f"b{i}", "tokens": s[:cut[i]], "want": [cut[i] - 1]} for i, s in enumerate(seqs)], "end": []})
    expect = {3: [(i, cut[i] - 1) for i in range(3)]}
    for t in range(8):
        live = [i for i in range(3) if cut[i] + t < len(seqs[i])]
        steps.append({"step": 4 + t, "entries": [{"id": f"b{i}", "tokens": [seqs[i][cut[i] + t]], "want": [0] if t % 2 == 0 else []} for i in live],
                      "end": [f"b{i}" for i in live if cut[i] + t + 1 == len(seqs[i])]})
        if t % 2 == 0:
            expect[4 + t] = [(i, cut[i] + t) for i in live]
    text = "".join(json.dumps(st) + "\n" for st in steps)
    proc = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", "bfloat16", "--out",
                           str(tmp_path), "--max-tokens", str(sum(len(s) for s in seqs))], input=text, capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [w for st in steps for w in ("done", str(st["step"]))]
    scale = max(float(r.abs().max()) for r in ref)

    def read(step):
        return torch.from_numpy(np.fromfile(tmp_path / f"{step}.f32", dtype="<f4").reshape(-1, vocab).copy())
    for i, r in enumerate(ref):
        got = read(i)
        assert got.shape[0] == 2 and float((got - r[[0, len(r) - 1]]).abs().max()) <= 2e-2 * scale
    for step, rows in expect.items():
        got = read(step)
        assert got.shape[0] == len(rows)
        for j, (i, pos) in enumerate(rows):
            assert float((got[j] - ref[i][pos]).abs().max()) <= 2e-2 * scale, f"step {step}, request {i}, position {pos}"
    assert not (tmp_path / "5.f32").exists()
