"""Nazulorn on the GPU against the plain implementation: every mechanism alone, then whole models in every way of
cutting the work, keys at the edges of windows and pages, a far key among hundreds, long decoding, and greedy
generation through the entry point."""

import math

import pytest
import torch

import nazulorn_cases as cases
from conftest import random_tokens
from helpers import assert_close, make_session, run_ragged_batches, run_tail_by_one, run_whole
from plain import nazulorn_plain as plain
from starter_b200.cache import Cache
from starter_b200.config import (DiffAttentionSpec, GatedMLPSpec, GLASpec, GroupedNormSpec, MoESpec, ScaledHalfRopeSpec,
                                  StreamNormSpec)
from starter_b200.engine import Engine
from starter_b200.engine.context import Runtime, StepContext, StreamResidual
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


def run_mixer(rt, part, h, cuts, max_step_tokens=1024, pages=16):
    """The mixer over one sequence whose rows h come in pieces of the given sizes; rows of all pieces, in order, and the
    cache it ran on."""
    cache = Cache([part.cache_request()], n_slots=2, max_tokens=64 * pages, dtype=rt.dtype, device="cuda", max_step_tokens=max_step_tokens)
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
    return torch.cat(outs), cache, slot


def cuttings(n):
    """Whole; a tail token by token; portions of two; two unequal portions; every token alone."""
    return [[n], [n - 9] + [1] * 9, [2] * (n // 2) + [1] * (n % 2), [n // 3, n - n // 3], [1] * n]


# ---- the streams --------------------------------------------------------------------------------------------

@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("streams, width", [(1, 96), (2, 41), (3, 96), (4, 1032), (8, 2560), (2, 4104)])
def test_stream_read_and_return(mode, streams, width):
    rt = runtime(mode)
    S = streams
    w = {"weight": rand((width,), 1, 0.1, 1.0), "in": rand((S,), 2, 0.5, 0.5), "out": rand((S,), 3, 0.5, 0.5), "mix": rand((S, S), 4, 0.4, 0.3)}
    part = build_part("norm", StreamNormSpec(size=width, eps=2e-5, streams=S, mult=0.4), {k: v.to(rt.dtype).cuda() for k, v in w.items()}, rt)
    X = rand((S, 7, width), 5, 3.0) + 1e-4 * rand((S, 7, width), 6)          # a 32-bit residual is no bfloat16 number
    stream = StreamResidual(X.permute(1, 0, 2).reshape(7, S * width).contiguous().cuda(), S)
    close(part.read(stream), plain.rms_norm(plain.stream_read(X, w["in"]), w["weight"], 2e-5), mode, "read")
    y = rand((7, width), 7)
    part.write(stream, y.to(rt.dtype).cuda())
    X2 = plain.stream_write(X, w["mix"], w["out"], y, 0.4)
    n = part.read(stream)                                                      # takes the waiting return first
    assert stream.x.dtype == torch.float32 and stream.pending is None
    close(stream.x.view(7, S, width).permute(1, 0, 2), X2, mode, "streams after the return stay 32-bit", rel=2e-6)
    close(n, plain.rms_norm(plain.stream_read(X2, w["in"]), w["weight"], 2e-5), mode, "read after the return")
    part.write(stream, y.to(rt.dtype).cuda())
    final = build_part("norm", GroupedNormSpec(size=width, eps=2e-5), {"weight": w["weight"].to(rt.dtype).cuda()}, rt)
    rows = torch.tensor([5, 0], dtype=torch.int32, device="cuda")
    got = stream.at_rows(rt.ops, rows).normed(final)                           # what the output head reads: the sum of the streams
    X3 = plain.stream_write(X2, w["mix"], w["out"], y, 0.4)
    close(got, plain.rms_norm(X3.sum(0), w["weight"], 2e-5)[[5, 0]], mode, "sum of the streams at chosen rows")


def test_plain_residual_is_one_stream_without_weights():
    rt = runtime("float32")
    part = build_part("norm", StreamNormSpec(size=48, eps=1e-5, streams=0, mult=0.6), {"weight": rand((48,), 1, 0.1, 1.0).cuda()}, rt)
    x, y = rand((5, 48), 2, 2.0), rand((5, 48), 3)
    stream = StreamResidual(x.clone().cuda(), 1)
    part.write(stream, y.cuda())
    part.read(stream)
    close(stream.x, x + 0.6 * y, "float32", "x += mult * y", rel=1e-6)


@pytest.mark.parametrize("mode", MODES)
def test_scaled_embedding_in_copies(mode):
    rt = runtime(mode)
    table = rand((50, 72), 1)
    tokens = torch.tensor([3, 49, 0, 3], dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = rt.ops.embed_streams(tokens, table.to(rt.dtype).cuda(), status, 0.37, 3)
    assert out.dtype == torch.float32 and tuple(out.shape) == (4, 216) and int(status.item()) == 0
    want = (table[tokens.long().cpu()] * torch.tensor(0.37)).repeat(1, 3)
    assert torch.equal(out.cpu(), want)
    rt.ops.embed_streams(torch.tensor([50], dtype=torch.int32, device="cuda"), table.to(rt.dtype).cuda(), status, 1.0, 1)
    assert int(status.item()) == 1                                             # a token outside the table raises the bit


# ---- attention with two maps ----------------------------------------------------------------------------------

def diff_spec(H, G, D, V, window, dims, scaling=None, diff=0.5, width=80, base=10000.0):
    pos = None
    if dims:
        sc = scaling or (None, None, None, None)
        pos = ScaledHalfRopeSpec(theta=base, rotary_dim=dims, factor=sc[0], original=sc[1], fast=sc[2], slow=sc[3])
    return DiffAttentionSpec(hidden_size=width, num_heads=H, num_kv_heads=G, head_dim=D, v_dim=V, scale=D ** -0.5, diff=diff,
                             norm_eps=1e-5, window=window, position=pos)


def diff_weights(s, seed):
    H, G, D, V, h = s.num_heads, s.num_kv_heads, s.head_dim, s.v_dim, s.hidden_size
    w = {"q": rand((H * 2 * D, h), seed, h ** -0.5), "k": rand((G * 2 * D, h), seed + 1, h ** -0.5), "v": rand((G * V, h), seed + 2, h ** -0.5),
         "o": rand((h, H * V), seed + 3, (H * V) ** -0.5)}
    for i, n in enumerate(("lq1", "lk1", "lq2", "lk2")):
        w[n] = rand((D,), seed + 4 + i, 0.3)
    return w


def diff_entry(s):
    m = {"heads": s.num_heads, "kv_heads": s.num_kv_heads, "dim": s.head_dim, "vdim": s.v_dim, "scale": s.scale, "diff": s.diff}
    if s.window:
        m["mask"] = {"size": s.window}
    if s.position is not None:
        p = s.position
        m["rot"] = {"base": p.theta, "dims": p.rotary_dim}
        if p.factor is not None:
            m["rot"]["scaling"] = {"factor": p.factor, "original": p.original, "fast": p.fast, "slow": p.slow}
    return m


DIFF_SIZES = [
    dict(H=6, G=2, D=16, V=24, window=20, dims=8, scaling=(8.0, 16.0, 4.0, 1.0), diff=0.3),     # the general kernel
    dict(H=8, G=2, D=32, V=64, window=64, dims=32, scaling=(6.0, 256.0, 16.0, 2.0), diff=0.45),  # the tensor-core kernels, a window of one page
    dict(H=2, G=1, D=64, V=128, window=100, dims=32),                                           # part of a map turns
    dict(H=1, G=1, D=20, V=12, window=None, dims=0, diff=0.8),                                  # no window, nothing turned
    dict(H=8, G=4, D=128, V=128, window=70, dims=128, base=1e6),
    dict(H=3, G=3, D=32, V=64, window=7, dims=16),                                              # three heads per key head: not a size the 16-row kernel takes
]


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("sizes", DIFF_SIZES)
def test_two_map_attention_alone(mode, sizes):
    rt = runtime(mode)
    spec = diff_spec(**sizes)
    w = diff_weights(spec, 20)
    part = build_part("mixer", spec, {k: v.to(rt.dtype).cuda() for k, v in w.items()}, rt)
    n = 150
    h = rand((n, spec.hidden_size), 3)
    want = plain.differential_attention(h, w, diff_entry(spec), 1e-5)
    for cuts in cuttings(n):
        got, _, _ = run_mixer(rt, part, h, cuts, max_step_tokens=48)            # rings of pages wrap; steps of 48 rows at most
        close(got, want, mode, f"cut {cuts[:3]}..")


def test_query_rows_are_reordered_by_key_head_and_map():
    """The cache keeps a key head per (key/value head, map) and one value head per key/value head; the turned keys in it
    are the plain implementation's, at positions beyond the first page too."""
    rt = runtime("float32")
    spec = diff_spec(H=4, G=2, D=16, V=24, window=None, dims=12, scaling=(4.0, 64.0, 8.0, 1.0))
    w = diff_weights(spec, 30)
    part = build_part("mixer", spec, {k: v.cuda() for k, v in w.items()}, rt)
    h = rand((70, 80), 1)
    _, cache, slot = run_mixer(rt, part, h, [70])
    k = plain.rotate_half((h @ w["k"].T).reshape(70, 4, 16), torch.arange(70), diff_entry(spec)["rot"])
    v = (h @ w["v"].T).reshape(70, 2, 24)
    g = cache.layers[0].group
    assert tuple(g.k.shape[2:]) == (4, 64, 16) and tuple(g.v.shape[2:]) == (2, 64, 24)
    for pos in (0, 63, 64, 69):
        page = int(g.table[slot, pos // 64])
        close(g.k[0, page, :, pos % 64], k[pos], "float32", f"keys at {pos}")
        close(g.v[0, page, :, pos % 64], v[pos], "float32", f"values at {pos}", rel=1e-6)


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("window, loud", [(48, 16), (48, 17), (64, 0), (64, 1), (7, 57), (7, 58), (100, 30), (None, 2)])
def test_a_loud_key_at_the_window_edge(mode, window, loud):
    """One token's input is many times larger than the others', so its key takes a map's whole softmax wherever that
    map's score with it is positive: a window that is one position off shows at once.  The queries just inside and just
    outside the window stand at page borders and inside pages, in a prompt and decoded one by one."""
    rt = runtime(mode)
    spec = diff_spec(H=8, G=4, D=32, V=64, window=window, dims=32)
    w = diff_weights(spec, 40)
    part = build_part("mixer", spec, {k: v.to(rt.dtype).cuda() for k, v in w.items()}, rt)
    n = 420 if window is None else loud + window + 12
    h = rand((n, 80), 5)
    h[loud] *= 25.0
    want = plain.differential_attention(h, w, diff_entry(spec), 1e-5)
    edge = n - 1 if window is None else loud + window          # the first query that no longer sees the loud key
    quiet = h.clone()
    quiet[loud] /= 25.0
    base = plain.differential_attention(quiet, w, diff_entry(spec), 1e-5)
    assert float((want[edge - 1] - base[edge - 1]).abs().max()) > 0.05 * float(want.abs().max())     # the loud key matters where seen
    if window is not None:
        assert float((want[edge] - base[edge]).abs().max()) < 1e-4                                   # and not a position later
    for cuts in ([n], [edge - 3] + [1] * (n - edge + 3), [edge] + [n - edge]):
        got, _, _ = run_mixer(rt, part, h, cuts)
        for pos in (edge - 1, edge, n - 1):
            close(got[pos:pos + 1], want[pos:pos + 1], mode, f"window {window}, loud {loud}, cut {cuts[:2]}, position {pos}",
                  rel=REL[mode] * float(want.abs().max()) / float(want[pos].abs().max()))


# ---- gated linear attention -------------------------------------------------------------------------------------

def gla_weights(s, seed):
    h, kd, vd, r = s.hidden_size, s.num_heads * s.head_dim, s.num_heads * s.v_dim, s.decay_rank
    w = {"q": rand((kd, h), seed, h ** -0.5), "k": rand((kd, h), seed + 1, h ** -0.5), "v": rand((vd, h), seed + 2, h ** -0.5),
         "g": rand((vd, h), seed + 3, h ** -0.5), "o": rand((h, vd), seed + 4, vd ** -0.5), "norm": rand((s.v_dim,), seed + 5, 0.1, 1.0),
         "a1": rand((r, h), seed + 6, h ** -0.5), "a2": rand((kd, r), seed + 7, r ** -0.5), "a2_bias": rand((kd,), seed + 8, 1.5, 2.0)}
    return w


GLA_SIZES = [(2, 24, 40, 8.0, 8), (2, 64, 64, 16.0, 16), (1, 32, 128, 4.0, 8), (1, 40, 72, 2.0, 3), (4, 128, 64, 16.0, 16),
             (1, 136, 20, 1.0, 4), (2, 16, 300, 3.0, 8), (3, 8, 8, 0.5, 2)]


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("sizes", GLA_SIZES)
def test_gated_linear_attention_alone(mode, sizes):
    rt = runtime(mode)
    H, D, V, tau, rank = sizes
    spec = GLASpec(hidden_size=72, num_heads=H, head_dim=D, v_dim=V, tau=tau, decay_rank=rank, norm_eps=1e-5)
    w = gla_weights(spec, 50)
    part = build_part("mixer", spec, {k: v.to(rt.dtype).cuda() for k, v in w.items()}, rt)
    n = 75
    h = rand((n, 72), 4)
    named = {**{k: v for k, v in w.items() if k != "a2_bias"}, "a2.b": w["a2_bias"]}
    want, state = plain.gated_linear_attention(h, named, {"heads": H, "dim": D, "vdim": V, "tau": tau}, 1e-5)
    for cuts in cuttings(n):
        got, cache, slot = run_mixer(rt, part, h, cuts)
        close(got, want, mode, f"cut {cuts[:3]}..")
        close(cache.layers[0].state[slot].view(H, D, V), state, mode, f"state after cut {cuts[:3]}..")
        assert cache.layers[0].state.dtype == torch.float32


def test_a_step_of_several_sequences_keeps_their_states_apart():
    rt = runtime("float32")
    spec = GLASpec(hidden_size=72, num_heads=2, head_dim=64, v_dim=64, tau=16.0, decay_rank=16, norm_eps=1e-5)
    w = gla_weights(spec, 60)
    named = {**{k: v for k, v in w.items() if k != "a2_bias"}, "a2.b": w["a2_bias"]}
    part = build_part("mixer", spec, {k: v.cuda() for k, v in w.items()}, rt)
    cache = Cache([part.cache_request()], n_slots=3, max_tokens=64 * 8, dtype=rt.dtype, device="cuda")
    slots = [cache.alloc() for _ in range(3)]
    lens = [40, 3, 17]
    hs = [rand((n + 5, 72), 70 + i) for i, n in enumerate(lens)]
    ctx = context(rt, cache, slots, lens)
    first = part.forward(ctx, torch.cat([h[:n] for h, n in zip(hs, lens)]).cuda(), cache.layers[0])
    rt.ops.advance_lengths(ctx)
    for s, n in zip(slots, lens):
        cache.advance_host(s, n)
    tails = []
    for t in range(5):                                   # then five steps of one token each, in another order of slots
        order = [2, 0, 1]
        ctx = context(rt, cache, [slots[i] for i in order], [1, 1, 1])
        out = part.forward(ctx, torch.stack([hs[i][lens[i] + t] for i in order]).cuda(), cache.layers[0])
        rt.ops.advance_lengths(ctx)
        for i in order:
            cache.advance_host(slots[i], 1)
        tails.append({i: out[j] for j, i in enumerate(order)})
    at = 0
    for i, n in enumerate(lens):
        want, _ = plain.gated_linear_attention(hs[i], named, {"heads": 2, "dim": 64, "vdim": 64, "tau": 16.0}, 1e-5)
        close(first[at:at + n], want[:n], "float32", f"sequence {i} in the ragged step")
        close(torch.stack([tails[t][i] for t in range(5)]), want[n:], "float32", f"sequence {i} decoded")
        at += n


# ---- experts ---------------------------------------------------------------------------------------------------

def moe_spec(width, E, I, top, ff, limit, shared=None, scale=1.7):
    gated = lambda f, lim: GatedMLPSpec(hidden_size=width, intermediate_size=f, activation="clamped_swish", limit=lim, alpha=1.702)
    return MoESpec(hidden_size=width, n_experts=E, n_identity=I, top=top, route_scale=scale, expert=gated(ff, limit),
                   shared=gated(*shared) if shared else None)


def moe_weights(s, seed):
    h, ff = s.hidden_size, s.expert.intermediate_size
    w = {"router": rand((s.n_experts + s.n_identity, h), seed, 3.0 * h ** -0.5), "correction": rand((s.n_experts + s.n_identity,), seed + 1, 0.05)}
    for e in range(s.n_experts):
        w[f"e{e}_gate"], w[f"e{e}_up"] = rand((ff, h), seed + 10 + 3 * e, 2.0 * h ** -0.5), rand((ff, h), seed + 11 + 3 * e, 2.0 * h ** -0.5)
        w[f"e{e}_down"] = rand((h, ff), seed + 12 + 3 * e, ff ** -0.5)
    if s.shared is not None:
        f = s.shared.intermediate_size
        w["shared_gate"], w["shared_up"], w["shared_down"] = rand((f, h), seed + 2, h ** -0.5), rand((f, h), seed + 3, h ** -0.5), rand((h, f), seed + 4, f ** -0.5)
    return w


def moe_plain(s, w, h, choice=None):
    named = {k.replace("_", "."): v for k, v in w.items()}
    mlp = {"router": {"experts": s.n_experts, "identity": s.n_identity, "top": s.top, "scale": s.route_scale},
           "expert": {"limit": s.expert.limit}}
    if s.shared is not None:
        mlp["shared"] = {"limit": s.shared.limit}
    return plain.expert_mixture(h, named, mlp, choice), plain.route(h, named["router"], named["correction"], mlp["router"])


MOE_SIZES = [dict(width=72, E=5, I=2, top=3, ff=40, limit=0.8, shared=(56, 1.2)), dict(width=128, E=4, I=0, top=1, ff=72, limit=2.0),
             dict(width=40, E=2, I=3, top=4, ff=24, limit=0.5, shared=(16, 3.0)), dict(width=64, E=0, I=3, top=2, ff=8, limit=1.0),
             dict(width=256, E=40, I=1, top=8, ff=64, limit=1.0, shared=(96, 1.3)),
             dict(width=36, E=3, I=1, top=2, ff=20, limit=1.0, shared=(12, 1.0))]      # rows that 16-byte reads do not fit


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("sizes", MOE_SIZES)
@pytest.mark.parametrize("rows", [1, 5, 40, 300])     # a few pairs: every pair streams its expert; many (bfloat16): pairs in the order of their experts
def test_experts_alone(mode, sizes, rows):
    rt = runtime(mode)
    spec = moe_spec(**sizes)
    w = moe_weights(spec, 80)
    part = build_part("ff", spec, {k: v.to(rt.dtype).cuda() for k, v in w.items()}, rt)
    h = rand((rows, spec.hidden_size), 9)
    want, (chosen, weights) = moe_plain(spec, w, h)
    assert float((h @ w.get("e0_gate", torch.zeros(1, spec.hidden_size)).T).max()) > spec.expert.limit or spec.n_experts == 0   # the clamp bites
    got_chosen, got_weights = rt.ops.moe_route(h.to(rt.dtype).cuda(), part.router, part.correction, spec.top, spec.route_scale)
    assert torch.equal(got_chosen.long().cpu().sort(dim=1).values, chosen.sort(dim=1).values)      # the inputs are bfloat16 numbers: no close call
    order = torch.argsort(got_chosen.long().cpu(), dim=1), torch.argsort(chosen, dim=1)
    close(torch.gather(got_weights.cpu(), 1, order[0]), torch.gather(weights, 1, order[1]), "float32", "weights", rel=1e-5)
    close(part.forward(None, h.to(rt.dtype).cuda()), want, mode, f"{rows} rows")


def test_router_prefers_the_lowest_index_among_equals_and_honours_the_correction():
    rt = runtime("float32")
    router = torch.zeros(6, 16)
    router[4, 0] = 1.0                                    # output 4 has the largest score ...
    correction = torch.tensor([0.0, 0.0, 0.5, 0.0, 0.0, 0.0])      # ... output 2 the largest choice score
    h = torch.zeros(2, 16)
    h[:, 0] = 1.0
    chosen, weight = rt.ops.moe_route(h.cuda(), router.cuda(), correction.cuda(), 3, 2.0)
    assert chosen.tolist() == [[2, 4, 0]] * 2             # then the score, then the lowest index among equals
    s = torch.softmax(h @ router.T, dim=-1)[0]
    want = s[[2, 4, 0]] / s[[2, 4, 0]].sum() * 2.0        # the weights use the scores without the correction
    close(weight[0], want, "float32", "weights", rel=1e-6)


# ---- whole models ----------------------------------------------------------------------------------------------

@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name in cases.CASES:
        out[name] = cases.write_folder(name, tmp_path_factory.mktemp(f"nazulorn_gpu_{name}"))
    return out


def mostly_close(got, ref, what, share=0.9, rel=3e-2):
    """bfloat16: a chosen expert may differ from the 32-bit choice where two choice scores nearly meet, and the rows
    after it then differ too.  Most rows stay within rounding of the plain result, and no row strays far."""
    scale = max(float(r.abs().max()) for r in ref)
    errs = torch.cat([(g - r).abs().max(dim=1).values for g, r in zip(got, ref)]) / scale
    assert float((errs <= rel).float().mean()) >= share and float(errs.max()) < 0.5, \
        f"{what}: {float((errs <= rel).float().mean()):.2f} of the rows within {rel}, worst {float(errs.max()):.3g}"


@pytest.mark.parametrize("name", list(cases.CASES))
def test_every_cutting_matches_plain_float32(folders, name):
    folder = folders[name]
    seqs = random_tokens(cases.CASES[name]["vocab"], (5, 150, 41, 1, 64, 65, 2), seed=3)
    ref = cases.plain_logits(folder, seqs)
    sess = make_session(folder, "float32", max_tokens=64 * 16, max_seqs=4, max_step_tokens=48, max_rows=100)
    assert_close(run_whole(sess, seqs), ref, "float32", "alone and whole")
    assert_close(run_whole(sess, seqs[:3], together=True), ref[:3], "float32", "one ragged step")
    assert_close(run_tail_by_one(sess, seqs, tail=40), ref, "float32", "tail one by one")
    assert_close(run_ragged_batches(sess, seqs, batch_size=3, poison=True), ref, "float32", "ragged batches, freed pages poisoned")
    assert sess.cache.slots.n_held == 0


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_every_cutting_stays_near_plain_bfloat16(folders, name):
    folder = folders[name]
    seqs = random_tokens(cases.CASES[name]["vocab"], (5, 150, 41, 1, 64, 65, 2), seed=3)
    ref = cases.plain_logits(folder, seqs)
    sess = make_session(folder, "bfloat16", max_tokens=64 * 16, max_seqs=4, max_step_tokens=48, max_rows=100)
    mostly_close(run_whole(sess, seqs), ref, "alone and whole")
    mostly_close(run_tail_by_one(sess, seqs, tail=40), ref, "tail one by one")
    mostly_close(run_ragged_batches(sess, seqs, batch_size=3, poison=True), ref, "ragged batches, freed pages poisoned")


def test_portions_down_to_two_tokens(folders):
    seqs = random_tokens(211, (37,), seed=4)
    ref = cases.plain_logits(folders["A"], seqs)
    for portion in (2, 3, 7, 20, 21):
        sess = make_session(folders["A"], "float32", max_tokens=64 * 4, max_seqs=2, max_step_tokens=portion)
        assert_close(run_whole(sess, seqs), ref, "float32", f"portions of {portion}")


def test_a_batch_against_each_request_alone_through_long_decoding(folders):
    """Three unequal requests decoded together for 150 tokens (windows pass over decoded tokens, rings of pages wrap)
    against the plain model on each alone."""
    seqs = random_tokens(300, (230, 170, 151), seed=7)
    ref = cases.plain_logits(folders["B"], seqs)
    sess = make_session(folders["B"], "float32", max_tokens=64 * 16, max_seqs=3)
    assert_close(run_ragged_batches(sess, seqs, batch_size=3, prefix_fraction=0.3), ref, "float32", "batch of three, decoded together")


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name", ["B", "C"])
def test_greedy_generation_through_the_entry_point(folders, name, graphs):
    cfg, tensors = plain.read_folder(folders[name])
    prompts = random_tokens(cases.CASES[name]["vocab"], (3, 11, 1), seed=6)
    want = plain.generate(cfg, tensors, prompts, 10)
    engine = Engine(folders[name], dtype="float32", max_batch=4, max_context=128, use_graphs=graphs)
    assert engine.generate_all(prompts, 10) == want
    assert engine.session.cache.slots.n_held == 0


def test_captured_decoding_gives_the_tokens_of_eager_decoding_bfloat16(folders):
    prompts = random_tokens(300, (70, 5, 33), seed=8)
    eager = Engine(folders["B"], dtype="bfloat16", max_batch=4, max_context=256, use_graphs=False).generate_all(prompts, 40)
    captured = Engine(folders["B"], dtype="bfloat16", max_batch=4, max_context=256, use_graphs=True).generate_all(prompts, 40)
    assert eager == captured


def test_replay_through_the_trace_runner_and_generation_from_the_command_line(folders, tmp_path):
    """bin/trace_run as a user drives it (a prompt in two portions, then two requests decoded in one batch, logits in
    files), and ``python -m starter_b200 generate`` on the same folder."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    import numpy as np
    root = Path(__file__).resolve().parent.parent
    folder, vocab = folders["A"], 211
    a, b = random_tokens(vocab, (75, 9), seed=12)
    ref = cases.plain_logits(folder, [a, b])
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:40], "want": [0, 39]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[40:70], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": b[:4], "want": [3]}], "end": []}]
    for t in range(5):
        steps.append({"step": 3 + t, "entries": [{"id": "a", "tokens": [a[70 + t]], "want": [0]}, {"id": "b", "tokens": [b[4 + t]], "want": [0]}],
                      "end": ["a", "b"] if t == 4 else []})
    proc = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out",
                           str(tmp_path), "--max-tokens", "256"], input="".join(json.dumps(s) + "\n" for s in steps),
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
    read = lambda n: torch.from_numpy(np.fromfile(tmp_path / f"{n}.f32", dtype="<f4").reshape(-1, vocab).copy())
    tol = 1e-4 * float(ref[0].abs().max())
    assert float((read(0) - ref[0][[0, 39]]).abs().max()) <= tol and not (tmp_path / "1.f32").exists()
    assert float((read(2) - ref[1][[3]]).abs().max()) <= tol
    for t in range(5):
        assert float((read(3 + t) - torch.stack([ref[0][70 + t], ref[1][4 + t]])).abs().max()) <= tol, f"decoded token {t}"
    cfg, tensors = plain.read_folder(folder)
    want = plain.generate(cfg, tensors, [a[:6], b[:3]], 4)
    proc = subprocess.run([sys.executable, "-m", "starter_b200", "generate", "--model", str(folder), "--dtype", "float32", "--input-ids",
                           ",".join(map(str, a[:6])) + ";" + ",".join(map(str, b[:3])), "--max-new-tokens", "4", "--max-batch", "4",
                           "--max-context", "128"],
                          capture_output=True, text=True, timeout=600, cwd=str(root))
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [json.loads(line) for line in proc.stdout.splitlines()] == want
