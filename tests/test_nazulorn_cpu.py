"""Nazulorn through the library's own cache, step function and generation loop on a CPU (the kernels' meaning restated
in torch, tests/emulated_ops.py), against the plain implementation: what is tested here is the host side, i.e. the
configuration, the streams, the cache and state records, the cutting of work into steps."""

import copy
import json

import pytest
import torch

import nazulorn_cases as cases
from conftest import random_tokens
from emulated_ops import EmulatedOps
from helpers import assert_close, run_ragged_batches, run_tail_by_one, run_whole
from plain import nazulorn_plain as plain
from starter_b200.cache import KVGroup, StateGroup
from starter_b200.config import ConfigError, config_from_dict, load_config
from starter_b200.engine import Engine
from starter_b200.engine.session import Session


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: cases.write_folder(name, tmp_path_factory.mktemp(f"nazulorn_{name}"), dtype=torch.float32) for name in cases.CASES}


def session(folder, **kw):
    args = dict(dtype="float32", device="cpu", ops=EmulatedOps(), max_tokens=64 * 12, max_seqs=4)
    args.update(kw)
    return Session(folder, **args)


def test_configuration_round_trip_and_parts(folders):
    cfg = load_config(folders["A"])
    assert cfg.architecture == "Nazulorn" and config_from_dict(cfg.to_dict()) == cfg
    spec = cfg.model_spec()
    assert spec.streams == 3 and spec.embedding_scale == 0.7 and spec.logit_scale == 1.5 and not spec.tie_embeddings
    assert [b.mixer.kind for b in spec.layers] == ["diff_attention", "gla", "diff_attention", "gla"]
    assert spec.layers[3].ff is None and spec.layers[0].ff.n_identity == 2 and spec.layers[0].ff.shared.limit == 1.2
    assert spec.layers[0].mixer.position.factor == 8.0 and spec.layers[2].mixer.position.factor is None
    assert spec.layers[0].mixer_norm.mult == 0.4 and spec.layers[0].mixer.window == 20
    names = cfg.tensor_names()
    assert names.layers[1]["mixer"]["a2_bias"] == "l1.mix.a2.b" and names.layers[0]["ff"]["e4_down"] == "l0.mlp.e4.down"
    assert names.layers[2]["mixer_norm"]["mix"] == "l2.hc1.mix" and "ff" not in names.layers[3]
    plain_residual = cases.config("C")
    assert plain_residual.model_spec().streams == 1 and "in" not in plain_residual.tensor_names().layers[0]["mixer_norm"]
    assert plain_residual.model_spec().layers[1].mixer.window is None and plain_residual.model_spec().layers[1].mixer.position is None


def test_decay_rank_comes_from_the_tensor_shape(folders, tmp_path):
    raw = json.loads((folders["C"] / "config.json").read_text())
    del raw["layers"][0]["mixer"]["decay_rank"]
    (tmp_path / "config.json").write_text(json.dumps(raw))
    (tmp_path / "model.safetensors").write_bytes((folders["C"] / "model.safetensors").read_bytes())
    sess = session(tmp_path)
    assert sess.model.blocks[0].mixer.spec.decay_rank == 3
    seqs = random_tokens(97, (9,), seed=1)
    assert_close(run_whole(sess, seqs), cases.plain_logits(folders["C"], seqs), "float32", "rank from shape")


@pytest.mark.parametrize("change, what", [
    (lambda r: r["layers"][0].update(type="conv"), "unknown"),
    (lambda r: r["layers"][0]["mixer"].pop("diff"), "diff"),
    (lambda r: r["layers"][1]["mixer"].pop("tau"), "tau"),
    (lambda r: r["layers"][1]["mixer"].update(tau=0.0), "tau"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=4), "evenly"),
    (lambda r: r["layers"][0]["mlp"].update(kind="dense"), "moe"),
    (lambda r: r["layers"][0]["mlp"]["router"].update(top=9), "chooses"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=18), "rotat"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=3), "rotat"),
    (lambda r: r["layers"][0]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda r: r.update(streams=0), "streams"),
])
def test_bad_configurations_are_refused(change, what):
    raw = copy.deepcopy(cases.CASES["A"])
    change(raw)
    with pytest.raises(ConfigError, match=what):
        config_from_dict(raw)


def test_cache_entries_and_state_records(folders):
    sess = session(folders["A"])
    layers = sess.cache.layers
    assert len(layers) == 4
    assert isinstance(layers[0].group, KVGroup) and isinstance(layers[1].group, StateGroup)
    assert layers[0].group is not layers[2].group and layers[1].group is not layers[3].group    # other sizes, other groups
    g = layers[0].group
    assert g.ring_pages > 0 and g.request.num_kv_heads == 4 and g.v_heads == 2      # a key head per map, the maps share values
    assert g.k.shape[-1] == 16 and g.v.shape[-1] == 24 and g.v.shape[-3] == 2 and g.k.shape[-3] == 4
    assert layers[1].state.shape[-1] == 2 * 24 * 40 and layers[1].state.dtype == torch.float32
    full = session(folders["C"]).cache.layers[1].group
    assert full.ring_pages == 0                                                     # no window: every key stays


@pytest.mark.parametrize("name", list(cases.CASES))
def test_every_cutting_matches_plain(folders, name):
    folder = folders[name]
    seqs = random_tokens(cases.CASES[name]["vocab"], (5, 90, 41, 1, 64, 65, 2), seed=3)
    ref = cases.plain_logits(folder, seqs)
    sess = session(folder, max_step_tokens=24, max_rows=50)     # prompts go through in portions of 24 tokens at most
    assert_close(run_whole(sess, seqs), ref, "float32", "alone and whole")
    assert_close(run_whole(sess, seqs[:3], together=True), ref[:3], "float32", "one ragged step")
    assert_close(run_tail_by_one(sess, seqs, tail=30), ref, "float32", "tail one by one")
    assert_close(run_ragged_batches(sess, seqs, batch_size=3, poison=True), ref, "float32", "ragged batches, freed pages poisoned")
    assert sess.cache.slots.n_held == 0


def test_portions_down_to_two_tokens(folders):
    seqs = random_tokens(211, (37,), seed=4)
    ref = cases.plain_logits(folders["A"], seqs)
    for portion in (2, 3, 7, 20, 21):
        sess = session(folders["A"], max_step_tokens=portion)
        assert_close(run_whole(sess, seqs), ref, "float32", f"portions of {portion}")


def test_state_of_a_freed_slot_does_not_leak(folders):
    """A slot that held a long sequence is used again: the recurrence starts from zeros."""
    sess = session(folders["B"], max_seqs=1)
    seqs = random_tokens(300, (70, 9), seed=5)
    ref = cases.plain_logits(folders["B"], seqs)
    assert_close(run_whole(sess, seqs), ref, "float32", "second sequence in the first one's slot")


def test_layers_match_plain_stream_sums(folders):
    """The sum of the streams after every layer, taken from the library's own residual, beside the plain model's."""
    cfg, tensors = plain.read_folder(folders["A"])
    tokens = random_tokens(211, (19,), seed=9)[0]
    _, want = plain.forward(cfg, tensors, tokens, return_layers=True)
    sess = session(folders["A"])
    seen = []
    for block in sess.model.blocks:
        inner = block.forward

        def spy(ctx, stream, layer_cache, inner=inner):
            inner(ctx, stream, layer_cache)
            snap = stream.x.clone()
            pending = stream.pending
            sess.runtime.ops.stream_norm(snap, stream.streams, pending, None, None, 0.0, torch.float32)
            seen.append(snap.view(snap.shape[0], stream.streams, -1).sum(1))
        block.forward = spy
    run_whole(sess, [tokens])
    for i, (got, ref) in enumerate(zip(seen, want)):
        assert float((got - ref).abs().max()) <= 1e-4 * float(ref.abs().max()), f"layer {i}"


def test_greedy_generation_through_the_entry_point(folders):
    cfg, tensors = plain.read_folder(folders["C"])
    prompts = random_tokens(97, (3, 11, 1), seed=6)
    want = plain.generate(cfg, tensors, prompts, 10)
    engine = Engine.from_session(session(folders["C"]), use_graphs=False)
    assert engine.generate_all(prompts, 10) == want
    assert engine.session.cache.slots.n_held == 0


def test_random_weights_from_the_command_line(tmp_path):
    from starter_b200.cli import main
    (tmp_path / "config.json").write_text(json.dumps(cases.CASES["D"]))
    assert main(["random-weights", "--config", str(tmp_path / "config.json"), "--seed", "3", "--out", str(tmp_path / "model")]) == 0
    sess = session(tmp_path / "model")
    assert sess.model.spec.vocab_size == 64 and len(sess.model.blocks) == 2 and sess.model.spec.streams == 1
    seqs = random_tokens(64, (12,), seed=8)
    assert_close(run_whole(sess, seqs), cases.plain_logits(tmp_path / "model", seqs), "float32", "folder from the command line")
