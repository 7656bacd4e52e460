"""Kudazen through the library's own cache, step function and generation loop on a CPU (the kernels' meaning restated
in torch, tests/emulated_ops.py), against the plain implementation: what is tested here is the host side, i.e. the
configuration, the layer schedule with shared weights, the cache and state records, the cutting of work into steps."""

import copy
import json

import pytest
import torch

import kudazen_cases as cases
from conftest import random_tokens
from emulated_ops import EmulatedOps
from helpers import assert_close, run_ragged_batches, run_tail_by_one, run_whole
from plain import kudazen_plain as plain
from starter_b200.cache import KVGroup, StateGroup
from starter_b200.config import ConfigError, config_from_dict, load_config
from starter_b200.engine import Engine
from starter_b200.engine.session import Session


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: cases.write_folder(name, tmp_path_factory.mktemp(f"kudazen_{name}"), dtype=torch.float32) for name in cases.CASES}


def session(folder, **kw):
    args = dict(dtype="float32", device="cpu", ops=EmulatedOps(), max_tokens=64 * 12, max_seqs=4)
    args.update(kw)
    return Session(folder, **args)


def test_configuration_round_trip_and_schedule(folders):
    cfg = load_config(folders["A"])
    assert cfg.architecture == "Kudazen" and config_from_dict(cfg.to_dict()) == cfg
    spec = cfg.model_spec()
    assert spec.schedule == (0, 1, 2, 1, 2, 3) and len(spec.layers) == 4 and spec.residual_float32
    assert spec.layers[3].ff is None and spec.layers[0].ff.limit == 2.0 and spec.layers[1].ff.limit == 1.0
    names = cfg.tensor_names()
    assert names.layers[3]["mixer"]["dq_norm"] == "l5.mix.dq.norm" and "ff" not in names.layers[3]


def test_decay_rank_comes_from_the_tensor_shape(folders, tmp_path):
    raw = json.loads((folders["C"] / "config.json").read_text())
    del raw["layers"][0]["mixer"]["decay_rank"]
    (tmp_path / "config.json").write_text(json.dumps(raw))
    (tmp_path / "model.safetensors").write_bytes((folders["C"] / "model.safetensors").read_bytes())
    sess = session(tmp_path)
    assert sess.model.blocks[0].mixer.spec.decay_rank == 5
    seqs = random_tokens(97, (9,), seed=1)
    assert_close(run_whole(sess, seqs), cases.plain_logits(folders["C"], seqs, "float32"), "float32", "rank from shape")


@pytest.mark.parametrize("change, what", [
    (lambda r: r["layers"][0].update(type="conv"), "unknown"),
    (lambda r: r["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda r: r["layers"][3].update(weights_of=0), "another type"),
    (lambda r: r["layers"][2]["mixer"].update(kv_heads=4), "evenly"),
    (lambda r: r["norm"].update(groups=5), "groups"),
    (lambda r: r["layers"][0]["mlp"].update(kind="experts"), "dense"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=10), "rotat"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=3), "rotat"),
])
def test_bad_configurations_are_refused(change, what):
    raw = copy.deepcopy(cases.CASES["A"])
    change(raw)
    with pytest.raises(ConfigError, match=what):
        config_from_dict(raw)


def test_each_layer_run_has_a_cache_or_state_of_its_own(folders):
    sess = session(folders["A"])
    layers = sess.cache.layers
    assert len(layers) == 6
    assert isinstance(layers[1].group, StateGroup) and layers[1].group is layers[3].group and layers[1].index != layers[3].index
    assert isinstance(layers[2].group, KVGroup) and layers[2].group is layers[4].group and layers[2].index != layers[4].index
    assert layers[2].group.ring_pages > 0 and layers[0].group.ring_pages == 0    # a chunked layer keeps a ring of pages
    assert layers[0].group.v is None and layers[0].group.request.head_dim == 56 + 8   # one row per token: latent | rotated part
    assert layers[2].group.v.shape[-1] == 24 and layers[2].group.k.shape[-1] == 16


@pytest.mark.parametrize("name", list(cases.CASES))
def test_every_cutting_matches_plain(folders, name):
    folder = folders[name]
    seqs = random_tokens(cases.CASES[name]["vocab"], (5, 90, 41, 1, 64, 65, 2), seed=3)
    ref = cases.plain_logits(folder, seqs, "float32")
    sess = session(folder, max_step_tokens=24, max_rows=50)     # prompts go through in portions of 24 tokens at most
    assert_close(run_whole(sess, seqs), ref, "float32", "alone and whole")
    assert_close(run_whole(sess, seqs[:3], together=True), ref[:3], "float32", "one ragged step")
    assert_close(run_tail_by_one(sess, seqs, tail=30), ref, "float32", "tail one by one")
    assert_close(run_ragged_batches(sess, seqs, batch_size=3, poison=True), ref, "float32", "ragged batches, freed pages poisoned")
    assert sess.cache.slots.n_held == 0


def test_portions_down_to_two_tokens(folders):
    seqs = random_tokens(211, (37,), seed=4)
    ref = cases.plain_logits(folders["A"], seqs, "float32")
    for portion in (2, 3, 7, 20, 21):
        sess = session(folders["A"], max_step_tokens=portion)
        assert_close(run_whole(sess, seqs), ref, "float32", f"portions of {portion}")


def test_state_of_a_freed_slot_does_not_leak(folders):
    """A slot that held a long sequence is used again: the recurrence and the blend start from zeros."""
    sess = session(folders["B"], max_seqs=1)
    seqs = random_tokens(300, (70, 9), seed=5)
    ref = cases.plain_logits(folders["B"], seqs, "float32")
    assert_close(run_whole(sess, seqs), ref, "float32", "second sequence in the first one's slot")


def test_greedy_generation_through_the_entry_point(folders):
    cfg, tensors = plain.read_folder(folders["C"])
    prompts = random_tokens(97, (3, 11, 1), seed=6)
    want = plain.generate(cfg, tensors, prompts, 12, "float32")
    engine = Engine.from_session(session(folders["C"]), use_graphs=False)
    assert engine.generate_all(prompts, 12) == want
    assert engine.session.cache.slots.n_held == 0


def test_random_weights_from_the_command_line(tmp_path):
    from starter_b200.cli import main
    (tmp_path / "config.json").write_text(json.dumps(cases.CASES["C"]))
    assert main(["random-weights", "--config", str(tmp_path / "config.json"), "--seed", "3", "--out", str(tmp_path / "model")]) == 0
    sess = session(tmp_path / "model")
    assert sess.model.spec.vocab_size == 97 and len(sess.model.blocks) == 3
    seqs = random_tokens(97, (12,), seed=8)
    assert_close(run_whole(sess, seqs), cases.plain_logits(tmp_path / "model", seqs, "float32"), "float32", "folder from the command line")


def test_replay_sizes_its_cache_for_whole_pages():
    from starter_b200.engine.replay import cache_room
    tokens, slots = cache_room(1728, 128)
    assert slots == 128 and tokens >= 1728 + 128 * 63        # every live request may leave a page all but empty
    assert cache_room(5, 128) == (5 + 5 * 63, 5)              # never more requests than tokens
