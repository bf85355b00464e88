"""Rizitar without a GPU: configuration, weight rules, cache plan, and the plain
implementation's own pieces checked by hand."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import plain_rizitar as plain
from ayaka_b200.cache.storage import plan_cache
from ayaka_b200.config.rizitar import RizitarConfig
from ayaka_b200.errors import AyakaError
from ayaka_b200.models import build_model
from ayaka_b200.models.rizitar import DEFAULT_DECAY_RANK, RIZITAR
from ayaka_b200.parts.pooled_attention import blended_frequencies
from ayaka_b200.weights.loader import TensorSource, load_into
from ayaka_b200.weights.random_init import random_state
from rizitar_cases import (LOUD, TINY_A, TINY_B, TINY_C, TINY_D, attention, delta, dense, layer,
                           model, moe)


@pytest.mark.parametrize("config", [TINY_A, TINY_B, TINY_C, TINY_D])
def test_a_configuration_reads_back_as_itself(config):
    parsed = RizitarConfig.from_json_dict(config)
    again = RizitarConfig.from_json_dict(parsed.to_json_dict())
    assert again == parsed
    assert len(parsed.layers) == len(config["layers"])


def test_keys_that_may_be_left_out():
    parsed = RizitarConfig.from_json_dict(TINY_B)
    assert parsed.embedding_scale == 1.0 and parsed.side_dim == 0
    no_window = parsed.layers[1]
    assert (no_window.window, no_window.pool, no_window.rot) == (0, 0, None)
    assert parsed.layers[3].pool == 0 and parsed.layers[3].window == 7
    assert parsed.layers[4].rot.factor == 1.0
    bare = {"type": "attention", "mixer": {"heads": 2, "dim": 8, "scale": 0.5}, "mlp": None}
    only = RizitarConfig.from_json_dict(model(10, 16, 1e-5, [bare])).layers[0]
    assert (only.kv_heads, only.vdim, only.window) == (2, 8, 0)


@pytest.mark.parametrize("spoil", [
    lambda c: c["layers"][0]["mixer"].pop("scale"),
    lambda c: c["layers"][0]["mixer"].update(kv_heads=3),
    lambda c: c["layers"][0]["mixer"].update(vdim=24),
    lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7),
    lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18),
    lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("slow"),
    lambda c: c["layers"][1].update(type="attention_with_a_hat"),
    lambda c: c["layers"][1]["mlp"]["router"].update(top=7),
    lambda c: c["layers"][3]["mlp"].update(kind="sparse"),
    lambda c: c["norm"].update(eps=0.0),
    lambda c: c.pop("width"),
])
def test_what_is_refused(spoil):
    import copy

    config = copy.deepcopy(TINY_A)
    spoil(config)
    with pytest.raises(AyakaError):
        RizitarConfig.from_json_dict(config)


def test_the_cache_plan_keeps_pooled_rows_beside_the_pages():
    built, _, _ = build_model(TINY_A, "float32", "meta")
    plan = plan_cache(built.spec.order, built.needs())
    needs = built.needs()
    assert needs[0][0].pool == 4 and needs[0][0].window == 0  # every page stays
    assert needs[2][0].pool == 5 and needs[1][0] is None and needs[1][1] is not None
    assert needs[1][1].shape == (2 * 12 * 12,) and needs[3][1].shape == (20 * 20,)
    assert len(plan.groups) == 2
    # a page of 16 tokens holds 4 pooled rows of blocks of 4, and 4 of blocks of 5
    assert plan.bytes_per_page(0, 4, 16) == 2 * (16 + 4) * (16 + 16) * 4
    assert plan.bytes_per_page(1, 4, 16) == 1 * (16 + 4) * (10 + 10) * 4
    # without blocks the window is the cache's again
    built, _, _ = build_model(TINY_B, "float32", "meta")
    needs = built.needs()
    assert (needs[3][0].window, needs[3][0].pool) == (7, 0)
    assert (needs[1][0].window, needs[1][0].pool) == (0, 0)
    assert (needs[4][0].window, needs[4][0].pool) == (0, 11)


@pytest.mark.parametrize("config", [TINY_A, TINY_B])
def test_random_tensors_fill_the_model_exactly(config):
    state = random_state(config, 3, LOUD)
    built, architecture, parsed = build_model(config, "float32", "cpu")
    load_into(built, architecture.weight_rules(parsed), TensorSource(tensors=state))
    stored = sum(t.numel() for name, t in state.items() if name != "side.embed")
    held = sum(p.tensor.numel() for name, p in built.named_params() if "side.table" not in name)
    assert stored == held
    first = built.blocks[0].mixer
    if config is TINY_A:
        assert torch.equal(first.proj_weight[:64], state["l0.mix.q"])
        assert torch.equal(first.proj_weight[64:], state["l0.mix.k"])
        second = built.blocks[1].mixer
        assert torch.equal(second.proj_weight[second.a_at:second.a_at + 24], state["l1.mix.a"])
        assert torch.equal(second.proj_weight[second.low_at:], state["l1.mix.w1"])
        experts = built.blocks[1].feed_forward
        assert torch.equal(experts.in_weight[3 * 24:4 * 24], state["l1.mlp.e3.up"])
        assert torch.equal(built.blocks[2].side.table, state["side.embed"][:, 12:18])


def test_the_decay_rank_comes_from_the_stored_tensor_when_the_file_is_silent():
    config = model(50, 32, 1e-5, [layer(delta(2, 8), dense(16))])
    state = random_state(config, 1, LOUD)
    assert state["l0.mix.w1"].shape == (DEFAULT_DECAY_RANK, 32)
    state["l0.mix.w1"] = state["l0.mix.w1"][:5].clone()
    state["l0.mix.w2"] = state["l0.mix.w2"][:, :5].clone()
    shapes = {name: tuple(t.shape) for name, t in state.items()}
    built, architecture, parsed = build_model(config, "float32", "cpu", shapes.get)
    assert parsed.layers[0].decay_rank == 5
    load_into(built, architecture.weight_rules(parsed), TensorSource(tensors=state))
    assert RIZITAR.config_json(parsed)["layers"][0]["mixer"]["decay_rank"] == 5
    with pytest.raises(AyakaError):
        build_model(config, "float32", "cpu")  # neither the file nor a tensor gives it


def test_the_plain_mask_at_its_edges():
    tokens, blocks = plain.pooled_mask(40, 9, 4)
    assert tokens[20, 20] and tokens[20, 12] and not tokens[20, 11] and not tokens[20, 21]
    # block 2 holds 8..11: seen when 11 <= p - 9
    assert blocks[20, 2] and not blocks[19, 2] and blocks[20, 0] and not blocks[20, 3]
    # position 11 is neither in the window of 21 nor in a seen block of 22's neighbour 23
    assert not tokens[23, 14] and not blocks[23, 3] and blocks[24, 3]
    assert not blocks[:12].any() and blocks.shape == (40, 10)
    tokens, blocks = plain.pooled_mask(10, 0, 4)
    assert tokens[9, 0] and blocks.shape == (10, 0)
    tokens, blocks = plain.pooled_mask(6, 1, 1)
    assert [int(tokens[5].sum()), int(blocks[5].sum())] == [1, 5]


def test_blended_frequencies_are_the_plain_tables():
    for rot in ({"dims": 8, "base": 100.0,
                 "scaling": {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 0.5}},
                {"dims": 16, "base": 500.0}):
        scaling = rot.get("scaling") or {}
        freq, gain = blended_frequencies(rot["dims"], rot["base"], **scaling)
        cos, sin = plain.rotary_tables(np.array([0, 1, 7, 300]), rot)
        want = np.array([0, 1, 7, 300])[:, None] * np.array(freq)[None, :]
        assert np.allclose(cos, np.cos(want) * gain, atol=1e-12)
        assert np.allclose(sin, np.sin(want) * gain, atol=1e-12)
    freq, gain = blended_frequencies(8, 100.0, factor=4.0, original=32, fast=8.0, slow=0.5)
    assert gain == pytest.approx(0.1 * math.log(4.0) + 1.0)
    assert freq[0] == 1.0 and freq[3] == pytest.approx(100.0 ** -0.75 / 4.0)  # kept, slowed
    assert 100.0 ** -0.25 / 4.0 < freq[1] < 100.0 ** -0.25  # between the two


def test_the_plain_pieces_by_hand():
    assert plain.xielu(np.array([2.0]), 0.0, 0.0)[0] == pytest.approx(math.log(2) * 4 + 1)
    assert plain.xielu(np.array([-1.0]), 0.0, 1.0)[0] == pytest.approx(
        (0.5 + math.log1p(math.e)) * (math.exp(-1) - 1 + 1) - 0.5)
    # one head of two channels, one step from a known state
    t = {"r": np.eye(2), "k": np.eye(2), "v": np.eye(2), "g": np.zeros((2, 2)),
         "a": np.zeros((2, 2)), "a.b": np.zeros(2), "w1": np.zeros((1, 2)),
         "w2": np.zeros((2, 1)), "w0": np.zeros(2), "norm": np.ones(2), "o": np.eye(2)}
    state = np.array([[[1.0, 2.0], [3.0, 4.0]]])
    h = np.array([[1.0, 0.0]])
    plain.delta_rule(h, t, "", {"heads": 1, "dim": 2}, 1e-6, state)
    w = math.exp(-math.exp(-0.5) * 0.5)
    u0 = 1.0 / math.sqrt(1.0 + 1e-6)
    # row 0: decayed, minus a u (u^T S) with a = 1/2, plus k v^T; row 1: decayed only
    assert np.allclose(state[0, 0], [w * 1 - 0.5 * u0 * u0 * 1 + 1, w * 2 - 0.5 * u0 * u0 * 2])
    assert np.allclose(state[0, 1], [w * 3, w * 4])
    # the mixture weighs by the softmax over all experts, not over the chosen
    t = {"router": np.array([[2.0], [1.0], [0.0]]), **{
        f"e{e}.up": np.array([[1.0]]) for e in range(3)}, **{
        f"e{e}.down": np.array([[float(e + 1)]]) for e in range(3)}}
    got = plain.mixture(np.array([[1.0]]), t, "", moe(3, 2, 1))
    z = np.exp([2.0, 1.0, 0.0])
    assert got[0, 0] == pytest.approx((z[0] * 1 + z[1] * 2) / z.sum())
