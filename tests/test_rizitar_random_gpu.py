"""Drawn Rizitar models through drawn schedules: a seed draws every size and constant (widths
that are no multiple of 8, one to six heads in one to three key/value heads, heads rotated
wholly, partly or not at all with plain or blended frequencies, windows from 1 to beyond the
prompt, blocks from 1 to longer than the window, delta layers with one to three heads of 4 to
70 channels, experts of which one to all are chosen, layers without feed-forward, with or
without the token input, the order of the mixers), the requests, the page size, the pool and
every step's cut; the engine must agree with the plain model on every position.
``RIZITAR_RANDOM_SEEDS`` widens the run."""

from __future__ import annotations

import os
import random

import pytest

import engine_support as support
from cases import random_tokens
from rizitar_cases import attention, delta, dense, layer, model, moe, plain_logits
from ayaka_b200.weights.rules import RandomInit

pytestmark = pytest.mark.gpu

SEEDS = range(int(os.environ.get("RIZITAR_RANDOM_SEEDS", "12")))


def draw_mlp(rng: random.Random):
    kind = rng.choice(["none", "dense", "moe", "moe"])
    if kind == "none":
        return None
    if kind == "dense":
        return dense(rng.choice([16, 40, 70, 128]))
    experts = rng.randint(1, 12)
    return moe(experts, rng.randint(1, min(experts, 4)), rng.choice([8, 12, 24, 40]))


def draw_model(rng: random.Random) -> dict:
    width = rng.choice([24, 40, 50, 64, 72, 96, 130])
    layers = []
    for _ in range(rng.randint(1, 5)):
        if rng.random() < 0.6:
            kv_heads = rng.choice([1, 1, 2, 3])
            dim = rng.choice([4, 8, 12, 16, 24, 32])
            window = rng.choice([0, 1, 2, 5, 16, 17, 31, 40, 200])
            pool = rng.choice([None, 0, 1, 2, 3, 7, 12, 16, 20, 64])
            rot = rng.choice([0, 2, dim // 2 - dim // 2 % 2, dim])
            scaling = rng.choice([None, (rng.choice([2.0, 8.0, 32.0]), rng.choice([16, 64, 512]),
                                         rng.choice([4.0, 32.0]), rng.choice([0.5, 1.0, 2.0]))])
            entry = attention(kv_heads * rng.randint(1, 3), kv_heads, dim, window, pool,
                              rot=rot, base=rng.choice([37.0, 1000.0, 10000.0]), scaling=scaling,
                              scale=rng.choice([None, 0.2, 0.5]))
        else:
            entry = delta(rng.randint(1, 3), rng.choice([4, 7, 12, 16, 33, 70]),
                          rng.choice([1, 3, 8, 16]))
        layers.append(layer(entry, draw_mlp(rng)))
    return model(rng.choice([17, 64, 101, 300]), width, rng.choice([1e-5, 1e-6, 1e-3]), layers,
                 embed_scale=rng.choice([None, 1.0, 3.0, 12.0]),
                 # (a token input of one or two entries is left out: its branch is one or two
                 # vectors times as many gates, and the norm behind it blows gates near zero up
                 # to full size, so that the plain model itself moves by 1e-4 under weight
                 # noise of 1e-7)
                 side=rng.choice([None, 3, 4, 10]))


def draw_steps(rng: random.Random, sequences: dict[str, list[int]], pool_tokens: int
               ) -> list[dict]:
    sizes = tuple(rng.choice([1, 1, 2, 2, 3, 5, 8, 15, 16, 17, 31, 33, 64]) for _ in range(9))
    kind = rng.choice(["whole", "tail", "portions", "mixed", "mixed"])
    if kind == "whole":
        return support.schedule_whole(sequences)
    if kind == "tail":
        return support.schedule_tail(sequences, tail=rng.choice([1, 7, 40]))
    if kind == "portions":
        return support.schedule_portions(sequences, sizes=sizes)
    return support.schedule_mixed(sequences, pool_tokens=pool_tokens,
                                  live_limit=rng.choice([2, 3, 4]),
                                  decode_tail=rng.choice([0, 3, 20]), sizes=sizes)


@pytest.mark.parametrize("seed", SEEDS)
def test_a_drawn_model_through_a_drawn_schedule(tmp_path, seed):
    rng = random.Random(3000 + seed)
    config = draw_model(rng)
    init = RandomInit(weight_std=rng.choice([0.08, 0.15]) * (64 / config["width"]) ** 0.5,
                      scale_residual_projections=False, bias_std=rng.choice([0.0, 0.1]),
                      norm_std=0.1)
    lengths = [rng.choice([1, 2, 3, 15, 16, 17, 33, 60, 97, 140]) for _ in range(rng.randint(1, 6))]
    sequences = {f"s{i}": random_tokens(config["vocab"], n, 7 * seed + i)
                 for i, n in enumerate(lengths)}
    page = rng.choice([8, 16, 16, 32])
    pool_tokens = max(-(-n // 64) * 64 for n in lengths) + rng.choice([0, 64, 256])
    steps = draw_steps(rng, sequences, pool_tokens)
    folder, state = support.make_model(tmp_path / "model", config, seed, init, "float32")
    core = support.build_core(folder, "float32",
                              num_blocks=max(pool_tokens // page + 1 + 8 // page, 6),
                              block_size=page, max_running=4,
                              max_tokens_per_step=max(256, page))
    got = support.replay(core, steps)
    expected = plain_logits(state, config, sequences)
    support.assert_logits_close(got, expected, "float32", "rizitar-drawn", page=page)
    assert not core.manager.live_requests()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["attention", "window", "pooled", "delta", "dense", "experts",
                                   "side"])
def test_each_mechanism_alone_in_a_model_of_one_layer(tmp_path, which, dtype):
    """A model that has the one mechanism and as little else as the design allows."""
    mixer = {"attention": attention(4, 2, 16, 0, scale=0.4),
             "window": attention(4, 2, 16, 19, rot=16, base=100.0),
             "pooled": attention(2, 1, 32, 19, 6, rot=8, base=100.0,
                                 scaling=(4.0, 32, 8.0, 1.0)),
             "delta": delta(2, 16, 4)}.get(which, attention(1, 1, 16, 1))
    mlp = {"dense": dense(48), "experts": moe(8, 2, 32)}.get(which)
    config = model(120, 64, 1e-5, [layer(mixer, mlp)], side=8 if which == "side" else None,
                   embed_scale=4.0 if which == "side" else None)
    init = RandomInit(weight_std=0.12, scale_residual_projections=False, bias_std=0.1,
                      norm_std=0.1)
    folder, state = support.make_model(tmp_path / "m", config, 2, init, dtype)
    sequences = {f"r{i}": random_tokens(120, n, 30 + i) for i, n in enumerate((70, 2, 33))}
    expected = plain_logits(state, config, sequences)
    core = support.build_core(folder, dtype, num_blocks=12)
    got = support.replay(core, support.schedule_mixed(sequences, pool_tokens=128))
    if which == "experts" and dtype == "bfloat16":
        from test_rizitar_engine_gpu import assert_mostly_close

        assert_mostly_close(got, expected, "rizitar-one/experts")
    else:
        support.assert_logits_close(got, expected, dtype, f"rizitar-one/{which}")
