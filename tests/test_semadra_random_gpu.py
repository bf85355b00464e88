"""Drawn Semadra models through drawn schedules: a seed draws every size and constant (widths
that are no multiple of 8, one to six heads in one to three key/value heads, key and value
sizes of their own, windows from 1 to beyond the prompt, kept stretches shorter and longer
than the window, latents read by later layers with other windows, experts in groups of one
to four, layers without feed-forward, with or without the token input, the order of the
mixers), the requests, the page size, the pool and every step's cut; the engine must agree
with the plain model on every position. ``SEMADRA_RANDOM_SEEDS`` widens the run."""

from __future__ import annotations

import os
import random

import pytest

import engine_support as support
from cases import random_tokens
from semadra_cases import attention, dense, latent, layer, model, moe, plain_logits
from ayaka_b200.weights.rules import RandomInit

pytestmark = pytest.mark.gpu

SEEDS = range(int(os.environ.get("SEMADRA_RANDOM_SEEDS", "12")))


def draw_mlp(rng: random.Random):
    kind = rng.choice(["none", "dense", "moe", "moe"])
    if kind == "none":
        return None
    if kind == "dense":
        return dense(rng.choice([16, 40, 70, 128]))
    groups = rng.choice([1, 1, 2, 3, 4])
    per = rng.randint(1, 4)
    keep = rng.randint(1, groups)
    top = rng.randint(1, min(keep * per, 4))
    return moe(groups * per, top, rng.choice([8, 12, 24, 40]),
               groups=None if groups == 1 and rng.random() < 0.5 else groups,
               keep=keep, scale=rng.choice([1.0, 0.5, 2.5]),
               shared=rng.choice([None, 8, 20, 48]))


def draw_model(rng: random.Random) -> dict:
    width = rng.choice([24, 40, 50, 64, 72, 96, 130])
    layers, owners = [], {}
    for index in range(rng.randint(1, 5)):
        if rng.random() < 0.5:
            kv_heads = rng.choice([1, 1, 2, 3])
            window = rng.choice([0, 1, 2, 5, 16, 17, 31, 40, 200])
            keep = rng.choice([None, 0, 1, 4, 16, 19, 50])
            entry = attention(kv_heads * rng.randint(1, 3), kv_heads,
                              rng.choice([4, 8, 12, 16, 24, 32]), rng.choice([4, 8, 10, 16, 32]),
                              window, keep, scale=rng.choice([None, 0.2, 0.5]))
        else:
            source = rng.choice(list(owners)) if owners and rng.random() < 0.4 else None
            rank = owners[source] if source is not None else rng.choice([6, 8, 14, 16, 24, 40, 64])
            entry = latent(rng.randint(1, 6), rng.choice([4, 8, 12, 16, 24]),
                           rng.choice([4, 8, 10, 16, 32]), rng.choice([6, 8, 16, 20, 48]), rank,
                           rng.choice([0, 1, 2, 5, 16, 17, 31, 40, 200]), kv_from=source,
                           scale=rng.choice([None, 0.2, 0.5]))
            if source is None:
                owners[index] = rank
        layers.append(layer(entry, draw_mlp(rng)))
    return model(rng.choice([17, 64, 101, 300]), width, rng.choice([1e-5, 1e-6, 1e-3]), layers,
                 embed_scale=rng.choice([None, 1.0, 3.0, 12.0]),
                 mult=rng.choice([None, 1.0, 0.3, 0.7]), side=rng.choice([None, 1, 4, 10]))


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
    rng = random.Random(2000 + seed)
    config = draw_model(rng)
    init = RandomInit(weight_std=rng.choice([0.08, 0.15]) * (64 / config["width"]) ** 0.5,
                      scale_residual_projections=False, bias_std=0.0, norm_std=0.1)
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
    support.assert_logits_close(got, expected, "float32", "semadra-drawn", page=page)
    assert not core.manager.live_requests()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["attention", "latent", "shared_latent", "experts", "side"])
def test_each_mechanism_alone_in_a_model_of_one_layer(tmp_path, which, dtype):
    """A model that has the one mechanism and as little else as the design allows."""
    if which == "attention":
        layers = [layer(attention(4, 2, 16, 32, 19, 7, scale=0.4))]
    elif which == "latent":
        layers = [layer(latent(2, 16, 32, 24, 40, 19, scale=0.4))]
    elif which == "shared_latent":
        layers = [layer(latent(2, 16, 32, 24, 40, 19)),
                  layer(latent(4, 32, 16, 8, 40, 45, kv_from=0, scale=0.3))]
    else:
        layers = [layer(latent(1, 16, 16, 16, 16, 1),
                        moe(8, 2, 32, groups=4, keep=2, scale=1.5, shared=16)
                        if which == "experts" else None)]
    config = model(120, 64, 1e-5, layers, side=8 if which == "side" else None,
                   embed_scale=4.0 if which == "side" else None,
                   mult=0.5 if which in ("side", "experts") else None)
    init = RandomInit(weight_std=0.12, scale_residual_projections=False, bias_std=0.0,
                      norm_std=0.1)
    folder, state = support.make_model(tmp_path / "m", config, 2, init, dtype)
    sequences = {f"r{i}": random_tokens(120, n, 30 + i) for i, n in enumerate((70, 2, 33))}
    expected = plain_logits(state, config, sequences)
    core = support.build_core(folder, dtype, num_blocks=12)
    got = support.replay(core, support.schedule_mixed(sequences, pool_tokens=128))
    if which == "experts" and dtype == "bfloat16":
        from test_semadra_engine_gpu import assert_mostly_close

        assert_mostly_close(got, expected, "semadra-one/experts")
    else:
        support.assert_logits_close(got, expected, dtype, f"semadra-one/{which}")
