"""Tiny Rizitar configurations for the tests. Each differs from the others in every size and
constant, and none makes equal what a model could happen to make equal: query and key/value
heads, a head's size and its rotated part, window and pooled block (a block longer than the
window, a block of one, a window of one), layers with and without window, pooling, rotation,
blended frequencies, feed-forward and token input, the first layer's kind, top and 1."""

from __future__ import annotations

import numpy as np
import torch

import plain_rizitar as plain
from ayaka_b200.weights.rules import RandomInit

NAME = "Rizitar"


def attention(heads, kv_heads, dim, window, pool=None, *, rot=None, base=10000.0, scaling=None,
              scale=None):
    mask = {}
    if window:
        mask["size"] = window
    if pool is not None:
        mask["pool"] = pool
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
             "scale": scale if scale is not None else dim ** -0.5, "mask": mask}
    if rot:
        mixer["rot"] = {"dims": rot, "base": base}
        if scaling is not None:
            factor, original, fast, slow = scaling
            mixer["rot"]["scaling"] = {"factor": factor, "original": original, "fast": fast,
                                       "slow": slow}
    return {"type": "attention", "mixer": mixer}


def delta(heads, dim, rank=None):
    mixer = {"heads": heads, "dim": dim}
    if rank is not None:
        mixer["decay_rank"] = rank
    return {"type": "general_delta", "mixer": mixer}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def layer(entry, mlp=None):
    return {**entry, "mlp": mlp}


def model(vocab, width, eps, layers, *, embed_scale=None, side=None):
    out = {"architecture": NAME, "vocab": vocab, "width": width, "norm": {"eps": eps},
           "layers": layers}
    if embed_scale is not None:
        out["embedding"] = {"scale": embed_scale}
    if side is not None:
        out["token_side"] = {"dim": side}
    return out


#: both mixers, grouped heads, part of a head rotated with blended frequencies, a head wholly
#: rotated with plain ones, blocks shorter than the window, every kind of feed-forward
TINY_A = model(131, 64, 1e-5, [
    layer(attention(4, 2, 16, 9, 4, rot=8, base=100.0, scaling=(4.0, 32, 8.0, 0.5)), dense(96)),
    layer(delta(2, 12, 5), moe(6, 2, 24)),
    layer(attention(3, 1, 10, 21, 5, rot=10, base=37.0, scale=0.3)),
    layer(delta(1, 20, 3), dense(40)),
], embed_scale=4.0, side=6)

#: starts with a delta layer; no window at all; a window of one with blocks of one; a window
#: without blocks; a block longer than the window; one expert chosen; all but one chosen; no
#: token input; no scale on the table
TINY_B = model(257, 96, 1e-6, [
    layer(delta(3, 8, 7), dense(72)),
    layer(attention(2, 2, 12, 0), moe(5, 1, 20)),
    layer(attention(2, 1, 8, 1, 1, rot=4, base=50.0, scaling=(2.0, 16, 4.0, 1.0), scale=0.21),
          moe(4, 3, 12)),
    layer(attention(4, 4, 6, 7), dense(24)),
    layer(attention(2, 1, 16, 5, 11, rot=16, base=500.0)),
])

#: sizes the bfloat16 tensor-core products and attention kernels take (multiples of 16), no
#: experts: a bfloat16 run has no choice that a rounding could turn
TINY_C = model(320, 128, 2e-5, [
    layer(attention(4, 2, 32, 40, 8, rot=16, base=1000.0, scaling=(8.0, 64, 16.0, 1.0)),
          dense(256)),
    layer(delta(2, 32, 16), dense(192)),
    layer(attention(2, 2, 64, 70, 12, rot=64, base=10000.0, scale=0.11), dense(128)),
    layer(delta(4, 16, 8)),
], embed_scale=8.0, side=16)

#: the same kind of sizes with experts (bfloat16 runs of it are held to most positions only)
TINY_D = model(200, 128, 1e-5, [
    layer(attention(4, 4, 32, 33, 16, rot=32, base=300.0, scaling=(4.0, 48, 8.0, 2.0)),
          moe(8, 2, 64)),
    layer(delta(2, 32, 16), moe(6, 3, 32)),
], embed_scale=8.0, side=8)

LOUD = RandomInit(weight_std=0.16, scale_residual_projections=False, bias_std=0.1, norm_std=0.1)
LOUD_WIDE = RandomInit(weight_std=0.1, scale_residual_projections=False, bias_std=0.1,
                       norm_std=0.1)


def numpy_state(state: dict) -> dict[str, np.ndarray]:
    return {name: tensor.detach().cpu().to(torch.float64).numpy()
            for name, tensor in state.items()}


def plain_logits(state: dict, config: dict, sequences: dict[str, list[int]]
                 ) -> dict[str, torch.Tensor]:
    wide = numpy_state(state)
    return {rid: torch.from_numpy(plain.logits(config, wide, np.asarray(tokens))).float()
            for rid, tokens in sequences.items()}


def greedy_generate(state: dict, config: dict, prompt: list[int], count: int) -> list[int]:
    """``count`` tokens by arg-max (ties to the smaller id), the whole sequence run again for
    every token."""
    wide = numpy_state(state)
    tokens, out = list(prompt), []
    for _ in range(count):
        last = plain.logits(config, wide, np.asarray(tokens))[-1]
        out.append(int(np.argmax(last)))
        tokens.append(out[-1])
    return out
