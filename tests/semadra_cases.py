"""Tiny Semadra configurations for the tests. Each differs from the others in every size and
constant, and none makes equal what a model could happen to make equal: query and key/value
heads, a head's key and value sizes, the two latents' ranks, a reader's window and its
owner's, experts per group, kept groups and all groups, top and 1, factors and 1."""

from __future__ import annotations

import torch

import plain_semadra as plain
from ayaka_b200.weights.rules import RandomInit

NAME = "Semadra"


def attention(heads, kv_heads, dim, vdim, window, keep_first, scale=None):
    mask = {}
    if window:
        mask["size"] = window
    if keep_first is not None:
        mask["keep_first"] = keep_first
    return {"type": "attention", "mixer": {
        "heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
        "scale": scale if scale is not None else dim ** -0.5, "mask": mask}}


def latent(heads, dim, vdim, q_rank, kv_rank, window, kv_from=None, scale=None):
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
             "scale": scale if scale is not None else dim ** -0.5}
    if window:
        mixer["mask"] = {"size": window}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, *, groups=None, keep=None, scale=1.0, shared=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups, "keep": keep}
    out = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def layer(entry, mlp=None):
    return {**entry, "mlp": mlp}


def model(vocab, width, eps, layers, *, embed_scale=None, mult=None, side=None):
    out = {"architecture": NAME, "vocab": vocab, "width": width, "norm": {"eps": eps},
           "layers": layers}
    if embed_scale is not None:
        out["embedding"] = {"scale": embed_scale}
    if mult is not None:
        out["residual_mult"] = mult
    if side is not None:
        out["token_side"] = {"dim": side}
    return out


#: both mixers, a reader of another layer's latents with a wider window than its owner's,
#: grouped heads, a window shorter than the kept stretch is long, every kind of feed-forward
TINY_A = model(131, 64, 1e-5, [
    layer(latent(2, 16, 24, 20, 32, 11), dense(96)),
    layer(attention(4, 2, 16, 8, 9, 13, scale=0.3), moe(6, 2, 24, groups=3, keep=2, scale=1.5,
                                                       shared=40)),
    layer(latent(3, 8, 16, 12, 32, 37, kv_from=0, scale=0.4)),
    layer(attention(2, 2, 24, 24, 21, 3), moe(4, 1, 16, scale=0.7)),
], embed_scale=4.0, mult=0.4, side=6)

#: starts with an attention layer; one key/value head for all; no kept tokens; a window of
#: one; an attention without a window; groups of one expert; no side input; factors left out
TINY_B = model(257, 96, 1e-6, [
    layer(attention(3, 1, 8, 20, 1, 0), dense(72)),
    layer(latent(1, 24, 8, 40, 24, 1000)),
    layer(attention(2, 1, 12, 6, 0, None, scale=0.21), moe(5, 3, 20, groups=5, keep=4,
                                                          scale=2.5)),
    layer(latent(4, 6, 10, 8, 24, 5, kv_from=1, scale=0.5), moe(8, 2, 12, groups=2, keep=1,
                                                               shared=8)),
    layer(latent(2, 12, 12, 16, 16, 17), dense(40)),
])

#: sizes the bfloat16 tensor-core products and attention kernels take (multiples of 16), no
#: experts: a bfloat16 run has no choice that a rounding could turn
TINY_C = model(320, 128, 2e-5, [
    layer(latent(4, 32, 16, 48, 64, 48), dense(256)),
    layer(attention(4, 2, 32, 16, 40, 24), dense(192)),
    layer(latent(2, 64, 32, 32, 64, 30, kv_from=0), dense(128)),
    layer(attention(2, 2, 64, 64, 70, 5, scale=0.11)),
], embed_scale=8.0, mult=0.5, side=16)

#: the same sizes with experts (bfloat16 runs of it are held to most positions only)
TINY_D = model(200, 128, 1e-5, [
    layer(attention(4, 4, 32, 32, 33, 16), moe(8, 2, 64, groups=4, keep=2, scale=2.0,
                                               shared=64)),
    layer(latent(2, 32, 32, 32, 48, 25), moe(6, 3, 32, groups=2, keep=2, shared=32)),
], embed_scale=8.0, mult=0.3, side=8)

LOUD = RandomInit(weight_std=0.16, scale_residual_projections=False, bias_std=0.0, norm_std=0.1)
LOUD_WIDE = RandomInit(weight_std=0.1, scale_residual_projections=False, bias_std=0.0,
                       norm_std=0.1)


def plain_logits(state: dict, config: dict, sequences: dict[str, list[int]]
                 ) -> dict[str, torch.Tensor]:
    wide = plain.cast_state(state, torch.float64)
    return {rid: plain.logits(wide, config, tokens).float()
            for rid, tokens in sequences.items()}
