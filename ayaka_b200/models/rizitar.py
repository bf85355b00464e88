"""Rizitar as data: its parts, its checkpoint names, its random weights.

A layer is ``x += post1(mixer(pre1(x))); x += post2(mlp(pre2(x))); x += side(x)`` (block
``sandwich_norm``; all norms ``rms(y) * w`` with plain weights). The mixer is a softmax
attention with grouped heads whose values are its keys as projected, a norm per head on
queries and keys, rotary positions on part of each head with frequencies blended for long
contexts, a sliding window behind which blocks of positions are seen as the means of their
keys and values, and a sink in the softmax (``parts/pooled_attention.py``); or a generalised
delta rule with a decay and a removal rate per key channel (``parts/recurrent.py``). The
feed-forward is a dense one with biases and a learned quadratic-exponential unit
(``parts/feed_forward.py``), a mixture of ungated experts with squared relu, routed by the
softmax over all experts without renormalising (``parts/experts.py``), or absent. ``side`` is
a gated embedding of the row's own token (``parts/token_input.py``). The token table is scaled
on the way in and used as it is for the logits: ``logits = embed @ final_norm(x)``.

Checkpoint names: ``embed``, ``side.embed`` (``[vocab, layers * dim]``, layer ``i`` owns
columns ``i * dim .. (i + 1) * dim``), ``final.norm`` and per layer ``l<i>.norm1``,
``norm1b``, ``norm2``, ``norm2b`` (in front of and behind the mixer and the feed-forward),
``l<i>.mix.*``, ``l<i>.mlp.*`` (``up``, ``up.b``, ``down``, ``down.b``, ``act``; ``router``,
``e<j>.up``, ``e<j>.down``), ``l<i>.side.gate`` / ``.proj`` / ``.norm``; linear weights
``[out, in]``. Stored matrices that multiply the same input are stacked into one parameter.
"""

from __future__ import annotations

import hashlib
import math
from collections.abc import Callable, Iterator, Mapping
from dataclasses import replace

import torch

from ayaka_b200.config.rizitar import RizitarConfig, RizitarLayer
from ayaka_b200.errors import ModelLoadError
from ayaka_b200.models.registry import Architecture, register_architecture
from ayaka_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, Run
from ayaka_b200.weights.rules import RandomInit, WeightRule, WeightRules

__all__ = ["RIZITAR", "rizitar_model_spec", "rizitar_weight_rules"]

#: The design has no table of positions and no longest sequence; the engine bounds a
#: sequence by its cache instead (positions are int32 on the device).
UNBOUNDED_POSITIONS = 1 << 30
#: The factor on ``sigmoid(z)`` in the exponent of the delta rule's decay: the design fixes it.
DECAY_RATE = math.exp(-0.5)
#: inner width of the decay's projections when neither the configuration nor a stored tensor
#: gives it (random models)
DEFAULT_DECAY_RANK = 16


def _mixer_spec(layer: RizitarLayer, width: int, eps: float) -> PartSpec:
    if layer.kind == "attention":
        rot = layer.rot
        rotation = {} if rot is None else dict(
            rot_dims=rot.dims, rot_base=rot.base, rot_factor=rot.factor,
            rot_original=rot.original, rot_fast=rot.fast, rot_slow=rot.slow)
        return PartSpec("pooled_window_attention", width=width, num_heads=layer.heads,
                        num_kv_heads=layer.kv_heads, head_dim=layer.dim, scale=layer.scale,
                        window=layer.window, pool=layer.pool, qk_norm=True, eps=eps, sink=True,
                        values_from_keys=True, **rotation)
    if layer.decay_rank is None:
        raise ModelLoadError("a general_delta layer needs decay_rank in config.json or the "
                             "stored tensor mix.w1 that gives it")
    return PartSpec("delta_rule", width=width, num_heads=layer.heads, dim=layer.dim,
                    columns=layer.dim, decay_rank=layer.decay_rank, decay_rate=DECAY_RATE,
                    eps=eps)


def _feed_forward_spec(layer: RizitarLayer, width: int) -> PartSpec:
    mlp = layer.mlp
    if mlp is None:
        return PartSpec("none")
    if mlp.kind == "dense":
        return PartSpec("dense", width=width, inner=mlp.ff, activation="xielu", bias=True)
    return PartSpec("experts", width=width, experts=mlp.experts, top=mlp.top, inner=mlp.ff,
                    unit="relu_squared", scoring="softmax_all")


def rizitar_model_spec(config: RizitarConfig) -> ModelSpec:
    """The model as parts. Every size comes from ``config``."""
    width, eps = config.width, config.eps
    norm = PartSpec("rms_norm", width=width, eps=eps)
    side = None if not config.side_dim else PartSpec(
        "token_gated", width=width, dim=config.side_dim, vocab_size=config.vocab,
        activation="gelu_tanh", eps=eps)
    layers = [LayerSpec(block="sandwich_norm", mixer=_mixer_spec(layer, width, eps),
                        feed_forward=_feed_forward_spec(layer, width), mixer_norm=norm,
                        feed_forward_norm=norm, side=side)
              for layer in config.layers]
    return ModelSpec(
        hidden_size=width,
        vocab_size=config.vocab,
        max_positions=UNBOUNDED_POSITIONS,
        embedding=PartSpec("token", vocab_size=config.vocab, width=width,
                           scale=config.embedding_scale),
        position=PartSpec("none"),
        layers=tuple(layers),
        order=tuple(Run(layer=index) for index in range(len(config.layers))),
        final_norm=norm,
        head=PartSpec("linear", vocab_size=config.vocab, width=width, tied=True),
        eos_token_id=None,
    )


def _stacked(dst: str, pieces: list[tuple[str, int]]) -> dict[str, WeightRule]:
    """Rules that put stored tensors one under the other into parameter ``dst``."""
    rules, at = {}, 0
    for name, rows in pieces:
        rules[name] = WeightRule(dst, dim=0, offset=at)
        at += rows
    return rules


def rizitar_weight_rules(config: RizitarConfig) -> WeightRules:
    rules: dict[str, WeightRule | tuple[WeightRule, ...]] = {
        "embed": WeightRule("embedding.weight"),
        "final.norm": WeightRule("final_norm.weight"),
    }
    width, dim = config.width, config.side_dim
    ignore: list[str] = []
    if dim:
        rules["side.embed"] = tuple(
            WeightRule(f"layers.{index}.side.table", dim=1, take=(index * dim, (index + 1) * dim))
            for index in range(len(config.layers)))
    for index, layer in enumerate(config.layers):
        src, dst = f"l{index}.", f"layers.{index}."
        mix, mixer = f"{src}mix.", f"{dst}mixer."
        rules[f"{src}norm1"] = WeightRule(f"{dst}mixer_norm.weight")
        rules[f"{src}norm1b"] = WeightRule(f"{dst}mixer_post_norm.weight")
        if layer.kind == "attention":
            rules.update(_stacked(f"{mixer}proj.weight", [
                (f"{mix}q", layer.heads * layer.dim), (f"{mix}k", layer.kv_heads * layer.dim)]))
            rules[f"{mix}q.norm"] = WeightRule(f"{mixer}q_norm.weight")
            rules[f"{mix}k.norm"] = WeightRule(f"{mixer}k_norm.weight")
            rules[f"{mix}sink"] = WeightRule(f"{mixer}sink")
        else:
            inner = layer.heads * layer.dim
            # the order of DeltaRule's fused projection
            rules.update(_stacked(f"{mixer}proj.weight", [
                (f"{mix}r", inner), (f"{mix}k", inner), (f"{mix}a", inner), (f"{mix}v", inner),
                (f"{mix}g", inner), (f"{mix}w1", layer.decay_rank or 0)]))
            rules[f"{mix}a.b"] = WeightRule(f"{mixer}rate.bias")
            rules[f"{mix}w2"] = WeightRule(f"{mixer}decay_up.weight")
            rules[f"{mix}w0"] = WeightRule(f"{mixer}decay_up.bias")
            rules[f"{mix}norm"] = WeightRule(f"{mixer}norm.weight")
        rules[f"{mix}o"] = WeightRule(f"{mixer}out.weight")
        mlp = layer.mlp
        if mlp is None:
            # a layer without a feed-forward may still store the norms that would go with it
            ignore += [rf"l{index}\.norm2", rf"l{index}\.norm2b"]
        else:
            rules[f"{src}norm2"] = WeightRule(f"{dst}feed_forward_norm.weight")
            rules[f"{src}norm2b"] = WeightRule(f"{dst}feed_forward_post_norm.weight")
            ff = f"{dst}feed_forward."
            if mlp.kind == "dense":
                rules[f"{src}mlp.up"] = WeightRule(f"{ff}up.weight")
                rules[f"{src}mlp.up.b"] = WeightRule(f"{ff}up.bias")
                rules[f"{src}mlp.down"] = WeightRule(f"{ff}down.weight")
                rules[f"{src}mlp.down.b"] = WeightRule(f"{ff}down.bias")
                rules[f"{src}mlp.act"] = WeightRule(f"{ff}act.numbers")
            else:
                rules[f"{src}mlp.router"] = WeightRule(f"{ff}router.weight")
                for e in range(mlp.experts):
                    rules[f"{src}mlp.e{e}.up"] = WeightRule(f"{ff}in.weight", dim=0,
                                                            offset=e * mlp.ff)
                    rules[f"{src}mlp.e{e}.down"] = WeightRule(f"{ff}out.weight", dim=0,
                                                              offset=e * width)
        if dim:
            rules[f"{src}side.gate"] = WeightRule(f"{dst}side.gate.weight")
            rules[f"{src}side.proj"] = WeightRule(f"{dst}side.proj.weight")
            rules[f"{src}side.norm"] = WeightRule(f"{dst}side.norm.weight")
    return WeightRules(rules=rules, ignore=tuple(ignore))


def _complete(config: RizitarConfig,
              shape_of: Callable[[str], tuple[int, ...] | None]) -> RizitarConfig:
    """Fill the sizes that only stored tensors give: a delta layer's decay rank."""
    layers = []
    for index, layer in enumerate(config.layers):
        if layer.kind == "general_delta" and layer.decay_rank is None:
            shape = shape_of(f"l{index}.mix.w1")
            if shape is not None and len(shape) == 2:
                layer = replace(layer, decay_rank=int(shape[0]))
        layers.append(layer)
    return replace(config, layers=tuple(layers))


def _generator(seed: int, name: str) -> torch.Generator:
    digest = hashlib.blake2b(f"{seed}:{name}".encode(), digest_size=8).digest()
    return torch.Generator().manual_seed(int.from_bytes(digest, "big") & ((1 << 63) - 1))


def _random_tensors(config: RizitarConfig, seed: int,
                    init: RandomInit) -> Iterator[tuple[str, torch.Tensor]]:
    """Random float32 tensors under checkpoint names. A matrix is drawn with deviation
    ``weight_std * sqrt(width / fan_in)`` (a product keeps the size of its input; the norms
    behind the sublayers make the size of most of them immaterial), norm weights with
    ``norm_std`` around one, biases with ``bias_std``, sinks and the units' two numbers around
    zero with deviation one half, the token table so that a scaled row has entries of size
    one. Each tensor has its own generator, seeded from ``seed`` and its name."""
    width = config.width
    loud = init.weight_std * math.sqrt(width)

    def normal(name: str, shape: tuple[int, ...], std: float, mean: float = 0.0) -> torch.Tensor:
        if std == 0.0:
            return torch.full(shape, mean, dtype=torch.float32)
        values = torch.randn(shape, generator=_generator(seed, name), dtype=torch.float32)
        return values.mul_(std).add_(mean)

    def matrix(name: str, rows: int, cols: int, gain: float = 1.0) -> torch.Tensor:
        return normal(name, (rows, cols), gain * loud / math.sqrt(cols))

    yield "embed", normal("embed", (config.vocab, width),
                          1.0 / max(abs(config.embedding_scale), 1e-3))
    if config.side_dim:
        yield "side.embed", normal("side.embed",
                                   (config.vocab, len(config.layers) * config.side_dim), 1.0)
    for index, layer in enumerate(config.layers):
        p, m = f"l{index}.", f"l{index}.mix."
        yield f"{p}norm1", normal(f"{p}norm1", (width,), init.norm_std, 1.0)
        yield f"{p}norm1b", normal(f"{p}norm1b", (width,), init.norm_std, 1.0)
        if layer.kind == "attention":
            yield f"{m}q", matrix(f"{m}q", layer.heads * layer.dim, width)
            yield f"{m}k", matrix(f"{m}k", layer.kv_heads * layer.dim, width)
            yield f"{m}q.norm", normal(f"{m}q.norm", (layer.dim,), init.norm_std, 1.0)
            yield f"{m}k.norm", normal(f"{m}k.norm", (layer.dim,), init.norm_std, 1.0)
            yield f"{m}sink", normal(f"{m}sink", (layer.heads,), 0.5)
            yield f"{m}o", matrix(f"{m}o", width, layer.heads * layer.dim)
        else:
            inner = layer.heads * layer.dim
            rank = layer.decay_rank or DEFAULT_DECAY_RANK
            for name in ("r", "k", "v", "g", "a"):
                yield f"{m}{name}", matrix(f"{m}{name}", inner, width)
            yield f"{m}a.b", normal(f"{m}a.b", (inner,), max(init.bias_std, 0.1))
            yield f"{m}w1", matrix(f"{m}w1", rank, width)
            yield f"{m}w2", matrix(f"{m}w2", inner, rank)
            yield f"{m}w0", normal(f"{m}w0", (inner,), 1.0)
            yield f"{m}norm", normal(f"{m}norm", (inner,), init.norm_std, 1.0)
            yield f"{m}o", matrix(f"{m}o", width, inner)
        mlp = layer.mlp
        if mlp is not None:
            yield f"{p}norm2", normal(f"{p}norm2", (width,), init.norm_std, 1.0)
            yield f"{p}norm2b", normal(f"{p}norm2b", (width,), init.norm_std, 1.0)
            f = f"{p}mlp."
            if mlp.kind == "dense":
                yield f"{f}up", matrix(f"{f}up", mlp.ff, width)
                yield f"{f}up.b", normal(f"{f}up.b", (mlp.ff,), init.bias_std)
                yield f"{f}down", matrix(f"{f}down", width, mlp.ff)
                yield f"{f}down.b", normal(f"{f}down.b", (width,), init.bias_std)
                yield f"{f}act", normal(f"{f}act", (2,), 0.5)
            else:
                yield f"{f}router", matrix(f"{f}router", mlp.experts, width, 2.0)
                for e in range(mlp.experts):
                    yield f"{f}e{e}.up", matrix(f"{f}e{e}.up", mlp.ff, width)
                    yield f"{f}e{e}.down", matrix(f"{f}e{e}.down", width, mlp.ff)
        if config.side_dim:
            s = f"{p}side."
            yield f"{s}gate", matrix(f"{s}gate", config.side_dim, width)
            yield f"{s}proj", matrix(f"{s}proj", width, config.side_dim)
            yield f"{s}norm", normal(f"{s}norm", (width,), init.norm_std, 1.0)
    yield "final.norm", normal("final.norm", (width,), init.norm_std, 1.0)


def _parse(config_json: Mapping[str, object]) -> RizitarConfig:
    return RizitarConfig.from_json_dict(config_json)


def _config_json(config: RizitarConfig) -> dict[str, object]:
    """What a written model folder says: a random model states its decay ranks."""
    filled = replace(config, layers=tuple(
        replace(layer, decay_rank=layer.decay_rank or DEFAULT_DECAY_RANK)
        if layer.kind == "general_delta" else layer for layer in config.layers))
    return filled.to_json_dict()


RIZITAR = register_architecture(Architecture(
    name="Rizitar",
    parse_config=_parse,
    model_spec=rizitar_model_spec,  # type: ignore[arg-type]
    weight_rules=rizitar_weight_rules,  # type: ignore[arg-type]
    random_tensors=_random_tensors,  # type: ignore[arg-type]
    config_json=_config_json,  # type: ignore[arg-type]
    complete_config=_complete,  # type: ignore[arg-type]
))
