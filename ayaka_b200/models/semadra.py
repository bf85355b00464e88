"""Semadra as data: its parts, its checkpoint names, its random weights.

A layer is ``x += m * norm1(mixer(x)); x += m * norm2(mlp(x)); x += m * side(x)`` (block
``output_norm``: the sublayers read the stream itself, the norms ``rms(y) * (1 + w)`` stand on
their outputs, ``m`` is ``residual_mult``). The mixer is a softmax attention with grouped
heads, norms over the whole query and key projections, no positions in its scores, a sliding
window that keeps the sequence's first tokens in sight and an output gate per entry
(``parts/gated_attention.py``), or a latent attention whose queries go through a latent of
their own and whose cached latents a later layer may read instead of projecting its own
(``parts/latent.py``). The feed-forward is a gated dense one (silu), a mixture of such experts
routed by sigmoid scores among the best groups with a shared expert beside them
(``parts/experts.py``), or absent. ``side`` is a gated embedding of the row's own token
(``parts/token_input.py``). The token table is scaled on the way in and used as it is for the
logits: ``logits = embed @ final_norm(x)``.

Checkpoint names: ``embed``, ``side.embed`` (``[vocab, layers * dim]``, layer ``i`` owns
columns ``i * dim .. (i + 1) * dim``), ``final.norm`` and per layer ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*`` (``gate``, ``up``, ``down``; ``router``,
``e<j>.*``, ``shared.*``), ``l<i>.side.gate`` / ``.proj`` / ``.norm``; linear weights
``[out, in]``. Stored matrices that multiply the same input are stacked into one parameter.
"""

from __future__ import annotations

import hashlib
import math
from collections.abc import Iterator, Mapping

import torch

from ayaka_b200.config.semadra import SemadraConfig, SemadraLayer
from ayaka_b200.models.registry import Architecture, register_architecture
from ayaka_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, Run
from ayaka_b200.weights.rules import RandomInit, WeightRule, WeightRules

__all__ = ["SEMADRA", "semadra_model_spec", "semadra_weight_rules"]

#: The design has no table of positions and no longest sequence; the engine bounds a
#: sequence by its cache instead (positions are int32 on the device).
UNBOUNDED_POSITIONS = 1 << 30


def _mixer_spec(layer: SemadraLayer, width: int, eps: float) -> PartSpec:
    if layer.kind == "attention":
        return PartSpec("gated_attention", width=width, num_heads=layer.heads,
                        num_kv_heads=layer.kv_heads, head_dim=layer.dim, value_dim=layer.vdim,
                        scale=layer.scale, window=layer.window, keep_first=layer.keep_first,
                        qk_norm=True, eps=eps, gate=True)
    return PartSpec("latent_attention", width=width, num_heads=layer.heads, dim=layer.dim,
                    rot=0, value_dim=layer.vdim, rank=layer.kv_rank, scale=layer.scale,
                    window=layer.window, eps=eps, query_rank=layer.q_rank, gate=False,
                    shares_latent=layer.kv_from is not None)


def _feed_forward_spec(layer: SemadraLayer, width: int) -> PartSpec:
    mlp = layer.mlp
    if mlp is None:
        return PartSpec("none")
    if mlp.kind == "dense":
        return PartSpec("gated_dense", width=width, inner=mlp.ff, activation="silu")
    return PartSpec("experts", width=width, experts=mlp.experts, top=mlp.top, inner=mlp.ff,
                    unit="silu", scoring="sigmoid", groups=mlp.groups, keep_groups=mlp.keep,
                    route_scale=mlp.route_scale, renormalise=False, shared_inner=mlp.shared_ff)


def semadra_model_spec(config: SemadraConfig) -> ModelSpec:
    """The model as parts. Every size comes from ``config``."""
    width, eps = config.width, config.eps
    norm = PartSpec("rms_norm", width=width, eps=eps, offset=1.0)
    side = None if not config.side_dim else PartSpec(
        "token_gated", width=width, dim=config.side_dim, vocab_size=config.vocab,
        activation="gelu_tanh", eps=eps)
    layers = [LayerSpec(block="output_norm", mixer=_mixer_spec(layer, width, eps),
                        feed_forward=_feed_forward_spec(layer, width), mixer_norm=norm,
                        feed_forward_norm=norm, residual_factor=config.residual_mult, side=side)
              for layer in config.layers]
    return ModelSpec(
        hidden_size=width,
        vocab_size=config.vocab,
        max_positions=UNBOUNDED_POSITIONS,
        embedding=PartSpec("token", vocab_size=config.vocab, width=width,
                           scale=config.embedding_scale),
        position=PartSpec("none"),
        layers=tuple(layers),
        order=tuple(Run(layer=index, reads_cache_of=layer.kv_from)
                    for index, layer in enumerate(config.layers)),
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


def _gated_rules(src: str, dst: str, ff: int) -> dict[str, WeightRule]:
    rules = _stacked(f"{dst}in.weight", [(f"{src}gate", ff), (f"{src}up", ff)])
    rules[f"{src}down"] = WeightRule(f"{dst}out.weight")
    return rules


def semadra_weight_rules(config: SemadraConfig) -> WeightRules:
    rules: dict[str, WeightRule | tuple[WeightRule, ...]] = {
        "embed": WeightRule("embedding.weight"),
        "final.norm": WeightRule("final_norm.weight"),
    }
    width, dim = config.width, config.side_dim
    if dim:
        rules["side.embed"] = tuple(
            WeightRule(f"layers.{index}.side.table", dim=1, take=(index * dim, (index + 1) * dim))
            for index in range(len(config.layers)))
    for index, layer in enumerate(config.layers):
        src, dst = f"l{index}.", f"layers.{index}."
        mix, mixer = f"{src}mix.", f"{dst}mixer."
        rules[f"{src}norm1"] = WeightRule(f"{dst}mixer_norm.weight")
        if layer.kind == "attention":
            q, k = layer.heads * layer.dim, layer.kv_heads * layer.dim
            v, joined = layer.kv_heads * layer.vdim, layer.heads * layer.vdim
            rules.update(_stacked(f"{mixer}proj.weight", [
                (f"{mix}q", q), (f"{mix}k", k), (f"{mix}v", v), (f"{mix}g", joined)]))
            rules[f"{mix}q.norm"] = WeightRule(f"{mixer}q_norm.weight")
            rules[f"{mix}k.norm"] = WeightRule(f"{mixer}k_norm.weight")
        else:
            pieces = [(f"{mix}dq", layer.q_rank)]
            if layer.kv_from is None:
                pieces.append((f"{mix}dkv", layer.kv_rank))
                rules[f"{mix}dkv.norm"] = WeightRule(f"{mixer}latent_norm.weight")
            rules.update(_stacked(f"{mixer}proj.weight", pieces))
            rules[f"{mix}dq.norm"] = WeightRule(f"{mixer}q_norm.weight")
            rules[f"{mix}uq"] = WeightRule(f"{mixer}q_up.weight")
            rules[f"{mix}uk"] = WeightRule(f"{mixer}up_key.weight")
            rules[f"{mix}uv"] = WeightRule(f"{mixer}up_value.weight")
        rules[f"{mix}o"] = WeightRule(f"{mixer}out.weight")
        mlp = layer.mlp
        if mlp is not None:
            rules[f"{src}norm2"] = WeightRule(f"{dst}feed_forward_norm.weight")
            ff = f"{dst}feed_forward."
            if mlp.kind == "dense":
                rules.update(_gated_rules(f"{src}mlp.", ff, mlp.ff))
            else:
                rules[f"{src}mlp.router"] = WeightRule(f"{ff}router.weight")
                for e in range(mlp.experts):
                    at = e * 2 * mlp.ff
                    rules[f"{src}mlp.e{e}.gate"] = WeightRule(f"{ff}in.weight", dim=0, offset=at)
                    rules[f"{src}mlp.e{e}.up"] = WeightRule(f"{ff}in.weight", dim=0,
                                                            offset=at + mlp.ff)
                    rules[f"{src}mlp.e{e}.down"] = WeightRule(f"{ff}out.weight", dim=0,
                                                              offset=e * width)
                if mlp.shared_ff:
                    rules.update(_gated_rules(f"{src}mlp.shared.", f"{ff}shared.",
                                              mlp.shared_ff))
        if dim:
            rules[f"{src}side.gate"] = WeightRule(f"{dst}side.gate.weight")
            rules[f"{src}side.proj"] = WeightRule(f"{dst}side.proj.weight")
            rules[f"{src}side.norm"] = WeightRule(f"{dst}side.norm.weight")
    # a layer without a feed-forward may still store the norm that would go with it
    ignore = tuple(rf"l{index}\.norm2" for index, layer in enumerate(config.layers)
                   if layer.mlp is None)
    return WeightRules(rules=rules, ignore=ignore)


def _generator(seed: int, name: str) -> torch.Generator:
    digest = hashlib.blake2b(f"{seed}:{name}".encode(), digest_size=8).digest()
    return torch.Generator().manual_seed(int.from_bytes(digest, "big") & ((1 << 63) - 1))


def _random_tensors(config: SemadraConfig, seed: int,
                    init: RandomInit) -> Iterator[tuple[str, torch.Tensor]]:
    """Random float32 tensors under checkpoint names. A matrix is drawn with deviation
    ``weight_std * sqrt(width / fan_in)`` (a product keeps the size of its input; the norms on
    the sublayers' outputs make the size of most of them immaterial), norm weights with
    ``norm_std`` around zero (the one-plus norms) or around one (the plain ones), the token
    table so that a scaled row has entries of size one. Each tensor has its own generator,
    seeded from ``seed`` and its name."""
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
        yield f"{p}norm1", normal(f"{p}norm1", (width,), init.norm_std)
        if layer.kind == "attention":
            q, k = layer.heads * layer.dim, layer.kv_heads * layer.dim
            for name, rows in (("q", q), ("k", k), ("v", layer.kv_heads * layer.vdim),
                               ("g", layer.heads * layer.vdim)):
                yield f"{m}{name}", matrix(f"{m}{name}", rows, width)
            yield f"{m}q.norm", normal(f"{m}q.norm", (q,), init.norm_std, 1.0)
            yield f"{m}k.norm", normal(f"{m}k.norm", (k,), init.norm_std, 1.0)
        else:
            yield f"{m}dq", matrix(f"{m}dq", layer.q_rank, width)
            yield f"{m}dq.norm", normal(f"{m}dq.norm", (layer.q_rank,), init.norm_std, 1.0)
            yield f"{m}uq", matrix(f"{m}uq", layer.heads * layer.dim, layer.q_rank)
            if layer.kv_from is None:
                yield f"{m}dkv", matrix(f"{m}dkv", layer.kv_rank, width)
                yield f"{m}dkv.norm", normal(f"{m}dkv.norm", (layer.kv_rank,), init.norm_std,
                                             1.0)
            yield f"{m}uk", matrix(f"{m}uk", layer.heads * layer.dim, layer.kv_rank)
            yield f"{m}uv", matrix(f"{m}uv", layer.heads * layer.vdim, layer.kv_rank)
        yield f"{m}o", matrix(f"{m}o", width, layer.heads * layer.vdim)
        mlp = layer.mlp
        if mlp is not None:
            yield f"{p}norm2", normal(f"{p}norm2", (width,), init.norm_std)
            f = f"{p}mlp."
            names = [(f, mlp.ff)] if mlp.kind == "dense" else \
                [(f"{f}e{e}.", mlp.ff) for e in range(mlp.experts)] + \
                ([(f"{f}shared.", mlp.shared_ff)] if mlp.shared_ff else [])
            if mlp.kind == "moe":
                yield f"{f}router", matrix(f"{f}router", mlp.experts, width, 2.0)
            for prefix, ff in names:
                yield f"{prefix}gate", matrix(f"{prefix}gate", ff, width)
                yield f"{prefix}up", matrix(f"{prefix}up", ff, width)
                yield f"{prefix}down", matrix(f"{prefix}down", width, ff)
        if config.side_dim:
            s = f"{p}side."
            yield f"{s}gate", matrix(f"{s}gate", config.side_dim, width)
            yield f"{s}proj", matrix(f"{s}proj", width, config.side_dim)
            yield f"{s}norm", normal(f"{s}norm", (width,), init.norm_std, 1.0)
    yield "final.norm", normal("final.norm", (width,), init.norm_std)


def _parse(config_json: Mapping[str, object]) -> SemadraConfig:
    return SemadraConfig.from_json_dict(config_json)


SEMADRA = register_architecture(Architecture(
    name="Semadra",
    parse_config=_parse,
    model_spec=semadra_model_spec,  # type: ignore[arg-type]
    weight_rules=semadra_weight_rules,  # type: ignore[arg-type]
    random_tensors=_random_tensors,  # type: ignore[arg-type]
    config_json=lambda config: config.to_json_dict(),  # type: ignore[attr-defined]
))
