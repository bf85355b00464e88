"""The typed configuration of a Rizitar model, read from its own ``config.json`` keys.

Rizitar is a decoder with a norm in front of and behind every sublayer:
``x += post1(mixer(pre1(x))); x += post2(mlp(pre2(x)))``, then a small gated embedding of the
row's own token joins the stream. ``config.json``::

    {"architecture": "Rizitar", "vocab": V, "width": D, "norm": {"eps": e},
     "embedding": {"scale": s}, "token_side": {"dim": d},
     "layers": [{"type": "attention" | "general_delta", "mixer": {...},
                 "mlp": {"kind": "dense", "ff": F}
                      | {"kind": "moe", "expert": {"ff": F}, "router": {"experts": E, "top": k}}
                      | null}, ...]}

``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size`` (the
window), ``mask.pool`` (positions per pooled block behind the window), ``rot.dims``,
``rot.base`` and ``rot.scaling`` (``factor``, ``original``, ``fast``, ``slow``).
``general_delta``: ``heads``, ``dim`` and optionally ``decay_rank`` (the inner width of the
decay's two projections; when absent it is the row count of the stored ``l<i>.mix.w1``).

Keys whose absence has one natural meaning may be left out: ``kv_heads`` (= ``heads``),
``vdim`` (= ``dim``), ``mask`` or ``mask.size`` (no window, nothing pooled), ``mask.pool``
(nothing pooled), ``rot`` (no rotation), ``rot.scaling`` (plain frequencies), ``token_side``
(no token input), ``embedding.scale`` (1). Every other key is required.
"""

from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass

from ayaka_b200.config.semadra import _count, _number, _object, _require
from ayaka_b200.errors import ConfigError, ModelLoadError

__all__ = ["RizitarConfig", "RizitarLayer", "RizitarMlp", "RizitarRotation"]


@dataclass(frozen=True, slots=True)
class RizitarMlp:
    """A layer's feed-forward. ``dense``: ``ff`` is its inner width. ``moe``: ``ff`` is an
    expert's inner width, ``experts`` of which each row uses ``top``."""

    kind: str
    ff: int
    experts: int = 0
    top: int = 0


@dataclass(frozen=True, slots=True)
class RizitarRotation:
    """Rotary positions on the first ``dims`` entries of a head. ``factor`` 1: plain
    frequencies; else blended for contexts beyond ``original`` between the pairs that make
    ``fast`` and ``slow`` turns over ``original`` positions."""

    dims: int
    base: float
    factor: float = 1.0
    original: float = 0.0
    fast: float = 0.0
    slow: float = 0.0


@dataclass(frozen=True, slots=True)
class RizitarLayer:
    """One entry of ``layers``. ``attention`` uses ``kv_heads``, ``vdim``, ``scale``,
    ``window`` (0: none), ``pool`` (0: none) and ``rot``; ``general_delta`` uses
    ``decay_rank`` (``None`` until a stored tensor gives it)."""

    kind: str
    heads: int
    dim: int
    kv_heads: int = 0
    vdim: int = 0
    scale: float = 0.0
    window: int = 0
    pool: int = 0
    rot: RizitarRotation | None = None
    decay_rank: int | None = None
    mlp: RizitarMlp | None = None


@dataclass(frozen=True, slots=True)
class RizitarConfig:
    """Everything ``config.json`` says. ``side_dim`` 0: no per-layer token input."""

    architecture: str
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    side_dim: int
    layers: tuple[RizitarLayer, ...]

    @classmethod
    def from_json_dict(cls, config: Mapping[str, object]) -> RizitarConfig:
        _require(config, ("architecture", "vocab", "width", "norm", "layers"), "config.json")
        eps = _number(_object(config["norm"], "model.norm").get("eps"), "model.norm.eps")
        if eps <= 0:
            raise ConfigError("model.norm.eps", "INVALID_RANGE", "must be positive")
        entries = config["layers"]
        if not isinstance(entries, (list, tuple)) or not entries:
            raise ConfigError("model.layers", "WRONG_TYPE", "must be a non-empty list")
        layers = tuple(_layer(_object(entry, f"model.layers[{index}]"), index)
                       for index, entry in enumerate(entries))
        embedding = config.get("embedding")
        scale = 1.0 if embedding is None or _object(embedding, "model.embedding").get("scale") \
            is None else _number(embedding["scale"], "model.embedding.scale")  # type: ignore
        side = config.get("token_side")
        architecture = config["architecture"]
        if not isinstance(architecture, str) or not architecture:
            raise ConfigError("model.architecture", "WRONG_TYPE", "must be a non-empty string")
        return cls(
            architecture=architecture, vocab=_count(config["vocab"], "model.vocab"),
            width=_count(config["width"], "model.width"), eps=eps, embedding_scale=scale,
            side_dim=0 if side is None else _count(
                _object(side, "model.token_side").get("dim"), "model.token_side.dim"),
            layers=layers)

    def to_json_dict(self) -> dict[str, object]:
        """The ``config.json`` content that reads back as this configuration."""
        entries: list[dict[str, object]] = []
        for layer in self.layers:
            mixer: dict[str, object] = {"heads": layer.heads, "dim": layer.dim}
            if layer.kind == "attention":
                mask: dict[str, object] = {}
                if layer.window:
                    mask["size"] = layer.window
                    if layer.pool:
                        mask["pool"] = layer.pool
                mixer.update(kv_heads=layer.kv_heads, vdim=layer.vdim, scale=layer.scale,
                             mask=mask)
                rot = layer.rot
                if rot is not None:
                    stored: dict[str, object] = {"dims": rot.dims, "base": rot.base}
                    if rot.factor != 1.0:
                        stored["scaling"] = {"factor": rot.factor, "original": rot.original,
                                             "fast": rot.fast, "slow": rot.slow}
                    mixer["rot"] = stored
            elif layer.decay_rank is not None:
                mixer["decay_rank"] = layer.decay_rank
            mlp = layer.mlp
            kept: dict[str, object] | None = None
            if mlp is not None and mlp.kind == "dense":
                kept = {"kind": "dense", "ff": mlp.ff}
            elif mlp is not None:
                kept = {"kind": "moe", "expert": {"ff": mlp.ff},
                        "router": {"experts": mlp.experts, "top": mlp.top}}
            entries.append({"type": layer.kind, "mixer": mixer, "mlp": kept})
        out: dict[str, object] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.eps}, "embedding": {"scale": self.embedding_scale},
            "layers": entries}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        return out


def _mlp(value: object, where: str) -> RizitarMlp | None:
    if value is None:
        return None
    mlp = _object(value, where)
    kind = mlp.get("kind")
    if kind == "dense":
        return RizitarMlp("dense", _count(mlp.get("ff"), f"{where}.ff"))
    if kind != "moe":
        raise ModelLoadError(f"{where}.kind {kind!r} is not a feed-forward of this design; "
                             "known: dense, moe")
    _require(mlp, ("expert", "router"), where)
    router = _object(mlp["router"], f"{where}.router")
    _require(router, ("experts", "top"), f"{where}.router")
    experts = _count(router["experts"], f"{where}.router.experts")
    top = _count(router["top"], f"{where}.router.top")
    if top > experts:
        raise ConfigError(f"{where}.router.top", "INVALID_RANGE", "must be at most experts")
    return RizitarMlp(
        "moe", _count(_object(mlp["expert"], f"{where}.expert").get("ff"), f"{where}.expert.ff"),
        experts=experts, top=top)


def _rotation(value: object, dim: int, path: str) -> RizitarRotation | None:
    if value is None:
        return None
    rot = _object(value, path)
    _require(rot, ("dims", "base"), path)
    dims = _count(rot["dims"], f"{path}.dims", minimum=0)
    if dims == 0:
        return None
    base = _number(rot["base"], f"{path}.base")
    if dims % 2 or dims > dim or base <= 1.0:
        raise ConfigError(path, "INVALID_RANGE",
                          "dims must be even and at most dim, base greater than 1")
    scaling = rot.get("scaling")
    if scaling is None:
        return RizitarRotation(dims, base)
    scaling = _object(scaling, f"{path}.scaling")
    _require(scaling, ("factor", "original", "fast", "slow"), f"{path}.scaling")
    numbers = {key: _number(scaling[key], f"{path}.scaling.{key}")
               for key in ("factor", "original", "fast", "slow")}
    if min(numbers.values()) <= 0:
        raise ConfigError(f"{path}.scaling", "INVALID_RANGE", "every entry must be positive")
    return RizitarRotation(dims, base, **numbers)


def _layer(entry: Mapping[str, object], index: int) -> RizitarLayer:
    where = f"model.layers[{index}]"
    kind = entry.get("type")
    if kind not in ("attention", "general_delta"):
        raise ModelLoadError(f"{where}.type {kind!r} is not a mixer of this design; known: "
                             "attention, general_delta")
    path = f"{where}.mixer"
    mixer = _object(entry.get("mixer"), path)
    _require(mixer, ("heads", "dim") + (("scale",) if kind == "attention" else ()), path)
    heads = _count(mixer["heads"], f"{path}.heads")
    dim = _count(mixer["dim"], f"{path}.dim")
    mlp = _mlp(entry.get("mlp"), f"{where}.mlp")
    if kind == "general_delta":
        rank = mixer.get("decay_rank")
        return RizitarLayer("general_delta", heads, dim, mlp=mlp, decay_rank=None
                            if rank is None else _count(rank, f"{path}.decay_rank"))
    kv_heads = heads if mixer.get("kv_heads") is None \
        else _count(mixer["kv_heads"], f"{path}.kv_heads")
    if heads % kv_heads:
        raise ConfigError(f"{path}.kv_heads", "INVALID_RANGE", "must divide heads")
    vdim = dim if mixer.get("vdim") is None else _count(mixer["vdim"], f"{path}.vdim")
    if vdim != dim:
        raise ConfigError(f"{path}.vdim", "INVALID_RANGE",
                          "the values are the keys as projected: vdim must equal dim")
    mask = mixer.get("mask")
    mask = {} if mask is None else _object(mask, f"{path}.mask")
    window = 0 if mask.get("size") is None else _count(mask["size"], f"{path}.mask.size")
    pool = 0 if mask.get("pool") is None or not window \
        else _count(mask["pool"], f"{path}.mask.pool", minimum=0)
    return RizitarLayer("attention", heads, dim, kv_heads=kv_heads, vdim=vdim,
                        scale=_number(mixer["scale"], f"{path}.scale"), window=window, pool=pool,
                        rot=_rotation(mixer.get("rot"), dim, f"{path}.rot"), mlp=mlp)
