"""The typed configuration of a Semadra model, read from its own ``config.json`` keys.

Semadra is a decoder whose sublayers read the residual stream itself and are normed on their
*output*: ``x += m * norm1(mixer(x)); x += m * norm2(mlp(x))``, then a small gated embedding of
the row's own token joins the stream. ``config.json``::

    {"architecture": "Semadra", "vocab": V, "width": D, "norm": {"eps": e},
     "embedding": {"scale": s}, "residual_mult": m, "token_side": {"dim": d},
     "layers": [{"type": "attention" | "latent_attention", "mixer": {...},
                 "mlp": {"kind": "dense", "ff": F}
                      | {"kind": "moe", "expert": {"ff": F}, "router": {"experts": E, "top": k,
                         "scale": r, "groups": {"count": g, "keep": n}}, "shared": {"ff": S}}
                      | null}, ...]}

``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size``,
``mask.keep_first``. ``latent_attention``: ``heads``, ``dim``, ``vdim``, ``q_rank``,
``kv_rank``, ``scale``, ``mask.size`` and optionally ``kv_from`` (the index of an earlier
latent layer whose cached latents this layer reads instead of projecting its own).

Keys whose absence has one natural meaning may be left out: ``kv_heads`` (= ``heads``),
``mask`` or ``mask.size`` (no window), ``mask.keep_first`` (0), ``router.groups`` (one group),
``shared`` (no shared expert), ``token_side`` (no token input), ``embedding.scale`` and
``residual_mult`` (1). Every other key is required.
"""

from __future__ import annotations

import math
from collections.abc import Mapping
from dataclasses import dataclass

from ayaka_b200.errors import ConfigError, ModelLoadError

__all__ = ["SemadraConfig", "SemadraLayer", "SemadraMlp"]


def _number(value: object, path: str) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or \
            not math.isfinite(value):
        raise ConfigError(path, "WRONG_TYPE", f"must be a finite number, got {value!r}")
    return float(value)


def _count(value: object, path: str, minimum: int = 1) -> int:
    if type(value) is not int:
        raise ConfigError(path, "WRONG_TYPE", f"must be an integer, got {value!r}")
    if value < minimum:
        raise ConfigError(path, "INVALID_RANGE", f"must be at least {minimum}, got {value}")
    return value


def _object(value: object, path: str) -> Mapping[str, object]:
    if not isinstance(value, Mapping):
        raise ConfigError(path, "WRONG_TYPE", "must be an object")
    return value


def _require(mapping: Mapping[str, object], keys: tuple[str, ...], path: str) -> None:
    lacking = [key for key in keys if mapping.get(key) is None]
    if lacking:
        raise ModelLoadError(f"{path} lacks " + ", ".join(lacking),
                             context={"missing": tuple(lacking)})


@dataclass(frozen=True, slots=True)
class SemadraMlp:
    """A layer's feed-forward. ``kind`` ``dense``: ``ff`` is its inner width. ``moe``: ``ff``
    is an expert's inner width, ``experts`` of which each row uses ``top``, in ``groups`` equal
    groups of which the best ``keep`` may be chosen from, weights ``route_scale * score``;
    ``shared_ff`` > 0: a shared expert of that inner width."""

    kind: str
    ff: int
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1
    route_scale: float = 1.0
    shared_ff: int = 0


@dataclass(frozen=True, slots=True)
class SemadraLayer:
    """One entry of ``layers``. ``kind`` ``attention`` uses ``kv_heads`` and ``keep_first``;
    ``latent_attention`` uses ``q_rank``, ``kv_rank`` and ``kv_from`` (``None``: its own
    latents). ``window`` 0: no window."""

    kind: str
    heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    kv_heads: int = 0
    keep_first: int = 0
    q_rank: int = 0
    kv_rank: int = 0
    kv_from: int | None = None
    mlp: SemadraMlp | None = None


@dataclass(frozen=True, slots=True)
class SemadraConfig:
    """Everything ``config.json`` says. ``side_dim`` 0: no per-layer token input."""

    architecture: str
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    residual_mult: float
    side_dim: int
    layers: tuple[SemadraLayer, ...]

    @classmethod
    def from_json_dict(cls, config: Mapping[str, object]) -> SemadraConfig:
        _require(config, ("architecture", "vocab", "width", "norm", "layers"), "config.json")
        eps = _number(_object(config["norm"], "model.norm").get("eps"), "model.norm.eps")
        if eps <= 0:
            raise ConfigError("model.norm.eps", "INVALID_RANGE", "must be positive")
        entries = config["layers"]
        if not isinstance(entries, (list, tuple)) or not entries:
            raise ConfigError("model.layers", "WRONG_TYPE", "must be a non-empty list")
        layers: list[SemadraLayer] = []
        for index, entry in enumerate(entries):
            layers.append(_layer(_object(entry, f"model.layers[{index}]"), index, layers))
        embedding = config.get("embedding")
        scale = 1.0 if embedding is None or _object(embedding, "model.embedding").get("scale") \
            is None else _number(embedding["scale"], "model.embedding.scale")  # type: ignore
        mult = config.get("residual_mult")
        side = config.get("token_side")
        architecture = config["architecture"]
        if not isinstance(architecture, str) or not architecture:
            raise ConfigError("model.architecture", "WRONG_TYPE", "must be a non-empty string")
        return cls(
            architecture=architecture, vocab=_count(config["vocab"], "model.vocab"),
            width=_count(config["width"], "model.width"), eps=eps, embedding_scale=scale,
            residual_mult=1.0 if mult is None else _number(mult, "model.residual_mult"),
            side_dim=0 if side is None else _count(
                _object(side, "model.token_side").get("dim"), "model.token_side.dim"),
            layers=tuple(layers))

    def to_json_dict(self) -> dict[str, object]:
        """The ``config.json`` content that reads back as this configuration."""
        entries: list[dict[str, object]] = []
        for layer in self.layers:
            mask: dict[str, object] = {}
            if layer.window:
                mask["size"] = layer.window
            mixer: dict[str, object] = {"heads": layer.heads, "dim": layer.dim,
                                        "vdim": layer.vdim, "scale": layer.scale, "mask": mask}
            if layer.kind == "attention":
                mixer["kv_heads"] = layer.kv_heads
                mask["keep_first"] = layer.keep_first
            else:
                mixer["q_rank"], mixer["kv_rank"] = layer.q_rank, layer.kv_rank
                if layer.kv_from is not None:
                    mixer["kv_from"] = layer.kv_from
            mlp = layer.mlp
            stored: dict[str, object] | None = None
            if mlp is not None and mlp.kind == "dense":
                stored = {"kind": "dense", "ff": mlp.ff}
            elif mlp is not None:
                stored = {"kind": "moe", "expert": {"ff": mlp.ff},
                          "router": {"experts": mlp.experts, "top": mlp.top,
                                     "scale": mlp.route_scale,
                                     "groups": {"count": mlp.groups, "keep": mlp.keep}}}
                if mlp.shared_ff:
                    stored["shared"] = {"ff": mlp.shared_ff}
            entries.append({"type": layer.kind, "mixer": mixer, "mlp": stored})
        out: dict[str, object] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.eps}, "embedding": {"scale": self.embedding_scale},
            "residual_mult": self.residual_mult, "layers": entries}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        return out


def _mlp(value: object, where: str) -> SemadraMlp | None:
    if value is None:
        return None
    mlp = _object(value, where)
    kind = mlp.get("kind")
    if kind == "dense":
        return SemadraMlp("dense", _count(mlp.get("ff"), f"{where}.ff"))
    if kind != "moe":
        raise ModelLoadError(f"{where}.kind {kind!r} is not a feed-forward of this design; "
                             "known: dense, moe")
    _require(mlp, ("expert", "router"), where)
    router = _object(mlp["router"], f"{where}.router")
    _require(router, ("experts", "top"), f"{where}.router")
    experts = _count(router["experts"], f"{where}.router.experts")
    top = _count(router["top"], f"{where}.router.top")
    groups, keep = 1, 1
    if router.get("groups") is not None:
        grouping = _object(router["groups"], f"{where}.router.groups")
        groups = _count(grouping.get("count"), f"{where}.router.groups.count")
        keep = _count(grouping.get("keep"), f"{where}.router.groups.keep")
    if experts % groups or keep > groups or top > keep * (experts // groups):
        raise ConfigError(f"{where}.router", "INVALID_RANGE",
                          "groups.count must divide experts, groups.keep be at most "
                          "groups.count, and the kept groups hold at least top experts")
    shared = mlp.get("shared")
    return SemadraMlp(
        "moe", _count(_object(mlp["expert"], f"{where}.expert").get("ff"), f"{where}.expert.ff"),
        experts=experts, top=top, groups=groups, keep=keep,
        route_scale=1.0 if router.get("scale") is None
        else _number(router["scale"], f"{where}.router.scale"),
        shared_ff=0 if shared is None
        else _count(_object(shared, f"{where}.shared").get("ff"), f"{where}.shared.ff"))


def _layer(entry: Mapping[str, object], index: int, before: list[SemadraLayer]) -> SemadraLayer:
    where = f"model.layers[{index}]"
    kind = entry.get("type")
    if kind not in ("attention", "latent_attention"):
        raise ModelLoadError(f"{where}.type {kind!r} is not a mixer of this design; known: "
                             "attention, latent_attention")
    mixer = _object(entry.get("mixer"), f"{where}.mixer")
    keys = ("heads", "dim", "vdim", "scale") + \
        (() if kind == "attention" else ("q_rank", "kv_rank"))
    _require(mixer, keys, f"{where}.mixer")
    path = f"{where}.mixer"
    mask = mixer.get("mask")
    mask = {} if mask is None else _object(mask, f"{path}.mask")
    window = 0 if mask.get("size") is None else _count(mask["size"], f"{path}.mask.size")
    common = dict(heads=_count(mixer["heads"], f"{path}.heads"),
                  dim=_count(mixer["dim"], f"{path}.dim"),
                  vdim=_count(mixer["vdim"], f"{path}.vdim"),
                  scale=_number(mixer["scale"], f"{path}.scale"), window=window,
                  mlp=_mlp(entry.get("mlp"), f"{where}.mlp"))
    if kind == "attention":
        kv_heads = common["heads"] if mixer.get("kv_heads") is None \
            else _count(mixer["kv_heads"], f"{path}.kv_heads")
        if common["heads"] % kv_heads:  # type: ignore[operator]
            raise ConfigError(f"{path}.kv_heads", "INVALID_RANGE", "must divide heads")
        keep = 0 if mask.get("keep_first") is None \
            else _count(mask["keep_first"], f"{path}.mask.keep_first", minimum=0)
        return SemadraLayer("attention", kv_heads=kv_heads, keep_first=keep,
                            **common)  # type: ignore[arg-type]
    kv_rank = _count(mixer["kv_rank"], f"{path}.kv_rank")
    source = mixer.get("kv_from")
    if source is not None:
        source = _count(source, f"{path}.kv_from", minimum=0)
        if source >= index or before[source].kind != "latent_attention" or \
                before[source].kv_from is not None or before[source].kv_rank != kv_rank:
            raise ModelLoadError(
                f"{path}.kv_from must name an earlier latent attention layer that projects "
                "its own latents, of the same kv_rank")
    return SemadraLayer("latent_attention", q_rank=_count(mixer["q_rank"], f"{path}.q_rank"),
                        kv_rank=kv_rank, kv_from=source, **common)  # type: ignore[arg-type]
