"""Arrangements: how one layer wires its norms, its mixer and its feed-forward."""

from __future__ import annotations

import torch

from ayaka_b200.kernels import ops
from ayaka_b200.parts.base import BuildContext, Part, build_part, register_part
from ayaka_b200.parts.context import LayerCache, StepContext, Workspace
from ayaka_b200.parts.spec import LayerSpec

__all__ = ["Block", "OutputNormBlock", "ParallelBlock", "PreNormBlock", "SandwichNormBlock"]


class Block(Part):
    """Interface of an arrangement: ``forward(residual, step, cache)`` updates the fp32
    residual stream ``[N, width]`` in place. ``mixer`` is exposed for the cache planner."""

    mixer: Part

    def forward(self, residual: torch.Tensor, step: StepContext, cache: LayerCache) -> None:
        raise NotImplementedError


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    """``x += mixer(norm(x)); x += feed_forward(norm(x))`` — GPT-2's block
    (``python/ayaka/models/gpt2.py:99-101``). The sums happen in fp32 inside the last matrix
    product of each half.

    With ``spec.layer_scale`` each half's result is multiplied element by element by a vector
    of the model's width (``mixer_scale``, ``feed_forward_scale``) before the sum: a part that
    has ``forward_scaled(hidden, residual, step[, cache], scale)`` applies the vector in its
    own last kernel; any other part writes into a scratch row that one more kernel scales and
    adds."""

    def __init__(self, spec: LayerSpec, ctx: BuildContext, position: Part | None) -> None:
        super().__init__(ctx)
        self.mixer_norm = self.add_child(
            "mixer_norm", build_part("norm", spec.mixer_norm.kind, spec.mixer_norm, ctx))
        self.mixer = self.add_child(
            "mixer", build_part("mixer", spec.mixer.kind, spec.mixer, ctx, position))
        # a layer without a feed-forward has no second norm either
        self.feed_forward_norm = None if spec.feed_forward.kind == "none" else self.add_child(
            "feed_forward_norm",
            build_part("norm", spec.feed_forward_norm.kind, spec.feed_forward_norm, ctx))
        self.feed_forward = self.add_child(
            "feed_forward",
            build_part("feed_forward", spec.feed_forward.kind, spec.feed_forward, ctx))
        self.width = int(spec.mixer_norm.width)  # type: ignore[arg-type]
        self.mixer_scale = self.feed_forward_scale = None
        if spec.layer_scale:
            self.mixer_scale = self.add_param("mixer_scale", (self.width,), "vector")
            if spec.feed_forward.kind != "none":
                self.feed_forward_scale = self.add_param("feed_forward_scale", (self.width,),
                                                         "vector")

    def native_run(self, workspace: Workspace):  # noqa: ANN201
        """``(attention part, feed-forward part)`` for the C++ host code when both halves of
        this layer can run there (fusable norms, parts that know how to pack themselves),
        else ``None``; see ``kernels/native.py``."""
        if self.mixer_scale is not None:
            return None
        if not (_plain_norm(self.mixer_norm) and _plain_norm(self.feed_forward_norm)
                and hasattr(self.mixer, "native_part")
                and hasattr(self.feed_forward, "native_part")):
            return None
        attention = self.mixer.native_part(self.mixer_norm, workspace)  # type: ignore
        mlp = self.feed_forward.native_part(self.feed_forward_norm, workspace)  # type: ignore
        return None if attention is None or mlp is None else (attention, mlp)

    def forward(self, residual: torch.Tensor, step: StepContext, cache: LayerCache) -> None:
        n = step.num_rows
        hidden = step.workspace.buffer("block.normed", self.width, self.ctx.dtype)
        if self.mixer_scale is not None:
            self._forward_scaled(hidden, residual, step, cache)
            return
        # a part that can apply the norm itself gets the residual and the norm part
        if hasattr(self.mixer, "forward_normed") and _plain_norm(self.mixer_norm):
            self.mixer.forward_normed(self.mixer_norm, residual, step, cache)  # type: ignore
        else:
            self.mixer_norm.forward(residual, hidden, count=n)  # type: ignore[attr-defined]
            self.mixer.forward(hidden, residual, step, cache)  # type: ignore[attr-defined]
        if self.feed_forward_norm is None:
            return
        if hasattr(self.feed_forward, "forward_normed") and _plain_norm(self.feed_forward_norm):
            self.feed_forward.forward_normed(  # type: ignore[attr-defined]
                self.feed_forward_norm, residual, step)
        else:
            self.feed_forward_norm.forward(residual, hidden, count=n)  # type: ignore
            self.feed_forward.forward(hidden, residual, step)  # type: ignore[attr-defined]


    def _forward_scaled(self, hidden: torch.Tensor, residual: torch.Tensor, step: StepContext,
                        cache: LayerCache) -> None:
        n = step.num_rows
        self.mixer_norm.forward(residual, hidden, count=n)  # type: ignore[attr-defined]
        if hasattr(self.mixer, "forward_scaled"):
            self.mixer.forward_scaled(hidden, residual, step, cache,  # type: ignore
                                      self.mixer_scale)
        else:
            branch = self._empty_branch(step)
            self.mixer.forward(hidden, branch, step, cache)  # type: ignore[attr-defined]
            ops.scale_add(branch, self.mixer_scale, residual, rows=n)
        if self.feed_forward_scale is None or self.feed_forward_norm is None:
            return
        self.feed_forward_norm.forward(residual, hidden, count=n)  # type: ignore
        if hasattr(self.feed_forward, "forward_scaled"):
            self.feed_forward.forward_scaled(hidden, residual, step,  # type: ignore
                                             self.feed_forward_scale)
        else:
            branch = self._empty_branch(step)
            self.feed_forward.forward(hidden, branch, step)  # type: ignore[attr-defined]
            ops.scale_add(branch, self.feed_forward_scale, residual, rows=n)

    def _empty_branch(self, step: StepContext) -> torch.Tensor:
        """A zeroed fp32 scratch row per row of the step (parts add into what they get)."""
        branch = step.workspace.buffer("block.branch", self.width, torch.float32)
        branch[:step.num_rows].zero_()
        return branch


@register_part("block", "parallel")
class ParallelBlock(Block):
    """``h = norm(x); x += mixer(h) + feed_forward(h)``: one norm, and both halves read its
    output. Each half adds its result into the fp32 residual stream in the epilogue of its
    last matrix product, the mixer first. The layer's norm is ``spec.mixer_norm``
    (``spec.feed_forward_norm`` is not built)."""

    def __init__(self, spec: LayerSpec, ctx: BuildContext, position: Part | None) -> None:
        super().__init__(ctx)
        self.mixer_norm = self.add_child(
            "mixer_norm", build_part("norm", spec.mixer_norm.kind, spec.mixer_norm, ctx))
        self.mixer = self.add_child(
            "mixer", build_part("mixer", spec.mixer.kind, spec.mixer, ctx, position))
        self.feed_forward = self.add_child(
            "feed_forward",
            build_part("feed_forward", spec.feed_forward.kind, spec.feed_forward, ctx))
        self.width = int(spec.mixer_norm.width)  # type: ignore[arg-type]

    def forward(self, residual: torch.Tensor, step: StepContext, cache: LayerCache) -> None:
        # a buffer of its own: the halves' own scratch must not overwrite what both read
        hidden = step.workspace.buffer("block.shared_normed", self.width, self.ctx.dtype)
        self.mixer_norm.forward(residual, hidden, count=step.num_rows)  # type: ignore
        self.mixer.forward(hidden, residual, step, cache)  # type: ignore[attr-defined]
        self.feed_forward.forward(hidden, residual, step)  # type: ignore[attr-defined]


def _can_follow(norm: object) -> bool:
    """Whether ``norm`` is a root-mean-square norm that ``ops.norm_add`` can apply on its way
    out (``weight``, ``offset``, ``eps`` and ``width``)."""
    return all(hasattr(norm, name) for name in ("weight", "offset", "eps", "width"))


def _plain_norm(norm: Part | None) -> bool:
    """Whether ``norm`` declares itself a LayerNorm that a fused kernel can apply from its
    (weight, bias, eps); see ``parts/norm.py``."""
    return bool(getattr(norm, "fusable_layer_norm", False))


@register_part("block", "output_norm")
class OutputNormBlock(Block):
    """``x += f * norm1(mixer(x)); x += f * norm2(feed_forward(x))`` and, with a ``side``
    part, ``x += f * side(x)``: the norms stand on the sublayers' *outputs*, the sublayers
    read the residual stream itself, and ``f`` is ``spec.residual_factor``.

    The stream is fp32; a sublayer's matrix operand is its rounding to the compute type, kept
    in one scratch tensor that every kernel which updates the stream also refreshes
    (``ops.norm_add`` with ``copy``), so only a model's first layer pays a pass of its own for
    it. In float32 the sublayers read the stream directly. A sublayer writes into a scratch
    branch (``forward_into`` where the part has it, else a zeroed branch it adds into)."""

    def __init__(self, spec: LayerSpec, ctx: BuildContext, position: Part | None) -> None:
        super().__init__(ctx)
        self.mixer_norm = self.add_child(
            "mixer_norm", build_part("norm", spec.mixer_norm.kind, spec.mixer_norm, ctx))
        self.mixer = self.add_child(
            "mixer", build_part("mixer", spec.mixer.kind, spec.mixer, ctx, position))
        self.feed_forward_norm = None if spec.feed_forward.kind == "none" else self.add_child(
            "feed_forward_norm",
            build_part("norm", spec.feed_forward_norm.kind, spec.feed_forward_norm, ctx))
        self.feed_forward = self.add_child(
            "feed_forward",
            build_part("feed_forward", spec.feed_forward.kind, spec.feed_forward, ctx))
        self.side = None if spec.side is None else self.add_child(
            "side", build_part("side", spec.side.kind, spec.side, ctx))
        self.width = int(spec.mixer_norm.width)  # type: ignore[arg-type]
        self.factor = float(spec.residual_factor)
        for norm in (self.mixer_norm, self.feed_forward_norm):
            if norm is not None and not hasattr(norm, "add_normed"):
                raise ValueError("an output_norm block needs norms that can add their result "
                                 "to the stream (add_normed)")

    def forward(self, residual: torch.Tensor, step: StepContext, cache: LayerCache) -> None:
        n, work = step.num_rows, step.workspace
        rounded = self.ctx.dtype != torch.float32
        if rounded:
            stream = work.buffer("block.stream", self.width, self.ctx.dtype)
            if not step.extra.get("block.stream_copy"):
                ops.cast_rows(residual, stream, rows=n)
            step.extra["block.stream_copy"] = True
        else:
            stream = residual
        copy = stream if rounded else None
        branch = work.buffer("block.branch", self.width, torch.float32)
        if hasattr(self.mixer, "forward_into"):
            self.mixer.forward_into(stream, branch, step, cache)  # type: ignore[attr-defined]
        else:
            branch[:n].zero_()
            self.mixer.forward(stream, branch, step, cache)  # type: ignore[attr-defined]
        self.mixer_norm.add_normed(branch, residual, factor=self.factor,  # type: ignore
                                   count=n, copy=copy)
        if self.feed_forward_norm is not None:
            if hasattr(self.feed_forward, "forward_into"):
                self.feed_forward.forward_into(stream, branch, step)  # type: ignore
            else:
                branch[:n].zero_()
                self.feed_forward.forward(stream, branch, step)  # type: ignore[attr-defined]
            self.feed_forward_norm.add_normed(branch, residual,  # type: ignore[attr-defined]
                                              factor=self.factor, count=n, copy=copy)
        if self.side is not None:
            self.side.forward(stream, residual, step, factor=self.factor,  # type: ignore
                              copy=copy)


@register_part("block", "sandwich_norm")
class SandwichNormBlock(Block):
    """``x += post1(mixer(pre1(x))); x += post2(feed_forward(pre2(x)))`` and, with a ``side``
    part, ``x += f * side(x)``: a norm in front of every sublayer and another on its output.
    The norms in front are ``spec.mixer_norm`` / ``spec.feed_forward_norm`` (children
    ``mixer_norm``, ``feed_forward_norm``); the ones behind have the same kind and sizes and
    weights of their own (children ``mixer_post_norm``, ``feed_forward_post_norm``). ``f`` is
    ``spec.residual_factor`` and stands on everything that joins the stream.

    The stream is fp32. A sublayer reads its norm's output in the compute type and writes a
    fp32 branch (``forward_into`` where the part has it, else a zeroed branch it adds into);
    the norm behind it adds ``f * norm(branch)`` to the stream in one launch, and for a side
    part that launch also leaves the new stream rounded once to the compute type.

    The norm in front of a sublayer is applied by the launch that last updated the stream (the
    norm behind the sublayer before it, or the side part's), which holds the new row in
    registers: the mixer's by the layer before (the model names the next layer's norm in
    ``step.extra["block.next_norm"]`` and this block marks ``step.extra["block.normed_by"]``
    when it has applied it), the feed-forward's by this layer's own first half. Only a
    model's first layer launches a norm of its own."""

    def __init__(self, spec: LayerSpec, ctx: BuildContext, position: Part | None) -> None:
        super().__init__(ctx)
        has_ff = spec.feed_forward.kind != "none"

        def norm(name: str, part: object) -> Part:
            return self.add_child(name, build_part("norm", part.kind, part, ctx))  # type: ignore

        self.mixer_norm = norm("mixer_norm", spec.mixer_norm)
        self.mixer = self.add_child(
            "mixer", build_part("mixer", spec.mixer.kind, spec.mixer, ctx, position))
        self.mixer_post_norm = norm("mixer_post_norm", spec.mixer_norm)
        self.feed_forward_norm = norm("feed_forward_norm", spec.feed_forward_norm) \
            if has_ff else None
        self.feed_forward = self.add_child(
            "feed_forward",
            build_part("feed_forward", spec.feed_forward.kind, spec.feed_forward, ctx))
        self.feed_forward_post_norm = norm("feed_forward_post_norm", spec.feed_forward_norm) \
            if has_ff else None
        self.side = None if spec.side is None else self.add_child(
            "side", build_part("side", spec.side.kind, spec.side, ctx))
        self.width = int(spec.mixer_norm.width)  # type: ignore[arg-type]
        self.factor = float(spec.residual_factor)
        for post in (self.mixer_post_norm, self.feed_forward_post_norm):
            if post is not None and not hasattr(post, "add_normed"):
                raise ValueError("a sandwich_norm block needs norms that can add their result "
                                 "to the stream (add_normed)")

    def forward(self, residual: torch.Tensor, step: StepContext, cache: LayerCache) -> None:
        n, work = step.num_rows, step.workspace
        rounded = self.ctx.dtype != torch.float32
        hidden = work.buffer("block.normed", self.width, self.ctx.dtype)
        branch = work.buffer("block.branch", self.width, torch.float32)
        # the side part reads the stream itself: the last norm behind a sublayer leaves it a
        # copy in the compute type (in float32 it reads the stream)
        copy = work.buffer("block.stream", self.width, self.ctx.dtype) \
            if rounded and self.side is not None else None
        last_is_mixer = self.feed_forward_norm is None
        # the norm of the layer that follows, if the model named one this block can apply
        following = step.extra.pop("block.next_norm", None)
        if not (_can_follow(following) and following.width == self.width):
            following = None
        if step.extra.pop("block.normed_by", None) is not self.mixer_norm:
            self.mixer_norm.forward(residual, hidden, count=n)  # type: ignore[attr-defined]
        if hasattr(self.mixer, "forward_into"):
            self.mixer.forward_into(hidden, branch, step, cache)  # type: ignore[attr-defined]
        else:
            branch[:n].zero_()
            self.mixer.forward(hidden, branch, step, cache)  # type: ignore[attr-defined]
        # which norm the launch that updates the stream applies on its way out, into `hidden`
        fused_second = not last_is_mixer and _can_follow(self.feed_forward_norm)
        after_mixer = self.feed_forward_norm if fused_second else (
            following if last_is_mixer and self.side is None else None)
        self.mixer_post_norm.add_normed(branch, residual, factor=self.factor,  # type: ignore
                                        count=n, copy=copy if last_is_mixer else None,
                                        then=after_mixer, then_out=hidden)
        if self.feed_forward_norm is not None:
            if not fused_second:
                self.feed_forward_norm.forward(residual, hidden, count=n)  # type: ignore
            if hasattr(self.feed_forward, "forward_into"):
                self.feed_forward.forward_into(hidden, branch, step)  # type: ignore
            else:
                branch[:n].zero_()
                self.feed_forward.forward(hidden, branch, step)  # type: ignore[attr-defined]
            self.feed_forward_post_norm.add_normed(  # type: ignore[union-attr]
                branch, residual, factor=self.factor, count=n, copy=copy,
                then=following if self.side is None else None, then_out=hidden)
        if self.side is not None:
            self.side.forward(copy if rounded else residual, residual, step,  # type: ignore
                              factor=self.factor, then=following, then_out=hidden)
        if following is not None:
            step.extra["block.normed_by"] = following
