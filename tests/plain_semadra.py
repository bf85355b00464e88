"""Semadra, plainly: whole sequences in float64, one function per mechanism, no cache.

The model is a ``config.json`` dictionary and a dictionary of tensors under checkpoint names.
Nothing here is shared with the engine; it is the slow statement of the equations that the
engine's kernels are compared with.
"""

from __future__ import annotations

import math

import torch

__all__ = ["attention_layer", "cast_state", "dense", "expert_choice", "forward", "gelu_tanh",
           "greedy_generate", "latent", "latent_attention_layer", "logits", "mixture", "rms",
           "router_margins", "side_input", "softmax_attention", "visible"]

F64 = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """``x / sqrt(mean(x^2) + eps)`` over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def visible(length: int, size: int, keep_first: int = 0) -> torch.Tensor:
    """``[query, key]`` booleans: key ``j`` is seen from ``i`` when it is not later and either
    closer than ``size`` or among the first ``keep_first`` of the sequence."""
    i = torch.arange(length)[:, None]
    j = torch.arange(length)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                      mask: torch.Tensor) -> torch.Tensor:
    """``q`` ``[T, H, d]``, ``k`` ``[T, G, d]``, ``v`` ``[T, G, e]``; head ``h`` uses key/value
    head ``h // (H / G)``. Returns ``[T, H * e]``."""
    length, heads, _ = q.shape
    per = heads // k.shape[1]
    out = []
    for h in range(heads):
        g = h // per
        scores = (q[:, h] @ k[:, g].T) * scale
        scores = scores.masked_fill(~mask, -math.inf)
        out.append(torch.softmax(scores, dim=-1) @ v[:, g])
    return torch.cat(out, dim=-1)


def attention_layer(h: torch.Tensor, w: dict[str, torch.Tensor], p: str, mixer: dict,
                    eps: float) -> torch.Tensor:
    heads, groups = mixer["heads"], mixer.get("kv_heads", mixer["heads"])
    dim, vdim = mixer["dim"], mixer["vdim"]
    length = h.shape[0]
    q = rms(h @ w[p + "q"].T, eps) * w[p + "q.norm"]
    k = rms(h @ w[p + "k"].T, eps) * w[p + "k.norm"]
    v = h @ w[p + "v"].T
    mask = visible(length, (mixer.get("mask") or {}).get("size") or length,
                   (mixer.get("mask") or {}).get("keep_first", 0))
    joined = softmax_attention(q.view(length, heads, dim), k.view(length, groups, dim),
                               v.view(length, groups, vdim), mixer["scale"], mask)
    return (joined * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def latent(h: torch.Tensor, w: dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    """The cached rows of a latent attention layer that owns a down-projection."""
    return rms(h @ w[p + "dkv"].T, eps) * w[p + "dkv.norm"]


def latent_attention_layer(h: torch.Tensor, c: torch.Tensor, w: dict[str, torch.Tensor], p: str,
                           mixer: dict, eps: float) -> torch.Tensor:
    heads, dim, vdim = mixer["heads"], mixer["dim"], mixer["vdim"]
    length = h.shape[0]
    cq = rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).view(length, heads, dim)
    k = (c @ w[p + "uk"].T).view(length, heads, dim)
    v = (c @ w[p + "uv"].T).view(length, heads, vdim)
    joined = softmax_attention(q, k, v, mixer["scale"],
                               visible(length, (mixer.get("mask") or {}).get("size") or length))
    return joined @ w[p + "o"].T


def dense(h: torch.Tensor, w: dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def expert_choice(scores: torch.Tensor, top: int, count: int, keep: int) -> torch.Tensor:
    """Indices ``[T, top]`` of the chosen experts: the largest scores among the experts of the
    ``keep`` groups (of ``count`` equal groups of neighbours) whose two largest scores sum
    highest."""
    length, experts = scores.shape
    grouped = scores.view(length, count, experts // count)
    group_score = grouped.topk(min(2, experts // count), dim=-1).values.sum(-1)
    best = group_score.topk(keep, dim=-1).indices
    allowed = torch.zeros(length, count, dtype=torch.bool)
    allowed.scatter_(1, best, True)
    allowed = allowed[:, :, None].expand_as(grouped).reshape(length, experts)
    return scores.masked_fill(~allowed, -math.inf).topk(top, dim=-1).indices


def choice_margin(scores: torch.Tensor, top: int, count: int, keep: int) -> torch.Tensor:
    """Per row, how close the choice was: the smaller of the gap between the last kept and the
    first dropped group's score and the gap between the last chosen and the first unchosen
    score among the kept groups' experts (scores lie in (0, 1))."""
    length, experts = scores.shape
    margin = torch.full((length,), float("inf"), dtype=scores.dtype)
    grouped = scores.view(length, count, experts // count)
    group_score = grouped.topk(min(2, experts // count), dim=-1).values.sum(-1)
    if keep < count:
        ordered = group_score.sort(dim=-1, descending=True).values
        margin = torch.minimum(margin, ordered[:, keep - 1] - ordered[:, keep])
    best = group_score.topk(keep, dim=-1).indices
    allowed = torch.zeros(length, count, dtype=torch.bool).scatter_(1, best, True)
    allowed = allowed[:, :, None].expand_as(grouped).reshape(length, experts)
    ordered = scores.masked_fill(~allowed, -1.0).sort(dim=-1, descending=True).values
    if top < experts and top < keep * (experts // count):
        margin = torch.minimum(margin, ordered[:, top - 1] - ordered[:, top])
    return margin


def mixture(h: torch.Tensor, w: dict[str, torch.Tensor], p: str, mlp: dict,
            margins: list[torch.Tensor] | None = None) -> torch.Tensor:
    router = mlp["router"]
    scores = torch.sigmoid(h @ w[p + "router"].T)
    groups = router.get("groups") or {"count": 1, "keep": 1}
    chosen = expert_choice(scores, router["top"], groups["count"], groups["keep"])
    if margins is not None:
        margins.append(choice_margin(scores, router["top"], groups["count"], groups["keep"]))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            out[t] += scores[t, e] * router["scale"] * dense(h[t:t + 1], w, f"{p}e{e}.")[0]
    if mlp.get("shared") is not None:
        out = out + dense(h, w, p + "shared.")
    return out


def side_input(x: torch.Tensor, tokens: torch.Tensor, w: dict[str, torch.Tensor], p: str,
               index: int, dim: int, eps: float) -> torch.Tensor:
    """The normed per-layer token input (before the residual factor)."""
    e = w["side.embed"][tokens, index * dim:(index + 1) * dim]
    y = (gelu_tanh(x @ w[p + "gate"].T) * e) @ w[p + "proj"].T
    return rms(y, eps) * w[p + "norm"]


def forward(config: dict, weights: dict[str, torch.Tensor], tokens: list[int],
            layers_out: list[torch.Tensor] | None = None,
            margins: list[torch.Tensor] | None = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one sequence; ``layers_out`` collects the residual stream after
    every layer, ``margins`` every router's closeness of choice."""
    w = {name: t.to(F64) if t.is_floating_point() else t for name, t in weights.items()}
    eps, m = config["norm"]["eps"], config.get("residual_mult", 1.0)
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"][ids] * (config.get("embedding") or {}).get("scale", 1.0)
    latents: dict[int, torch.Tensor] = {}
    side = config.get("token_side")
    for i, layer in enumerate(config["layers"]):
        p, mixer = f"l{i}.", layer["mixer"]
        if layer["type"] == "attention":
            y = attention_layer(x, w, p + "mix.", mixer, eps)
        else:
            source = mixer.get("kv_from")
            if source is None:
                latents[i] = latent(x, w, p + "mix.", eps)
                source = i
            y = latent_attention_layer(x, latents[source], w, p + "mix.", mixer, eps)
        x = x + m * rms(y, eps) * (1.0 + w[p + "norm1"])
        mlp = layer.get("mlp")
        if mlp is not None:
            y = dense(x, w, p + "mlp.") if mlp["kind"] == "dense" \
                else mixture(x, w, p + "mlp.", mlp, margins)
            x = x + m * rms(y, eps) * (1.0 + w[p + "norm2"])
        if side is not None:
            x = x + m * side_input(x, ids, w, p + "side.", i, side["dim"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rms(x, eps) * (1.0 + w["final.norm"])
    return x @ w["embed"].T


def cast_state(state: dict, dtype: torch.dtype) -> dict:
    return {name: t.to(dtype) if t.is_floating_point() else t for name, t in state.items()}


def logits(state: dict, config: dict, tokens: torch.Tensor) -> torch.Tensor:
    return forward(config, state, tokens)


def router_margins(state: dict, config: dict, tokens: torch.Tensor) -> torch.Tensor:
    """Per position, the smallest closeness of choice over the layers' routers. Where it is
    below the rounding of an engine's arithmetic the model is discontinuous: another expert
    may rightly be chosen there, and the logits jump."""
    margins: list[torch.Tensor] = []
    forward(config, state, tokens, margins=margins)
    out = torch.full((len(tokens),), float("inf"), dtype=F64)
    for margin in margins:
        out = torch.minimum(out, margin)
    return out


def greedy_generate(state: dict, config: dict, prompt: list[int], count: int) -> list[int]:
    """``count`` tokens, each the largest logit (smallest id on ties) of the whole sequence
    so far run from scratch."""
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(torch.argmax(forward(config, state, tokens)[-1])))
    return tokens[len(prompt):]
