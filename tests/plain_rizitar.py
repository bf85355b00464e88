"""A plain float64 Rizitar: whole sequences, no cache, one function per mechanism.

It shares no code with the engine. ``tensors`` maps checkpoint names to numpy arrays,
``config`` is the ``config.json`` content as a dict.

Notation: ``x`` is the residual stream ``[T, width]``; a layer is
``x += post1(mixer(pre1(x))); x += post2(ff(pre2(x))); x += side(x)``.
"""

from __future__ import annotations

import math

import numpy as np

__all__ = [
    "attention", "delta_rule", "dense", "forward", "logits", "mixture", "pooled_mask",
    "rms", "rotary_tables", "side_input", "xielu",
]


def rms(x: np.ndarray, weight: np.ndarray | None, eps: float) -> np.ndarray:
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return y if weight is None else y * weight


def gelu_tanh(z: np.ndarray) -> np.ndarray:
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z: float) -> float:
    return max(z, 0.0) + math.log1p(math.exp(-abs(z)))


def sigmoid(z: np.ndarray) -> np.ndarray:
    return 1.0 / (1.0 + np.exp(-z))


def xielu(z: np.ndarray, p: float, q: float) -> np.ndarray:
    """Positive side ``softplus(p) z^2 + z/2``, other side ``(1/2 + softplus(q)) (e^z - 1 - z)
    + z/2``."""
    up = softplus(p) * z * z + 0.5 * z
    down = (0.5 + softplus(q)) * (np.expm1(np.minimum(z, 0.0)) - z) + 0.5 * z
    return np.where(z > 0, up, down)


def rotary_tables(positions: np.ndarray, rot: dict) -> tuple[np.ndarray, np.ndarray]:
    """cos and sin ``[T, dims / 2]`` with the long-context blend of frequencies."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    i = np.arange(half, dtype=np.float64)
    freq = base ** (-2.0 * i / dims)
    gain = 1.0
    scaling = rot.get("scaling")
    if scaling:
        factor, original = float(scaling["factor"]), float(scaling["original"])

        def turn_dim(turns: float) -> float:
            return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
        hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
        ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        freq = freq / factor * ramp + freq * (1.0 - ramp)
        gain = 0.1 * math.log(factor) + 1.0
    angle = positions[:, None].astype(np.float64) * freq[None, :]
    return np.cos(angle) * gain, np.sin(angle) * gain


def rotate(x: np.ndarray, cos: np.ndarray, sin: np.ndarray, dims: int) -> np.ndarray:
    """``x`` ``[T, heads, dim]``; entry ``i`` pairs with ``i + dims / 2``."""
    half = dims // 2
    out = x.copy()
    a, b = x[..., :half], x[..., half:dims]
    out[..., :half] = a * cos[:, None, :] - b * sin[:, None, :]
    out[..., half:dims] = b * cos[:, None, :] + a * sin[:, None, :]
    return out


def pooled_mask(count: int, size: int, pool: int) -> tuple[np.ndarray, np.ndarray]:
    """``tokens[i, j]``: query ``i`` sees key ``j``; ``blocks[i, b]``: it sees the mean of
    block ``b`` (positions ``b * pool .. b * pool + pool - 1``, all at least ``size`` back)."""
    i = np.arange(count)[:, None]
    j = np.arange(count)[None, :]
    tokens = (i - j >= 0) & ((i - j < size) if size else True)
    nblocks = count // pool if (size and pool) else 0
    b = np.arange(nblocks)[None, :]
    blocks = (b * pool + pool - 1 <= i - size) if nblocks else np.zeros((count, 0), bool)
    return tokens, blocks


def attention(h: np.ndarray, t: dict, prefix: str, mixer: dict, eps: float) -> np.ndarray:
    heads, kv_heads = int(mixer["heads"]), int(mixer.get("kv_heads") or mixer["heads"])
    dim, vdim = int(mixer["dim"]), int(mixer["vdim"])
    count = h.shape[0]
    q = (h @ t[prefix + "q"].T).reshape(count, heads, dim)
    k = (h @ t[prefix + "k"].T).reshape(count, kv_heads, dim)
    v = k.copy()  # the values are the keys as projected
    q = rms(q, t[prefix + "q.norm"], eps)
    k = rms(k, t[prefix + "k.norm"], eps)
    rot = mixer.get("rot")
    if rot and int(rot["dims"]):
        cos, sin = rotary_tables(np.arange(count), rot)
        q, k = rotate(q, cos, sin, int(rot["dims"])), rotate(k, cos, sin, int(rot["dims"]))
    mask = mixer.get("mask") or {}
    size, pool = int(mask.get("size") or 0), int(mask.get("pool") or 0)
    tokens, blocks = pooled_mask(count, size, pool)
    nblocks = blocks.shape[1]
    kb = k[:nblocks * pool].reshape(nblocks, max(pool, 1), kv_heads, dim).sum(axis=1) / max(pool, 1)
    vb = v[:nblocks * pool].reshape(nblocks, max(pool, 1), kv_heads, vdim).sum(axis=1) / max(pool, 1)
    scale = float(mixer["scale"])
    sink = t.get(prefix + "sink")
    out = np.zeros((count, heads, vdim))
    for head in range(heads):
        g = head // (heads // kv_heads)
        s_tok = np.where(tokens, q[:, head] @ k[:, g].T * scale, -np.inf)
        s_blk = np.where(blocks, q[:, head] @ kb[:, g].T * scale, -np.inf)
        s = np.concatenate([s_tok, s_blk], axis=1)
        top = s.max(axis=1, keepdims=True)
        if sink is not None:
            top = np.maximum(top, float(sink[head]))
        w = np.exp(s - top)
        below = w.sum(axis=1, keepdims=True)
        if sink is not None:
            below = below + np.exp(float(sink[head]) - top)
        w = w / below
        out[:, head] = w[:, :count] @ v[:, g] + w[:, count:] @ vb[:, g]
    return out.reshape(count, heads * vdim) @ t[prefix + "o"].T


def delta_rule(h: np.ndarray, t: dict, prefix: str, mixer: dict, eps: float,
               state: np.ndarray | None = None) -> np.ndarray:
    """``S <- diag(w) S - (a u)(u^T S) + k v^T`` with both terms reading the old ``S``;
    ``o = S^T r``."""
    heads, dim = int(mixer["heads"]), int(mixer["dim"])
    count = h.shape[0]
    r = (h @ t[prefix + "r"].T).reshape(count, heads, dim)
    k = (h @ t[prefix + "k"].T).reshape(count, heads, dim)
    v = (h @ t[prefix + "v"].T).reshape(count, heads, dim)
    raw = np.tanh(h @ t[prefix + "w1"].T) @ t[prefix + "w2"].T + t[prefix + "w0"]
    w = np.exp(-math.exp(-0.5) * sigmoid(raw)).reshape(count, heads, dim)
    a = sigmoid(h @ t[prefix + "a"].T + t[prefix + "a.b"]).reshape(count, heads, dim)
    u = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
    out = np.zeros((count, heads, dim))
    S = np.zeros((heads, dim, dim)) if state is None else state
    for step in range(count):
        for head in range(heads):
            old = S[head]
            uu = u[step, head]
            S[head] = w[step, head][:, None] * old \
                - np.outer(a[step, head] * uu, uu @ old) + np.outer(k[step, head], v[step, head])
            out[step, head] = S[head].T @ r[step, head]
    out = rms(out, None, eps).reshape(count, heads * dim) * t[prefix + "norm"]
    out = out * sigmoid(h @ t[prefix + "g"].T)
    return out @ t[prefix + "o"].T


def dense(h: np.ndarray, t: dict, prefix: str) -> np.ndarray:
    p, q = (float(z) for z in t[prefix + "act"])
    inner = xielu(h @ t[prefix + "up"].T + t[prefix + "up.b"], p, q)
    return inner @ t[prefix + "down"].T + t[prefix + "down.b"]


def mixture(h: np.ndarray, t: dict, prefix: str, mlp: dict) -> np.ndarray:
    experts, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    z = h @ t[prefix + "router"].T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z) / np.exp(z).sum(axis=-1, keepdims=True)
    out = np.zeros((h.shape[0], t[prefix + "e0.down"].shape[0]))
    for row in range(h.shape[0]):
        order = sorted(range(experts), key=lambda e: (-s[row, e], e))[:top]
        for e in order:
            inner = np.maximum(h[row] @ t[f"{prefix}e{e}.up"].T, 0.0) ** 2
            out[row] += s[row, e] * (inner @ t[f"{prefix}e{e}.down"].T)
    return out


def side_input(x: np.ndarray, tokens: np.ndarray, t: dict, layer: int, dim: int,
               eps: float) -> np.ndarray:
    e = t["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    g = gelu_tanh(x @ t[f"l{layer}.side.gate"].T) * e
    y = g @ t[f"l{layer}.side.proj"].T
    return rms(y, t[f"l{layer}.side.norm"], eps)


def forward(config: dict, t: dict, tokens: np.ndarray,
            keep: list[np.ndarray] | None = None) -> np.ndarray:
    """The residual stream after the last layer; ``keep`` collects it after every layer."""
    t = {name: np.asarray(value, dtype=np.float64) for name, value in t.items()}
    tokens = np.asarray(tokens)
    eps = float(config["norm"]["eps"])
    scale = float((config.get("embedding") or {}).get("scale") or 1.0)
    side_dim = int((config.get("token_side") or {}).get("dim") or 0)
    x = t["embed"][tokens] * scale
    for index, layer in enumerate(config["layers"]):
        p = f"l{index}."
        h = rms(x, t[p + "norm1"], eps)
        if layer["type"] == "attention":
            y = attention(h, t, p + "mix.", layer["mixer"], eps)
        else:
            y = delta_rule(h, t, p + "mix.", layer["mixer"], eps)
        x = x + rms(y, t[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms(x, t[p + "norm2"], eps)
            y = dense(h, t, p + "mlp.") if mlp["kind"] == "dense" \
                else mixture(h, t, p + "mlp.", mlp)
            x = x + rms(y, t[p + "norm2b"], eps)
        if side_dim:
            x = x + side_input(x, tokens, t, index, side_dim, eps)
        if keep is not None:
            keep.append(x.copy())
    return x


def logits(config: dict, t: dict, tokens: np.ndarray) -> np.ndarray:
    x = forward(config, t, tokens)
    eps = float(config["norm"]["eps"])
    final = rms(x, np.asarray(t["final.norm"], dtype=np.float64), eps)
    return final @ np.asarray(t["embed"], dtype=np.float64).T
