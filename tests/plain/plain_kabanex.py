"""A plain, slow implementation of the Kabanex decoder: whole sequences, no cache, no state carried between
calls, float64 on the CPU, one function per mechanism.  It shares no code with models_b200; it is what the
engine is compared with.

Notation: T tokens, W model width, H query heads, G key/value heads, D key size, Dv value size.
"""

from __future__ import annotations

import math

import torch

from .plain_llama import read_model_folder  # noqa: F401  (reads config.json and the safetensors file)

F = torch.float64


def layer_norm(x: torch.Tensor, gain: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(var + eps) * gain + bias with var = mean((x - mean)^2)."""
    mean = x.mean(dim=-1, keepdim=True)
    centred = x - mean
    var = (centred * centred).mean(dim=-1, keepdim=True)
    return centred / torch.sqrt(var + eps) * gain + bias


def rotate(t: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """t [T, heads, D]: coordinate i < dims/2 of every head is paired with coordinate i + dims/2; the pair
    (u, v) at position p turns by the angle p * base^(-2i/dims).  Coordinates from `dims` on stay."""
    if dims == 0:
        return t
    half = dims // 2
    out = t.clone()
    for i in range(half):
        angle = positions.to(F) * (base ** (-2.0 * i / dims))
        cos, sin = torch.cos(angle)[:, None], torch.sin(angle)[:, None]
        u, v = t[..., i], t[..., i + half]
        out[..., i] = u * cos - v * sin
        out[..., i + half] = v * cos + u * sin
    return out


def visible(tokens: int, window, keep_first: int) -> torch.Tensor:
    """[T, T] bool: query i sees key j iff j <= i and (i - j < window or j < keep_first); window None: j <= i."""
    mask = torch.zeros((tokens, tokens), dtype=torch.bool)
    for i in range(tokens):
        for j in range(i + 1):
            mask[i, j] = window is None or i - j < window or j < keep_first
    return mask


def talking_attention(q, k, v, talk, gate_logits, scale: float, window, keep_first: int) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, Dv] (already rotated), talk [H, H] or None, gate_logits [T, H] or
    None.  Returns [T, H, Dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    per = H // G
    mask = visible(T, window, keep_first)
    weights = torch.zeros((H, T, T), dtype=F)
    for h in range(H):
        scores = (q[:, h, :] @ k[:, h // per, :].T) * scale
        scores = scores.masked_fill(~mask, -math.inf)
        weights[h] = torch.softmax(scores, dim=-1)
    if talk is not None:
        weights = torch.einsum("hg,gij->hij", talk, weights)
    out = torch.stack([weights[h] @ v[:, h // per, :] for h in range(H)], dim=1)
    if gate_logits is not None:
        out = out * torch.sigmoid(gate_logits)[:, :, None]
    return out


def min_gru(z_in: torch.Tensor, x_in: torch.Tensor, start=None):
    """z_in, x_in [T, R] (biases already added).  Returns the states S_1..S_T [T, R]; S_0 = start or zero."""
    z = torch.sigmoid(z_in)
    candidate = torch.where(x_in >= 0, x_in + 0.5, torch.sigmoid(x_in))
    state = torch.zeros(z_in.shape[1], dtype=F) if start is None else start.to(F)
    states = []
    for t in range(z_in.shape[0]):
        state = (1.0 - z[t]) * state + z[t] * candidate[t]
        states.append(state)
    return torch.stack(states)


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def dense_feed_forward(h, up, down) -> torch.Tensor:
    """down . relu(up . h)^2"""
    return (torch.relu(h @ up.T) ** 2) @ down.T


def left_mixer(h, weights, prefix: str, c: dict) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, Dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    w = lambda name: weights[prefix + name].to(F)  # noqa: E731
    q = (h @ w("q").T).reshape(T, H, D)
    k = (h @ w("k").T).reshape(T, G, D)
    v = (h @ w("v").T).reshape(T, G, Dv)
    positions = torch.arange(T)
    rot = c.get("rot") or {"dims": 0, "base": 1.0}
    q, k = rotate(q, positions, rot["dims"], rot.get("base", 1.0)), rotate(k, positions, rot["dims"], rot.get("base", 1.0))
    mask = c.get("mask")
    out = talking_attention(q, k, v, w("talk"), h @ w("g").T, c["scale"], mask["size"] if mask else None,
                            (mask.get("keep_first") or 0) if mask else 0)
    return out.reshape(T, H * Dv) @ w("o").T


def right_mixer(h, weights, prefix: str) -> torch.Tensor:
    w = lambda name: weights[prefix + name].to(F)  # noqa: E731
    states = min_gru(h @ w("z").T + w("z.b"), h @ w("x").T + w("x.b"))
    return (states * silu(h @ w("g").T)) @ w("o").T


def forward(config: dict, weights: dict, tokens, hidden_out=None) -> torch.Tensor:
    """Logits [T, vocab] (float64) of the whole sequence.  `hidden_out`, a list, receives the residual
    stream after every layer."""
    eps = config["norm"]["eps"]
    x = weights["embed"].to(F)[torch.tensor(list(tokens), dtype=torch.long)]
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = layer_norm(x, weights[p + "norm1"].to(F), weights[p + "norm1.b"].to(F), eps)
        mixer = layer["mixer"]
        delta = mixer["left_scale"] * left_mixer(h, weights, p + "mix.left.", mixer["left"])
        delta = delta + mixer["right_scale"] * right_mixer(h, weights, p + "mix.right.")
        if layer.get("mlp") is not None:
            delta = delta + dense_feed_forward(h, weights[p + "mlp.up"].to(F), weights[p + "mlp.down"].to(F))
        x = x + delta
        if hidden_out is not None:
            hidden_out.append(x.clone())
    x = layer_norm(x, weights["final.norm"].to(F), weights["final.norm.b"].to(F), eps)
    return x @ weights["head"].to(F).T
