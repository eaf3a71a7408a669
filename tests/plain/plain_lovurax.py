"""A plain, slow statement of the Lovurax decoder: whole sequences, no cache, float64 on the CPU, one
function per mechanism, written from the design's equations and sharing nothing with the package.

A layer is pre-norm with gated residuals: with h = rmsnorm(x),
    x <- x + sigmoid(Rg h + rb) * sublayer(h)
first for the mixer, then (if the layer has one) for the feed-forward.  Mixers: `retention` (a linear
recurrence with a fixed decay per head), `attention` (grouped heads, sigmoid weights, no softmax) and
`latent_attention` (keys and values expanded from one low-rank row per position, softmax).  Weights are a
dict name -> tensor; a configuration is the dict of the model's config.json.
"""

from __future__ import annotations

import math

import torch

from .plain_llama import read_model_folder  # noqa: F401  (reads config.json and the safetensors file)

F = torch.float64


def rms_norm(x, weight=None, eps=1e-6):
    """x / sqrt(mean(x^2) + eps) over the last axis, times `weight` when there is one."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0.0)


def xielu(z, p, q):
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2."""
    ap, aq = softplus(p), 0.5 + softplus(q)
    return torch.where(z > 0, ap * z * z + 0.5 * z, aq * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z)


def rotate_half(x, positions, dims, base, angle_dtype=F):
    """x [T, heads, dim]: coordinate i of the first `dims` is paired with i + dims/2; the pair (u, v) at
    position p becomes (u cos a - v sin a, v cos a + u sin a), a = p * base^(-2i/dims).  The rest passes.
    `angle_dtype` float32: the frequency and the angle are rounded to 32 bits, as the design computes them (far from
    zero the angle's last bits are worth more than a float32 comparison forgives)."""
    if dims == 0:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=F)
    angle = (positions.to(angle_dtype)[:, None] * (base ** (-2.0 * i / dims)).to(angle_dtype)[None, :]).to(F)
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def retention_states(q, k, v, decay, start=None):
    """The recurrence itself, token by token, for one head: S_t = decay S_(t-1) + k_t v_t^T from `start` (zeros by
    default), o_t = S_t^T q_t.  q, k [T, D], v [T, Dv].  Returns o [T, Dv] and the last state."""
    S = torch.zeros(q.shape[1], v.shape[1], dtype=F) if start is None else start.clone()
    out = torch.zeros(q.shape[0], v.shape[1], dtype=F)
    for t in range(q.shape[0]):
        S = decay * S + torch.outer(k[t], v[t])
        out[t] = S.T @ q[t]
    return out, S


def retention_sums(q, k, v, decay):
    """The same o_t from a zero state, written out as sums: o_t = sum over j <= t of decay^(t - j) (q_t . k_j) v_j."""
    T = q.shape[0]
    t = torch.arange(T)
    distance = (t[:, None] - t[None, :]).clamp(min=0).to(F)
    weight = torch.where(t[:, None] >= t[None, :], torch.full((), float(decay), dtype=F) ** distance, torch.zeros((), dtype=F))
    return ((q @ k.T) * weight) @ v


def retention(h, w, m, eps):
    """Per head S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, from S = 0 at the start of the sequence, with q and k
    rotated and k times dim^(-1/2); o divided by its root mean square per head, times silu(G h), then the output matrix."""
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rotate_half((h @ w["q"].T).view(T, H, D), pos, rot["dims"], rot["base"])
    k = rotate_half((h @ w["k"].T).view(T, H, D), pos, rot["dims"], rot["base"]) * D ** -0.5
    v = (h @ w["v"].T).view(T, H, Dv)
    out = torch.stack([retention_sums(q[:, head], k[:, head], v[:, head], m["decay"][head]) for head in range(H)], dim=1)
    out = rms_norm(out, None, eps).reshape(T, H * Dv)
    g = h @ w["g"].T
    return (out * (g * sigmoid(g))) @ w["o"].T


def sigmoid_attention(h, w, m, eps):
    """Grouped heads; queries and keys RMS-normed per head with a gain shared by the heads; the query at
    position p times 1 + coef ln(floor((p + 1) / every) + 1); weight of key j <= i:
    sigmoid(scale q.k - slope_h (i - j) + pb_h), slope_h = 2^(-8 (h + 1) / H); no normalisation over keys;
    the heads side by side times sigmoid(G h), then the output matrix."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm((h @ w["q"].T).view(T, H, D), w["q.norm"], eps)
    k = rms_norm((h @ w["k"].T).view(T, G, D), w["k.norm"], eps)
    v = (h @ w["v"].T).view(T, G, Dv)
    pos = torch.arange(T)
    temp = m.get("q_temp")
    if temp:
        q = q * (1.0 + temp["coef"] * torch.log(torch.floor((pos + 1).to(F) / temp["every"]) + 1.0))[:, None, None]
    out = torch.zeros(T, H, Dv, dtype=F)
    distance = (pos[:, None] - pos[None, :]).to(F)
    visible = distance >= 0
    for head in range(H):
        c = head // (H // G)
        slope = 2.0 ** (-8.0 * (head + 1) / H)
        score = (q[:, head] @ k[:, c].T) * m["scale"] - slope * distance
        weight = torch.where(visible, sigmoid(score + w["pb"][head]), torch.zeros((), dtype=F))
        out[:, head] = weight @ v[:, c]
    return (out.reshape(T, H * Dv) * sigmoid(h @ w["g"].T)) @ w["o"].T


def latent_attention(h, w, m, eps):
    """c = rmsnorm(Dkv h) (the only thing a cache would keep); per head k = Uk c, v = Uv c; softmax over
    j <= i of scale q.k; head h's result times sigmoid((G h)_h); then the output matrix."""
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).view(T, H, D)
    c = rms_norm(h @ w["dkv"].T, w["dkv.norm"], eps)
    k = (c @ w["uk"].T).view(T, H, D)
    v = (c @ w["uv"].T).view(T, H, Dv)
    pos = torch.arange(T)
    visible = pos[:, None] >= pos[None, :]
    gate = sigmoid(h @ w["g"].T)
    out = torch.zeros(T, H, Dv, dtype=F)
    for head in range(H):
        score = (q[:, head] @ k[:, head].T) * m["scale"]
        score = torch.where(visible, score, torch.full((), -math.inf, dtype=F))
        out[:, head] = torch.softmax(score, dim=-1) @ v[:, head] * gate[:, head:head + 1]
    return out.reshape(T, H * Dv) @ w["o"].T


def dense_feed_forward(h, w):
    return xielu(h @ w["up"].T, w["act"][0], w["act"][1]) @ w["down"].T


MIXERS = {"retention": retention, "attention": sigmoid_attention, "latent_attention": latent_attention}


def sub(weights, prefix):
    """The tensors under `prefix`, as float64, with the prefix taken off their names."""
    return {name[len(prefix):]: t.to(F) for name, t in weights.items() if name.startswith(prefix)}


def forward(config, weights, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence; `layers_out` (a list) receives the stream after every layer."""
    eps = config["norm"]["eps"]
    W = {n: t.to(F) for n, t in weights.items()}
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = rms_norm(x, W[p + "norm1"], eps)
        mixed = MIXERS[layer["type"]](h, sub(weights, p + "mix."), layer["mixer"], eps)
        x = x + sigmoid(h @ W[p + "rg1"].T + W[p + "rg1.b"]) * mixed
        if layer.get("mlp") is not None:
            h = rms_norm(x, W[p + "norm2"], eps)
            x = x + sigmoid(h @ W[p + "rg2"].T + W[p + "rg2.b"]) * dense_feed_forward(h, sub(weights, p + "mlp."))
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, W["final.norm"], eps) @ W["embed"].T * config.get("logit_scale", 1.0)
